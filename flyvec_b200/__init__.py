"""flyvec_b200: FlyVec trainer and hasher for NVIDIA B200 behind the reference's API."""
__version__ = "0.1.0"
from .core import FlyVec  # noqa: F401
from .tokenizer import GensimTokenizer, VocabTokenizer  # noqa: F401
