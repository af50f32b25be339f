"""``flyvec``: the reference's import name (flyvec/__init__.py:2-5 exports ``FlyVec`` and
``GensimTokenizer``) over the B200 library, so that ``from flyvec import FlyVec`` keeps working
for code written against bhoov/flyvec."""
from flyvec_b200 import __version__  # noqa: F401
from flyvec_b200.core import FlyVec
from flyvec_b200.tokenizer import GensimTokenizer

__all__ = ["FlyVec", "GensimTokenizer"]
