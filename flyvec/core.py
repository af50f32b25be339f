"""``flyvec.core``: the reference's module name for :class:`FlyVec` and its helpers (flyvec/core.py)."""
from flyvec_b200.core import *  # noqa: F401,F403
from flyvec_b200.core import FlyVec, normalize_synapses, softmax  # noqa: F401
