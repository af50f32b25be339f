"""ctypes access to oracle/_build/liboracle.so and oracle/_ref/prune_input.so
(test infrastructure only; see oracle/build_oracle.py)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import build_oracle

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = build_oracle.build_oracle_lib()
        L = C.CDLL(str(path))
        L.orc_train_step.restype = C.c_int
        L.orc_train_step.argtypes = [C.c_int] * 6 + [C.c_void_p] * 4 + [C.c_float, C.c_float] + [C.c_void_p] * 5
        L.orc_hash_tokens.restype = C.c_int
        L.orc_hash_tokens.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
        L.orc_num_threads.restype = C.c_int
        _lib = L
    return _lib


def num_threads() -> int:
    return lib().orc_num_threads()


class StepRunner:
    """Holds the scratch memory for repeated calls of the C train step."""

    def __init__(self, K, N, V, W, B, G):
        self.dims = (K, N, V, W, B, G)
        self.scratch = np.empty((G + 1) * K * N, np.float32)

    def step(self, Wm, idx, nwin, f, eps, prec=1e-30):
        """``Wm`` float32 [K][N] is updated in place.  Returns (win [G][B], xx [G][K], nc, s)."""
        K, N, V, W, B, G = self.dims
        assert Wm.dtype == np.float32 and Wm.flags.c_contiguous and Wm.shape == (K, N)
        idx = np.ascontiguousarray(idx, np.int32).reshape(G, B, W)
        nwin = np.ascontiguousarray(nwin, np.int32)
        f = np.ascontiguousarray(f, np.float32)
        win = np.empty((G, B), np.int32)
        xx = np.empty((G, K), np.float32)
        nc, s = C.c_float(0), C.c_float(0)
        rc = lib().orc_train_step(K, N, V, W, B, G, Wm.ctypes.data, idx.ctypes.data, nwin.ctypes.data, f.ctypes.data,
                                  C.c_float(eps), C.c_float(prec), win.ctypes.data, xx.ctypes.data,
                                  C.addressof(nc), C.addressof(s), self.scratch.ctypes.data)
        assert rc == 0
        return win, xx, np.float32(nc.value), np.float32(s.value)


def hash_tokens(syn, V, ids, h):
    syn = np.ascontiguousarray(syn, np.float32)
    ids = np.ascontiguousarray(ids, np.int32)
    K, N = syn.shape
    out = np.empty((ids.size, K), np.int8)
    rc = lib().orc_hash_tokens(syn.ctypes.data, K, N, V, ids.ctypes.data, ids.size, h, out.ctypes.data)
    assert rc == 0
    return out


def reference_enumerate_windows(offsets, W):
    """The reference's own getnum_samples / compute_offset_phrases
    (flyvec/src/prune_input.cpp:63-122) from oracle/_ref/prune_input.so.
    Returns None when that library has not been built."""
    path = build_oracle.REF_OUT / "prune_input.so"
    if not path.exists():
        if build_oracle.build_reference_prune_input() is None:
            return None
    L = C.CDLL(str(path))
    L.getnum_samples.restype = C.c_uint64
    L.getnum_samples.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64]
    L.compute_offset_phrases.restype = None
    L.compute_offset_phrases.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64]
    off = np.ascontiguousarray(offsets, np.uint64)
    nch = off.size - 1
    n = L.getnum_samples(off.ctypes.data, nch, W)
    out = np.zeros(n + 1, np.uint64)
    L.compute_offset_phrases(out.ctypes.data, off.ctypes.data, nch, W)
    return out[:n]
