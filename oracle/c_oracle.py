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


def set_num_threads(n: int) -> None:
    """OpenMP threads of the C oracle (overrides an inherited OMP_NUM_THREADS)."""
    L = lib()
    L.orc_set_num_threads.restype = None
    L.orc_set_num_threads.argtypes = [C.c_int]
    L.orc_set_num_threads(int(n))


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


# ---------------------------------------------------------------------------
# The reference's own training kernels on the host (oracle/_ref/ref_kernels_host.so)
# ---------------------------------------------------------------------------
_refk = None


def reference_kernels():
    """ctypes handle of the host build of the reference's kernels, or None when it
    neither exists nor can be built (no reference checkout)."""
    global _refk
    if _refk is None:
        path = build_oracle.build_reference_kernels()
        if path is None or not path.exists():
            return None
        L = C.CDLL(str(path))
        L.refk_train_step.restype = C.c_int
        L.refk_train_step.argtypes = ([C.c_int] * 7 + [C.c_void_p] * 3 + [C.c_uint64] + [C.c_void_p] * 2
                                      + [C.c_float] * 3 + [C.c_void_p] * 10)
        L.refk_get_max.restype = C.c_int
        L.refk_get_max.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        _refk = L
    return _refk


def reference_winners(a, m=2):
    """``get_max_and_m_max_kernel_2`` (flyvec/src/cuda_funcs.cu:488-561) as the reference
    launches it (64 threads per window), on activations ``a`` [Num][hid].
    Returns (winner, m-th winner) or None without the host build."""
    L = reference_kernels()
    if L is None:
        return None
    a = np.array(a, np.float32, order="C", copy=True)
    ids = np.zeros((a.shape[0], 2), np.int32)
    assert L.refk_get_max(a.shape[0], a.shape[1], m, a.ctypes.data, ids.ctypes.data) == 0
    return ids[:, 0].copy(), ids[:, 1].copy()


def reference_train_step(Wm, tokens, starts, order, f, V, W, B, G, eps, delta=0.0, prec=1e-30, m=2):
    """One global step through the reference's own kernels, in the reference's launch
    sequence (see oracle/ref_kernels_host.cpp).  ``order`` holds at least ``G*B`` window
    ids; device ``g`` takes ``order[g*B:(g+1)*B]``.  Returns a dict or None without the
    host build."""
    L = reference_kernels()
    if L is None:
        return None
    Wm = np.ascontiguousarray(Wm, np.float32)
    K, N = Wm.shape
    tokens = np.ascontiguousarray(tokens, np.int32)
    starts = np.ascontiguousarray(starts, np.uint64)
    order = np.ascontiguousarray(order[:G * B], np.uint64)
    assert order.size == G * B
    f = np.ascontiguousarray(f, np.float32)
    out = dict(idx=np.zeros((G, B, W), np.int32), a_w=np.zeros((G, B, K), np.float32), a_r=np.zeros((G, B, K), np.float32),
               ids=np.zeros((G, B, 2), np.int32), xx=np.zeros((G, K), np.float32), D=np.zeros((K, N), np.float32),
               W=np.zeros((K, N), np.float32))
    nc, s, same = C.c_float(0), C.c_float(0), C.c_int(0)
    rc = L.refk_train_step(K, N, V, W, B, G, m, Wm.ctypes.data, tokens.ctypes.data, starts.ctypes.data, starts.size,
                           order.ctypes.data, f.ctypes.data, C.c_float(eps), C.c_float(delta), C.c_float(prec),
                           out["idx"].ctypes.data, out["a_w"].ctypes.data, out["a_r"].ctypes.data, out["ids"].ctypes.data,
                           out["xx"].ctypes.data, out["D"].ctypes.data, out["W"].ctypes.data, C.addressof(nc), C.addressof(s),
                           C.addressof(same))
    assert rc == 0
    out.update(nc=np.float32(nc.value), s=np.float32(s.value), replicas_identical=bool(same.value),
               win=out["ids"][:, :, 0], mmax=out["ids"][:, :, 1])
    return out
