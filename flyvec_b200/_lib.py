"""ctypes binding of ``libflyvec_b200.so`` (declared in ``include/flyvec_b200.h``).

The reference binds its five shared objects the same way
(flyvec/train_flyvec.py:62-139) but assigns its prototypes to a misspelt
attribute, so none are applied; here every entry point gets real ``argtypes``
and ``restype`` and a non-zero status raises.

There is no fallback: if the library has not been built, or a call fails,
an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

CSRC = Path(__file__).resolve().parent / "csrc"
LIB_PATH = CSRC / "libflyvec_b200.so"
HEADER = Path(__file__).resolve().parent.parent / "include" / "flyvec_b200.h"

FV_FLAG_COUNT_FP32 = 1
FV_FLAG_ACC_FP64 = 2
FV_FLAG_FOLD_EVERY_STEP = 4
FV_FLAG_EMULATE_RANKS = 8
FV_HASH_PACKED = 0
FV_HASH_BYTES = 1
FV_HASH_RAW = 2
FV_HASH_NO_UNK = 4
FV_HASH_EXACT = 8

STATUS_NAMES = {1: "FV_ERR_INVALID", 2: "FV_ERR_CUDA", 3: "FV_ERR_COMM", 4: "FV_ERR_STATE", 5: "FV_ERR_DATA",
                6: "FV_ERR_TIMEOUT"}


class FlyvecError(RuntimeError):
    """A library call returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


class FvConfig(C.Structure):
    _fields_ = [
        ("struct_size", C.c_uint32), ("device", C.c_int32), ("rank", C.c_int32), ("world", C.c_int32),
        ("hid", C.c_uint32), ("vocab", C.c_uint32), ("window", C.c_uint32), ("batch", C.c_uint32),
        ("lr0", C.c_float), ("delta", C.c_float), ("prec", C.c_float),
        ("m", C.c_uint32), ("maxlen", C.c_uint32), ("flags", C.c_uint32),
    ]


class FvRunStats(C.Structure):
    _fields_ = [
        ("steps", C.c_uint64), ("windows", C.c_uint64), ("seconds", C.c_double), ("fwd_seconds", C.c_double),
        ("exch_seconds", C.c_double), ("upd_seconds", C.c_double), ("kernel_launches", C.c_uint64),
        ("last_nc", C.c_float), ("last_scale", C.c_float), ("device_error", C.c_uint32), ("timed_steps", C.c_uint32),
    ]

    def as_dict(self):
        return {k: getattr(self, k) for k, _ in self._fields_}


_P = C.c_void_p
_PROTOTYPES = {
    "fv_version": ([], C.c_int),
    "fv_last_error": ([], C.c_char_p),
    "fv_device_count": ([C.POINTER(C.c_int)], C.c_int),
    "fv_enumerate_windows": ([_P, C.c_uint64, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint64), _P], C.c_int),
    "fv_inverse_frequency": ([_P, C.c_uint64, C.c_uint32, C.c_int, _P], C.c_int),
    "fv_trainer_create": ([C.POINTER(FvConfig), C.POINTER(_P)], C.c_int),
    "fv_trainer_destroy": ([_P], C.c_int),
    "fv_trainer_set_corpus": ([_P, _P, C.c_uint64, _P, C.c_uint64], C.c_int),
    "fv_trainer_set_corpus_windows": ([_P, _P, C.c_uint64, _P, C.c_uint64], C.c_int),
    "fv_trainer_get_window_starts": ([_P, _P], C.c_int),
    "fv_trainer_num_windows": ([_P, C.POINTER(C.c_uint64)], C.c_int),
    "fv_trainer_get_inverse_frequency": ([_P, _P], C.c_int),
    "fv_trainer_set_inverse_frequency": ([_P, _P], C.c_int),
    "fv_trainer_set_weights": ([_P, _P], C.c_int),
    "fv_trainer_get_weights": ([_P, _P], C.c_int),
    "fv_trainer_set_permutation": ([_P, _P, C.c_uint64], C.c_int),
    "fv_trainer_shuffle": ([_P, C.c_uint64], C.c_int),
    "fv_trainer_get_permutation": ([_P, _P], C.c_int),
    "fv_trainer_run_epoch": ([_P, C.c_uint64, C.c_uint64, C.POINTER(FvRunStats)], C.c_int),
    "fv_trainer_run_steps": ([_P, C.c_uint64, C.c_uint64, C.c_float, _P, _P, C.POINTER(FvRunStats)], C.c_int),
    "fv_trainer_run_steps_timed": ([_P, C.c_uint64, C.c_uint64, C.c_uint64, C.c_float, C.POINTER(FvRunStats)], C.c_int),
    "fv_trainers_link": ([C.POINTER(_P), C.c_int32], C.c_int),
    "fv_trainers_run_steps": ([C.POINTER(_P), C.c_int32, C.c_uint64, C.c_uint64, C.c_uint64, C.c_float, _P, _P,
                               C.POINTER(FvRunStats)], C.c_int),
    "fv_trainers_run_epoch": ([C.POINTER(_P), C.c_int32, C.c_uint64, C.c_uint64, C.POINTER(FvRunStats)], C.c_int),
    "fv_trainer_last_packets": ([_P, _P, _P], C.c_int),
    "fv_trainer_run_steps_host": ([_P, _P, C.c_uint64, C.c_float, _P, _P, C.POINTER(FvRunStats)], C.c_int),
    "fv_trainer_run_steps_host_local": ([_P, _P, C.c_uint64, C.c_float, _P, _P, C.POINTER(FvRunStats)], C.c_int),
    "fv_trainer_step_debug": ([_P, C.c_uint64, C.c_float, _P, _P, C.POINTER(C.c_float), C.POINTER(C.c_float)],
                              C.c_int),
    "fv_trainer_time_forward": ([_P, C.c_uint64, C.c_uint32, C.POINTER(C.c_double)], C.c_int),
    "fv_comm_unique_id": ([_P], C.c_int),
    "fv_trainer_init_comm": ([_P, _P], C.c_int),
    "fv_trainer_set_option": ([_P, C.c_char_p, C.c_double], C.c_int),
    "fv_trainer_get_counter": ([_P, C.c_char_p, C.POINTER(C.c_uint64)], C.c_int),
    "fv_trainer_comm_mode": ([_P, C.POINTER(C.c_int)], C.c_int),
    "fv_shard_range": ([C.c_uint64, C.c_uint32, C.c_int32, C.c_int32, C.c_uint64, C.POINTER(C.c_uint64),
                        C.POINTER(C.c_uint64)], C.c_int),
    "fv_hasher_create": ([_P, C.c_uint32, C.c_uint32, C.c_int, C.c_float, C.c_int, C.POINTER(_P)], C.c_int),
    "fv_hasher_destroy": ([_P], C.c_int),
    "fv_hasher_get_weights": ([_P, _P], C.c_int),
    "fv_hash_tokens": ([_P, _P, C.c_uint64, C.c_uint32, C.c_uint32, _P], C.c_int),
    "fv_hash_tokens_static": ([_P, _P, C.c_uint64, C.c_uint32, C.c_uint32, _P], C.c_int),
    "fv_hash_windows": ([_P, _P, C.c_uint64, C.c_uint32, _P, C.c_uint32, C.c_uint32, _P], C.c_int),
    "fv_hash_tokens_device": ([_P, _P, C.c_uint64, C.c_uint32, C.c_uint32, _P, C.POINTER(C.c_double)], C.c_int),
    "fv_hash_windows_device": ([_P, _P, C.c_uint64, C.c_uint32, C.c_int, C.c_uint32, C.c_uint32, _P,
                                C.POINTER(C.c_double)], C.c_int),
    "fv_hasher_set_inverse_frequency": ([_P, _P, C.c_uint32], C.c_int),
    "fv_device_alloc": ([C.c_int, C.c_size_t, C.POINTER(_P)], C.c_int),
    "fv_device_free": ([C.c_int, _P], C.c_int),
    "fv_host_alloc_pinned": ([C.c_size_t, C.POINTER(_P)], C.c_int),
    "fv_host_free_pinned": ([_P], C.c_int),
    "fv_device_mem_info": ([C.c_int, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)], C.c_int),
    "fv_copy_to_device": ([C.c_int, _P, _P, C.c_size_t], C.c_int),
    "fv_copy_to_host": ([C.c_int, _P, _P, C.c_size_t], C.c_int),
    "fv_flush_l2": ([C.c_int, C.c_size_t], C.c_int),
    "fv_probe_read_bandwidth": ([C.c_int, C.c_int, C.c_size_t, C.c_uint32, C.c_uint32, C.POINTER(C.c_double)], C.c_int),
}

_lib = None


def build(verbose: bool = False) -> Path:
    """Compile the library in-tree for sm_100a (what ``flyvec_compile`` runs)."""
    res = subprocess.run(["make", "-C", str(CSRC), "-j4"], capture_output=True, text=True)
    if verbose or res.returncode != 0:
        print(res.stdout)
        print(res.stderr)
    if res.returncode != 0:
        raise RuntimeError("building libflyvec_b200.so failed")
    make_ref_abi_links()
    return LIB_PATH


#: the five shared objects the reference's driver loads (flyvec/train_flyvec.py:62-66)
REF_ABI_NAMES = ("model_descriptor.so", "model_arrays.so", "cuda_helpers.so", "cuda_funcs.so", "prune_input.so")
REF_ABI_DIR = CSRC / "ref_abi"


def make_ref_abi_links() -> Path:
    """Directory in which the reference's five library names all resolve to this library, for running
    the reference's own ``train_flyvec.py`` unmodified (set its ``BIN`` there)."""
    REF_ABI_DIR.mkdir(exist_ok=True)
    for name in REF_ABI_NAMES:
        link = REF_ABI_DIR / name
        if link.is_symlink() or link.exists():
            link.unlink()
        link.symlink_to(Path("..") / LIB_PATH.name)
    return REF_ABI_DIR


def lib() -> C.CDLL:
    """The loaded library with prototypes applied.  Raises if it is not built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: run `flyvec_compile` (or `make -C {CSRC}`) first; there is no CPU fallback")
        handle = C.CDLL(str(LIB_PATH), mode=os.RTLD_GLOBAL if hasattr(os, "RTLD_GLOBAL") else C.DEFAULT_MODE)
        for name, (argtypes, restype) in _PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise FlyvecError(status, lib().fv_last_error().decode("utf-8", "replace"))


def ptr(a: np.ndarray):
    return C.c_void_p(a.ctypes.data)


def as_c(a, dtype) -> np.ndarray:
    """C-contiguous array of ``dtype`` (no copy when it already is one)."""
    return np.ascontiguousarray(a, dtype=dtype)


def pinned_empty(shape, dtype) -> np.ndarray:
    """numpy view over page-locked host memory (flyvec/train_flyvec.py:159-163
    does the same over ``do_gpu_cudaHostAlloc``).  The memory lives until exit."""
    n = int(np.prod(shape)) * np.dtype(dtype).itemsize
    p = C.c_void_p()
    check(lib().fv_host_alloc_pinned(n, C.byref(p)))
    buf = (C.c_char * n).from_address(p.value)
    return np.frombuffer(buf, dtype=dtype).reshape(shape)


def device_free_bytes(device: int = 0) -> int:
    """Free device memory as cudaMemGetInfo reports it."""
    free, total = C.c_size_t(0), C.c_size_t(0)
    check(lib().fv_device_mem_info(device, C.byref(free), C.byref(total)))
    return free.value


def device_count() -> int:
    n = C.c_int(0)
    check(lib().fv_device_count(C.byref(n)))
    return n.value
