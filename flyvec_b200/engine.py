"""Thin Python objects over the C ABI: one :class:`Trainer` per GPU (rank) and a
:class:`Hasher`.  They only marshal numpy arrays; all arithmetic runs in the
CUDA library."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import FvConfig, FvRunStats, as_c, check, ptr


class Trainer:
    """One data-parallel rank of the FlyVec trainer (the role of the reference's
    ``model_descriptor`` + ``model_arrays`` pair, flyvec/train_flyvec.py:141-229)."""

    def __init__(self, hid: int, vocab: int, window: int = 11, batch: int = 10000, lr0: float = 0.002,
                 delta: float = 0.0, prec: float = 1e-30, device: int = 0, rank: int = 0, world: int = 1,
                 flags: int = 0, maxlen: int = 0, m: int = 2):
        self._h = C.c_void_p()
        self.cfg = FvConfig(C.sizeof(FvConfig), device, rank, world, hid, vocab, window, batch, lr0, delta, prec, m,
                            maxlen, flags)
        self.K, self.V, self.N, self.W, self.B, self.G, self.rank = hid, vocab, 2 * vocab, window, batch, world, rank
        check(_lib.lib().fv_trainer_create(C.byref(self.cfg), C.byref(self._h)))

    # -- lifetime -----------------------------------------------------------
    def close(self):
        if self._h:
            _lib.lib().fv_trainer_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- data ---------------------------------------------------------------
    def set_corpus(self, encodings: np.ndarray, offsets: np.ndarray) -> int:
        enc = as_c(encodings, np.int32)
        off = as_c(offsets, np.uint64)
        check(_lib.lib().fv_trainer_set_corpus(self._h, ptr(enc), enc.size, ptr(off), off.size))
        return self.num_windows

    @property
    def num_windows(self) -> int:
        n = C.c_uint64(0)
        check(_lib.lib().fv_trainer_num_windows(self._h, C.byref(n)))
        return n.value

    def window_starts(self) -> np.ndarray:
        st = np.empty(self.num_windows, np.uint64)
        check(_lib.lib().fv_trainer_get_window_starts(self._h, ptr(st)))
        return st

    @property
    def steps_per_epoch(self) -> int:
        per = self.G * self.B
        return (self.num_windows + per - 1) // per

    def inverse_frequency(self) -> np.ndarray:
        f = np.empty(self.V, np.float32)
        check(_lib.lib().fv_trainer_get_inverse_frequency(self._h, ptr(f)))
        return f

    def set_inverse_frequency(self, f: np.ndarray):
        f = as_c(f, np.float32)
        assert f.size == self.V
        check(_lib.lib().fv_trainer_set_inverse_frequency(self._h, ptr(f)))

    def set_weights(self, w: np.ndarray):
        w = as_c(w, np.float32)
        if w.shape != (self.K, self.N):
            raise ValueError(f"weights must have shape ({self.K}, {self.N}), got {w.shape}")
        check(_lib.lib().fv_trainer_set_weights(self._h, ptr(w)))

    def get_weights(self) -> np.ndarray:
        w = np.empty((self.K, self.N), np.float32)
        check(_lib.lib().fv_trainer_get_weights(self._h, ptr(w)))
        return w

    def set_permutation(self, perm: np.ndarray):
        perm = as_c(perm, np.uint64)
        check(_lib.lib().fv_trainer_set_permutation(self._h, ptr(perm), perm.size))

    def shuffle(self, seed: int):
        check(_lib.lib().fv_trainer_shuffle(self._h, C.c_uint64(seed & (2 ** 64 - 1))))

    def get_permutation(self) -> np.ndarray:
        perm = np.empty(self.num_windows, np.uint64)
        check(_lib.lib().fv_trainer_get_permutation(self._h, ptr(perm)))
        return perm

    # -- running ------------------------------------------------------------
    def run_epoch(self, epoch: int, nep: int) -> dict:
        st = FvRunStats()
        check(_lib.lib().fv_trainer_run_epoch(self._h, epoch, nep, C.byref(st)))
        return st.as_dict()

    def run_steps(self, first_step: int, nsteps: int, eps: float, want_log: bool = False):
        st = FvRunStats()
        nc = np.empty(nsteps, np.float32) if want_log else None
        sc = np.empty(nsteps, np.float32) if want_log else None
        check(_lib.lib().fv_trainer_run_steps(self._h, first_step, nsteps, eps, ptr(nc) if want_log else None,
                                              ptr(sc) if want_log else None, C.byref(st)))
        d = st.as_dict()
        if want_log:
            d["nc"], d["scale"] = nc, sc
        return d

    def run_steps_host(self, idx_host: np.ndarray, nsteps: int, eps: float, nc_out: np.ndarray | None = None):
        """``idx_host``: int32 ``[nsteps, world*batch, window]`` input ids in host
        (ideally pinned) memory; uploaded inside the call."""
        assert idx_host.dtype == np.int32 and idx_host.flags.c_contiguous
        assert idx_host.size == nsteps * self.G * self.B * self.W
        st = FvRunStats()
        check(_lib.lib().fv_trainer_run_steps_host(self._h, ptr(idx_host), nsteps, eps,
                                                   ptr(nc_out) if nc_out is not None else None, None, C.byref(st)))
        return st.as_dict()

    def run_steps_host_local(self, idx_local: np.ndarray, nsteps: int, eps: float, nc_out: np.ndarray | None = None):
        """``idx_local``: int32 ``[nsteps, batch, window]`` input ids of THIS rank's windows only; the ranks'
        ids are all-gathered on the GPUs, a block of steps ahead of the step loop."""
        assert idx_local.dtype == np.int32 and idx_local.flags.c_contiguous
        assert idx_local.size == nsteps * self.B * self.W
        st = FvRunStats()
        check(_lib.lib().fv_trainer_run_steps_host_local(self._h, ptr(idx_local), nsteps, eps,
                                                         ptr(nc_out) if nc_out is not None else None, None, C.byref(st)))
        return st.as_dict()

    def step_debug(self, step: int, eps: float):
        win = np.empty(self.G * self.B, np.int32)
        xx = np.empty((self.G, self.K), np.float32)
        nc, sc = C.c_float(0), C.c_float(0)
        check(_lib.lib().fv_trainer_step_debug(self._h, step, eps, ptr(win), ptr(xx), C.byref(nc), C.byref(sc)))
        return win.reshape(self.G, self.B), xx, np.float32(nc.value), np.float32(sc.value)

    def run_steps_timed(self, first_step: int, nsteps: int, warmup: int, eps: float) -> dict:
        """``nsteps`` steps in one call, the first ``warmup`` of them outside the timed region."""
        st = FvRunStats()
        check(_lib.lib().fv_trainer_run_steps_timed(self._h, first_step, nsteps, warmup, eps, C.byref(st)))
        return st.as_dict()

    def last_packets(self):
        """Winners ``[world][batch]`` and xx ``[world][K]`` of the last step as this rank holds them."""
        win = np.empty(self.G * self.B, np.int32)
        xx = np.empty((self.G, self.K), np.float32)
        check(_lib.lib().fv_trainer_last_packets(self._h, ptr(win), ptr(xx)))
        return win.reshape(self.G, self.B), xx

    def time_forward(self, step: int, reps: int = 50) -> float:
        """Seconds per launch of the fused gather/arg-max kernel, back-to-back launches."""
        sec = C.c_double(0)
        check(_lib.lib().fv_trainer_time_forward(self._h, step, reps, C.byref(sec)))
        return sec.value

    # -- multi-GPU ----------------------------------------------------------
    @staticmethod
    def comm_unique_id() -> bytes:
        buf = (C.c_uint8 * 128)()
        check(_lib.lib().fv_comm_unique_id(buf))
        return bytes(buf)

    def init_comm(self, uid: bytes):
        assert len(uid) == 128
        buf = (C.c_uint8 * 128).from_buffer_copy(uid)
        check(_lib.lib().fv_trainer_init_comm(self._h, buf))


    def set_option(self, key: str, value: float):
        """Tuning knobs that change no result: ``spin_limit``, ``tag_variant``."""
        check(_lib.lib().fv_trainer_set_option(self._h, key.encode(), float(value)))

    def counter(self, key: str) -> int:
        """Counters since creation, e.g. ``matrix_scans``."""
        v = C.c_uint64(0)
        check(_lib.lib().fv_trainer_get_counter(self._h, key.encode(), C.byref(v)))
        return v.value

    @property
    def comm_mode(self) -> int:
        """0 = single rank, 1 = NCCL all-gather per step, 2 = peer-memory mailboxes."""
        m = C.c_int(0)
        check(_lib.lib().fv_trainer_comm_mode(self._h, C.byref(m)))
        return m.value


class TrainerGroup:
    """All ranks of a data-parallel job in ONE process (the reference's arrangement,
    flyvec/train_flyvec.py:141-229): ``devices[r]`` is rank ``r``'s GPU.  Distinct devices run
    concurrently, one host thread each; the same device repeated runs the ranks phase by phase
    on one GPU (for tests)."""

    def __init__(self, devices, hid: int, vocab: int, window: int = 11, batch: int = 10000, lr0: float = 0.002,
                 delta: float = 0.0, prec: float = 1e-30, flags: int = 0, maxlen: int = 0, shard: bool | None = None):
        n = len(devices)
        self.ranks = [Trainer(hid, vocab, window, batch, lr0, delta, prec, device=dev, rank=r, world=n, flags=flags,
                              maxlen=maxlen) for r, dev in enumerate(devices)]
        self.n = n
        self._arr = (C.c_void_p * n)(*[t._h for t in self.ranks])
        check(_lib.lib().fv_trainers_link(self._arr, n))
        if shard is not None and n > 1:
            for t in self.ranks:
                t.set_option("shard", 1 if shard else 0)

    def close(self):
        for t in self.ranks:
            t.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def set_corpus(self, encodings, offsets) -> int:
        return [t.set_corpus(encodings, offsets) for t in self.ranks][0]

    def set_weights(self, w):
        for t in self.ranks:
            t.set_weights(w)

    def set_permutation(self, perm):
        for t in self.ranks:
            t.set_permutation(perm)

    def shuffle(self, seed: int):
        for t in self.ranks:
            t.shuffle(seed)

    @property
    def steps_per_epoch(self) -> int:
        return self.ranks[0].steps_per_epoch

    def run_steps(self, first_step: int, nsteps: int, eps: float, warmup: int = 0, want_log: bool = False):
        stats = (FvRunStats * self.n)()
        nc = np.empty(nsteps, np.float32) if want_log else None
        sc = np.empty(nsteps, np.float32) if want_log else None
        check(_lib.lib().fv_trainers_run_steps(self._arr, self.n, first_step, nsteps, warmup, eps,
                                               ptr(nc) if want_log else None, ptr(sc) if want_log else None, stats))
        out = [s.as_dict() for s in stats]
        if want_log:
            out[0]["nc"], out[0]["scale"] = nc, sc
        return out

    def run_epoch(self, epoch: int, nep: int):
        stats = (FvRunStats * self.n)()
        check(_lib.lib().fv_trainers_run_epoch(self._arr, self.n, epoch, nep, stats))
        return [s.as_dict() for s in stats]

    def step_debug(self, step: int, eps: float):
        """One step; winners ``[world][batch]`` and xx ``[world][K]`` as rank 0 received them, nc, scale."""
        st = self.run_steps(step, 1, eps, want_log=True)
        win, xx = self.ranks[0].last_packets()
        return win, xx, st[0]["nc"][0], st[0]["scale"][0]

    def get_weights(self, rank: int = 0) -> np.ndarray:
        return self.ranks[rank].get_weights()


def shard_range(num_windows: int, batch: int, world: int, rank: int, step: int):
    """Windows ``[first, first+count)`` of the current order that ``rank`` owns in
    global step ``step`` (flyvec/src/cuda_funcs.cu:1667-1670)."""
    a, b = C.c_uint64(0), C.c_uint64(0)
    check(_lib.lib().fv_shard_range(num_windows, batch, world, rank, step, C.byref(a), C.byref(b)))
    return a.value, b.value


def enumerate_windows(offsets: np.ndarray, window: int, maxlen: int = 0) -> np.ndarray:
    off = as_c(offsets, np.uint64)
    n = C.c_uint64(0)
    nch = max(off.size - 1, 0)
    check(_lib.lib().fv_enumerate_windows(ptr(off), nch, window, maxlen, C.byref(n), None))
    starts = np.empty(n.value, np.uint64)
    check(_lib.lib().fv_enumerate_windows(ptr(off), nch, window, maxlen, C.byref(n), ptr(starts)))
    return starts


def inverse_frequency(encodings: np.ndarray, vocab: int, saturate: bool = False) -> np.ndarray:
    enc = as_c(encodings, np.int32)
    f = np.empty(vocab, np.float32)
    check(_lib.lib().fv_inverse_frequency(ptr(enc), enc.size, vocab, int(saturate), ptr(f)))
    return f


class Hasher:
    """Synapses resident on one GPU plus the two hashing entry points."""

    def __init__(self, synapses: np.ndarray, normalize: bool = False, prec: float = 1.0e-32, device: int = 0):
        w = as_c(synapses, np.float32)
        if w.ndim != 2 or w.shape[1] % 2:
            raise ValueError("synapses must be float32 [K][2V]")
        self.K, self.N = w.shape
        self.V = self.N // 2
        self.device = device
        self._h = C.c_void_p()
        check(_lib.lib().fv_hasher_create(ptr(w), self.K, self.N, int(normalize), prec, device, C.byref(self._h)))

    def close(self):
        if self._h:
            _lib.lib().fv_hasher_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def weights(self) -> np.ndarray:
        w = np.empty((self.K, self.N), np.float32)
        check(_lib.lib().fv_hasher_get_weights(self._h, ptr(w)))
        return w

    def code_bytes(self, packed: bool) -> int:
        return (self.K + 7) // 8 if packed else self.K

    def _out(self, out, n: int, packed: bool) -> np.ndarray:
        """Result array: the caller's (uint8, C-contiguous, e.g. page-locked) or a fresh one."""
        shape = (n, self.code_bytes(packed))
        if out is None:
            return np.empty(shape, np.uint8)
        if out.dtype != np.uint8 or not out.flags.c_contiguous or out.shape != shape:
            raise ValueError(f"out must be a C-contiguous uint8 array of shape {shape}")
        return out

    def hash_tokens(self, ids, hash_length: int = 50, packed: bool = False, zero_unknown: bool = True,
                    out: np.ndarray | None = None) -> np.ndarray:
        ids = as_c(ids, np.int32).reshape(-1)
        flags = (_lib.FV_HASH_PACKED if packed else _lib.FV_HASH_BYTES) | (0 if zero_unknown else _lib.FV_HASH_NO_UNK)
        out = self._out(out, ids.size, packed)
        check(_lib.lib().fv_hash_tokens(self._h, ptr(ids), ids.size, hash_length, flags, ptr(out)))
        return out if packed else out.view(np.int8)

    #: size of the library's fixed staging area used by :meth:`hash_tokens_static`
    STATIC_SCRATCH_BYTES = 8 << 20

    def hash_tokens_static(self, ids, hash_length: int = 50, packed: bool = False) -> np.ndarray:
        """Like :meth:`hash_tokens`, but through the entry point that allocates no device
        memory: for hashing small batches while a trainer is busy on the same GPU, or when
        another pool owns the device memory.  The batch must fit the fixed staging area
        (``len(ids) * (4 + bytes per code) + 256 <= 8 MiB``); concurrent calls on one GPU
        must be serialised by the caller."""
        ids = as_c(ids, np.int32).reshape(-1)
        flags = _lib.FV_HASH_PACKED if packed else _lib.FV_HASH_BYTES
        out = np.empty((ids.size, self.code_bytes(packed)), np.uint8)
        check(_lib.lib().fv_hash_tokens_static(self._h, ptr(ids), ids.size, hash_length, flags, ptr(out)))
        return out if packed else out.view(np.int8)

    def hash_windows(self, idx, inv_freq=None, hash_length: int = 50, packed: bool = False,
                     exact: bool = False, out: np.ndarray | None = None) -> np.ndarray:
        """``exact``: sum every window in double like the reference instead of certifying float sums
        first (same codes, slower)."""
        idx = as_c(idx, np.int32)
        assert idx.ndim == 2
        flags = (_lib.FV_HASH_PACKED if packed else _lib.FV_HASH_BYTES) | (_lib.FV_HASH_EXACT if exact else 0)
        f = None
        if inv_freq is None:
            flags |= _lib.FV_HASH_RAW
        else:
            f = as_c(inv_freq, np.float32)
            assert f.size == self.V
        out = self._out(out, idx.shape[0], packed)
        check(_lib.lib().fv_hash_windows(self._h, ptr(idx), idx.shape[0], idx.shape[1], ptr(f) if f is not None else None,
                                         hash_length, flags, ptr(out)))
        return out if packed else out.view(np.int8)

    def set_inverse_frequency(self, f):
        f = as_c(f, np.float32)
        check(_lib.lib().fv_hasher_set_inverse_frequency(self._h, ptr(f), f.size))

    # device-resident forms, used by the benchmark
    def hash_tokens_device(self, d_ids: int, n: int, hash_length: int, d_out: int, packed: bool = True) -> float:
        sec = C.c_double(0)
        flags = _lib.FV_HASH_PACKED if packed else _lib.FV_HASH_BYTES
        check(_lib.lib().fv_hash_tokens_device(self._h, C.c_void_p(d_ids), n, hash_length, flags, C.c_void_p(d_out),
                                               C.byref(sec)))
        return sec.value

    def hash_windows_device(self, d_idx: int, nwin: int, window: int, weighted: bool, hash_length: int, d_out: int,
                            packed: bool = True) -> float:
        sec = C.c_double(0)
        flags = _lib.FV_HASH_PACKED if packed else _lib.FV_HASH_BYTES
        check(_lib.lib().fv_hash_windows_device(self._h, C.c_void_p(d_idx), nwin, window, int(weighted), hash_length,
                                                flags, C.c_void_p(d_out), C.byref(sec)))
        return sec.value


class DeviceBuffer:
    """Raw device allocation through the C ABI (benchmark helper)."""

    def __init__(self, nbytes: int, device: int = 0):
        self.device, self.nbytes = device, nbytes
        p = C.c_void_p()
        check(_lib.lib().fv_device_alloc(device, nbytes, C.byref(p)))
        self.ptr = p.value

    def upload(self, a: np.ndarray):
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes
        check(_lib.lib().fv_copy_to_device(self.device, C.c_void_p(self.ptr), ptr(a), a.nbytes))

    def download(self, shape, dtype) -> np.ndarray:
        out = np.empty(shape, dtype)
        assert out.nbytes <= self.nbytes
        check(_lib.lib().fv_copy_to_host(self.device, ptr(out), C.c_void_p(self.ptr), out.nbytes))
        return out

    def free(self):
        if self.ptr:
            _lib.lib().fv_device_free(self.device, C.c_void_p(self.ptr))
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def flush_l2(device: int = 0, nbytes: int = 256 << 20):
    check(_lib.lib().fv_flush_l2(device, nbytes))


def probe_read_bandwidth(pattern: str, footprint: int, row_bytes: int = 1600, reps: int = 20, device: int = 0) -> float:
    """GB/s this GPU delivers right now for ``pattern`` = "stream" or "gather" over ``footprint`` bytes."""
    out = C.c_double(0)
    check(_lib.lib().fv_probe_read_bandwidth(device, {"stream": 0, "gather": 1}[pattern], footprint, row_bytes, reps,
                                             C.byref(out)))
    return out.value
