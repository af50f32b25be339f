"""CPU oracle for the FlyVec train/hash hot path -- TEST INFRASTRUCTURE ONLY.

This module is a numpy restatement of what the reference (bhoov/flyvec)
computes on its live training path and in its hashing API.  It exists to
check the CUDA library; nothing in the product imports it.  Only the test
suite, the smoke check and the CPU-baseline leg of the benchmark may use it.

Every function cites the reference lines it follows (paths are relative to
the reference project root).  The restatement is literal on purpose: it keeps
the reference's dense ``ds`` matrix, its float/double conversion points and its
per-device "mean over active replicas" combine, so it is only practical at
small and medium sizes.

Pinning status
--------------
* window enumeration: pinned against the reference's own ``prune_input.cpp``
  compiled for the host (see ``oracle/build_oracle.py`` and
  ``tests/test_oracle.py``).
* hashing: pinned against golden vectors produced by executing the reference's
  unmodified ``flyvec/core.py`` (see ``tests/golden/make_hash_golden.py``).
* training step: the reference ships no test, golden vector or fixture for its
  CUDA trainer.  The pin is the reference's own kernel text executed on the host:
  ``oracle/build_oracle.py`` cuts the ``__global__`` functions of the live path
  out of ``flyvec/src/cuda_funcs.cu`` and ``cu_special_reduction.cu`` where they
  lie, compiles them against a CUDA-on-host execution model
  (``oracle/cuda_on_host.h``: blocks in order, threads as lock-step fibers, the
  warp shuffle as the hardware performs it) and ``tests/test_oracle.py`` compares
  every stage of :func:`train_step` with that build bit for bit (input ids,
  activations, winner and second winner incl. exact ties, ``xx``, combine, ``nc``,
  step size, updated synapses; 1-3 replicas, ``delta`` zero and non-zero).  The
  reference's complete trainer binary was not run on a GPU; the host-side launch
  sequence is restated in ``oracle/ref_kernels_host.cpp`` from the cited lines.
  Where the hardware leaves an order open (float atomics) the host model applies
  them in thread order within block order, one admissible order.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
F64 = np.float64

#: chunks this long or longer are dropped whole (flyvec/src/prune_input.cpp:7)
MAXLEN = 214
#: value written over a found maximum while searching for the m-th one
#: (flyvec/src/cuda_funcs.cu:539)
MASK_VALUE = F32(-9999.9999)


# --------------------------------------------------------------------------
# T1  window enumeration            flyvec/src/prune_input.cpp:63-122
# --------------------------------------------------------------------------
def enumerate_windows(offsets: np.ndarray, W: int, maxlen: int = MAXLEN) -> np.ndarray:
    """Start index of every length-``W`` window that stays inside one chunk.

    Follows ``getnum_samples`` (prune_input.cpp:63-84) and
    ``compute_offset_phrases`` (prune_input.cpp:87-122): a chunk contributes
    ``len-W+1`` windows iff ``W <= len < maxlen``; starts are counted from a
    running total of chunk lengths (``global_count``), not from ``offsets[s]``.
    """
    offsets = np.asarray(offsets, dtype=np.uint64)
    if offsets.size < 2:
        return np.zeros(0, dtype=np.uint64)
    lengths = (offsets[1:] - offsets[:-1]).astype(np.int64)
    base = np.concatenate(([0], np.cumsum(lengths)[:-1])).astype(np.int64)
    keep = (lengths >= W) & (lengths < maxlen)
    nwin = np.where(keep, lengths - W + 1, 0)
    total = int(nwin.sum())
    if total == 0:
        return np.zeros(0, dtype=np.uint64)
    first = np.repeat(base, nwin)
    seg_start = np.repeat(np.cumsum(nwin) - nwin, nwin)
    return (first + (np.arange(total, dtype=np.int64) - seg_start)).astype(np.uint64)


# --------------------------------------------------------------------------
# T2  inverse word frequency        flyvec/src/model_arrays.cu:395-424
# --------------------------------------------------------------------------
def inverse_word_frequency(tokens: np.ndarray, V: int, saturate_fp32: bool = True) -> np.ndarray:
    """``f[v] = 1/count(v)`` (0 for unseen ids); negative ids are ignored.

    The reference counts with ``float += 1.0`` (model_arrays.cu:413-416), which
    stops growing at 2**24; ``saturate_fp32`` reproduces that.  The reciprocal
    is a double division rounded to float (model_arrays.cu:419-424).
    """
    tokens = np.asarray(tokens)
    counts = np.bincount(tokens[tokens >= 0].astype(np.int64), minlength=V)[:V].astype(np.int64)
    if saturate_fp32:
        counts = np.minimum(counts, 1 << 24)
    f = np.zeros(V, dtype=F32)
    nz = counts != 0
    f[nz] = (1.0 / counts[nz].astype(F64)).astype(F32)
    return f


# --------------------------------------------------------------------------
# T4  window -> sparse input ids     flyvec/src/cuda_funcs.cu:915-936
# --------------------------------------------------------------------------
def build_idx(tokens: np.ndarray, starts: np.ndarray, window_ids: np.ndarray, W: int, V: int) -> np.ndarray:
    """``idx[j][c] = token(window_j, c)`` with ``+V`` at the centre ``c == W//2``;
    a token of -1 stays -1."""
    window_ids = np.asarray(window_ids, dtype=np.int64)
    pos = starts[window_ids].astype(np.int64)[:, None] + np.arange(W, dtype=np.int64)[None, :]
    idx = np.asarray(tokens)[pos].astype(np.int32)
    mid = W // 2
    centre = idx[:, mid]
    idx[:, mid] = np.where(centre == -1, -1, centre + V)
    return idx


# --------------------------------------------------------------------------
# T6  activations                    flyvec/src/cuda_funcs.cu:248-263, 289-305
# --------------------------------------------------------------------------
def activations(ds: np.ndarray, idx: np.ndarray, f: np.ndarray | None, V: int) -> np.ndarray:
    """``a[j][mu] = (float) sum_c (double)(ds[mu][idx_jc] [*_fp32 f[idx_jc % V]])``.

    The product with the inverse frequency is a float product
    (cuda_funcs.cu:298-299); the running sum is a double, visited in window
    order ``c = 0..W-1``; the store rounds to float (cuda_funcs.cu:302).
    ``f is None`` gives the unweighted overload (cuda_funcs.cu:248-263).
    """
    B, W = idx.shape
    K = ds.shape[0]
    acc = np.zeros((B, K), dtype=F64)
    for c in range(W):
        col = idx[:, c]
        ok = col != -1
        safe = np.where(ok, col, 0)
        vals = ds[:, safe].T  # (B, K) float32
        if f is not None:
            vals = vals * f[safe % V][:, None]  # float32 * float32 -> float32
        acc += np.where(ok[:, None], vals.astype(F64), 0.0)
    return acc.astype(F32)


# --------------------------------------------------------------------------
# T7  winner and m-th winner         flyvec/src/cuda_funcs.cu:488-561
# --------------------------------------------------------------------------
def tie_rank(K: int) -> np.ndarray:
    """Rank of every unit in the reference's tie order (smaller wins among equal maxima).

    ``get_max_and_m_max_kernel_2`` runs 64 threads per window.  Thread ``t`` scans units
    ``t, t+64, ...`` with a strict ``>``, so it keeps its lowest index (cuda_funcs.cu:507-512).
    The warp reduction uses ``__shfl_down_sync`` with offsets 16, 8, 4, 2, 1 and a strict
    ``>`` (515-522): lane ``l`` keeps its own candidate against lane ``l+offset``, so lane 0
    ends with the candidate whose lane has the smallest 5-bit *reversed* number (lane
    priority 0, 16, 8, 24, 4, ...).  Thread 0 then prefers warp 0 over warp 1 (535-540).
    Key: ``(thread // 32, bitreverse5(thread % 32), index)`` with ``thread = index % 64``.
    Every thread starts from ``(data[0], 0)`` (505-506), which the key covers: unit 0 has
    the smallest key of all.
    """
    i = np.arange(K, dtype=np.int64)
    t = i % 64
    lane = t % 32
    rev = np.zeros(K, dtype=np.int64)
    for b in range(5):
        rev |= ((lane >> b) & 1) << (4 - b)
    return ((t // 32) * 32 + rev) * (K + 1) + i


def _argmax_ref_order(a: np.ndarray) -> np.ndarray:
    """Row-wise arg-max with the reference's tie order (see :func:`tie_rank`)."""
    K = a.shape[1]
    mx = a.max(axis=1, keepdims=True)
    key = tie_rank(K)
    masked = np.where(a == mx, key[None, :], np.iinfo(np.int64).max)
    return (masked.min(axis=1) % (K + 1)).astype(np.int32)


def winners(a_sel: np.ndarray, m: int = 2) -> tuple[np.ndarray, np.ndarray]:
    """Index of the largest and of the ``m``-th largest activation per window.

    Each found maximum is overwritten with -9999.9999 before the next search
    (cuda_funcs.cu:539) and restored afterwards (551-553).
    """
    work = a_sel.copy()
    rows = np.arange(work.shape[0])
    first = _argmax_ref_order(work)
    last = first
    for _ in range(1, m):
        work[rows, last] = MASK_VALUE
        last = _argmax_ref_order(work)
    return first, last


# --------------------------------------------------------------------------
# Phase A on one device: steps 1-8    flyvec/src/cuda_funcs.cu:1664-1742
# --------------------------------------------------------------------------
def device_phase(Wm: np.ndarray, idx: np.ndarray, f: np.ndarray, V: int, delta: float = 0.0, m: int = 2):
    """What one GPU computes before the cross-device combine.

    Returns ``(ds, xx, win, mmax, a_w)``.  ``ds`` is the dense K x N matrix the
    reference hands to its reduction.
    """
    K, N = Wm.shape
    delta = F32(delta)
    ds0 = Wm  # p == 2: ds = W exactly (cuda_funcs.cu:234-245, 1685-1688)
    a_w = activations(ds0, idx, f, V)  # cuda_funcs.cu:1700
    a_r = activations(ds0, idx, None, V)  # cuda_funcs.cu:1701
    win, mmax = winners(a_r, m)  # cuda_funcs.cu:1719 (raw activations select)
    xx = np.zeros(K, dtype=F32)  # cuda_funcs.cu:1715
    rows = np.arange(idx.shape[0])
    if delta != 0:
        # one thread per window adds both terms back to back (cuda_funcs.cu:726-735)
        for j in rows:
            xx[win[j]] = F32(xx[win[j]] + a_w[j, win[j]])
            xx[mmax[j]] = F32(xx[mmax[j]] + F32(-delta * a_w[j, mmax[j]]))
    else:
        np.add.at(xx, win, a_w[rows, win])  # sequential float adds, window order
    # cuda_funcs.cu:394-406
    ds = np.where((xx != 0)[:, None], (-xx)[:, None] * Wm, F32(0)).astype(F32)
    # cuda_funcs.cu:657-672
    B, W = idx.shape
    flat = idx.reshape(-1)
    ok = flat != -1
    fv = f[np.where(ok, flat, 0) % V]
    r1 = np.repeat(win, W)
    if delta != 0:
        # a thread adds both terms of its (window, position) back to back (cuda_funcs.cu:665-668);
        # windows in block order, positions in thread order: one admissible order of the atomics
        r2 = np.repeat(mmax, W)
        rows = np.stack([r1[ok], r2[ok]], axis=1).reshape(-1)
        cols = np.repeat(flat[ok], 2)
        vals = np.stack([fv[ok], (-delta * fv[ok]).astype(F32)], axis=1).reshape(-1)
        np.add.at(ds, (rows, cols), vals)
    else:
        np.add.at(ds, (r1[ok], flat[ok]), fv[ok])
    return ds, xx, win, mmax, a_w


# --------------------------------------------------------------------------
# Phases B and C                     flyvec/src/cu_special_reduction.cu:26-99, 316-354
# --------------------------------------------------------------------------
def combine_and_update(Wm: np.ndarray, ds_list, xx_list, eps: float, prec: float):
    """Mean of ``ds`` over the devices where the row was active, abs-max,
    scaled update.  Returns ``(W_new, nc, s)``.

    * ``nnz[h]`` counts devices with ``xx_dev[h] != 0`` (cu_special_reduction.cu:42-50);
    * ``D = (float)( (float)(sum of doubles) * (1.0/nnz) )`` (60-67);
    * ``nc = max|D|`` (69-70, 153-189, 257-261);
    * ``s = eps / max(prec, nc)`` (cuda_funcs.cu:1797-1799);
    * ``W += s*D`` where the row is active and ``|s*D| > 1e-10``
      (cu_special_reduction.cu:336-348).
    """
    K, N = Wm.shape
    act = np.stack([(xx != 0) for xx in xx_list])  # (G, K)
    nnz = act.sum(axis=0)
    total = np.zeros((K, N), dtype=F64)
    for ds, a in zip(ds_list, act):
        total += np.where(a[:, None], ds.astype(F64), 0.0)
    inv = np.where(nnz > 0, 1.0 / np.maximum(nnz, 1).astype(F64), 1.0)
    D = (total.astype(F32).astype(F64) * inv[:, None]).astype(F32)
    D[nnz == 0] = 0
    nc = F32(np.abs(D).max()) if D.size else F32(0)
    eps = F32(eps)
    prec = F32(prec)
    s = F32(eps / prec) if prec > nc else F32(eps / nc)
    val = (s * D).astype(F32)
    upd = (np.abs(val).astype(F64) > 1.0e-10) & (nnz > 0)[:, None]
    W_new = np.where(upd, (Wm + val).astype(F32), Wm)
    return W_new, nc, s


def train_step(Wm, idx_per_device, f, V, eps, delta=0.0, prec=1e-30, m=2):
    """One global minibatch step over ``len(idx_per_device)`` devices.

    Devices with no windows behave like a device whose ``xx`` is all zero.
    Returns ``(W_new, info)`` with the per-device winners, ``xx``, ``nc``, ``s``.
    """
    ds_list, xx_list, wins, mmaxs, aws = [], [], [], [], []
    K = Wm.shape[0]
    for idx in idx_per_device:
        if idx.shape[0] == 0:
            ds_list.append(np.zeros_like(Wm))
            xx_list.append(np.zeros(K, dtype=F32))
            wins.append(np.zeros(0, np.int32))
            mmaxs.append(np.zeros(0, np.int32))
            aws.append(np.zeros((0, K), F32))
            continue
        ds, xx, win, mmax, a_w = device_phase(Wm, idx, f, V, delta, m)
        ds_list.append(ds)
        xx_list.append(xx)
        wins.append(win)
        mmaxs.append(mmax)
        aws.append(a_w)
    W_new, nc, s = combine_and_update(Wm, ds_list, xx_list, eps, prec)
    return W_new, dict(win=wins, mmax=mmaxs, xx=xx_list, nc=nc, s=s, a_w=aws)


# --------------------------------------------------------------------------
# Schedules                          flyvec/src/cuda_funcs.cu:1229-1230
# --------------------------------------------------------------------------
def epoch_eps(lr0: float, epoch: int, nep: int) -> np.float32:
    """``eps = lr0 * (1 - epoch/Nep)``: float quotient, double product, float store."""
    q = F32(F32(epoch) / F32(nep))
    return F32(F64(F32(lr0)) * (1.0 - F64(q)))


def epoch_delta(delta: float, epoch: int, nep: int) -> np.float32:
    """``delta * 0.5 * (1 + tanh((epoch - Nep/8) / 10))``."""
    arg = (F64(F32(epoch)) - 0.125 * nep) / 10.0
    return F32(F64(F32(delta)) * 0.5 * (1.0 + np.tanh(arg)))


def run_epoch(Wm, tokens, starts, perm, f, V, W, batch, ngpus, eps, delta=0.0, prec=1e-30, m=2,
              max_steps=None, collect=False):
    """The step loop (cuda_funcs.cu:1662-1812) with the true tail: global step
    ``t`` covers permuted windows ``[t*G*B, (t+1)*G*B)``, device ``g`` takes the
    ``g``-th block of ``B`` clipped to ``Ns``.  (The reference replays stale rows
    of the previous batch in a partial last step, cuda_funcs.cu:1667-1680 against
    1700-1732; inputs whose window count is a multiple of ``G*B`` behave the same
    in both.)
    """
    Ns = len(perm)
    infos = []
    step = 0
    for k in range(0, Ns, batch * ngpus):
        if max_steps is not None and step >= max_steps:
            break
        idxs = []
        for g in range(ngpus):
            lo = min(k + g * batch, Ns)
            hi = min(lo + batch, Ns)
            idxs.append(build_idx(tokens, starts, perm[lo:hi], W, V))
        Wm, info = train_step(Wm, idxs, f, V, eps, delta, prec, m)
        if collect:
            infos.append(info)
        step += 1
    return Wm, infos


# --------------------------------------------------------------------------
# H1  hashing                        flyvec/core.py:22-36, 139-185
# --------------------------------------------------------------------------
def normalize_synapses(syn: np.ndarray, prec: float = 1.0e-32, p: int = 2) -> np.ndarray:
    """Row-wise p-norm normalisation, same expression as flyvec/core.py:33-36."""
    K, N = syn.shape
    nc = np.power(np.sum(syn ** p, axis=1), 1 / p).reshape(K, 1)
    return syn / np.tile(nc + prec, (1, N))


def threshold_code(act: np.ndarray, hash_length: int) -> np.ndarray:
    """Binary code of one activation vector (flyvec/core.py:155-158): threshold
    at the float midpoint of the ``h``-th and ``(h+1)``-th largest, strict ``>``."""
    srt = np.sort(act)[::-1]
    thr = (srt[hash_length - 1] + srt[hash_length]) / 2.0
    return (act > thr).astype(np.int8)


def hash_tokens(syn: np.ndarray, V: int, ids: np.ndarray, hash_length: int) -> np.ndarray:
    """Context-independent codes for a batch of token ids: column ``V+id`` of
    ``syn`` (flyvec/core.py:179), id 0 (unknown) gives all zeros
    (flyvec/core.py:120-125, 151)."""
    ids = np.asarray(ids, dtype=np.int64)
    K = syn.shape[0]
    out = np.zeros((ids.size, K), dtype=np.int8)
    for n, t in enumerate(ids):
        if t == 0:
            continue
        out[n] = threshold_code(syn[:, V + t], hash_length)
    return out


def hash_tokens_fast(syn: np.ndarray, V: int, ids: np.ndarray, hash_length: int) -> np.ndarray:
    """Vectorised form of :func:`hash_tokens` (same rule, np.partition for the
    two order statistics).  Used as the multi-core "strong CPU" baseline."""
    ids = np.asarray(ids, dtype=np.int64)
    K = syn.shape[0]
    out = np.zeros((ids.size, K), dtype=np.int8)
    CH = 8192
    for lo in range(0, ids.size, CH):
        sl = ids[lo:lo + CH]
        act = syn[:, V + sl].T  # (n, K)
        part = -np.partition(-act, (hash_length - 1, hash_length), axis=1)
        thr = (part[:, hash_length - 1] + part[:, hash_length]) / F32(2.0)
        code = (act > thr[:, None]).astype(np.int8)
        code[sl == 0] = 0
        out[lo:lo + CH] = code
    return out


# --------------------------------------------------------------------------
# H2  window hashing (no reference function; composition of T4+T6 with H1's rule)
# --------------------------------------------------------------------------
def hash_windows(syn: np.ndarray, V: int, idx: np.ndarray, f: np.ndarray | None, hash_length: int) -> np.ndarray:
    """Context-dependent codes: activation of T6 (weighted when ``f`` is given,
    cuda_funcs.cu:289-305, else raw, 248-263) thresholded by H1's rule
    (flyvec/core.py:155-158)."""
    act = activations(syn, idx, f, V)
    out = np.zeros(act.shape, dtype=np.int8)
    for j in range(act.shape[0]):
        out[j] = threshold_code(act[j], hash_length)
    return out


def pack_codes(codes: np.ndarray) -> np.ndarray:
    """Bit-pack {0,1} codes little-endian within each byte: unit ``mu`` is bit
    ``mu % 8`` of byte ``mu // 8``."""
    return np.packbits(codes.astype(np.uint8), axis=-1, bitorder="little")


# --------------------------------------------------------------------------
# The same step in the form the CUDA kernels use (no dense ds): what a rank can
# rebuild from the winners and xx vectors of all ranks plus the shared corpus.
# --------------------------------------------------------------------------
def closed_form_update(Wm, idx_per_device, win_per_device, xx_per_device, f, V, eps, prec=1e-30):
    """``W_mu <- (1 - s X_mu) W_mu + s S_mu`` for units active on at least one rank.

    ``X_mu`` is the mean of ``xx_dev[mu]`` over the ranks where it is non-zero and
    ``S_mu,i`` the mean over those ranks of ``count_dev(mu, i) * f_i``; this is
    cu_special_reduction.cu:42-67 applied to ``ds = -xx W + scatter``
    (cuda_funcs.cu:394-406, 657-672) and the update of
    cu_special_reduction.cu:336-348, evaluated in double instead of following the
    reference's float rounding steps.  Returns ``(W_new, nc, s)``.
    """
    K, N = Wm.shape
    xx = np.stack(xx_per_device).astype(F64)
    act = xx != 0
    n = act.sum(axis=0)
    X = np.where(n > 0, xx.sum(axis=0, where=act) / np.maximum(n, 1), 0.0)
    S = np.zeros((K, N), dtype=F64)
    for idx, win, a in zip(idx_per_device, win_per_device, act):
        if idx.shape[0] == 0:
            continue
        rows = np.repeat(win, idx.shape[1])
        flat = idx.reshape(-1)
        ok = (flat >= 0) & a[rows]
        np.add.at(S, (rows[ok], flat[ok]), f[flat[ok] % V].astype(F64))
    S /= np.maximum(n, 1)[:, None]
    D = np.where((n > 0)[:, None], -X[:, None] * Wm.astype(F64) + S, 0.0)
    nc = F32(np.abs(D).max())
    s = F32(F32(eps) / F32(prec)) if F32(prec) > nc else F32(F32(eps) / nc)
    W_new = np.where((n > 0)[:, None], Wm.astype(F64) + F64(s) * D, Wm.astype(F64)).astype(F32)
    return W_new, nc, s
