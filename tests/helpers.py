"""Shared pieces of the parity tests: small seeded problems and comparison rules."""
import numpy as np

from flyvec_b200 import synth
from oracle import flyvec_oracle as orc


def small_problem(K=64, V=512, W=11, ntok=30000, seed=7, sigma=1.0, mean_len=25.0, zipf_s=1.0):
    enc, off = synth.make_corpus(ntok, V, s=zipf_s, mean_len=mean_len, min_len=W, seed=seed)
    starts = orc.enumerate_windows(off, W)
    f = orc.inverse_word_frequency(enc, V, saturate_fp32=False)
    W0 = synth.make_weights(K, 2 * V, seed=seed + 1, sigma=sigma)
    rng = np.random.Generator(np.random.PCG64(seed + 2))
    perm = rng.permutation(len(starts)).astype(np.uint64)
    return dict(enc=enc, off=off, starts=starts, f=f, W0=W0, perm=perm, K=K, V=V, W=W)


def top2_margin(a_row):
    """Relative gap between the two largest entries of one activation row."""
    part = np.partition(a_row, -2)
    a1, a2 = float(part[-1]), float(part[-2])
    return (a1 - a2) / max(abs(a1), 1e-30)


def check_winners(win_gpu, win_ref, a_raw, rel_margin=1e-6):
    """Winners must agree except where the top-2 gap is below ``rel_margin``
    relative (the tolerance the parity target states for near ties)."""
    bad = np.nonzero(win_gpu != win_ref)[0]
    for j in bad:
        m = top2_margin(a_raw[j])
        assert m < rel_margin, f"window {j}: gpu {win_gpu[j]} ref {win_ref[j]} margin {m:.3e}"
    return len(bad)


def rel_err(a, b):
    """max |a-b| relative to the largest magnitude of the reference."""
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64))) / max(float(np.max(np.abs(b))), 1e-30))
