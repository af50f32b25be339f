"""CPU tests of the oracle itself: its pins against the reference's own code and
golden vectors, and the agreement of its numpy and C restatements."""
from pathlib import Path

import numpy as np
import pytest

from flyvec_b200 import synth
from oracle import c_oracle
from oracle import flyvec_oracle as orc
from tests.helpers import small_problem

GOLDEN = Path(__file__).resolve().parent / "golden"


# ---- T1: window enumeration, pinned on the reference's prune_input.cpp ------------
def ragged_offsets(rng, n, W):
    lens = np.concatenate([rng.integers(1, 40, n), [W - 1, W, W + 1, 213, 214, 215, 300, 0, 0, W]])
    rng.shuffle(lens)
    return np.concatenate([[0], np.cumsum(lens)]).astype(np.uint64)


@pytest.mark.parametrize("W", [1, 5, 11, 15])
def test_windows_match_reference_binary(W):
    rng = np.random.default_rng(W)
    off = ragged_offsets(rng, 500, W)
    ref = c_oracle.reference_enumerate_windows(off, W)
    if ref is None:
        pytest.skip("oracle/_ref/prune_input.so not built (no reference checkout)")
    np.testing.assert_array_equal(orc.enumerate_windows(off, W), ref)


def test_windows_known_case():
    # chunk lengths [11,5,12,213,214,300,20] at W=11: 1 + 0 + 2 + 203 + 0 + 0 + 10 windows
    lens = np.array([11, 5, 12, 213, 214, 300, 20])
    off = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint64)
    st = orc.enumerate_windows(off, 11)
    assert len(st) == 216
    assert st[0] == 0 and st[1] == 16 and st[2] == 17 and st[3] == 28
    assert st[-1] == off[-2] + 9


def test_windows_edge_cases():
    assert len(orc.enumerate_windows(np.array([0], np.uint64), 11)) == 0
    assert len(orc.enumerate_windows(np.array([0, 5], np.uint64), 11)) == 0
    assert len(orc.enumerate_windows(np.zeros(0, np.uint64), 11)) == 0
    np.testing.assert_array_equal(orc.enumerate_windows(np.array([0, 3], np.uint64), 1), [0, 1, 2])


# ---- T2 ---------------------------------------------------------------------------
def test_inverse_frequency_rules():
    enc = np.array([3, 3, 3, 1, -1, -1, 0, 0], np.int32)
    f = orc.inverse_word_frequency(enc, 5)
    np.testing.assert_array_equal(f, np.array([0.5, 1.0, 0.0, np.float32(1.0 / 3.0), 0.0], np.float32))
    assert f.dtype == np.float32


def test_inverse_frequency_saturates_like_a_float_counter():
    # a float counter incremented by 1.0 stops at 2**24 (flyvec/src/model_arrays.cu:413-416)
    c = np.float32(2 ** 24)
    assert np.float32(c + np.float32(1.0)) == c
    counts = np.array([2 ** 24 + 5, 7], np.int64)
    enc = np.repeat(np.arange(2, dtype=np.int32), [8, 7])  # small stand-in; the cap is applied on counts
    f_sat = orc.inverse_word_frequency(enc, 2, saturate_fp32=True)
    np.testing.assert_array_equal(f_sat, np.array([1 / 8, 1 / 7], np.float32))
    capped = np.minimum(counts, 1 << 24)
    assert capped[0] == 2 ** 24


# ---- H1: hashing, pinned on golden vectors from the reference's core.py -------------
def test_hash_oracle_matches_reference_golden():
    g = np.load(GOLDEN / "hash_golden.npz")
    K, V = int(g["K"]), int(g["V"])
    W = synth.make_weights(K, 2 * V, seed=int(g["seed"]))
    for normalize, key in ((True, "codes_norm"), (False, "codes_raw")):
        syn = orc.normalize_synapses(W) if normalize else W
        for hl, codes in zip(g["hash_lengths"], g[key]):
            np.testing.assert_array_equal(orc.hash_tokens(syn, V, g["ids"], int(hl)), codes)
            np.testing.assert_array_equal(orc.hash_tokens_fast(syn, V, g["ids"], int(hl)), codes)
            np.testing.assert_array_equal(c_oracle.hash_tokens(syn, V, g["ids"], int(hl)), codes)


def test_threshold_rule_with_ties():
    act = np.array([3, 3, 3, 1, 0], np.float32)
    # h=2: midpoint of 3 and 3 is 3, nothing is strictly greater
    assert orc.threshold_code(act, 2).sum() == 0
    assert orc.threshold_code(act, 3).sum() == 3
    np.testing.assert_array_equal(orc.pack_codes(np.array([[1, 0, 0, 0, 0, 0, 0, 0, 1]])), [[1, 1]])


# ---- training step: numpy restatement vs C restatement ------------------------------
@pytest.mark.parametrize("G", [1, 2, 3])
def test_numpy_and_c_oracle_agree_bitwise(G):
    p = small_problem(K=48, V=300, W=11, ntok=12000, seed=31 + G)
    B, eps = 100, np.float32(2e-4)
    runner = c_oracle.StepRunner(48, 600, 300, 11, B, G)
    Wn = p["W0"].copy()
    Wc = p["W0"].copy()
    for step in range(3):
        idxs = []
        for g in range(G):
            lo = (step * G + g) * B
            idxs.append(orc.build_idx(p["enc"], p["starts"], p["perm"][lo:lo + B], 11, 300))
        Wn, info = orc.train_step(Wn, idxs, p["f"], 300, eps)
        win, xx, nc, s = runner.step(Wc, np.stack(idxs), [B] * G, p["f"], eps)
        for g in range(G):
            np.testing.assert_array_equal(win[g], info["win"][g])
            np.testing.assert_array_equal(xx[g], info["xx"][g])
        assert nc == info["nc"] and s == info["s"]
        np.testing.assert_array_equal(Wc, Wn)


def test_step_properties():
    """Size-independent properties of the learning rule: rows that never win keep
    their weights, the largest update equals eps, the winner row moves towards
    its inputs."""
    p = small_problem(K=32, V=200, W=7, ntok=6000, seed=2)
    idx = orc.build_idx(p["enc"], p["starts"], p["perm"][:200], 7, 200)
    eps = np.float32(1e-3)
    W1, info = orc.train_step(p["W0"], [idx], p["f"], 200, eps)
    active = info["xx"][0] != 0
    np.testing.assert_array_equal(W1[~active], p["W0"][~active])
    assert np.isclose(np.abs(W1 - p["W0"]).max(), eps, rtol=1e-3)  # float subtraction of O(1) weights
    assert np.isclose(info["s"] * info["nc"], eps, rtol=1e-6)


def test_tie_order_of_winner():
    """Among equal maxima the reference keeps the smallest (thread // 32, bitreverse5(thread % 32), index),
    thread = index % 64 (cuda_funcs.cu:507-540)."""
    a = np.zeros((1, 200), np.float32)
    a[0, [70, 3]] = 5.0       # lanes 6 (reversed 12) and 3 (reversed 24): unit 70 survives the shuffle tree
    assert orc.winners(a)[0][0] == 70
    a[:] = 0
    a[0, [69, 130]] = 5.0     # lanes 5 (reversed 20) and 2 (reversed 8)
    assert orc.winners(a)[0][0] == 130
    a[:] = 0
    a[0, [1, 32]] = 5.0       # warp 0 beats warp 1 whatever the lane
    assert orc.winners(a)[0][0] == 1
    a[:] = 1.0                # all equal: index 0, then thread 0's next unit
    first, second = orc.winners(a)
    assert first[0] == 0 and second[0] == 64


# ---- T4-T13 pinned on the reference's own kernels, executed on the host --------------
def _need_reference_kernels():
    if c_oracle.reference_kernels() is None:
        pytest.skip("oracle/_ref/ref_kernels_host.so not built (no reference checkout)")


@pytest.mark.parametrize("K", [2, 5, 33, 64, 65, 100, 400, 1000])
def test_winners_match_reference_kernel_on_ties(K):
    """Tie-heavy activations through get_max_and_m_max_kernel_2 itself (64 lock-step threads,
    the shuffle tree as written)."""
    _need_reference_kernels()
    rng = np.random.default_rng(K)
    a = rng.integers(0, 3, (200, K)).astype(np.float32)
    a[::7] = 1.0          # every unit ties
    a[::5, 0] = 2.0       # unit 0 among the maxima
    a[1::11] -= 20000.0   # everything below the -9999.9999 mask of the second search
    for r in range(0, 200, 3):  # two-way exact ties on top of random values
        i, j = rng.choice(K, 2, replace=False)
        a[r, i] = a[r, j] = 7.0
    ref_w, ref_m = c_oracle.reference_winners(a)
    w, m = orc.winners(a)
    np.testing.assert_array_equal(w, ref_w)
    np.testing.assert_array_equal(m, ref_m)


@pytest.mark.parametrize("K,V,G,B,delta,ties", [
    (64, 512, 1, 256, 0.0, False), (64, 512, 2, 128, 0.0, False), (48, 300, 3, 100, 0.3, False),
    (16, 64, 3, 64, 0.5, True), (16, 64, 2, 128, 1.0, True), (8, 32, 1, 300, 0.0, True),
])
def test_train_step_matches_reference_kernels(K, V, G, B, delta, ties):
    """Every stage of one global step against the reference's own kernel text run on the host in
    the reference's launch sequence: input ids, weighted activations, winner and second winner,
    xx, the combined direction, nc, the step size and the updated synapses -- all bit for bit,
    on random weights and on a coarse grid of weights that produces exact ties everywhere."""
    _need_reference_kernels()
    p = small_problem(K=K, V=V, W=11, ntok=20000, seed=5)
    W0 = p["W0"]
    if ties:
        W0 = (np.round(np.random.default_rng(1).standard_normal(W0.shape) * 2) / 2).astype(np.float32)
    eps = np.float32(2e-4)
    ref = c_oracle.reference_train_step(W0, p["enc"], p["starts"], p["perm"], p["f"], V, 11, B, G, eps, delta=delta)
    assert ref["replicas_identical"]
    idxs = [orc.build_idx(p["enc"], p["starts"], p["perm"][g * B:(g + 1) * B], 11, V) for g in range(G)]
    Wn, info = orc.train_step(W0, idxs, p["f"], V, eps, delta=delta)
    for g in range(G):
        np.testing.assert_array_equal(ref["idx"][g], idxs[g])
        np.testing.assert_array_equal(ref["a_w"][g], info["a_w"][g])
        np.testing.assert_array_equal(ref["win"][g], info["win"][g])
        if delta != 0:
            np.testing.assert_array_equal(ref["mmax"][g], info["mmax"][g])
        np.testing.assert_array_equal(ref["xx"][g], info["xx"][g])
    assert ref["nc"] == info["nc"] and ref["s"] == info["s"]
    np.testing.assert_array_equal(ref["W"], Wn)


def test_c_oracle_matches_reference_kernels_over_steps():
    """The C restatement (the one the GPU parity tests at full shapes use) follows the
    reference's kernels bit for bit over consecutive steps, 1 and 3 replicas."""
    _need_reference_kernels()
    K, V, W, B = 32, 200, 11, 150
    p = small_problem(K=K, V=V, W=W, ntok=20000, seed=9)
    eps = np.float32(1e-3)
    for G in (1, 3):
        runner = c_oracle.StepRunner(K, 2 * V, V, W, B, G)
        Wc = p["W0"].copy()
        Wr = p["W0"].copy()
        for step in range(3):
            order = p["perm"][step * G * B:(step + 1) * G * B]
            idx = np.stack([orc.build_idx(p["enc"], p["starts"], order[g * B:(g + 1) * B], W, V) for g in range(G)])
            win, xx, nc, s = runner.step(Wc, idx, [B] * G, p["f"], eps)
            ref = c_oracle.reference_train_step(Wr, p["enc"], p["starts"], order, p["f"], V, W, B, G, eps)
            Wr = ref["W"]
            np.testing.assert_array_equal(win, ref["win"])
            np.testing.assert_array_equal(xx, ref["xx"])
            assert nc == ref["nc"] and s == ref["s"]
            np.testing.assert_array_equal(Wc, Wr)


def test_schedules():
    assert orc.epoch_eps(0.002, 0, 15) == np.float32(0.002)
    assert orc.epoch_eps(0.002, 15, 15) == 0
    assert np.isclose(orc.epoch_eps(2e-4, 3, 15), 2e-4 * 0.8, rtol=1e-6)
    assert orc.epoch_delta(0.0, 3, 15) == 0
