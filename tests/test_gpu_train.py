"""Parity of the CUDA trainer with the oracle (which restates
flyvec/src/cuda_funcs.cu:1662-1812 and cu_special_reduction.cu:26-99, 316-354).
All calls go through the C ABI."""
import numpy as np
import pytest

from flyvec_b200 import _lib
from flyvec_b200.engine import Trainer
from oracle import flyvec_oracle as orc
from tests.helpers import check_winners, rel_err, small_problem

pytestmark = pytest.mark.gpu

#: weights: relative to the largest |weight| of the reference result.  The parity
#: target for a whole epoch is 1e-4; single steps agree far better.
STEP_TOL = 2e-6
EPOCH_TOL = 1e-4


def make_trainer(p, batch, world=1, flags=0, lr0=2e-4):
    tr = Trainer(hid=p["K"], vocab=p["V"], window=p["W"], batch=batch, lr0=lr0, world=world, flags=flags)
    ns = tr.set_corpus(p["enc"], p["off"])
    assert ns == len(p["starts"])
    tr.set_weights(p["W0"])
    tr.set_permutation(p["perm"])
    return tr


def test_corpus_tables_match_oracle(built_lib):
    p = small_problem()
    tr = make_trainer(p, 256)
    np.testing.assert_array_equal(tr.inverse_frequency(), p["f"])
    np.testing.assert_array_equal(tr.get_permutation(), p["perm"])
    np.testing.assert_array_equal(tr.get_weights(), p["W0"])
    np.testing.assert_array_equal(tr.window_starts(), p["starts"])
    tr.close()


@pytest.mark.parametrize("V,W,nchunks,maxlen", [(300, 11, 5000, 0), (70000, 5, 3000, 40), (50, 3, 1, 0), (1000, 11, 2500, 12)])
def test_corpus_tables_built_on_gpu(built_lib, V, W, nchunks, maxlen):
    """Window table and 1/count come from GPU kernels; both must equal the oracle's (T1, T2) exactly,
    over empty chunks, chunks shorter than a window, chunks at and over the length limit, negative
    (padding) ids, and a vocabulary too large for the shared-memory histogram."""
    from flyvec_b200.engine import enumerate_windows
    rng = np.random.default_rng(V + W)
    lim = maxlen or orc.MAXLEN
    lens = rng.integers(0, lim + 8, nchunks)
    lens[rng.random(nchunks) < 0.1] = 0
    lens[rng.random(nchunks) < 0.05] = lim - 1
    lens[rng.random(nchunks) < 0.05] = lim
    lens[rng.random(nchunks) < 0.05] = W
    lens[rng.random(nchunks) < 0.05] = max(W - 1, 0)
    off = np.concatenate(([0], np.cumsum(lens))).astype(np.uint64)
    ntok = int(off[-1]) + 17
    enc = (rng.zipf(1.3, ntok) % V).astype(np.int32)
    enc[rng.random(ntok) < 0.01] = -1
    tr = Trainer(hid=8, vocab=V, window=W, batch=4, maxlen=maxlen)
    ns = tr.set_corpus(enc, off)
    want = orc.enumerate_windows(off, W, lim)
    assert ns == want.size
    np.testing.assert_array_equal(tr.window_starts(), want)
    np.testing.assert_array_equal(tr.window_starts(), enumerate_windows(off, W, maxlen))
    np.testing.assert_array_equal(tr.inverse_frequency(), orc.inverse_word_frequency(enc, V, saturate_fp32=False))
    np.testing.assert_array_equal(tr.get_permutation(), np.arange(ns, dtype=np.uint64))
    tr.close()


def test_corpus_errors_found_on_gpu(built_lib):
    tr = Trainer(hid=8, vocab=100, window=3, batch=4)
    enc = np.arange(60, dtype=np.int32)
    with pytest.raises(_lib.FlyvecError, match="backwards"):
        tr.set_corpus(enc, np.array([0, 30, 20, 60], np.uint64))
    bad = enc.copy()
    bad[41] = 100
    with pytest.raises(_lib.FlyvecError, match=">= vocab"):
        tr.set_corpus(bad, np.array([0, 30, 60], np.uint64))
    assert tr.set_corpus(enc, np.array([0, 30, 60], np.uint64)) == 56
    tr.close()


@pytest.mark.parametrize("K,V,W,batch", [(64, 512, 11, 256), (100, 300, 5, 97), (400, 1000, 11, 500), (130, 257, 15, 64)])
def test_teacher_forced_steps(built_lib, K, V, W, batch):
    """Each step is checked against the oracle started from the GPU's own weights
    of the step before, so rounding differences cannot pile up."""
    p = small_problem(K=K, V=V, W=W, ntok=20000)
    tr = make_trainer(p, batch)
    eps = np.float32(2e-4)
    Wcur = p["W0"]
    flips = 0
    for step in range(6):
        win, xx, nc, s = tr.step_debug(step, eps)
        Wgpu = tr.get_weights()
        lo = step * batch
        idx = orc.build_idx(p["enc"], p["starts"], p["perm"][lo:lo + batch], W, V)
        Wref, info = orc.train_step(Wcur, [idx], p["f"], V, eps)
        a_raw = orc.activations(Wcur, idx, None, V)
        flips += check_winners(win[0], info["win"][0], a_raw)
        if np.array_equal(win[0], info["win"][0]):
            np.testing.assert_allclose(xx[0], info["xx"][0], rtol=2e-5, atol=1e-7)
            np.testing.assert_allclose(nc, info["nc"], rtol=1e-5)
            np.testing.assert_allclose(s, info["s"], rtol=1e-5)
            assert rel_err(Wgpu, Wref) < STEP_TOL
        Wcur = Wgpu
    assert flips <= 1
    tr.close()


def test_first_step_winners_bit_exact_fp32_and_fp64_paths(built_lib):
    """From identical weights the float fast path, the forced double path and the
    oracle must pick the same winners (near ties included: the fast path hands
    them to the double path)."""
    p = small_problem(K=400, V=800, W=11, ntok=40000, seed=11)
    idx = orc.build_idx(p["enc"], p["starts"], p["perm"][:2000], 11, 800)
    a_raw = orc.activations(p["W0"], idx, None, 800)
    ref, _ = orc.winners(a_raw)
    for flags in (0, _lib.FV_FLAG_ACC_FP64):
        tr = make_trainer(p, 2000, flags=flags)
        win, _, _, _ = tr.step_debug(0, np.float32(2e-4))
        np.testing.assert_array_equal(win[0], ref)
        tr.close()


def test_exact_ties_follow_reference_order(built_lib):
    """Duplicate units tie exactly; the reference keeps the one with the smallest
    (thread // 32, bitreverse5(thread % 32), index), thread = index % 64 (cuda_funcs.cu:507-540)."""
    p = small_problem(K=200, V=300, W=7, ntok=8000, seed=5)
    W0 = p["W0"].copy()
    W0[70] = W0[3]      # lanes 6 (reversed 12) and 3 (reversed 24): unit 70 wins ties
    W0[130] = W0[69]    # lanes 2 (reversed 8) and 5 (reversed 20): unit 130 wins ties
    W0[33] = W0[1]      # warp 0 beats warp 1: unit 1 wins ties
    p["W0"] = W0
    idx = orc.build_idx(p["enc"], p["starts"], p["perm"][:1000], 7, 300)
    ref, _ = orc.winners(orc.activations(W0, idx, None, 300))
    assert (ref == 70).sum() + (ref == 130).sum() + (ref == 1).sum() > 0
    assert (ref == 3).sum() == 0 and (ref == 69).sum() == 0 and (ref == 33).sum() == 0
    tr = make_trainer(p, 1000)
    win, _, _, _ = tr.step_debug(0, np.float32(2e-4))
    np.testing.assert_array_equal(win[0], ref)
    tr.close()


@pytest.mark.parametrize("fold_every_step", [False, True])
def test_free_running_epoch(built_lib, fold_every_step):
    """A whole small epoch (with a ragged last step) against the oracle's epoch loop."""
    p = small_problem(K=64, V=512, W=11, ntok=30000)
    batch = 500
    flags = _lib.FV_FLAG_FOLD_EVERY_STEP if fold_every_step else 0
    tr = make_trainer(p, batch, flags=flags, lr0=2e-4)
    st = tr.run_epoch(0, 1)
    Wgpu = tr.get_weights()
    eps = orc.epoch_eps(2e-4, 0, 1)
    Wref, _ = orc.run_epoch(p["W0"], p["enc"], p["starts"], p["perm"], p["f"], p["V"], p["W"], batch, 1, eps)
    assert st["steps"] == (len(p["starts"]) + batch - 1) // batch
    assert st["windows"] == len(p["starts"])
    assert st["device_error"] == 0
    assert rel_err(Wgpu, Wref) < EPOCH_TOL
    # the update must have done something
    assert rel_err(Wgpu, p["W0"]) > 1e-4
    tr.close()


@pytest.mark.parametrize("world", [2, 4])
def test_cross_rank_combine_emulated(built_lib, world):
    """Mean over the ranks where a unit was active (cu_special_reduction.cu:42-67),
    with every rank's block computed in turn on one GPU."""
    p = small_problem(K=64, V=512, W=11, ntok=30000, seed=21)
    batch = 128
    tr = make_trainer(p, batch, world=world, flags=_lib.FV_FLAG_EMULATE_RANKS)
    eps = np.float32(2e-4)
    Wcur = p["W0"]
    for step in range(4):
        win, xx, nc, s = tr.step_debug(step, eps)
        Wgpu = tr.get_weights()
        idxs = []
        for g in range(world):
            lo = (step * world + g) * batch
            idxs.append(orc.build_idx(p["enc"], p["starts"], p["perm"][lo:lo + batch], p["W"], p["V"]))
        Wref, info = orc.train_step(Wcur, idxs, p["f"], p["V"], eps)
        same = True
        for g in range(world):
            a_raw = orc.activations(Wcur, idxs[g], None, p["V"])
            same &= check_winners(win[g], info["win"][g], a_raw) == 0
        if same:
            for g in range(world):
                np.testing.assert_allclose(xx[g], info["xx"][g], rtol=2e-5, atol=1e-7)
            np.testing.assert_allclose(nc, info["nc"], rtol=1e-5)
            assert rel_err(Wgpu, Wref) < STEP_TOL
        Wcur = Wgpu
    tr.close()


def test_inactive_rank_rows_are_dropped(built_lib):
    """A rank whose xx is zero for a unit is left out of that unit's mean
    (cu_special_reduction.cu:42-66).  Rank 1 only sees tokens whose inverse
    frequency is forced to zero, so all its xx vanish and every unit's mean runs
    over rank 0 alone (dividing by the number of ranks would halve the update)."""
    p = small_problem(K=32, V=200, W=5, ntok=6000, seed=3)
    enc = p["enc"].copy()
    half = 3000
    enc[:half] %= 100
    enc[half:] = 100 + enc[half:] % 100
    starts = p["starts"]
    first = np.nonzero(starts + 5 <= half)[0]
    second = np.nonzero(starts >= half)[0]
    chosen = np.concatenate([first[:64], second[:64]])
    rest = np.setdiff1d(np.arange(len(starts)), chosen)
    perm = np.concatenate([chosen, rest]).astype(np.uint64)
    f = orc.inverse_word_frequency(enc, 200, saturate_fp32=False)
    f[100:] = 0
    tr = Trainer(hid=32, vocab=200, window=5, batch=64, lr0=2e-4, world=2, flags=_lib.FV_FLAG_EMULATE_RANKS)
    tr.set_corpus(enc, p["off"])
    tr.set_inverse_frequency(f)
    tr.set_weights(p["W0"])
    tr.set_permutation(perm)
    eps = np.float32(2e-4)
    win, xx, nc, s = tr.step_debug(0, eps)
    idxs = [orc.build_idx(enc, starts, perm[g * 64:(g + 1) * 64], 5, 200) for g in range(2)]
    Wref, info = orc.train_step(p["W0"], idxs, f, 200, eps)
    assert not info["xx"][1].any() and info["xx"][0].any()
    for g in range(2):
        np.testing.assert_array_equal(win[g], info["win"][g])
        np.testing.assert_allclose(xx[g], info["xx"][g], rtol=2e-5, atol=1e-7)
    np.testing.assert_allclose(nc, info["nc"], rtol=1e-5)
    assert rel_err(tr.get_weights(), Wref) < STEP_TOL
    tr.close()


@pytest.mark.parametrize("delta", [0.0, 0.5])
def test_cancelled_unit_on_one_rank_leaves_the_counts(built_lib, delta):
    """A unit that wins windows on a rank while its activations there add up to exactly zero is
    inactive on that rank (cu_special_reduction.cu:42-66 tests xx != 0), so that rank's windows must
    not count in the scatter term although another rank, active for the same unit, touches the same
    matrix positions.  Rank 0 sees only tokens on which every weight is zero (unit 0 wins all ties
    with activation 0, unit 1 comes second); rank 1 mixes them with tokens units 0 and 1 respond to."""
    K, V, W, B = 8, 40, 3, 16
    zs = np.arange(10, 28, dtype=np.int32)                      # 18 tokens -> 16 windows of silent tokens
    mixed = np.empty(18, np.int32)
    mixed[0::2] = 1 + np.arange(9) % 5                          # tokens units 0 and 1 respond to
    mixed[1::2] = zs[:9]                                        # the same silent tokens as rank 0
    enc = np.concatenate([zs, mixed])
    off = np.array([0, 18, 36], np.uint64)
    W0 = np.zeros((K, 2 * V), np.float32)
    for blk in (0, V):
        W0[0, blk + 1:blk + 6] = 1.0
        W0[1, blk + 1:blk + 6] = 0.5
    tr = Trainer(hid=K, vocab=V, window=W, batch=B, lr0=2e-4, delta=delta, world=2, flags=_lib.FV_FLAG_EMULATE_RANKS)
    assert tr.set_corpus(enc, off) == 2 * B
    tr.set_weights(W0)
    eps = np.float32(2e-4)
    win, xx, nc, s = tr.step_debug(0, eps)
    starts = orc.enumerate_windows(off, W)
    f = orc.inverse_word_frequency(enc, V, saturate_fp32=False)
    idxs = [orc.build_idx(enc, starts, np.arange(g * B, (g + 1) * B, dtype=np.uint64), W, V) for g in range(2)]
    Wref, info = orc.train_step(W0, idxs, f, V, eps, delta=delta)
    assert info["xx"][0][0] == 0 and info["xx"][1][0] != 0 and (info["win"][0] == 0).all()
    for g in range(2):
        np.testing.assert_array_equal(win[g], info["win"][g])
        np.testing.assert_allclose(xx[g], info["xx"][g], rtol=2e-5, atol=1e-9)
    np.testing.assert_allclose(nc, info["nc"], rtol=1e-5)
    assert rel_err(tr.get_weights(), Wref) < STEP_TOL
    # the silent tokens of rank 0 must matter for the check: counting them changes the result
    both, _ = orc.train_step(W0, [np.concatenate(idxs)], f, V, eps, delta=delta)
    assert rel_err(both, Wref) > 5 * STEP_TOL
    tr.close()


@pytest.mark.parametrize("world", [1, 2])
def test_anti_hebbian_second_winner(built_lib, world):
    """delta != 0: the second-largest unit gets -delta times the Hebbian terms
    (cuda_funcs.cu:726-735 for xx, 665-668 for the scatter)."""
    p = small_problem(K=64, V=400, W=9, ntok=20000, seed=33)
    batch, delta = 160, 0.4
    flags = _lib.FV_FLAG_EMULATE_RANKS if world > 1 else 0
    tr = Trainer(hid=p["K"], vocab=p["V"], window=p["W"], batch=batch, lr0=2e-4, delta=delta, world=world, flags=flags)
    tr.set_corpus(p["enc"], p["off"])
    tr.set_weights(p["W0"])
    tr.set_permutation(p["perm"])
    eps = np.float32(2e-4)
    Wcur = p["W0"]
    for step in range(4):
        win, xx, nc, s = tr.step_debug(step, eps)
        Wgpu = tr.get_weights()
        idxs = []
        for g in range(world):
            lo = (step * world + g) * batch
            idxs.append(orc.build_idx(p["enc"], p["starts"], p["perm"][lo:lo + batch], p["W"], p["V"]))
        Wref, info = orc.train_step(Wcur, idxs, p["f"], p["V"], eps, delta=delta)
        for g in range(world):
            np.testing.assert_array_equal(win[g], info["win"][g])
            np.testing.assert_allclose(xx[g], info["xx"][g], rtol=5e-5, atol=1e-7)
        np.testing.assert_allclose(nc, info["nc"], rtol=1e-5)
        assert rel_err(Wgpu, Wref) < STEP_TOL
        Wcur = Wgpu
    # the term must matter: without it the weights differ visibly
    idx0 = orc.build_idx(p["enc"], p["starts"], p["perm"][:batch], p["W"], p["V"])
    Wplain, _ = orc.train_step(p["W0"], [idx0], p["f"], p["V"], eps)
    Wdelta, _ = orc.train_step(p["W0"], [idx0], p["f"], p["V"], eps, delta=delta)
    assert rel_err(Wplain, Wdelta) > 3 * STEP_TOL  # 7e-6 of max|W| in one step, well above the step tolerance
    tr.close()


def test_delta_epoch_schedule(built_lib):
    """run_epoch applies delta * 0.5 * (1 + tanh((epoch - Nep/8) / 10)) (cuda_funcs.cu:1230)."""
    p = small_problem(K=32, V=200, W=5, ntok=5000, seed=35)
    batch = 300
    tr = Trainer(hid=32, vocab=200, window=5, batch=batch, lr0=1e-3, delta=0.5)
    tr.set_corpus(p["enc"], p["off"])
    tr.set_weights(p["W0"])
    tr.set_permutation(p["perm"])
    tr.run_epoch(3, 8)
    Wgpu = tr.get_weights()
    tr.close()
    Wref, _ = orc.run_epoch(p["W0"], p["enc"], p["starts"], p["perm"], p["f"], 200, 5, batch, 1, orc.epoch_eps(1e-3, 3, 8),
                            delta=orc.epoch_delta(0.5, 3, 8))
    assert rel_err(Wgpu, Wref) < EPOCH_TOL


def test_streaming_mode_matches_resident_mode(built_lib):
    """Host-fed input ids (uploaded inside the call) give the same weights as the
    resident corpus, and the per-step normalisers come back."""
    p = small_problem(K=64, V=512, W=11, ntok=30000, seed=9)
    batch, nsteps = 256, 40
    a = make_trainer(p, batch)
    sa = a.run_steps(0, nsteps, 2e-4, want_log=True)
    Wa = a.get_weights()
    a.close()
    b = make_trainer(p, batch)
    idx = orc.build_idx(p["enc"], p["starts"], p["perm"][:nsteps * batch], p["W"], p["V"]).reshape(nsteps, batch, p["W"])
    pinned = _lib.pinned_empty(idx.shape, np.int32)
    pinned[...] = idx
    nc = np.empty(nsteps, np.float32)
    sb = b.run_steps_host(pinned, nsteps, 2e-4, nc_out=nc)
    Wb = b.get_weights()
    b.close()
    np.testing.assert_array_equal(Wa, Wb)
    np.testing.assert_array_equal(nc, sa["nc"])
    assert sb["windows"] == nsteps * batch
    # with one rank the rank-local feed is the same call
    c = make_trainer(p, batch)
    c.run_steps_host_local(pinned, nsteps, 2e-4)
    np.testing.assert_array_equal(c.get_weights(), Wa)
    c.close()
    # emulated ranks have no second process to gather from
    e = make_trainer(p, 64, world=2, flags=_lib.FV_FLAG_EMULATE_RANKS)
    with pytest.raises(_lib.FlyvecError, match="rank-local"):
        e.run_steps_host_local(np.ascontiguousarray(pinned[:4, :64]), 4, 2e-4)
    e.close()


def test_seeded_shuffle_is_a_permutation(built_lib):
    p = small_problem()
    tr = make_trainer(p, 256)
    tr.shuffle(1234)
    a = tr.get_permutation()
    tr.shuffle(1235)
    b = tr.get_permutation()
    tr.shuffle(1234)
    c = tr.get_permutation()
    n = len(p["starts"])
    np.testing.assert_array_equal(np.sort(a), np.arange(n, dtype=np.uint64))
    np.testing.assert_array_equal(np.sort(b), np.arange(n, dtype=np.uint64))
    np.testing.assert_array_equal(a, c)
    assert (a != b).mean() > 0.9
    assert (a != np.arange(n)).mean() > 0.9
    tr.close()


def test_error_paths(built_lib):
    with pytest.raises(_lib.FlyvecError, match="hid"):
        Trainer(hid=0, vocab=10)
    with pytest.raises(_lib.FlyvecError, match="m = 2"):
        Trainer(hid=8, vocab=10, delta=0.5, m=3)
    tr = Trainer(hid=8, vocab=10, window=3, batch=4)
    with pytest.raises(_lib.FlyvecError, match="weights"):
        tr.run_steps(0, 1, 1e-3)
    tr.set_weights(np.zeros((8, 20), np.float32))
    with pytest.raises(_lib.FlyvecError, match="corpus"):
        tr.run_steps(0, 1, 1e-3)
    enc = np.array([1, 2, 3, 11, 4, 5], np.int32)  # 11 >= vocab
    with pytest.raises(_lib.FlyvecError, match="token id"):
        tr.set_corpus(enc, np.array([0, 6], np.uint64))
    with pytest.raises(_lib.FlyvecError, match="offsets"):
        tr.set_corpus(np.zeros(6, np.int32), np.array([1, 6], np.uint64))
    tr.close()


def test_zero_weights_learn_nothing(built_lib):
    """sigma = 0 gives W = 0, every xx = 0, no unit active, no update (the reference's
    legacy default; cu_special_reduction.cu:336)."""
    p = small_problem(K=16, V=100, W=5, ntok=3000, sigma=0.0)
    tr = make_trainer(p, 100)
    st = tr.run_steps(0, 3, 2e-4)
    np.testing.assert_array_equal(tr.get_weights(), p["W0"])
    assert st["device_error"] == 0
    tr.close()


def test_cli_mirror_trains_and_resumes(built_lib, tmp_path):
    """flyvec_train's mirror: the reference's flags, file formats and checkpoint names
    (flyvec/train_flyvec.py:31-47, 186-189, 262-263); a run of three epochs equals two epochs plus a
    run resumed from the second checkpoint, and equals what the library API computes."""
    from flyvec_b200 import train_flyvec as cli

    p = small_problem(K=32, V=300, W=5, ntok=6000, seed=41)
    p["enc"][0] = 299  # max(encodings) + 1 is the vocabulary the CLI infers (train_flyvec.py:168)
    np.save(tmp_path / "encodings.npy", p["enc"].astype(np.int32))
    np.save(tmp_path / "offsets.npy", p["off"].astype(np.uint64))
    common = [str(tmp_path / "encodings.npy"), str(tmp_path / "offsets.npy"), "--hid", "32", "--W", "5", "-b", "128",
              "--initial_learning_rate", "0.0004", "--sigma", "1.0", "--seed", "7", "--Nep", "3"]
    quiet = lambda *a, **k: None
    base = cli.train(cli.parse_args(common + ["-o", str(tmp_path / "a")]), log=quiet)
    assert base.endswith("flyvec_model_H_32_W_5_LR_0.0004_")
    ck = [np.load(base + f"{ep}.npy") for ep in range(3)]
    assert all(c.shape == (32, 600) and c.dtype == np.float32 for c in ck)
    assert not np.array_equal(ck[0], ck[2])
    # resume from the second checkpoint: only epoch 2 runs, with the same order and learning rate
    resumed = cli.train(cli.parse_args(common + ["-o", str(tmp_path / "b"), "--starting_checkpoint", base + "1.npy"]), log=quiet)
    # the reference resumes at int(name.split('_')[-1]) = 1, i.e. it repeats epoch 1 (train_flyvec.py:236-239, 252)
    again = np.load(resumed + "1.npy")
    assert again.shape == (32, 600)
    # the library API gives the CLI's first epoch
    f = orc.inverse_word_frequency(p["enc"], 300, saturate_fp32=False)
    tr = Trainer(hid=32, vocab=300, window=5, batch=128, lr0=0.0004)
    tr.set_corpus(p["enc"], p["off"])
    tr.set_weights(np.float32(np.random.default_rng(7).normal(0.0, 1.0, (32, 600))))
    tr.shuffle(7 * 1000003 + 0)
    tr.run_epoch(0, 3)
    np.testing.assert_array_equal(tr.get_weights(), ck[0])
    np.testing.assert_array_equal(tr.inverse_frequency(), f)
    tr.close()
