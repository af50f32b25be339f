"""Several ranks driven by one process (fv_trainers_link): the peer-mailbox exchange and both forms
of the cross-rank update -- replicated (every rank rebuilds every rank's scatter) and sharded (every
rank owns the rows i % world == rank and sends the counts of their touched positions to its peers)
-- against the oracle's `ngpus = world` step.  All ranks sit on device 0 and are advanced phase by
phase, so these tests need one GPU; the kernels and the packets are those of a multi-GPU run."""
import numpy as np
import pytest

from flyvec_b200 import _lib, synth
from flyvec_b200.engine import Trainer, TrainerGroup
from oracle import c_oracle
from oracle import flyvec_oracle as orc
from tests.helpers import check_winners, small_problem
from tests.test_gpu_shapes import assert_weights_close

pytestmark = pytest.mark.gpu


def make_group(p, world, B, shard, delta=0.0, lr0=2e-4):
    g = TrainerGroup([0] * world, hid=p["K"], vocab=p["V"], window=p["W"], batch=B, lr0=lr0, delta=delta, shard=shard)
    assert g.set_corpus(p["enc"], p["off"]) == len(p["starts"])
    g.set_weights(p["W0"])
    g.set_permutation(p["perm"])
    assert all(t.comm_mode == 2 for t in g.ranks)
    return g


def replicas_identical(g):
    W0 = g.get_weights(0)
    for r in range(1, g.n):
        np.testing.assert_array_equal(g.get_weights(r), W0)
    return W0


@pytest.mark.parametrize("world,shard", [(2, False), (2, True), (3, True), (4, False), (4, True), (8, True)])
def test_linked_ranks_teacher_forced(built_lib, world, shard):
    p = small_problem(K=64, V=512, W=11, ntok=60000, seed=13)
    B = 200
    g = make_group(p, world, B, shard)
    eps = np.float32(2e-4)
    Wcur = p["W0"]
    for t in range(4):
        win, xx, nc, s = g.step_debug(t, eps)
        Wgpu = replicas_identical(g)
        order = p["perm"][t * world * B:(t + 1) * world * B]
        idxs = [orc.build_idx(p["enc"], p["starts"], order[r * B:(r + 1) * B], 11, 512) for r in range(world)]
        Wref, info = orc.train_step(Wcur, idxs, p["f"], 512, eps)
        for r in range(world):
            np.testing.assert_array_equal(win[r], info["win"][r])
            np.testing.assert_allclose(xx[r], info["xx"][r], rtol=2e-5, atol=1e-7)
        # every rank holds every rank's packet
        for t_r in g.ranks[1:]:
            w_r, x_r = t_r.last_packets()
            np.testing.assert_array_equal(w_r, win)
            np.testing.assert_array_equal(x_r, xx)
        np.testing.assert_allclose(nc, info["nc"], rtol=1e-5)
        assert_weights_close(Wgpu, Wref)
        Wcur = Wgpu
    g.close()


@pytest.mark.parametrize("shard", [False, True])
def test_linked_ranks_free_running_with_fold_and_ragged_tail(built_lib, shard):
    """A whole small epoch on 3 ranks: the scales are folded on the way (every 128 steps), the last
    global step is partial (one rank short, one rank empty)."""
    world, B, K, V, W = 3, 40, 48, 300, 7
    p = small_problem(K=K, V=V, W=W, ntok=26000, seed=17)
    ns = len(p["starts"])
    keep = (ns // (world * B)) * world * B - B - 7  # last step: rank 0 full, rank 1 short, rank 2 empty
    assert keep // (world * B) >= 130
    starts = p["starts"][:keep]
    g = TrainerGroup([0] * world, hid=K, vocab=V, window=W, batch=B, lr0=1e-3, shard=shard)
    for t in g.ranks:
        enc = _lib.as_c(p["enc"], np.int32)
        st = _lib.as_c(starts, np.uint64)
        _lib.check(_lib.lib().fv_trainer_set_corpus_windows(t._h, _lib.ptr(enc), enc.size, _lib.ptr(st), st.size))
    g.set_weights(p["W0"])
    perm = np.random.default_rng(5).permutation(keep).astype(np.uint64)
    g.set_permutation(perm)
    st = g.run_epoch(0, 1)
    assert st[0]["steps"] == (keep + world * B - 1) // (world * B)
    Wgpu = replicas_identical(g)
    g.close()
    Wref, _ = orc.run_epoch(p["W0"], p["enc"], starts, perm, p["f"], V, W, B, world, np.float32(1e-3))
    assert_weights_close(Wgpu, Wref)


def test_config2_shapes_eight_linked_ranks_sharded(built_lib):
    """Config 2's global step through the multi-GPU code itself: 8 ranks x 10000 windows, peer
    mailboxes, sharded update; teacher-forced against the oracle with ngpus = 8."""
    K, V, W, B, world, steps = 400, 20000, 11, 10000, 8, 3
    enc, off = synth.make_corpus(2_500_000, V, s=1.0, mean_len=25.0, min_len=W, seed=102)
    starts = orc.enumerate_windows(off, W)
    f = orc.inverse_word_frequency(enc, V, saturate_fp32=False)
    assert len(starts) >= steps * world * B
    perm = np.random.default_rng(202).permutation(len(starts)).astype(np.uint64)
    W0 = synth.make_weights(K, 2 * V, seed=2)
    p = dict(K=K, V=V, W=W, enc=enc, off=off, starts=starts, W0=W0, perm=perm)
    g = make_group(p, world, B, shard=True)
    runner = c_oracle.StepRunner(K, 2 * V, V, W, B, world)
    eps = np.float32(2e-4)
    Wcur = W0.copy()
    for t in range(steps):
        win, xx, nc, s = g.step_debug(t, eps)
        Wgpu = replicas_identical(g)
        order = perm[t * world * B:(t + 1) * world * B]
        idx = np.stack([orc.build_idx(enc, starts, order[r * B:(r + 1) * B], W, V) for r in range(world)])
        Wref = Wcur.copy()
        rwin, rxx, rnc, rs = runner.step(Wref, idx, [B] * world, f, eps)
        flips = 0
        for r in range(world):
            if not np.array_equal(win[r], rwin[r]):
                flips += check_winners(win[r], rwin[r], orc.activations(Wcur, idx[r], None, V))
        if flips == 0:
            np.testing.assert_allclose(xx, rxx, rtol=2e-5, atol=1e-7)
            np.testing.assert_allclose(nc, rnc, rtol=1e-5)
            assert_weights_close(Wgpu, Wref)
        assert flips <= 2
        Wcur = Wgpu
    g.close()


@pytest.mark.parametrize("slots", [2, 4, 8])
def test_batched_owner_tagging_on_duplicate_heavy_steps(built_lib, slots):
    """The tagging kernel with several slots per thread (owner-only form of the sharded update), forced at a
    small shape: a tiny vocabulary makes the same (unit, token) pair occur many times in one block round."""
    world, B = 3, 700
    p = small_problem(K=40, V=36, W=9, ntok=40000, seed=29, zipf_s=1.2)
    g = make_group(p, world, B, shard=True, lr0=5e-4)
    for t in g.ranks:
        t.set_option("tag_slots", slots)
    eps = np.float32(5e-4)
    Wcur = p["W0"]
    for t in range(3):
        win, xx, nc, s = g.step_debug(t, eps)
        Wgpu = replicas_identical(g)
        order = p["perm"][t * world * B:(t + 1) * world * B]
        idxs = [orc.build_idx(p["enc"], p["starts"], order[r * B:(r + 1) * B], 9, 36) for r in range(world)]
        Wref, info = orc.train_step(Wcur, idxs, p["f"], 36, eps)
        for r in range(world):
            np.testing.assert_array_equal(win[r], info["win"][r])
        np.testing.assert_allclose(nc, info["nc"], rtol=1e-5)
        assert_weights_close(Wgpu, Wref)
        Wcur = Wgpu
    g.close()


def test_sharded_and_replicated_updates_agree_bit_for_bit(built_lib):
    """Both forms of the update compute the same function of the exchanged data."""
    p = small_problem(K=100, V=400, W=11, ntok=80000, seed=23)
    out = []
    for shard in (False, True):
        g = make_group(p, 4, 500, shard)
        g.run_steps(0, 12, np.float32(5e-4))
        out.append(replicas_identical(g))
        g.close()
    np.testing.assert_array_equal(out[0], out[1])


def test_wait_for_a_silent_peer_runs_out(built_lib):
    """Rank 0 of a 2-rank job whose peer never sends anything: the bounded wait for the peer's
    winners gives up after `spin_limit` polls, the rest of the call falls through, the call returns
    FV_ERR_TIMEOUT, and the device stays usable."""
    p = small_problem(K=32, V=200, W=7, ntok=8000, seed=3)
    tr = Trainer(hid=32, vocab=200, window=7, batch=64, world=2, rank=0)
    tr.set_corpus(p["enc"], p["off"])
    tr.set_weights(p["W0"])
    tr.set_option("loopback_peers", 1)
    tr.set_option("spin_limit", 2000)
    with pytest.raises(_lib.FlyvecError, match="FV_ERR_TIMEOUT") as ei:
        tr.run_steps(0, 3, np.float32(1e-3))
    assert ei.value.status == 6
    tr.close()
    # a fresh trainer on the same device works
    t2 = Trainer(hid=32, vocab=200, window=7, batch=64)
    t2.set_corpus(p["enc"], p["off"])
    t2.set_weights(p["W0"])
    st = t2.run_steps(0, 3, np.float32(1e-3))
    assert st["steps"] == 3 and st["device_error"] == 0
    t2.close()
