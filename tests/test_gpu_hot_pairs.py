"""Requests for the rows of the most frequent tokens: counted per (row, unit) pair by the forward pass and
claimed once by the tagging kernel (the default where a step fits one round of the one-slot-per-thread
kernel), or claimed one by one like every other request (`"hot_pairs" = 0`).  The counts are integers, so
whole runs must agree bit for bit: weights, per-step normalisers and step sizes, with one rank, emulated
ranks, linked ranks (each counts its own windows and sends the counts to the others), the anti-Hebbian term,
and a corpus in which a handful of tokens make up almost everything."""
import numpy as np
import pytest

from flyvec_b200 import _lib, synth
from flyvec_b200.engine import Trainer, TrainerGroup
from oracle import flyvec_oracle as orc
from tests.helpers import small_problem

pytestmark = pytest.mark.gpu


def run_single(p, B, steps, hot, world=1, flags=0, lr0=1e-3, delta=0.0):
    tr = Trainer(hid=p["K"], vocab=p["V"], window=p["W"], batch=B, lr0=lr0, world=world, flags=flags, delta=delta)
    tr.set_option("hot_pairs", 1 if hot else 0)
    tr.set_corpus(p["enc"], p["off"])
    tr.set_weights(p["W0"])
    tr.set_permutation(p["perm"])
    log = tr.run_steps(0, steps, np.float32(lr0), want_log=True)
    W = tr.get_weights()
    tr.close()
    return W, log["nc"], log["scale"]


def skewed_problem(K, V, W, ntok, seed, s):
    enc, off = synth.make_corpus(ntok, V, s=s, mean_len=25.0, min_len=W, seed=seed)
    starts = orc.enumerate_windows(off, W)
    return dict(K=K, V=V, W=W, enc=enc, off=off, starts=starts, W0=synth.make_weights(K, 2 * V, seed=seed + 1),
                perm=np.random.default_rng(seed + 2).permutation(len(starts)).astype(np.uint64))


@pytest.mark.parametrize("K,V,W,B,steps,world,delta,s", [
    (64, 40, 11, 300, 140, 1, 0.0, 1.0),      # fewer tokens than hot rows: every row is hot
    (100, 400, 7, 200, 140, 1, 0.0, 1.0),
    (48, 300, 9, 150, 60, 3, 0.0, 1.0),       # emulated ranks: every rank's windows are counted by the one trainer
    (64, 200, 11, 250, 60, 1, 0.3, 1.0),      # anti-Hebbian term: second winners are counted as well
    (96, 500, 11, 1000, 40, 1, 0.0, 2.5),     # three tokens make up most of the corpus
    (400, 3000, 11, 2000, 40, 1, 0.0, 1.0),   # config-1 width
])
def test_counted_and_one_by_one_agree_bit_for_bit(built_lib, K, V, W, B, steps, world, delta, s):
    p = skewed_problem(K, V, W, 2 * steps * B * world + 40000, 51, s)
    assert len(p["starts"]) >= steps * B * world
    flags = _lib.FV_FLAG_EMULATE_RANKS if world > 1 else 0
    Wa, nca, sa = run_single(p, B, steps, True, world, flags, delta=delta)
    Wb, ncb, sb = run_single(p, B, steps, False, world, flags, delta=delta)
    np.testing.assert_array_equal(nca, ncb)
    np.testing.assert_array_equal(sa, sb)
    np.testing.assert_array_equal(Wa, Wb)
    assert not np.array_equal(Wa, p["W0"])


@pytest.mark.parametrize("world", [2, 3])
def test_linked_ranks_exchange_their_counts(built_lib, world):
    p = small_problem(K=64, V=300, W=11, ntok=200000, seed=53)
    B, steps = 150, 40
    out = []
    for hot in (1, 0):
        g = TrainerGroup([0] * world, hid=p["K"], vocab=p["V"], window=p["W"], batch=B, lr0=1e-3, shard=False)
        for t in g.ranks:
            t.set_option("hot_pairs", hot)
        g.set_corpus(p["enc"], p["off"])
        g.set_weights(p["W0"])
        g.set_permutation(p["perm"])
        st = g.run_steps(0, steps, np.float32(1e-3), want_log=True)
        Ws = [g.get_weights(r) for r in range(world)]
        for r in range(1, world):
            np.testing.assert_array_equal(Ws[r], Ws[0])
        out.append((Ws[0], st[0]["nc"]))
        g.close()
    np.testing.assert_array_equal(out[0][1], out[1][1])
    np.testing.assert_array_equal(out[0][0], out[1][0])


def test_config1_shapes_200_steps(built_lib):
    """Config 1 (10000 windows per step, Zipf(1.0)): the production case of the counted path, across a fold."""
    K, V, W, B, steps = 400, 20000, 11, 10000, 200
    p = skewed_problem(K, V, W, 4_000_000, 55, 1.0)
    assert len(p["starts"]) >= steps * B
    Wa, nca, sa = run_single(p, B, steps, True, lr0=2e-4)
    Wb, ncb, sb = run_single(p, B, steps, False, lr0=2e-4)
    np.testing.assert_array_equal(nca, ncb)
    np.testing.assert_array_equal(Wa, Wb)


def test_two_linked_ranks_at_config1_shapes_exchange_their_counts(built_lib):
    """Two ranks of 10000 windows each: a step of 220000 slots goes through the batched tagging kernel, every
    hot-row slot is skipped and the ranks' counts meet in the hotboxes.  Same bits as claiming one by one."""
    K, V, W, B, steps = 400, 20000, 11, 10000, 12
    p = skewed_problem(K, V, W, 1_500_000, 57, 1.0)
    assert len(p["starts"]) >= steps * B * 2
    out = []
    for hot in (1, 0):
        g = TrainerGroup([0, 0], hid=K, vocab=V, window=W, batch=B, lr0=2e-4, shard=False)
        for t in g.ranks:
            t.set_option("hot_pairs", hot)
        g.set_corpus(p["enc"], p["off"])
        g.set_weights(p["W0"])
        g.set_permutation(p["perm"])
        st = g.run_steps(0, steps, np.float32(2e-4), want_log=True)
        W0, W1 = g.get_weights(0), g.get_weights(1)
        np.testing.assert_array_equal(W0, W1)
        out.append((W0, st[0]["nc"]))
        g.close()
    np.testing.assert_array_equal(out[0][1], out[1][1])
    np.testing.assert_array_equal(out[0][0], out[1][0])
