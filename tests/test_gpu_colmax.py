"""The column maxima behind the normaliser, computed two ways: from the candidate lists kept from step to
step (the default) and by streaming the whole matrix in every step.  Both are exact, so whole runs must
agree bit for bit -- weights, per-step normalisers and step sizes -- whatever the shape, across folds of
the scales, with one rank, emulated ranks and linked ranks with the sharded update; and the same with the
evaluation and the apply kernel fused into one (the default) or apart."""
import numpy as np
import pytest

from flyvec_b200 import _lib, synth
from flyvec_b200.engine import Trainer, TrainerGroup
from oracle import flyvec_oracle as orc
from tests.helpers import small_problem

pytestmark = pytest.mark.gpu


def run_single(p, B, steps, lists, world=1, flags=0, lr0=1e-3, delta=0.0, fused=True):
    tr = Trainer(hid=p["K"], vocab=p["V"], window=p["W"], batch=B, lr0=lr0, world=world, flags=flags, delta=delta)
    tr.set_option("colmax_lists", 1 if lists else 0)
    tr.set_option("fused_update", 1 if fused else 0)
    tr.set_corpus(p["enc"], p["off"])
    tr.set_weights(p["W0"])
    tr.set_permutation(p["perm"])
    log = tr.run_steps(0, steps, np.float32(lr0), want_log=True)
    W = tr.get_weights()
    scans = (tr.counter("matrix_scans"), tr.counter("column_rescans"))
    tr.close()
    return W, log["nc"], log["scale"], scans


@pytest.mark.parametrize("K,V,W,B,steps,world,delta", [
    (64, 40, 11, 300, 140, 1, 0.0),      # tiny vocabulary: most rows of a unit are touched in every step
    (100, 400, 7, 200, 300, 1, 0.0),     # two folds on the way
    (48, 300, 9, 150, 150, 3, 0.0),      # emulated ranks
    (64, 200, 11, 250, 140, 1, 0.3),     # anti-Hebbian term
    (400, 3000, 11, 2000, 140, 1, 0.0),  # config-1 width
])
def test_lists_and_streaming_agree_bit_for_bit(built_lib, K, V, W, B, steps, world, delta):
    p = small_problem(K=K, V=V, W=W, ntok=2 * steps * B * world + 40000, seed=41)
    assert len(p["starts"]) >= steps * B * world
    flags = _lib.FV_FLAG_EMULATE_RANKS if world > 1 else 0
    Wa, nca, sa, scans_a = run_single(p, B, steps, True, world, flags, delta=delta)
    Wb, ncb, sb, scans_b = run_single(p, B, steps, False, world, flags, delta=delta)
    np.testing.assert_array_equal(nca, ncb)
    np.testing.assert_array_equal(sa, sb)
    np.testing.assert_array_equal(Wa, Wb)
    assert scans_b == (steps, 0)
    assert scans_a[0] == 1 + (steps - 1) // 128  # the first step and the step after every fold
    # and with evaluation and apply as two kernels instead of one
    Wc, ncc, sc, scans_c = run_single(p, B, steps, True, world, flags, delta=delta, fused=False)
    np.testing.assert_array_equal(ncc, nca)
    np.testing.assert_array_equal(Wc, Wa)
    assert scans_c == scans_a


def test_lists_spare_the_matrix_pass_at_config1_shapes(built_lib):
    """Config 1: 200 steps; with the lists the matrix is streamed only for the rebuilds after new weights
    and after the fold, a single unit's column is re-read in the rare step in which its candidates were
    all touched, and the run equals the streaming one bit for bit."""
    K, V, W, B, steps = 400, 20000, 11, 10000, 200
    enc, off = synth.make_corpus(4_000_000, V, s=1.0, mean_len=25.0, min_len=W, seed=105)
    starts = orc.enumerate_windows(off, W)
    assert len(starts) >= steps * B
    p = dict(K=K, V=V, W=W, enc=enc, off=off, starts=starts, W0=synth.make_weights(K, 2 * V, seed=5),
             perm=np.random.default_rng(205).permutation(len(starts)).astype(np.uint64))
    Wa, nca, sa, scans_a = run_single(p, B, steps, True, lr0=2e-4)
    Wb, ncb, sb, scans_b = run_single(p, B, steps, False, lr0=2e-4)
    np.testing.assert_array_equal(nca, ncb)
    np.testing.assert_array_equal(Wa, Wb)
    assert scans_b == (steps, 0)
    assert scans_a[0] == 2 and scans_a[1] <= steps // 8, f"{scans_a[1]} single columns were re-read in {steps} steps"
    print(f"with candidate lists: {scans_a[0]} matrix passes and {scans_a[1]} single-column reads in {steps} steps")


@pytest.mark.parametrize("world,shard", [(2, True), (4, True), (3, False)])
def test_lists_with_linked_ranks(built_lib, world, shard):
    p = small_problem(K=64, V=300, W=11, ntok=200000, seed=43)
    B, steps = 150, 135
    out = []
    for lists in (True, False):
        g = TrainerGroup([0] * world, hid=64, vocab=300, window=11, batch=B, lr0=1e-3, shard=shard)
        for t in g.ranks:
            t.set_option("colmax_lists", 1 if lists else 0)
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
