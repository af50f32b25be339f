"""World-size-2 run of the host-side multi-rank logic on CPU (gloo): every rank
computes the forward part of the oracle on its own shard of the step, the ranks
exchange only (winners, xx) -- what the library's all-gather carries -- and each
rebuilds the full update in closed form.  Both ranks must agree bit for bit with
each other and, to rounding, with the reference-style combine over dense ds
matrices (cu_special_reduction.cu:26-99, 316-354)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from oracle import flyvec_oracle as orc  # noqa: E402
from tests.helpers import rel_err, small_problem  # noqa: E402

WORLD, BATCH, STEPS = 2, 96, 3


def shard(ns, batch, world, rank, step):
    """Windows of the order that `rank` owns in global step `step`: the library's own rank
    arithmetic (fv_shard_range, host code, no device needed)."""
    from flyvec_b200.engine import shard_range

    first, count = shard_range(ns, batch, world, rank, step)
    return first, first + count


def _worker(rank, port, outdir):
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    p = small_problem(K=32, V=200, W=7, ntok=8000, seed=13)
    Wm = p["W0"]
    eps = np.float32(2e-4)
    ns = len(p["starts"])
    for step in range(STEPS):
        # every rank can rebuild everybody's input ids from the shared corpus and order
        idxs = []
        for g in range(WORLD):
            lo, hi = shard(ns, BATCH, WORLD, g, step)
            idxs.append(orc.build_idx(p["enc"], p["starts"], p["perm"][lo:hi], p["W"], p["V"]))
        _, xx, win, _, _ = orc.device_phase(Wm, idxs[rank], p["f"], p["V"])
        packet = torch.from_numpy(np.concatenate([win.astype(np.float32), xx]))  # B winners then K floats
        gathered = [torch.empty_like(packet) for _ in range(WORLD)]
        dist.all_gather(gathered, packet)
        wins = [g[:BATCH].numpy().astype(np.int32) for g in gathered]
        xxs = [g[BATCH:].numpy() for g in gathered]
        Wm, nc, s = orc.closed_form_update(Wm, idxs, wins, xxs, p["f"], p["V"], eps)
    np.save(Path(outdir) / f"w{rank}.npy", Wm)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_reference_combine(tmp_path):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(port, str(tmp_path)), nprocs=WORLD, join=True)
    w0, w1 = np.load(tmp_path / "w0.npy"), np.load(tmp_path / "w1.npy")
    np.testing.assert_array_equal(w0, w1)

    p = small_problem(K=32, V=200, W=7, ntok=8000, seed=13)
    Wref = p["W0"]
    ns = len(p["starts"])
    for step in range(STEPS):
        idxs = []
        for g in range(WORLD):
            lo, hi = shard(ns, BATCH, WORLD, g, step)
            idxs.append(orc.build_idx(p["enc"], p["starts"], p["perm"][lo:hi], p["W"], p["V"]))
        Wref, _ = orc.train_step(Wref, idxs, p["f"], p["V"], np.float32(2e-4))
    assert rel_err(w0, Wref) < 2e-6
    assert rel_err(w0, p["W0"]) > 1e-5


def test_closed_form_equals_dense_reference_form():
    """Single process, 1 and 3 devices, including a device with no windows."""
    p = small_problem(K=24, V=150, W=5, ntok=5000, seed=17)
    for sizes in ([80], [50, 0, 30]):
        idxs, lo = [], 0
        for b in sizes:
            idxs.append(orc.build_idx(p["enc"], p["starts"], p["perm"][lo:lo + b], p["W"], p["V"]))
            lo += b
        Wref, info = orc.train_step(p["W0"], idxs, p["f"], p["V"], np.float32(1e-3))
        Wcf, nc, s = orc.closed_form_update(p["W0"], idxs, info["win"], info["xx"], p["f"], p["V"], np.float32(1e-3))
        np.testing.assert_allclose(nc, info["nc"], rtol=1e-6)
        assert rel_err(Wcf, Wref) < 1e-6


def _ids_worker(rank, port, outdir):
    """Rank-local feed of input ids: every rank builds the ids of its own windows only, one all-gather
    lays the ranks' blocks of a chunk of steps side by side as [rank][step][batch*window], and block
    (step, rank) is read at offset rank * (steps * batch * window) + step * batch * window -- the
    addressing the library uses for fv_trainer_run_steps_host_local."""
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    p = small_problem(K=32, V=200, W=7, ntok=8000, seed=13)
    ns, Wd = len(p["starts"]), p["W"]
    own = []
    for step in range(STEPS):
        lo, hi = shard(ns, BATCH, WORLD, rank, step)
        own.append(orc.build_idx(p["enc"], p["starts"], p["perm"][lo:hi], Wd, p["V"]).reshape(-1))
    mine = torch.from_numpy(np.concatenate(own).astype(np.int32))
    gathered = [torch.empty_like(mine) for _ in range(WORLD)]
    dist.all_gather(gathered, mine)
    flat = torch.cat(gathered).numpy()
    rstride, own_ids = STEPS * BATCH * Wd, BATCH * Wd
    ok = True
    for step in range(STEPS):
        for g in range(WORLD):
            lo, hi = shard(ns, BATCH, WORLD, g, step)
            want = orc.build_idx(p["enc"], p["starts"], p["perm"][lo:hi], Wd, p["V"]).reshape(-1)
            got = flat[g * rstride + step * own_ids:g * rstride + (step + 1) * own_ids]
            ok = ok and np.array_equal(got, want)
    np.save(Path(outdir) / f"ids_ok{rank}.npy", np.array([ok]))
    dist.barrier()
    dist.destroy_process_group()


def test_rank_local_ids_meet_through_an_all_gather(tmp_path):
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_ids_worker, args=(port, str(tmp_path)), nprocs=WORLD, join=True)
    for r in range(WORLD):
        assert np.load(tmp_path / f"ids_ok{r}.npy")[0]
