"""Two real ranks (one process per GPU, NCCL exchange inside the library): the
replicas must stay bit-identical and follow the oracle's ngpus=2 semantics --
the mean over the ranks where a unit was active (cu_special_reduction.cu:42-67),
which is not what one rank with twice the batch computes."""
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from flyvec_b200 import _lib
from oracle import flyvec_oracle as orc
from tests.helpers import check_winners, rel_err, small_problem

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("exchange", ["mailbox", "mailbox-sharded", "nccl"])
def test_two_ranks_match_oracle(built_lib, tmp_path, exchange):
    """Packets written straight into the peer's memory with the replicated and with the sharded update,
    and one all-gather per step."""
    if _lib.device_count() < 2:
        pytest.skip("needs two GPUs")
    import os
    nsteps, batch, world = 4, 128, 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29541", str(ROOT / "tests" / "multi_rank_worker.py"),
           str(tmp_path), str(nsteps), str(batch)]
    env = dict(os.environ)
    env.pop("FV_COMM", None)
    env.pop("FV_SHARD", None)
    if exchange == "nccl":
        env["FV_COMM"] = "nccl"
    elif exchange == "mailbox-sharded":
        env["FV_SHARD"] = "1"
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    r0 = np.load(tmp_path / "rank0.npz")
    r1 = np.load(tmp_path / "rank1.npz")
    assert int(r0["mode"]) == (1 if exchange == "nccl" else 2)
    np.testing.assert_array_equal(r0["W"], r1["W"])       # replicas identical
    np.testing.assert_array_equal(r0["wins"], r1["wins"])  # both saw the same gathered winners
    assert int(r0["windows"]) == 3 * batch and int(r1["windows"]) == 3 * batch
    # ids fed per rank from host memory and all-gathered on the GPUs give what the resident corpus gives
    np.testing.assert_array_equal(r0["W_res"], r1["W_res"])
    np.testing.assert_array_equal(r0["W_loc"], r0["W_res"])
    np.testing.assert_array_equal(r1["W_loc"], r1["W_res"])
    assert not np.array_equal(r0["W_res"], r0["W"])

    p = small_problem(K=64, V=512, W=11, ntok=30000, seed=21)
    Wref = p["W0"]
    eps = np.float32(2e-4)
    for step in range(nsteps + 3):
        idxs = []
        for g in range(world):
            lo = (step * world + g) * batch
            idxs.append(orc.build_idx(p["enc"], p["starts"], p["perm"][lo:lo + batch], p["W"], p["V"]))
        Wprev = Wref
        Wref, info = orc.train_step(Wref, idxs, p["f"], p["V"], eps)
        if step < nsteps:
            for g in range(world):
                check_winners(r0["wins"][step][g], info["win"][g], orc.activations(Wprev, idxs[g], None, p["V"]),
                              rel_margin=1e-5)
            np.testing.assert_allclose(r0["ncs"][step], info["nc"], rtol=1e-4)
    assert rel_err(r0["W"], Wref) < 1e-5


def two_rank_oracle(p, batch, nsteps, eps):
    Wref, ncs = p["W0"], []
    for step in range(nsteps):
        idxs = []
        for g in range(2):
            lo = (step * 2 + g) * batch
            idxs.append(orc.build_idx(p["enc"], p["starts"], p["perm"][lo:lo + batch], p["W"], p["V"]))
        Wref, info = orc.train_step(Wref, idxs, p["f"], p["V"], eps)
        ncs.append(info["nc"])
    return Wref, np.array(ncs)


@pytest.mark.parametrize("shard", [False, True])
def test_one_process_drives_two_gpus(built_lib, shard):
    """The reference's arrangement (train_flyvec.py:141-146, cuda_funcs.cu:1664-1665): one process, one
    trainer and one host thread per GPU, the mailboxes mapped through CUDA peer access -- no NCCL, no
    launcher."""
    if _lib.device_count() < 2:
        pytest.skip("needs two GPUs")
    from flyvec_b200.engine import TrainerGroup

    p = small_problem(K=64, V=512, W=11, ntok=30000, seed=21)
    batch, nsteps, eps = 128, 6, np.float32(2e-4)
    g = TrainerGroup([0, 1], hid=p["K"], vocab=p["V"], window=p["W"], batch=batch, lr0=2e-4, shard=shard)
    assert g.set_corpus(p["enc"], p["off"]) == len(p["starts"])
    g.set_weights(p["W0"])
    g.set_permutation(p["perm"])
    assert all(t.comm_mode == 2 for t in g.ranks)
    st = g.run_steps(0, nsteps, eps, want_log=True)
    assert [s["windows"] for s in st] == [nsteps * batch] * 2
    W0, W1 = g.get_weights(0), g.get_weights(1)
    np.testing.assert_array_equal(W0, W1)
    Wref, ncs = two_rank_oracle(p, batch, nsteps, eps)
    np.testing.assert_allclose(st[0]["nc"], ncs, rtol=1e-4)
    assert rel_err(W0, Wref) < 1e-5
    g.close()


def test_cli_one_process_and_one_process_per_gpu_write_the_same_checkpoints(built_lib, tmp_path):
    """`flyvec_train --gpus 2` (one process drives both GPUs) and the same command as two launched ranks
    (socket rendezvous, NCCL only to hand round the mailbox handles) train the same replicas."""
    if _lib.device_count() < 2:
        pytest.skip("needs two GPUs")
    import os

    p = small_problem(K=64, V=512, W=11, ntok=30000, seed=22)
    np.save(tmp_path / "enc.npy", p["enc"].astype(np.int32))
    np.save(tmp_path / "off.npy", p["off"].astype(np.uint64))
    common = [str(tmp_path / "enc.npy"), str(tmp_path / "off.npy"), "--hid", "64", "-b", "128", "--Nep", "2", "--seed", "5",
              "--sigma", "1.0", "--initial_learning_rate", "0.001"]
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "FV_COMM", "FV_SHARD"):
        env.pop(k, None)
    one = subprocess.run([sys.executable, "-m", "flyvec_b200.train_flyvec", *common, "-o", str(tmp_path / "one"), "--gpus", "2"],
                         capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert one.returncode == 0, one.stdout[-2000:] + one.stderr[-4000:]
    per = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                          "127.0.0.1", "--master-port", "29547", "-m", "flyvec_b200.train_flyvec", *common, "-o",
                          str(tmp_path / "per")], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert per.returncode == 0, per.stdout[-2000:] + per.stderr[-4000:]
    names = sorted(f.name for f in (tmp_path / "one").iterdir())
    assert names == sorted(f.name for f in (tmp_path / "per").iterdir()) and len(names) == 2
    for n in names:
        a, b = np.load(tmp_path / "one" / n), np.load(tmp_path / "per" / n)
        assert a.shape == (64, 1024) and np.isfinite(a).all()
        np.testing.assert_array_equal(a, b)
    assert not np.array_equal(np.load(tmp_path / "one" / names[0]), np.load(tmp_path / "one" / names[1]))
