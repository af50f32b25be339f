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
