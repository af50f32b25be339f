"""One rank of the two-rank trainer test; launched by tests/test_gpu_multi.py through
``torch.distributed.run``.  Runs a few global steps with the library's own NCCL
exchange and writes this rank's weights and per-step winners to ``<out>/rank<r>.npz``."""
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from flyvec_b200.engine import Trainer  # noqa: E402
from tests.helpers import small_problem  # noqa: E402


def main():
    out = Path(sys.argv[1])
    nsteps, batch = int(sys.argv[2]), int(sys.argv[3])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    import torch.distributed as dist

    dist.init_process_group("gloo")
    p = small_problem(K=64, V=512, W=11, ntok=30000, seed=21)
    tr = Trainer(hid=p["K"], vocab=p["V"], window=p["W"], batch=batch, lr0=2e-4, device=local, rank=rank, world=world)
    box = [Trainer.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    tr.init_comm(box[0])
    tr.set_corpus(p["enc"], p["off"])
    tr.set_weights(p["W0"])
    tr.set_permutation(p["perm"])
    wins, ncs = [], []
    for step in range(nsteps):
        win, xx, nc, s = tr.step_debug(step, np.float32(2e-4))
        wins.append(win)
        ncs.append(nc)
    st = tr.run_steps(nsteps, 3, 2e-4)  # and a few more without the debug read-back
    W_a = tr.get_weights()
    # 40 more steps twice from the same weights: ids built on the GPU from the resident corpus, and ids of
    # this rank's windows fed from host memory and all-gathered on the GPUs (two chunks, the second partial)
    more, first = 40, nsteps + 3
    tr.run_steps(first, more, 2e-4)
    W_res = tr.get_weights()
    tr.set_weights(W_a)
    sel = p["perm"][first * world * batch:(first + more) * world * batch].reshape(more, world, batch)[:, rank, :].reshape(-1)
    pos = p["starts"][sel].astype(np.int64)[:, None] + np.arange(p["W"], dtype=np.int64)[None, :]
    ids = p["enc"][pos].astype(np.int32)
    ids[:, p["W"] // 2] += p["V"]
    tr.run_steps_host_local(np.ascontiguousarray(ids.reshape(more, batch, p["W"])), more, 2e-4)
    W_loc = tr.get_weights()
    np.savez(out / f"rank{rank}.npz", W=W_a, wins=np.stack(wins), ncs=np.array(ncs),
             windows=st["windows"], W_res=W_res, W_loc=W_loc, mode=tr.comm_mode)
    tr.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
