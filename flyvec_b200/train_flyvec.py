"""``flyvec_train`` / ``flyvec_compile``: the reference's training CLI
(flyvec/train_flyvec.py:25-263) over the CUDA library.

Flags, defaults, input formats (``encodings.npy`` int32 token ids, ``offsets.npy``
uint64 chunk boundaries) and the checkpoint name and layout
(``{prefix}_H_{hid}_W_{W}_LR_{lr}_{epoch}.npy``, float32 ``[K][2V]``) are the
reference's.  ``--seed`` and ``--gpus`` are additions.  Like the reference
(flyvec/train_flyvec.py:141-146) one process drives all GPUs: ``--gpus N`` makes
one trainer per device, links them, and the library runs one host thread per GPU.
When a launcher has started one process per GPU instead (``RANK`` and
``WORLD_SIZE`` in the environment) every process is one rank and the ranks meet
through :mod:`flyvec_b200.rendezvous`.  Nothing here needs PyTorch.
"""
from __future__ import annotations

import argparse
import os
import re
import time
from pathlib import Path

import numpy as np

__all__ = ["init", "main", "train", "parse_args"]


def init(argv=None):
    """``flyvec_compile``: build the CUDA library in-tree (the reference runs its
    ``short_make`` here, flyvec/train_flyvec.py:25-27)."""
    from . import _lib

    path = _lib.build(verbose=True)
    print(f"built {path}")


def parse_args(argv=None):
    p = argparse.ArgumentParser(prog="flyvec_train", description="Train FlyVec synapses on a tokenised corpus")
    p.add_argument("encodings_source", type=str, help="Path to the tokens encoded as IDs (np.int32)")
    p.add_argument("offsets_source", type=str,
                   help="Path to the chunk boundaries (np.uint64, first value 0, last value = number of tokens)")
    p.add_argument("-o", "--output_dir", type=str, default=".", help="Directory for the checkpoints")
    p.add_argument("-s", "--save_every", type=int, default=1, help="Epochs between checkpoints")
    p.add_argument("--ckpt_prefix", type=str, default="flyvec_model", help="Prefix of each checkpoint name")
    p.add_argument("--starting_checkpoint", type=str, default=None, help="Path to a saved .npy checkpoint")
    p.add_argument("--W", type=int, default=11, help="Size of the W-gram sliding window")
    p.add_argument("--hid", type=int, default=400, help="Number of hidden units (neurons)")
    p.add_argument("--initial_learning_rate", type=float, default=0.002, help="Initial learning rate")
    p.add_argument("--delta", type=float, default=0.0, help="Anti-Hebbian strength")
    p.add_argument("--mu", type=float, default=0.0, help="Mean of the random normal initialisation")
    p.add_argument("--sigma", type=float, default=0.02, help="Std of the random normal initialisation")
    p.add_argument("--Nep", type=int, default=15, help="Maximum number of epochs")
    p.add_argument("-b", "--batch_size", type=int, default=10000, help="Minibatch size per GPU")
    p.add_argument("--prec", type=float, default=1.0e-30, help="Precision, avoids dividing by 0")
    p.add_argument("--seed", type=int, default=None, help="Seed of the initial weights and the window order")
    p.add_argument("--gpus", type=int, default=1, help="Number of GPUs (data-parallel ranks)")
    return p.parse_args(argv)


def checkpoint_epoch(path: str) -> int:
    """Epoch encoded at the end of a checkpoint name.  The reference takes
    ``int(path.split('_')[-1])`` (flyvec/train_flyvec.py:236-239), which cannot
    parse a name that still carries its ``.npy`` suffix; both forms work here."""
    stem = re.sub(r"\.npy$", "", os.path.basename(path))
    return int(stem.split("_")[-1])


def train(args, log=print):
    """The body of ``main``.  One process drives ``--gpus`` devices, unless a launcher made this
    process one rank of several (then it drives its own device only)."""
    from .engine import Trainer, TrainerGroup
    from .rendezvous import Rendezvous, env

    rank, world, local = env()
    launched = world > 1
    if not launched:
        log = log if rank == 0 else (lambda *a, **k: None)
    output_dir = Path(args.output_dir)
    if rank == 0 and not output_dir.exists():
        output_dir.mkdir(parents=True)
    out_name = f"{args.ckpt_prefix}_H_{args.hid}_W_{args.W}_LR_{args.initial_learning_rate}_"
    out_base = str(output_dir / out_name)

    enc = np.load(args.encodings_source, mmap_mode="r")
    off = np.load(args.offsets_source, mmap_mode="r")
    vocab = int(np.max(enc)) + 1
    N = 2 * vocab
    log(f"Determined a vocabulary size of {vocab}")

    common = dict(hid=args.hid, vocab=vocab, window=args.W, batch=args.batch_size, lr0=args.initial_learning_rate,
                  delta=args.delta, prec=args.prec)
    rdv = None
    if launched:
        rdv = Rendezvous(rank, world)
        tr = Trainer(device=local, rank=rank, world=world, **common)
        tr.init_comm(rdv.broadcast(Trainer.comm_unique_id() if rank == 0 else None))
        ngpus = world
    elif args.gpus > 1:
        tr = TrainerGroup(list(range(args.gpus)), **common)
        ngpus = args.gpus
    else:
        tr = Trainer(device=0, **common)
        ngpus = 1

    ns = tr.set_corpus(np.asarray(enc), np.asarray(off))
    log(f"Number of phrases:  {ns}")

    epoch_start = 0
    if args.starting_checkpoint is not None:
        R = np.load(args.starting_checkpoint)
        epoch_start = checkpoint_epoch(args.starting_checkpoint)
    else:
        rng = np.random.default_rng(args.seed)
        R = np.float32(rng.normal(args.mu, args.sigma, (args.hid, N)))
    base_seed = args.seed if args.seed is not None else int(time.time())
    if rdv is not None:  # every replica starts from rank 0's weights and shuffles with rank 0's seed
        R = rdv.broadcast_array(R, (args.hid, N), np.float32)
        base_seed = int(rdv.broadcast_array(np.array([base_seed], np.int64), (1,), np.int64)[0])
    tr.set_weights(R)

    for i, ep in enumerate(range(epoch_start, args.Nep)):
        log(f"epoch ID =  {ep}")
        t1 = time.time()
        tr.shuffle(base_seed * 1000003 + ep)
        t11 = time.time()
        st = tr.run_epoch(ep, args.Nep)
        t2 = time.time()
        if isinstance(st, list):
            windows, seconds = sum(x["windows"] for x in st), max(x["seconds"] for x in st)
        else:
            windows, seconds = st["windows"] * ngpus, st["seconds"]
        log(f"time per epoch =  {t2 - t1} [s]   reshuffle time =  {t11 - t1} [s]   "
            f"windows/s = {windows / max(seconds, 1e-12):.4g}")
        if rank == 0 and (((i + 1) % args.save_every) == 0 or i == (args.Nep - 1)):
            np.save(out_base + str(ep), tr.get_weights())
    if rdv is not None:
        rdv.barrier()
        rdv.close()
    tr.close()
    return out_base


def main(argv=None):
    args = parse_args(argv)
    from .rendezvous import env

    rank, _, _ = env()
    train(args, log=print if rank == 0 else (lambda *a, **k: None))


if __name__ == "__main__":
    main()
