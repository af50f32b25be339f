"""The installable surface the reference has (settings.ini:19-20 console scripts, flyvec/__init__.py:2-5
import name) and the launcher-free rendezvous of the CLI's one-process-per-GPU mode.  CPU only."""
import multiprocessing as mp
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_reference_import_names():
    from flyvec import FlyVec, GensimTokenizer
    import flyvec.train_flyvec as t
    from flyvec_b200.core import FlyVec as Mine

    assert FlyVec is Mine and GensimTokenizer is not None
    assert callable(t.main) and callable(t.init)


def test_console_scripts_install_and_answer_help(tmp_path):
    """pip-installs the package (no index, no build isolation) into a scratch directory and runs the two
    commands the reference installs."""
    target = tmp_path / "site"
    res = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--quiet",
                          "--target", str(target), str(ROOT)], capture_output=True, text=True, timeout=600)
    if res.returncode != 0 and "No module named pip" in res.stderr:
        pytest.skip("pip is not available")
    assert res.returncode == 0, res.stderr[-3000:]
    assert (target / "bin" / "flyvec_train").exists() and (target / "bin" / "flyvec_compile").exists()
    assert (target / "flyvec_b200" / "csrc" / "flyvec_b200.h").exists(), "the public header must travel with the sources"
    env = dict(os.environ, PYTHONPATH=str(target))
    out = subprocess.run([sys.executable, str(target / "bin" / "flyvec_train"), "--help"], capture_output=True, text=True,
                         env=env, cwd=str(tmp_path), timeout=120)
    assert out.returncode == 0, out.stderr[-2000:]
    for flag in ("encodings_source", "offsets_source", "--output_dir", "--save_every", "--ckpt_prefix", "--starting_checkpoint",
                 "--W", "--hid", "--initial_learning_rate", "--delta", "--mu", "--sigma", "--Nep", "--batch_size", "--prec"):
        assert flag in out.stdout, f"{flag} missing from flyvec_train --help"


def _rank(rank, world, port, q):
    from flyvec_b200.rendezvous import Rendezvous

    r = Rendezvous(rank, world, addr="127.0.0.1", port=port, timeout=60)
    uid = r.broadcast(bytes(range(128)) if rank == 0 else None)
    w = r.broadcast_array(np.arange(12, dtype=np.float32).reshape(3, 4) if rank == 0 else None, (3, 4), np.float32)
    r.barrier()
    r.close()
    q.put((rank, uid == bytes(range(128)), float(w.sum())))


def test_rendezvous_carries_id_and_weights_between_processes():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 3, port, q)) for r in range(3)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == [(0, True, 66.0), (1, True, 66.0), (2, True, 66.0)]
