#!/usr/bin/env python
"""Benchmark of the FlyVec train step (and, on request, of the hashers) on B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference ...                      # the CPU arm

A "step" is one global minibatch step: every GPU processes ``batch`` = 10 000
windows of w = 11 tokens against K = 400 hidden units over a V = 20 000
vocabulary.  The corpus is synthetic (bounded Zipf(1.0) token ids, geometric
chunk lengths, seeds fixed); initial weights are N(0,1).  Rank 0 prints one JSON
line.  Under ``torch.distributed.run`` every process is one rank; the data path
uses the library's own NCCL communicator, ``torch.distributed`` (gloo) only
carries the rendezvous, the barriers and the max-over-ranks of the timings.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG = dict(K=400, V=20000, W=11, batch=10000, lr=2e-4, zipf_s=1.0, chunk_mean=25.0, tokens_per_gpu=50_000_000)
CORPUS_SEED, WEIGHT_SEED, PERM_SEED = 101, 1, 201
WORKLOAD = "train step, config 1 shapes: K=400 V=20000 w=11 batch=10000/GPU lr=2e-4 W0~N(0,1)"
METRIC = "train windows/sec (K=400,V=20k,w=11)"
CONFIG_ID = 1


def select_config(n: int):
    """`--config 3`: the large-model shapes (synapse matrix 400 MB, HBM-resident) instead of the headline
    configuration; a second measurement, not the line the metric is quoted on."""
    global WORKLOAD, METRIC, CONFIG_ID
    if n == 3:
        CFG.update(K=1000, V=50000, W=15, batch=20000, lr=2e-4, zipf_s=1.1, chunk_mean=40.0, tokens_per_gpu=50_000_000)
        WORKLOAD = "train step, config 3 shapes: K=1000 V=50000 w=15 batch=20000/GPU lr=2e-4 W0~N(0,1)"
        METRIC = "train windows/sec (K=1000,V=50k,w=15)"
        CONFIG_ID = 3


def forward_dram_traffic():
    """DRAM bytes (read + write) per launch of the forward kernel as the kept ncu capture of this
    workload measured them: the line ``dram_bytes_per_launch = <number>`` of
    profiles/k_forward_config1.md, or None when there is no such capture."""
    import re

    f = ROOT / "profiles" / "k_forward_config1.md"
    if not f.exists():
        return None
    m = re.search(r"^dram_bytes_per_launch\s*=\s*([0-9.eE+]+)", f.read_text(), re.M)
    return float(m.group(1)) if m else None


# ----------------------------------------------------------------------------
# helpers
# ----------------------------------------------------------------------------
def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


class Dist:
    """Rendezvous / barrier / max-reduce over gloo; a no-op for one rank."""

    def __init__(self, world):
        self.world = world
        self.dist = None
        if world > 1:
            import torch.distributed as dist

            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("gloo")
            self.dist = dist

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def bcast_obj(self, obj, src=0):
        if not self.dist:
            return obj
        box = [obj]
        self.dist.broadcast_object_list(box, src=src)
        return box[0]

    def max(self, x: float) -> float:
        if not self.dist:
            return x
        import torch

        t = torch.tensor([x], dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t[0])

    def sum(self, x: float) -> float:
        if not self.dist:
            return x
        import torch

        t = torch.tensor([x], dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t[0])

    def gather_obj(self, obj):
        """``obj`` of every rank, in rank order, on every rank."""
        if not self.dist:
            return [obj]
        box = [None] * self.world
        self.dist.all_gather_object(box, obj)
        return box

    def close(self):
        if self.dist:
            self.dist.destroy_process_group()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(smax)), "reasons": sorted(reasons),
                "samples": len(sm)}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s)"


def make_or_load_corpus(ntok: int, rank: int, dist: Dist):
    """Rank 0 draws the corpus once and shares it through /dev/shm."""
    from flyvec_b200 import synth

    if dist.world == 1:
        return synth.make_corpus(ntok, CFG["V"], s=CFG["zipf_s"], mean_len=CFG["chunk_mean"], min_len=CFG["W"],
                                 seed=CORPUS_SEED)
    tag = os.environ.get("MASTER_PORT", "0")
    base = Path("/dev/shm" if Path("/dev/shm").exists() else tempfile.gettempdir()) / f"fvbench_{tag}_{ntok}"
    if rank == 0:
        base.mkdir(exist_ok=True)
        enc, off = synth.make_corpus(ntok, CFG["V"], s=CFG["zipf_s"], mean_len=CFG["chunk_mean"], min_len=CFG["W"],
                                     seed=CORPUS_SEED)
        np.save(base / "enc.npy", enc)
        np.save(base / "off.npy", off)
    dist.barrier()
    enc = np.load(base / "enc.npy", mmap_mode="r")
    off = np.load(base / "off.npy", mmap_mode="r")
    dist.barrier()  # every rank has the files mapped: the names can go, the pages stay until the last unmap
    if rank == 0:
        import shutil

        shutil.rmtree(base, ignore_errors=True)
    return enc, off


def build_idx_host(enc, starts, perm, W, V):
    """Input ids of the given windows (token, centre token + V) as the streaming
    entry point takes them."""
    pos = starts[perm].astype(np.int64)[:, None] + np.arange(W, dtype=np.int64)[None, :]
    idx = np.asarray(enc)[pos].astype(np.int32)
    idx[:, W // 2] += V
    return idx


# ----------------------------------------------------------------------------
# this library
# ----------------------------------------------------------------------------
def bench_train(args):
    from flyvec_b200 import _lib, engine, synth

    rank, world, local = dist_env()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"
    dist = Dist(world)
    K, V, W, B = CFG["K"], CFG["V"], CFG["W"], CFG["batch"]
    steps, warmup = args.steps, args.warmup
    need_windows = (steps + warmup + 8 + max(steps, args.e2e_steps)) * world * B
    ntok = args.tokens or min(CFG["tokens_per_gpu"] * world, 400_000_000)
    enc, off = make_or_load_corpus(ntok, rank, dist)

    tr = engine.Trainer(hid=K, vocab=V, window=W, batch=B, lr0=CFG["lr"], device=local, rank=rank, world=world)
    if world > 1:
        uid = dist.bcast_obj(engine.Trainer.comm_unique_id() if rank == 0 else None)
        tr.init_comm(uid)
    ns = tr.set_corpus(np.asarray(enc), np.asarray(off))
    assert ns >= need_windows, f"corpus has {ns} windows, {need_windows} needed: raise --tokens"
    tr.set_weights(synth.make_weights(K, 2 * V, seed=WEIGHT_SEED))
    tr.shuffle(PERM_SEED)
    eps = np.float32(CFG["lr"])  # one epoch: eps = lr0 * (1 - 0/1)

    # ---- device-resident loop ------------------------------------------------
    # Warm-up and timed steps are ONE call: the library records its begin event on the stream between
    # step `warmup`-1 and step `warmup`, so exactly `steps` steps of a loop that is already in its
    # steady state (ids staged ahead, every rank in step with its peers) lie between the two events.
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    dist.barrier()
    t0 = time.perf_counter()
    st = tr.run_steps_timed(0, warmup + steps, warmup, eps)  # returns after the stream is idle
    wall = time.perf_counter() - t0
    dist.barrier()
    assert st["timed_steps"] == steps
    sec = dist.max(st["seconds"])
    wall = dist.max(wall)
    fwd_s = dist.max(st["fwd_seconds"])
    total_windows = steps * world * B
    value = total_windows / sec

    # ---- the replicas must have stayed identical ------------------------------------
    import zlib

    Wnow = tr.get_weights()
    digest = (zlib.crc32(Wnow.tobytes()), float(st["last_nc"]), float(st["last_scale"]))
    digests = dist.gather_obj(digest)
    replicas_identical = all(d == digests[0] for d in digests)

    # ---- end to end: ids streamed from pinned host memory, normalisers read back ----
    # its own step count: a call has fixed costs (control upload, final synchronisation, log read-back) that
    # a user's epoch of thousands of steps does not notice but 20 steps would
    e2e_steps = max(steps, args.e2e_steps)
    perm = tr.get_permutation()
    starts = engine.enumerate_windows(np.asarray(off), W)
    first = (warmup + steps) * world * B
    if first + e2e_steps * world * B > ns:
        first = 0
    # every rank feeds only its own windows (rank r's block of each global step); the ranks' ids meet on the GPUs
    sel = perm[first:first + e2e_steps * world * B].reshape(e2e_steps, world, B)[:, rank, :].reshape(-1)
    pinned = _lib.pinned_empty((e2e_steps, B, W), np.int32)
    pinned[...] = build_idx_host(enc, starts, sel, W, V).reshape(e2e_steps, B, W)
    nc_host = _lib.pinned_empty((e2e_steps,), np.float32)
    tr.run_steps_host_local(pinned[:min(8, e2e_steps)], min(8, e2e_steps), eps)  # warm the staging buffers
    dist.barrier()
    t0 = time.perf_counter()
    e2e_error = None
    try:
        tr.run_steps_host_local(pinned, e2e_steps, eps, nc_out=nc_host)
    except _lib.FlyvecError as exc:  # the line still carries the device-timed value; the failure is reported, not hidden
        e2e_error = str(exc)
    e2e_wall = dist.max(time.perf_counter() - t0)
    e2e_error = next((e for e in dist.gather_obj(e2e_error) if e), None)
    e2e_value = None if e2e_error else e2e_steps * world * B / e2e_wall
    clocks = sampler.stop() if rank == 0 else None

    # ---- roofline of the dominant kernel ---------------------------------------
    # k_forward is timed live as 50 back-to-back launches between two CUDA events on the trainer's
    # stream (an event pair around a single launch inside the step loop also counts the launch
    # latency that the pipelined loop hides).
    peak, peak_src = measured_peaks()
    fwd_bytes = B * W * K * 4 + B * (8 + 4 * W) + B * 8  # gathered rows + order entry and ids + winner and activation out
    if e2e_error is None:
        fwd_avg = dist.max(tr.time_forward(warmup + steps, reps=50))
    else:  # the trainers are void after a failed call: take the kernel's time inside the timed step loop instead
        fwd_avg = fwd_s / steps
    achieved = fwd_bytes / fwd_avg / 1e9
    step_bytes = B * W * K * 4 + 3 * K * 2 * V * 4 + B * (8 + 4 * W) + B * 2 + K * 4  # the reference schedule's figure
    # The synapse matrix (64 MB) lives in the L2, so the forward kernel's real ceiling is what the L2 gives
    # for its access pattern.  Both are measured here, in this run, with the library's probe: random
    # 1600-byte rows out of 64 MB (the gather), streaming over 64 MB (L2) and over 2 GiB (HBM).
    probes = None
    wt_mb = (2 * V * K * 4) >> 20
    gather_key = f"{'l2' if wt_mb <= 100 else 'hbm'}_gather_{K * 4}B_rows_of_{wt_mb}MB_gbs"
    if rank == 0:
        probes = {gather_key: engine.probe_read_bandwidth("gather", wt_mb << 20, K * 4, 40 if wt_mb <= 100 else 10, local),
                  "l2_stream_64MB_gbs": engine.probe_read_bandwidth("stream", 64 << 20, 16, 40, local),
                  "hbm_stream_2GiB_gbs": engine.probe_read_bandwidth("stream", 2 << 30, 16, 3, local)}

    # ---- parity of what was timed: 32 steps of this very workload against the oracle (one rank) ----
    parity = None
    if world == 1 and not args.no_cpu_baseline:
        parity = oracle_check(tr, enc, off, steps=32)

    out = {
        "metric": METRIC, "value": value, "unit": "windows/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": sec / steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "corpus_tokens": int(ntok), "windows": int(ns), "global_batch": world * B,
                   "parallelism": f"dp{world}",
                   "exchange": {0: "none", 1: "nccl all-gather per step", 2: "peer-memory mailboxes, flag-in-word packets"}[tr.comm_mode],
                   "timed_region": "steps [warmup, warmup+steps) of one run call; begin event recorded on the stream after the warm-up steps",
                   "l2": ("inputs larger than L2: corpus + window tables (>0.6 GB) stream through; the 64 MB synapse "
                          "matrix is re-read every step by design") if CONFIG_ID == 1 else
                         f"inputs larger than L2: the {wt_mb} MB synapse matrix is gathered from HBM (hot rows stay in the L2)"},
        "wall_ms_per_step": wall / steps * 1e3,
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "windows/s", "h2d_bytes_per_step": world * B * W * 4,
                "d2h_bytes_per_step": 4, "steps": e2e_steps, **({"error": e2e_error} if e2e_error else {}),
                "what": "fv_trainer_run_steps_host_local: every rank uploads the input ids of its own windows from pinned host "
                        "memory inside the call (all-gathered over NVLink when there are several ranks), per-step "
                        "normaliser copied back"},
        "gpu_launches": int(round(st["kernel_launches"] * steps / (steps + warmup))),
        "replicas_identical": replicas_identical,
        "roofline": {"kernel": "k_forward (fused gather-sum + arg-max)", "bound": "hbm", "achieved": achieved,
                     "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": forward_dram_traffic() if CONFIG_ID == 1 else None, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": fwd_bytes, "avg_launch_ms": fwd_avg * 1e3,
                     "measured_in_this_run": probes,
                     ("frac_of_l2_gather" if wt_mb <= 100 else "frac_of_hbm_gather"): (achieved / probes[gather_key]) if probes else None,
                     "note": ("rows are gathered from the L2-resident matrix, so achieved can exceed the HBM figure; "
                              "frac_of_l2_gather sets it against the same access pattern measured in this run") if wt_mb <= 100 else
                             ("the matrix exceeds the L2; the corpus is Zipf-distributed, so frequent rows are served by the L2 and "
                              "achieved can exceed what uniformly random rows (frac_of_hbm_gather's denominator) reach")},
        "phases_ms_per_step": {"forward": fwd_s / steps * 1e3, "xx kernel + all-gather (NCCL mode only; mailbox waits fall into update)": dist.max(st["exch_seconds"]) / steps * 1e3,
                               "update": dist.max(st["upd_seconds"]) / steps * 1e3},
        "step_algorithmic_gbs": step_bytes / (sec / steps) / 1e9,
        "last_nc": st["last_nc"],
    }
    if parity is not None:
        out["parity_check"] = parity
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_train_baseline(enc, off, seconds_limit=args.cpu_seconds)
    tr.close()
    if rank == 0 and world == 1 and not args.no_hash and CONFIG_ID == 1:
        out["hash"] = hash_summary(args)
    dist.close()
    if rank == 0:
        print(json.dumps(out))


def oracle_check(tr, enc, off, steps: int = 32):
    """The timed workload's first `steps` steps once more, from fresh weights, against the C oracle."""
    from flyvec_b200 import synth
    from oracle import c_oracle
    from oracle import flyvec_oracle as orc

    K, V, W, B = CFG["K"], CFG["V"], CFG["W"], CFG["batch"]
    W0 = synth.make_weights(K, 2 * V, seed=WEIGHT_SEED)
    eps = np.float32(CFG["lr"])
    tr.set_weights(W0)
    log = tr.run_steps(0, steps, eps, want_log=True)
    Wgpu = tr.get_weights()
    perm = tr.get_permutation()[:steps * B]
    starts = tr.window_starts()
    f = tr.inverse_frequency()
    runner = c_oracle.StepRunner(K, 2 * V, V, W, B, 1)
    Wref = W0.copy()
    nc = np.zeros(steps, np.float32)
    enc = np.asarray(enc)
    for t in range(steps):
        idx = orc.build_idx(enc, starts, perm[t * B:(t + 1) * B], W, V)
        _, _, nc[t], _ = runner.step(Wref, idx[None], [B], f, eps)
    err = np.abs(Wgpu.astype(np.float64) - Wref) / (np.abs(Wref) + 1e-2)
    return {"steps": steps, "against": "oracle/oracle_train.c on the same seeded inputs",
            "max_weight_err_rel_with_floor_1e-2": float(err.max()),
            "max_normaliser_rel_err": float((np.abs(log["nc"] - nc) / nc).max())}


def hash_summary(args):
    """Hashing figures for the default line: token hashing on config-0 shapes and window hashing at the
    config-4 hash lengths (a 4 M-window slice), each device-resident and end to end through host buffers."""
    import copy

    a = copy.copy(args)
    a.steps, a.warmup, a.cpu_seconds = 3, 3, min(args.cpu_seconds, 4.0)
    out = {}
    a.items, a.hash_length = 1_000_000, 50
    out["tokens_config0_hl50"] = hash_numbers(a, windows=False)
    a.items = 4_000_000
    state = {}
    for hl in (4, 16, 50, 128, 200):
        a.hash_length = hl
        a.no_cpu_baseline = args.no_cpu_baseline or hl != 50
        out[f"windows_config4_hl{hl}"] = hash_numbers(a, windows=True, state=state)
    return out


def bench_linked_ranks(args):
    """`--linked-ranks G`: the G ranks of a multi-GPU job as linked trainers on ONE GPU, advanced phase by
    phase (profiling aid, not a bench line): with FV_LOCKSTEP_TIMES=1 the library prints what each phase of
    one rank costs when it never has to wait for a peer."""
    from flyvec_b200 import engine, synth

    K, V, W, B = CFG["K"], CFG["V"], CFG["W"], CFG["batch"]
    G = args.linked_ranks
    enc, off = synth.make_corpus(args.tokens or 12_000_000, V, s=CFG["zipf_s"], mean_len=CFG["chunk_mean"], min_len=W,
                                 seed=CORPUS_SEED)
    g = engine.TrainerGroup([0] * G, hid=K, vocab=V, window=W, batch=B, lr0=CFG["lr"],
                            shard=None if args.shard < 0 else bool(args.shard))
    g.set_corpus(enc, off)
    g.set_weights(synth.make_weights(K, 2 * V, seed=WEIGHT_SEED))
    g.shuffle(PERM_SEED)
    st = g.run_steps(0, args.warmup + args.steps, np.float32(CFG["lr"]), warmup=args.warmup)
    print(json.dumps({"metric": "G linked ranks on one GPU, phase by phase", "ranks": G, "steps": args.steps,
                      "us_per_global_step_all_ranks": st[0]["seconds"] / args.steps * 1e6}))
    g.close()


def bench_update_emulated(args):
    """The replicated update (count, scan, apply) of `--emulate-ranks G` ranks' windows on ONE GPU: every rank's
    forward pass runs in turn, then one update over all G*B windows, exactly what each GPU of a G-GPU job does
    after the exchange.  For profiling the update kernels at multi-GPU sizes without a multi-GPU box."""
    from flyvec_b200 import _lib, engine, synth

    K, V, W, B = CFG["K"], CFG["V"], CFG["W"], CFG["batch"]
    G = args.emulate_ranks
    enc, off = synth.make_corpus(args.tokens or 12_000_000, V, s=CFG["zipf_s"], mean_len=CFG["chunk_mean"], min_len=W,
                                 seed=CORPUS_SEED)
    tr = engine.Trainer(hid=K, vocab=V, window=W, batch=B, lr0=CFG["lr"], world=G,
                        flags=_lib.FV_FLAG_EMULATE_RANKS if G > 1 else 0)
    tr.set_corpus(enc, off)
    tr.set_weights(synth.make_weights(K, 2 * V, seed=WEIGHT_SEED))
    tr.shuffle(PERM_SEED)
    eps = np.float32(CFG["lr"])
    tr.run_steps(0, args.warmup, eps)
    st = tr.run_steps(args.warmup, args.steps, eps)
    print(json.dumps({"metric": "update of G ranks' windows on one GPU (emulated ranks)", "ranks": G, "steps": args.steps,
                      "us_per_step": st["seconds"] / args.steps * 1e6, "update_us_per_step": st["upd_seconds"] / args.steps * 1e6,
                      "forward_us_per_step_all_ranks": st["fwd_seconds"] / args.steps * 1e6,
                      "config": {"workload": f"config 1 shapes, {G} x {B} windows per step"}}))


def hash_numbers(args, windows: bool, state: dict | None = None, device: int = 0, shard: tuple[int, int] = (0, 1)) -> dict:
    """Device-resident and end-to-end throughput of the token / window hasher.  End to end = the host-buffer
    entry point (fv_hash_tokens / fv_hash_windows) on page-locked ids and codes: upload, kernel and download
    of the whole batch inside the timed call.  `state` carries the inputs from one hash length to the next."""
    from flyvec_b200 import _lib, engine, synth

    K, V, W = CFG["K"], CFG["V"], CFG["W"]
    hl = args.hash_length
    state = state if state is not None else {}
    peak, peak_src = measured_peaks()
    code_b = (K + 7) // 8
    if "h" not in state:
        state["h"] = engine.Hasher(synth.make_weights(K, 2 * V, seed=WEIGHT_SEED), normalize=True, device=device)
        if windows:
            n = (args.items or 16_000_000) // shard[1]  # this rank's share: the items are independent, nothing is exchanged
            enc, off = synth.make_corpus(max(n // 2, 1_000_000), V, seed=104)
            starts = engine.enumerate_windows(off, W)
            sel = np.random.default_rng(204 + shard[0]).integers(0, len(starts), n)
            ids = _lib.pinned_empty((n, W), np.int32)
            ids[...] = build_idx_host(enc, starts, sel, W, V)
            state["inv_f"] = engine.inverse_frequency(enc, V)
            state["h"].set_inverse_frequency(state["inv_f"])
        else:
            n = (args.items or 1_000_000) // shard[1]
            ids = _lib.pinned_empty((n,), np.int32)
            ids[...] = synth.make_hash_ids(n, V, seed=100 + shard[0])
            state["inv_f"] = None
        state["ids"], state["n"] = ids, n
        state["codes"] = _lib.pinned_empty((n, code_b), np.uint8)
        state["d_in"] = engine.DeviceBuffer(ids.nbytes, device)
        state["d_in"].upload(ids)
        state["d_out"] = engine.DeviceBuffer(n * code_b, device)
    h, ids, n, inv_f, d_in, d_out = state["h"], state["ids"], state["n"], state["inv_f"], state["d_in"], state["d_out"]
    if windows:
        per_item = W * K * 4 + W * 4 + code_b
    else:
        # large batches go through the vocabulary table: an id in, a code gathered from the table and written out
        per_item = (4 + 2 * code_b) if n >= 4 * V else (K * 4 + code_b)
    run = (lambda: h.hash_windows_device(d_in.ptr, n, W, True, hl, d_out.ptr)) if windows else \
          (lambda: h.hash_tokens_device(d_in.ptr, n, hl, d_out.ptr))
    for _ in range(max(args.warmup, 3)):
        run()
    times = []
    for _ in range(max(args.steps, 1)):
        engine.flush_l2(device)
        times.append(run())
    t = float(np.mean(times))
    e2e = None
    for _ in range(3):  # the first call makes the staging buffers; best of the following
        t0 = time.perf_counter()
        if windows:
            h.hash_windows(ids, inv_freq=inv_f, hash_length=hl, packed=True, out=state["codes"])
        else:
            h.hash_tokens(ids, hash_length=hl, packed=True, out=state["codes"])
        dt = time.perf_counter() - t0
        e2e = dt if e2e is None or _ > 0 and dt < e2e else e2e
    assert np.array_equal(state["codes"], d_out.download((n, code_b), np.uint8)), "host-buffer and device-resident codes differ"
    cpu = None
    if not args.no_cpu_baseline:
        cpu = cpu_hash_baseline(h.weights(), V, np.asarray(ids), hl, windows, h_f=inv_f,
                                seconds_limit=args.cpu_seconds)
    pcie_bytes = int(ids.nbytes) + n * code_b
    out = {"metric": "hashed windows/sec" if windows else "hashed tokens/sec", "value": n / t,
           "unit": "windows/s" if windows else "tokens/s", "n_gpus": 1, "steps": len(times), "warmup": max(args.warmup, 3),
           "ms_per_step": t * 1e3, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
           "config": {"workload": ("config 4: window hashing" if windows else "config 0 shapes: token hashing"),
                      "items": n, "hash_length": hl, "l2": "L2 flushed between timed launches"},
           "e2e": {"value": n / e2e, "unit": "items/s", "h2d_bytes_per_step": int(ids.nbytes), "d2h_bytes_per_step": n * code_b,
                   "host_link_gbs": pcie_bytes / e2e / 1e9,
                   "what": "fv_hash_windows / fv_hash_tokens on page-locked host buffers: chunked upload, kernel and download "
                           "overlapped on two streams"},
           "roofline": {"kernel": "k_hash", "bound": "hbm", "achieved": per_item * n / t / 1e9, "peak": peak,
                        "unit": "GB/s", "frac": per_item * n / t / 1e9 / peak, "traffic": None, "peak_source": peak_src}}
    if cpu:
        out["cpu_baseline"] = cpu
    return out


def bench_hash(args, windows: bool):
    """One GPU, or `--gpus N` under torch.distributed.run: every rank hashes its own N-th of the items on its
    own GPU (the items are independent; there is no exchange), the line carries the sum over the ranks."""
    rank, world, local = dist_env()
    if world == 1:
        print(json.dumps(hash_numbers(args, windows)))
        return
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"
    dist = Dist(world)
    args.no_cpu_baseline = True
    dist.barrier()
    out = hash_numbers(args, windows, device=local, shard=(rank, world))
    n_local = out["config"]["items"]
    t = dist.max(out["ms_per_step"])
    e2e_t = dist.max(n_local / out["e2e"]["value"])
    dist.barrier()
    if rank == 0:
        out.update(value=world * n_local / (t * 1e-3), ms_per_step=t, n_gpus=world, scaling="weak")
        out["config"].update(items=world * n_local, parallelism=f"{world} independent shards, no exchange")
        out["e2e"].update(value=world * n_local / e2e_t, h2d_bytes_per_step=out["e2e"]["h2d_bytes_per_step"] * world,
                          d2h_bytes_per_step=out["e2e"]["d2h_bytes_per_step"] * world)
        out["roofline"]["note"] = "per GPU (rank 0)"
        print(json.dumps(out))
    dist.close()


def cpu_hash_baseline(syn, V, ids, hl, windows, h_f, seconds_limit: float = 15.0):
    """The oracle's numpy restatement of the reference's hashing rule on a bounded sample: for tokens the
    per-token loop shaped like FlyVec.get_sparse_embedding (flyvec/core.py:139-163, one core) and its
    vectorised form; for windows the weighted activation plus the same rule."""
    from oracle import flyvec_oracle as orc

    def timed(fn, items, first):
        n, done, spent = first, 0, 0.0
        while spent < seconds_limit / 2 and done < len(items):
            part = items[done:done + n]
            t0 = time.perf_counter()
            fn(part)
            spent += time.perf_counter() - t0
            done += len(part)
            n *= 2
        return done / spent, done, spent

    if windows:
        rate, done, spent = timed(lambda part: orc.hash_windows(syn, V, part, h_f, hl), ids, 256)
        return {"value": rate, "unit": "windows/s", "cores": 1, "kind": "port",
                "sample": f"{done} windows of the same workload, numpy restatement, {spent:.1f} s"}
    rate, done, spent = timed(lambda part: orc.hash_tokens(syn, V, part, hl), ids, 1024)
    fast, done_f, spent_f = timed(lambda part: orc.hash_tokens_fast(syn, V, part, hl), ids, 8192)
    return {"value": rate, "unit": "tokens/s", "cores": 1, "kind": "port",
            "sample": f"{done} tokens of the same workload, per-token numpy loop shaped like the reference's "
                      f"get_sparse_embedding, {spent:.1f} s",
            "vectorised_numpy_tokens_per_s": fast, "vectorised_sample": f"{done_f} tokens, {spent_f:.1f} s"}


# ----------------------------------------------------------------------------
# CPU arm: the oracle's C restatement of the reference step on the host cores
# ----------------------------------------------------------------------------
def cpu_train_baseline(enc, off, seconds_limit: float = 20.0, max_steps: int = 10 ** 9):
    """Times oracle/oracle_train.c (a literal restatement of the reference's step;
    the reference trainer itself is CUDA-only) on config-1 shapes."""
    from flyvec_b200 import synth
    from oracle import c_oracle
    from oracle import flyvec_oracle as orc

    K, V, W, B = CFG["K"], CFG["V"], CFG["W"], CFG["batch"]
    starts = orc.enumerate_windows(np.asarray(off[:200_000]), W)
    f = orc.inverse_word_frequency(np.asarray(enc), V, saturate_fp32=False)
    rng = np.random.default_rng(PERM_SEED)
    perm = rng.permutation(len(starts))
    Wm = synth.make_weights(K, 2 * V, seed=WEIGHT_SEED)
    runner = c_oracle.StepRunner(K, 2 * V, V, W, B, 1)
    nsteps, t_total = 0, 0.0
    while nsteps < max_steps and (nsteps < 2 or t_total < seconds_limit):
        idx = orc.build_idx(np.asarray(enc), starts, perm[(nsteps * B) % (len(perm) - B):][:B], W, V)
        t0 = time.perf_counter()
        runner.step(Wm, idx[None], [B], f, np.float32(CFG["lr"]))
        dt = time.perf_counter() - t0
        if nsteps > 0:  # the first call pages the scratch memory in
            t_total += dt
        nsteps += 1
    timed = nsteps - 1
    return {"value": timed * B / t_total, "unit": "windows/s", "cores": c_oracle.num_threads(), "kind": "port",
            "sample": f"{timed} full minibatch steps of {B} windows (config {CONFIG_ID} shapes), {t_total:.1f} s",
            "seconds_per_step": t_total / timed}


def bench_reference(args):
    rank, world, local = dist_env()
    if rank != 0:
        return
    from flyvec_b200 import synth

    from oracle import c_oracle

    # a launcher may have pinned OpenMP to one thread for its workers (torch.distributed.run does):
    # this arm is the CPU's turn and uses every core of the host, at any --gpus
    c_oracle.set_num_threads(os.cpu_count() or 1)
    K, V, W, B = CFG["K"], CFG["V"], CFG["W"], CFG["batch"]
    enc, off = synth.make_corpus(5_000_000, V, s=CFG["zipf_s"], mean_len=CFG["chunk_mean"], min_len=W, seed=CORPUS_SEED)
    limit = args.cpu_seconds_reference
    base = cpu_train_baseline(enc, off, seconds_limit=limit, max_steps=args.steps + 1)
    timed = int(base["sample"].split()[0])
    out = {"impl": "reference", "metric": METRIC, "value": base["value"],
           "unit": "windows/s", "n_gpus": args.gpus, "steps": timed, "warmup": 1,
           "ms_per_step": base["seconds_per_step"] * 1e3, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": WORKLOAD,
                      "note": "the reference trainer is CUDA-only; this arm times the C/OpenMP restatement of its "
                              "step (oracle/oracle_train.c) on the host cores, a bounded number of full steps"},
           "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
           "e2e": {"value": base["value"], "unit": "windows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["train", "hash_tokens", "hash_windows"], default="train")
    ap.add_argument("--emulate-ranks", type=int, default=0,
                    help="one GPU: time the update of this many ranks' windows (profiling aid, not a bench line)")
    ap.add_argument("--linked-ranks", type=int, default=0,
                    help="one GPU: run this many linked ranks phase by phase (profiling aid, not a bench line)")
    ap.add_argument("--shard", type=int, default=-1, help="with --linked-ranks: 1 sharded, 0 replicated update, -1 default")
    ap.add_argument("--config", type=int, choices=[1, 3], default=1,
                    help="1: the headline configuration; 3: the large-model shapes (K=1000, V=50000, w=15, batch 20000)")
    ap.add_argument("--tokens", type=int, default=0, help="corpus size (default 50M per GPU, at most 400M)")
    ap.add_argument("--items", type=int, default=0, help="hash workloads: number of tokens / windows")
    ap.add_argument("--hash-length", type=int, default=50)
    ap.add_argument("--e2e-steps", type=int, default=300, help="steps of the end-to-end measurement (at least --steps)")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--cpu-seconds-reference", type=float, default=90.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-hash", action="store_true", help="leave the hashing figures out of the train line")
    args = ap.parse_args()
    select_config(args.config)
    if args.impl == "reference":
        return bench_reference(args)
    if args.linked_ranks:
        return bench_linked_ranks(args)
    if args.emulate_ranks:
        return bench_update_emulated(args)
    if args.workload == "train":
        return bench_train(args)
    return bench_hash(args, windows=(args.workload == "hash_windows"))


if __name__ == "__main__":
    main()
