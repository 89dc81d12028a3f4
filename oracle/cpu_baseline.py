"""CPU baseline: the reference's CPU LoRA arithmetic timed on the host cores.  TEST/BENCH ONLY.

Restates how the reference spreads the LoRA delta over CPU cores: one single-threaded worker
process per core (runServerCPULoRA.py:83 pins each worker with numactl), each holding fp32
``down [H, r]`` / ``up [r, H]`` weights (lora_cpu/lora_shm_op/app.py:38-45) and computing
``(x.float() @ down @ up).half()`` for the rows it is handed (app.py:136-141).  Work items are
(layer, projection, adapter segment); they are dealt round-robin to the workers, which is the
reference's static slot -> worker binding.  Shared-memory doorbells are replaced by a barrier
so that only arithmetic is timed.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import time
from typing import Dict, List, Sequence, Tuple

import numpy as np


def _worker(wid, n_workers, items, x_by_proj, seed, start, stop, reps, out_q):
    import torch
    torch.set_num_threads(1)
    try:
        os.sched_setaffinity(0, {sorted(os.sched_getaffinity(0))[wid % len(os.sched_getaffinity(0))]})
    except (AttributeError, OSError):
        pass
    mine = items[wid::n_workers]
    g = torch.Generator().manual_seed(seed + wid)
    weights = []
    for (layer, pname, h_in, h_out, r, rows) in mine:
        down = (torch.randn(h_in, r, generator=g) / np.sqrt(h_in)).half().float()
        up = (torch.randn(r, h_out, generator=g) / np.sqrt(r)).half().float()
        weights.append((down, up))
    checksum = 0.0
    with torch.no_grad():
        for _ in range(reps):
            start.wait()
            for (layer, pname, h_in, h_out, r, rows), (down, up) in zip(mine, weights):
                x = x_by_proj[pname][rows]
                res = (x.float() @ down @ up).half()
                checksum += float(res[0, 0])
            stop.wait()
    out_q.put((wid, checksum))


def time_cpu_lora(wl, sample_layers: int = 1, n_workers: int = 0, reps: int = 3, seed: int = 2960):
    """Times ``sample_layers`` layers of workload ``wl`` (all four projections).

    Returns ``dict(seconds_per_layer, tokens_per_s, cores, sample)``; ``tokens_per_s`` scales
    the per-layer time to the workload's full depth.
    """
    import torch
    n_workers = n_workers or len(os.sched_getaffinity(0))
    g = torch.Generator().manual_seed(seed)
    t = wl.n_tokens
    x_qkv = torch.randn(t, wl.projections[0].h_in, generator=g).half()
    x_o = torch.randn(t, wl.projections[0].h_in, generator=g).half()
    x_by_proj = {p.name: (x_o if p.name == "o" else x_qkv) for p in wl.projections}
    order = np.argsort(wl.ids, kind="stable")
    uniq, starts = np.unique(wl.ids[order], return_index=True)
    ends = list(starts[1:]) + [t]
    items = []
    for layer in range(sample_layers):
        for p in wl.projections:
            for a, b, e in zip(uniq, starts, ends):
                items.append((layer, p.name, p.h_in, p.h_out, int(wl.ranks[a]), torch.from_numpy(order[b:e].copy())))
    # longest first so the round-robin deal is balanced
    items.sort(key=lambda it: -(it[4] * (it[2] + it[3])))
    ctx = mp.get_context("fork")
    start, stop = ctx.Barrier(n_workers + 1), ctx.Barrier(n_workers + 1)
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(w, n_workers, items, x_by_proj, seed, start, stop, reps, q), daemon=True)
             for w in range(n_workers)]
    for p in procs:
        p.start()
    times = []
    for _ in range(reps):
        start.wait()
        t0 = time.perf_counter()
        stop.wait()
        times.append(time.perf_counter() - t0)
    for _ in procs:
        q.get()
    for p in procs:
        p.join()
    best = float(np.median(times[1:])) if len(times) > 1 else times[0]
    per_layer = best / sample_layers
    return {
        "seconds_per_layer": per_layer,
        "tokens_per_s": t / (per_layer * wl.n_layers),
        "cores": n_workers,
        "sample": f"{sample_layers} of {wl.n_layers} layers x 4 projections, {len(uniq)} adapter segments, "
                  f"{reps} repeats (first discarded), one pinned single-thread worker per core",
    }
