"""Benchmark of the multi-LoRA delta path: one step = one full-model pass (every layer, q/k/v/o).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C] [--impl ours|reference]

Prints ONE JSON line (rank 0).

* ``value``        tokens/s with inputs resident in HBM: CUDA-graph replay of the whole pass, CUDA events
                   on the launching stream, median of several event pairs of K replays, max over ranks;
* ``e2e``          the same pass driven from pinned host buffers through the public ops, host<->device
                   copies inside the timed region;
* ``roofline``     the shrink + expand kernels of the pass (the pass without the plan kernel) against the
                   measured HBM copy bandwidth;
* ``gpu_reference``the reference's own GPU formulation in plain torch (cuBLAS) on the same GPU and tensors:
                   the batched-matmul pair of its prefill op, or the dense statement it left beside the
                   decode op, with a gather;
* ``cpu_baseline`` the reference's CPU LoRA worker processes timed on this host's cores;
* ``dropin``       the reference's own call pattern (3 x n_layers calls of ``add_lora_bgmv`` with a fresh
                   zero ``y`` each) beside the fused path on the same dense pools.

With N > 1 the default workload is placed by adapter (every adapter lives on one GPU, every token goes
where its adapter lives, no collective), and the two tensor-parallel workloads are run afterwards and
attached as ``tp``.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126e6
N_PAIRS = 5          # CUDA-event pairs per timed figure (median and spread are reported)

# DRAM bytes per kernel launch of workload 1 (dram__bytes_read.sum + dram__bytes_write.sum, mean over the
# launches of one layer) from the committed ncu summary of the BGMV kernels, and the digest of the kernel
# sources that capture was made from: the figure is reported only while the sources are the same.
TRAFFIC = {"bytes_per_launch": 41.3e6, "csrc_sha16": "eb0bd855e0ebe541"}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="override depth (0 = the workload's)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-gpu-reference", action="store_true")
    ap.add_argument("--no-dropin", action="store_true")
    ap.add_argument("--no-tp", action="store_true", help="N > 1: skip the tensor-parallel workloads")
    return ap.parse_args()


def csrc_digest() -> str:
    h = hashlib.sha256()
    d = os.path.join(ROOT, "ae-296_b200", "csrc")
    for f in sorted(os.listdir(d)):
        if f.endswith((".cu", ".cuh")):
            h.update(open(os.path.join(d, f), "rb").read())
    return h.hexdigest()[:16]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path))["hbm_gbs"], "measured"
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------
# CPU legs
# ------------------------------------------------------------------------------------------------

def cpu_legs(wl, steps: int, warmup: int):
    """The reference's CPU LoRA path on this host's cores.  ``kind: "reference"`` drives the reference's
    unmodified worker loop over shared memory (fetched copy under oracle/_ref); the oracle's port of the
    same arithmetic, grouped by adapter and without doorbells, is kept beside it as the best CPU case."""
    from oracle import ref_worker_baseline as RW
    from oracle.cpu_baseline import time_cpu_lora
    port = time_cpu_lora(wl, sample_layers=1, reps=4)
    best = {"value": port["tokens_per_s"], "unit": "tokens/s", "cores": port["cores"], "kind": "port", "sample": port["sample"]}
    if not RW.available():
        best["note"] = "oracle/_ref/app.py not fetched: the reference's own worker could not be timed"
        return best, port["seconds_per_layer"] * wl.n_layers
    ref = RW.time_reference_workers(wl, layers=wl.n_layers if wl.cfg != 2 else 4, steps=steps, warmup=warmup)
    out = {"value": ref["tokens_per_s"], "unit": "tokens/s", "cores": ref["cores"], "workers": ref["workers"],
           "kind": "reference", "sample": ref["sample"], "cpu_best": best}
    return out, ref["seconds_per_pass"]


def reference_arm(args, rank, world):
    if rank != 0:
        return
    from ae296_b200.workloads import make_workload
    wl = make_workload(args.workload)
    cpu, sec = cpu_legs(wl, steps=max(1, args.steps), warmup=max(1, min(args.warmup, 3)))
    out = {
        "impl": "reference", "metric": "lora_shrink_expand_tokens_per_s", "value": cpu["value"],
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"cfg{wl.cfg}:{wl.name}", "tokens_per_gpu": wl.n_tokens, "layers": wl.n_layers,
                   "adapters": wl.n_adapters, "projections": "q,k,v,o"},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------------
# helpers of the GPU legs
# ------------------------------------------------------------------------------------------------

class Timer:
    """CUDA-event timing of graph replays (or plain callables) on one stream."""

    def __init__(self, stream, world):
        self.stream, self.world = stream, world

    def run(self, fn, steps, warmup, pairs=N_PAIRS):
        import torch
        import torch.distributed as dist
        out = []
        with torch.cuda.stream(self.stream):
            for _ in range(warmup):
                fn()
            self.stream.synchronize()
            if self.world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            for _ in range(pairs):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(self.stream)
                for _ in range(steps):
                    fn()
                e1.record(self.stream)
                self.stream.synchronize()
                out.append(e0.elapsed_time(e1) / steps)
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier()
        return out          # ms per call of fn, one figure per event pair


def med(v):
    return float(statistics.median(v))


def spread(v):
    return {"min": float(min(v)), "max": float(max(v)), "pairs": len(v)}


def capture(stream, fn):
    import torch
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        with torch.cuda.graph(g, stream=stream):
            fn()
    return g


def numa_pin(dev_index: int):
    """Binds this process to the cores of the GPU's NUMA node (before pinned buffers are allocated, so
    that they land on that node).  Returns what was done, for the record."""
    try:
        import torch
        pr = torch.cuda.get_device_properties(dev_index)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read())
        if node < 0:
            return {"pci": bdf, "node": node, "pinned": False}
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
        return {"pci": bdf, "node": node, "pinned": bool(allowed), "cores": len(allowed)}
    except (OSError, ValueError, AttributeError):
        return None


# ------------------------------------------------------------------------------------------------
# the reference's GPU formulation in plain torch
# ------------------------------------------------------------------------------------------------

def gpu_reference_leg(wl, dev, stream, timer, n_layers, x_qkv, x_o, pools, steps, cycle=1):
    """cuBLAS on the same GPU: what the reference's GPU path computes with its own operators.

    prefill workload: ``torch.bmm(torch.bmm(x, A^T.contiguous()), B^T.contiguous())`` per projection on
    ``x [B, L, H]`` with every prompt padded to the longest (lightllm/models/lora_gpu.py:127-128; equal-length
    padding is the reference's layout, lightllm/server/io_struct.py:132-137).
    decode workloads: the dense statement left beside the decode op (lightllm/models/lora_gpu.py:136),
    ``bmm(bmm(x, down), up)`` with slot b <-> token b, fed by a gather of each token's adapter."""
    import numpy as np
    import torch
    names = [p.name for p in wl.projections]
    T = wl.n_tokens
    dt = x_qkv.dtype
    R = wl.r_max
    need = sum(wl.n_adapters * n_layers * R * (p.h_in + p.h_out) * 2 for p in wl.projections)
    free_b, _ = torch.cuda.mem_get_info()
    if wl.cfg == 3 or need > free_b * 0.6:
        return {"kind": "torch.bmm", "value": None, "note": "not run for this workload (dense padded pools do not fit, or mixed batch)"}
    dense = {}
    for p in wl.projections:
        wa = torch.zeros(wl.n_adapters, n_layers, R, p.h_in, dtype=dt, device=dev)
        wb = torch.zeros(wl.n_adapters, n_layers, p.h_out, R, dtype=dt, device=dev)
        for a in range(wl.n_adapters):
            r = int(wl.ranks[a])
            wa[a, :, :r].copy_(pools[p.name].a_block(a))
            wb[a, :, :, :r].copy_(pools[p.name].b_block(a))
        dense[p.name] = (wa, wb)
    scal = torch.from_numpy(wl.scalings).to(dev).to(dt)
    if wl.seq_lens is not None:                                   # prefill: padded [B, Lmax, H]
        B, Lm = len(wl.seq_lens), int(max(wl.seq_lens))
        starts = np.concatenate([[0], np.cumsum(wl.seq_lens)])
        xq = torch.zeros(n_layers, B, Lm, x_qkv.shape[-1], dtype=dt, device=dev)
        xo = torch.zeros_like(xq)
        for b in range(B):
            xq[:, b, :wl.seq_lens[b]].copy_(x_qkv[:, starts[b]:starts[b + 1]])
            xo[:, b, :wl.seq_lens[b]].copy_(x_o[:, starts[b]:starts[b + 1]])
        slot = torch.from_numpy(wl.ids[starts[:-1]].astype(np.int64)).to(dev)
        outs = {}

        def one_pass():
            for l in range(n_layers):
                for n in names:
                    wa, wb = dense[n]
                    x = xo[l] if n == "o" else xq[l]
                    # the reference's expression, with its two transposed copies
                    outs[n] = torch.bmm(torch.bmm(x, wa[slot, l].transpose(-1, -2).contiguous()),
                                        wb[slot, l].transpose(-1, -2).contiguous())
        what = f"torch.bmm pair on x [{B}, {Lm}, H] (prompts padded to the longest), transposed copies inside"
    else:
        ids = torch.from_numpy(wl.ids.astype(np.int64)).to(dev)
        outs = {}

        def one_pass():
            for l in range(n_layers):
                for n in names:
                    wa, wb = dense[n]
                    x = (x_o[l] if n == "o" else x_qkv[l]).unsqueeze(1)                  # [T, 1, H]
                    down = wa[ids, l].transpose(-1, -2)                                    # gather: [T, H, R]
                    up = wb[ids, l].transpose(-1, -2)                                      # [T, R, H_out]
                    outs[n] = torch.bmm(torch.bmm(x, down), up).squeeze(1) * scal[ids].unsqueeze(1)
        what = "dense bmm(bmm(x, down), up) with slot b <-> token b, adapters gathered per token (rank padded to the largest)"
    try:
        g = capture(stream, one_pass)
        ms = timer.run(g.replay, max(1, steps // 4), 2, pairs=3)
        mode = "cuda-graph"
    except Exception:                                              # not capturable: time eager launches
        ms = timer.run(one_pass, max(1, steps // 4), 2, pairs=3)
        mode = "eager"
    del dense
    ms = [v / cycle for v in ms]
    return {"kind": "torch.bmm", "what": what, "value": T / (med(ms) * 1e-3), "unit": "tokens/s",
            "ms_per_step": med(ms), "spread_ms": spread(ms), "timing": mode}


# ------------------------------------------------------------------------------------------------
# the reference's call pattern against this library's op
# ------------------------------------------------------------------------------------------------

def dropin_leg(wl, dev, stream, timer, steps):
    """32 layers x 3 calls of ``add_lora_bgmv(y, x, wa, wb, ids, layer, 1)`` with a fresh zero y per call
    (lightllm/models/lora_gpu.py:137-138,149-150,161-162) on dense uniform-rank pools of the workload's
    dimensions, eager and graph-replayed, beside the fused q/k/v apply and the ``Lora_GPU`` mirror (which
    fuses q/k/v behind the reference's three method calls) on the same pools."""
    import numpy as np
    import torch
    import ae296_b200 as L
    from ae296_b200 import _lib
    from ae296_b200.pool import AdapterPool
    p0 = wl.projections[0]
    H, T, N, nl, r = p0.h_in, wl.n_tokens, wl.n_adapters, wl.n_layers if wl.cfg != 0 else 32, 16
    dt = {"fp16": torch.float16, "bf16": torch.bfloat16}[wl.dtype]
    g = torch.Generator(device=dev).manual_seed(2960)
    pools = []
    for _ in range(3):
        wa = torch.empty(N, nl, r, H, dtype=dt, device=dev).normal_(0, 1.0 / float(np.sqrt(H)), generator=g)
        wb = torch.empty(N, nl, H, r, dtype=dt, device=dev).normal_(0, 0.25, generator=g)
        pools.append((wa, wb))
    x = torch.empty(nl, T, H, dtype=dt, device=dev).normal_(0, 1, generator=g)
    ids = torch.from_numpy(wl.ids.astype(np.int64)).to(dev)
    keep = []

    def reference_loop():
        keep.clear()
        for l in range(nl):
            for wa, wb in pools:
                y = torch.zeros(T, H, dtype=dt, device=dev)
                L.add_lora_bgmv(y, x[l], wa, wb, ids, l, 1)
                keep.append(y)

    views = [AdapterPool(wa, wb, None, None, None, N, nl, H, H, r, False, np.full(N, r, np.int32),
                         np.arange(N + 1, dtype=np.int64) * r) for wa, wb in pools]
    ad = L.ops._adapters_struct(N, nl, r, scale=1.0)
    batch = L.LoraBatch(T, N, H, 3, dev)
    batch.plan.build(ids, ad)
    y3 = torch.zeros(nl, 3, T, H, dtype=dt, device=dev)

    def fused_loop():
        y3.zero_()
        for l in range(nl):
            L.apply([(x[l], y3[l, i], views[i]) for i in range(3)], batch.plan, l, batch.workspace, _lib.NO_TENSOR, ad)

    # the reference sizes its pools and its index tensors with one number (batch_size)
    mirror = L.Lora_GPU({"n_layers": nl, "batch_size": max(N, T), "lora_rank": r, "hidden_dim": H, "tp_degree": 1,
                         "max_prefill_batch_size": 1}, dtype=dt)
    mirror.set_indices(ids)

    def mirror_loop():
        keep.clear()
        for l in range(nl):
            keep.append(mirror.invoke_one_layer_q(x[l], l))
            keep.append(mirror.invoke_one_layer_k(x[l], l))
            keep.append(mirror.invoke_one_layer_v(x[l], l))

    k = max(1, steps // 4)
    with torch.cuda.stream(stream):
        eager = timer.run(reference_loop, k, 2, pairs=3)
    out = {"calls_per_step": 3 * nl, "rank": r, "pool_gb": round(sum(a.numel() + b.numel() for a, b in pools) * 2 / 1e9, 2),
           "eager_ms": med(eager)}
    out["graph_ms"] = med(timer.run(capture(stream, reference_loop).replay, k, 2, pairs=3))
    out["fused_graph_ms"] = med(timer.run(capture(stream, fused_loop).replay, k, 2, pairs=3))
    out["mirror_graph_ms"] = med(timer.run(capture(stream, mirror_loop).replay, k, 2, pairs=3))
    out["graph_over_fused"] = out["graph_ms"] / out["fused_graph_ms"]
    bytes_qkv = sum(int(np.unique(wl.ids).size) * r * 2 * H * 2 + 3 * T * H * 2 + 4 * T for _ in range(3)) * nl
    out["graph_frac_of_hbm"] = bytes_qkv / (out["graph_ms"] * 1e-3) / 1e9 / hbm_peak()[0]
    return out


# ------------------------------------------------------------------------------------------------
# tensor-parallel workloads
# ------------------------------------------------------------------------------------------------

def tp_parity_check(wl, dev, rank, tp):
    """One layer, fp32 outputs: this rank's y shard from ``TPLora`` against the matching column slice of an
    unsharded apply of the same (seeded, hence identical on every rank) pool on this rank's GPU.
    Returns max-abs-error / RMS of the unsharded output, the larger of the projections."""
    import numpy as np
    import torch
    import ae296_b200 as L
    from ae296_b200.pool import AdapterPool
    from ae296_b200.tp import TPLora, column_slice
    from ae296_b200.workloads import torch_dtype
    dt = torch_dtype(wl.dtype)
    T = wl.n_tokens
    g = torch.Generator(device=dev).manual_seed(4242)           # the same draw on every rank
    ids = torch.from_numpy(wl.ids).to(dev)
    tiles = wl.seq_lens is not None
    worst = 0.0
    groups = [[p for p in wl.projections if p.name != "o"], [p for p in wl.projections if p.name == "o"]]
    for group in groups:
        h_in = group[0].h_in
        x = torch.empty(T, h_in, dtype=dt, device=dev).normal_(0, 1, generator=g)
        full, shard = [], []
        for p in group:
            pool = AdapterPool.empty(wl.n_adapters, 1, p.h_in, p.h_out, wl.ranks, wl.scalings, dtype=dt, device=dev)
            pool.wa.normal_(0, 1.0 / float(np.sqrt(p.h_in)), generator=g)
            pool.wb.normal_(0, 0.15, generator=g)
            full.append(pool)
            shard.append(pool.shard(tp, rank))
        ref = L.LoraBatch(T, wl.n_adapters, h_in, len(group), dev).set_ids(ids, full[0], tiles=tiles)
        y_full = [torch.zeros(T, p.h_out, dtype=torch.float32, device=dev) for p in group]
        ref.apply([(x, y, pool) for y, pool in zip(y_full, full)], 0)
        eng = TPLora(T, wl.n_adapters, h_in // tp, len(group), tp, rank, None, dev, exchange="peer").set_ids(ids, shard[0], tiles=tiles)
        y_sh = [torch.zeros(T, p.h_out // tp, dtype=torch.float32, device=dev) for p in group]
        eng.apply([(column_slice(x, tp, rank), y, sh) for y, sh in zip(y_sh, shard)], 0)
        torch.cuda.synchronize()
        eng.batch.workspace.check()
        for yf, ys in zip(y_full, y_sh):
            rms = float(yf.pow(2).mean().sqrt())
            worst = max(worst, float((column_slice(yf, tp, rank) - ys).abs().max()) / max(rms, 1e-30))
        eng.close()
        del ref, eng, full, shard
    return worst


def tensor_parallel_leg(args, wl, rank, local, world, dev):
    """Workloads 3 and 4 on N GPUs: A sharded along hidden, B along output, the fp32 shrink partials summed
    over the ranks between the two halves (the library's exchange over peer memory; the NCCL all-reduce is
    timed beside it).  Total work is fixed: strong scaling.  Returns the record."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from ae296_b200.pool import AdapterPool
    from ae296_b200.tp import TPLora
    from ae296_b200.workloads import SEED_BASE, torch_dtype

    tp = world
    parity = torch.tensor([tp_parity_check(wl, dev, rank, tp)], device=dev)
    dist.all_reduce(parity, op=dist.ReduceOp.MAX)
    torch.cuda.empty_cache()
    dt = torch_dtype(wl.dtype)
    T = wl.n_tokens
    n_layers = args.layers or wl.n_layers
    per_layer = wl.pool_bytes() // wl.n_layers // tp
    free_b, _ = torch.cuda.mem_get_info()
    fit = int((free_b * 0.8) // (per_layer + 1))
    note = None
    if n_layers > fit:
        note = f"pool trimmed to {fit} of {n_layers} layers to fit"
        n_layers = fit
    g = torch.Generator(device=dev).manual_seed(SEED_BASE + wl.cfg + 100 * rank)
    pools, ys = {}, {}
    for p in wl.projections:
        hi, ho = p.h_in // tp, p.h_out // tp
        pool = AdapterPool.empty(wl.n_adapters, n_layers, hi, ho, wl.ranks, wl.scalings, dtype=dt, device=dev)
        pool.wa.normal_(0, 1.0 / float(np.sqrt(p.h_in)), generator=g)
        pool.wb.normal_(0, 0.15, generator=g)
        pools[p.name] = pool
        ys[p.name] = torch.zeros(n_layers, T, ho, dtype=dt, device=dev)
    hi = wl.projections[0].h_in // tp
    x_qkv = torch.empty(n_layers, T, hi, dtype=dt, device=dev).normal_(0, 1, generator=g)
    x_o = torch.empty(n_layers, T, hi, dtype=dt, device=dev).normal_(0, 1, generator=g)
    ids = torch.from_numpy(wl.ids).to(dev)
    names = [p.name for p in wl.projections]
    stream = torch.cuda.Stream(dev)
    tiles = wl.seq_lens is not None
    timer = Timer(stream, world)

    def timed(exchange, sampler=None):
        eng = TPLora(T, wl.n_adapters, hi, 3, tp, rank, None, dev, exchange=exchange)

        def one_pass():
            eng.set_ids(ids, pools["q"], tiles=tiles)
            for l in range(n_layers):
                eng.apply([(x_qkv[l], ys[n][l], pools[n]) for n in names if n != "o"], l)
                eng.apply([(x_o[l], ys["o"][l], pools["o"])], l)

        mode = "cuda-graph"
        with torch.cuda.stream(stream):
            one_pass()
            stream.synchronize()
            dist.barrier()
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    one_pass()
                run = graph.replay
            except Exception:                       # a collective inside a graph refused: time eager launches
                mode = "eager"
                run = one_pass
        if sampler is not None:
            with sampler:
                ms_all = timer.run(run, args.steps, max(args.warmup, 3))
        else:
            ms_all = timer.run(run, args.steps, 3, pairs=3)
        tms = torch.tensor([med(ms_all)], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        eng.batch.workspace.check()
        eng.close()
        return float(tms.item()), ms_all, mode

    clk = ClockSampler(local)
    ms, ms_all, mode = timed("peer", clk)
    ms_nccl, _, mode_nccl = timed("nccl")
    peak, peak_src = hbm_peak()
    per_gpu = wl.bytes_per_layer(tp=tp) * n_layers + 2 * 4 * T * 64 * 4 * 2 * n_layers
    applies = n_layers * 2
    rec = {
        "workload": f"cfg{wl.cfg}:{wl.name}", "tp": tp, "tokens": T, "layers": n_layers, "adapters": wl.n_adapters,
        "ms_per_step": ms, "spread_ms": spread(ms_all), "tokens_per_s": T / (ms * 1e-3), "scaling": "strong",
        "dtype": "f32-accumulate/" + wl.dtype, "timing": mode,
        "parallelism": f"tp{tp}: A row-sharded, B column-sharded, one library call per apply; the fp32 shrink partials (rank columns of the rows present) are summed by the library's exchange kernels over peer memory",
        "with_nccl_all_reduce": {"ms_per_step": ms_nccl, "timing": mode_nccl},
        "per_gpu_gbs": per_gpu / (ms * 1e-3) / 1e9, "frac_of_hbm": per_gpu / (ms * 1e-3) / 1e9 / peak, "peak_source": peak_src,
        "tp_parity": float(parity.item()), "exchanges_per_step": applies,
        # per apply: shrink, exchange (adds up the split-K slots itself), expand; with prompts the tile kernels'
        # chain beside it: shrink half, exchange, expand half
        "gpu_launches_per_step": 1 + applies * (3 + (3 if tiles else 0)),
        "note": note, "clocks": clk.summary(),
    }
    del pools, ys, x_qkv, x_o
    torch.cuda.empty_cache()
    rec["replicated_a_scheme"] = replicated_a_leg(args, wl, rank, world, dev, n_layers)
    return rec


def replicated_a_leg(args, wl, rank, world, dev, n_layers):
    """The reference's own tensor-parallel layout for comparison: A replicated ``[r, h_in]``, B column-sharded
    ``[h_out/tp, r]``, every rank reads the full x and no collective is needed
    (lightllm/models/lora_gpu.py:25-26,33-34).  Costs tp x the A reads, saves the all-reduce and the split launches."""
    import numpy as np
    import torch
    import torch.distributed as dist
    import ae296_b200 as L
    from ae296_b200.pool import AdapterPool
    from ae296_b200.workloads import SEED_BASE, torch_dtype
    tp = world
    dt = torch_dtype(wl.dtype)
    T = wl.n_tokens
    rs = int(wl.ranks.astype(np.int64).sum())
    need = sum(rs * n_layers * (p.h_in + p.h_out // tp) * 2 for p in wl.projections)
    free_b, _ = torch.cuda.mem_get_info()
    fits = torch.tensor([1 if need < free_b * 0.8 else 0], device=dev)
    dist.all_reduce(fits, op=dist.ReduceOp.MIN)
    if int(fits.item()) == 0:
        return {"ms_per_step": None, "note": "replicated A does not fit beside B/tp on these GPUs"}
    g = torch.Generator(device=dev).manual_seed(SEED_BASE + wl.cfg + 100 * rank)
    pools, ys = {}, {}
    for p in wl.projections:
        pool = AdapterPool.empty(wl.n_adapters, n_layers, p.h_in, p.h_out // tp, wl.ranks, wl.scalings, dtype=dt, device=dev)
        pool.wa.normal_(0, 1.0 / float(np.sqrt(p.h_in)), generator=g)
        pool.wb.normal_(0, 0.15, generator=g)
        pools[p.name] = pool
        ys[p.name] = torch.zeros(n_layers, T, p.h_out // tp, dtype=dt, device=dev)
    h = wl.projections[0].h_in
    x_qkv = torch.empty(n_layers, T, h, dtype=dt, device=dev).normal_(0, 1, generator=g)
    x_o = torch.empty(n_layers, T, h, dtype=dt, device=dev).normal_(0, 1, generator=g)
    ids = torch.from_numpy(wl.ids).to(dev)
    batch = L.LoraBatch(T, wl.n_adapters, h, 3, dev)
    names = [p.name for p in wl.projections]
    stream = torch.cuda.Stream(dev)
    tiles = wl.seq_lens is not None

    def one_pass():
        batch.set_ids(ids, pools["q"], tiles=tiles)
        for l in range(n_layers):
            batch.apply([(x_qkv[l], ys[n][l], pools[n]) for n in names if n != "o"], l)
            batch.apply([(x_o[l], ys["o"][l], pools["o"])], l)

    ms_all = Timer(stream, world).run(capture(stream, one_pass).replay, args.steps, 3, pairs=3)
    tms = torch.tensor([med(ms_all)], device=dev)
    dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    batch.workspace.check()
    ms = float(tms.item())
    del pools, ys, x_qkv, x_o, batch
    torch.cuda.empty_cache()
    return {"ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "collectives_per_step": 0,
            "note": "A replicated, B column-sharded, full x on every rank (the reference's layout)"}


# ------------------------------------------------------------------------------------------------
# the default leg: one GPU, or N GPUs with the batch placed by adapter
# ------------------------------------------------------------------------------------------------

def placed_workload(base, world, rank):
    """N > 1: a global batch of ``world`` x the workload's tokens over ``world`` x its adapters (same
    distributions, seeded), split by ``place_by_adapter``; returns this rank's share as a workload of
    its own plus the placement's summary."""
    import dataclasses
    import numpy as np
    from ae296_b200.placement import place_by_adapter
    from ae296_b200.workloads import SEED_BASE, zipf_probs
    rng = np.random.default_rng(SEED_BASE + base.cfg + 1000 * world)
    n_g, t_g = base.n_adapters * world, base.n_tokens * world
    ranks = rng.choice(np.unique(base.ranks), n_g).astype(np.int32)
    ids = rng.choice(n_g, t_g, p=zipf_probs(n_g, 1.0)).astype(np.int32)
    pl = place_by_adapter(ids, world, n_g, "balanced", ranks=ranks)      # balances estimated bytes, not tokens
    mine = pl.adapters[rank]
    wl = dataclasses.replace(base, n_adapters=len(mine), ranks=ranks[mine], ids=pl.local_ids[rank].copy(),
                             n_decode=len(pl.tokens[rank]))
    info = {"policy": "balanced by estimated bytes (rank-weighted work segments)", "global_tokens": t_g, "global_adapters": n_g,
            "tokens_per_gpu": [int(len(t)) for t in pl.tokens], "adapters_per_gpu": [int(len(a)) for a in pl.adapters]}
    return wl, info, t_g


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        reference_arm(args, rank, world)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    import ae296_b200 as L
    from ae296_b200 import _lib
    from ae296_b200.workloads import make_workload, materialize_device

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = numa_pin(local)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"           # keeps NCCL's version banner off stdout: one JSON line only
        # a rank that fails alone must not keep the others (and the GPUs) waiting for NCCL's default ten minutes
        dist.init_process_group("nccl", device_id=dev, timeout=__import__("datetime").timedelta(seconds=180))

    base = make_workload(args.workload)
    if base.cfg in (3, 4) and world > 1:
        rec = tensor_parallel_leg(args, base, rank, local, world, dev)
        if rank == 0:
            out = {"metric": "lora_shrink_expand_tokens_per_s", "value": rec["tokens_per_s"], "unit": "tokens/s",
                   "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": rec["ms_per_step"],
                   "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": rec["dtype"], "data": "synthetic",
                   "config": {"workload": rec["workload"], "tokens": rec["tokens"], "layers": rec["layers"],
                              "parallelism": rec["parallelism"], "l2": "inputs larger than L2", "note": rec["note"]},
                   "roofline": {"bound": "hbm", "kernel": "whole pass per GPU (shrink + exchange + expand)",
                                "achieved": rec["per_gpu_gbs"], "peak": hbm_peak()[0], "unit": "GB/s", "frac": rec["frac_of_hbm"],
                                "traffic": None},
                   "tp": rec, "cpu_baseline": None, "e2e": None,
                   "gpu_launches": rec["gpu_launches_per_step"] * args.steps, "clocks": rec["clocks"]}
            print(json.dumps(out), flush=True)
        dist.destroy_process_group()
        return

    placement = None
    if world > 1:
        wl, placement, total_tokens = placed_workload(base, world, rank)
    else:
        wl, total_tokens = base, base.n_tokens
    # workload 0 is one layer: its steps cycle the layer index over a 32-layer pool so that a step's
    # weights come from HBM, not from the L2 the previous step filled
    cycle = 32 if wl.cfg == 0 else 1
    n_layers = (args.layers or wl.n_layers) * cycle
    free_b, _ = torch.cuda.mem_get_info()
    per_layer_pool = wl.pool_bytes() // wl.n_layers
    fit_layers = int((free_b * 0.8) // (per_layer_pool + 1))
    depth_note = None
    if n_layers > fit_layers:
        depth_note = f"pool trimmed to {fit_layers} of {n_layers} layers to fit one GPU"
        n_layers = fit_layers
    layers_per_step = n_layers // cycle
    T = wl.n_tokens
    x_qkv, x_o, pools = materialize_device(wl, dev, layers=n_layers)
    dt = x_qkv.dtype
    names = [p.name for p in wl.projections]
    ys = {p.name: torch.zeros(n_layers, T, p.h_out, dtype=dt, device=dev) for p in wl.projections}
    ids_host = torch.from_numpy(wl.ids).pin_memory()
    ids = ids_host.to(dev)
    batch = L.LoraBatch(T, wl.n_adapters, wl.projections[0].h_in, 3, dev)
    stream = torch.cuda.Stream(dev)
    timer = Timer(stream, world)
    use_tiles = wl.seq_lens is not None                # prompts (runs of >= 32 rows of one adapter) go to the tcgen05 tile kernel

    def graph_body(flags=0, plan=True):
        # `cycle` steps: each builds the plan (when asked) and applies its own layers
        for c in range(cycle):
            if plan:
                batch.set_ids(ids, pools["q"], tiles=use_tiles)
            for l in range(c * layers_per_step, (c + 1) * layers_per_step):
                batch.apply([(x_qkv[l], ys[n][l], pools[n]) for n in names if n != "o"], l, flags)
                batch.apply([(x_o[l], ys["o"][l], pools["o"])], l, flags)

    n_sm = torch.cuda.get_device_properties(dev).multi_processor_count

    def tile_launches(n_proj):
        # one launch, or three (shrink half cut along k, the kernel that adds the parts, expand half) when the
        # batch can hold fewer (tile, projection) pairs than the GPU has SMs
        return 0 if not use_tiles else (3 if (T // 128 + 1) * n_proj < n_sm else 1)

    launches_per_step = 1 + layers_per_step * (4 + tile_launches(3) + tile_launches(1))

    def timed_graph(flags=0, plan=True, steps=None, warmup=3):
        g = capture(stream, lambda: graph_body(flags, plan))
        return [v / cycle for v in timer.run(g.replay, steps or args.steps, warmup)]

    with ClockSampler(local) as clk:
        ms_all = timed_graph(0, True, warmup=max(args.warmup, 3))
        ms_noplan_all = timed_graph(0, False)
        ms_exp = med(timed_graph(_lib.ONLY_EXPAND, False))
        ms_shr = med(timed_graph(_lib.ONLY_SHRINK | _lib.KEEP_PARTIALS, False))
        ms_dta = med(timed_graph(_lib.DELTA_THEN_ADD, False))
    ms = med(ms_all)
    if world > 1:
        tms = torch.tensor([ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())

    def plan_only():
        for _ in range(8):
            batch.set_ids(ids, pools["q"], tiles=use_tiles)
    us_plan = med(timer.run(capture(stream, plan_only).replay, args.steps, 3, pairs=3)) * 1e3 / 8
    batch.workspace.check()

    peak, peak_src = hbm_peak()
    used = wl.distinct()
    rsum = int(wl.ranks[used].sum())
    e = 2
    exp_bytes = sum(rsum * p.h_out * e + 2 * T * p.h_out * e for p in wl.projections) * layers_per_step
    shr_bytes = sum(rsum * p.h_in * e + T * p.h_in * e + 4 * T for p in wl.projections) * layers_per_step
    ms_noplan = med(ms_noplan_all)
    n_apply = layers_per_step * 2
    n_launch = n_apply * 2
    pass_bytes = wl.bytes_per_layer() * layers_per_step
    digest = csrc_digest()
    traffic = TRAFFIC["bytes_per_launch"] if (wl.cfg == 1 and world == 1 and TRAFFIC["csrc_sha16"] == digest) else None
    ach = pass_bytes / (ms_noplan * 1e-3) / 1e9
    roofline = {
        "bound": "hbm",
        "kernel": ("" if not use_tiles else "sgmv_tile_kernel + ") + "bgmv_shrink_tma_kernel + bgmv_expand_tma_kernel",
        "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": traffic,
        "traffic_source": ("ncu capture summarised under profiles/, kernel sources " + str(TRAFFIC["csrc_sha16"])) if traffic else
                          "no ncu capture of these kernel sources (" + digest + ") on record",
        "peak_source": peak_src, "bytes_per_launch": pass_bytes / n_launch,
        "us_per_launch": ms_noplan * 1e3 / n_launch, "spread_ms": spread(ms_noplan_all), "frac_of_8TBs_nominal": ach / 8000.0,
        "expand_half": {"achieved": exp_bytes / (ms_exp * 1e-3) / 1e9, "frac": exp_bytes / (ms_exp * 1e-3) / 1e9 / peak,
                        "us_per_launch": ms_exp * 1e3 / n_apply},
        "shrink_half": {"achieved": shr_bytes / (ms_shr * 1e-3) / 1e9, "frac": shr_bytes / (ms_shr * 1e-3) / 1e9 / peak,
                        "us_per_launch": ms_shr * 1e3 / n_apply, "note": "shrink kernel alone (partial sums left unfolded)"},
        "plan_us": us_plan,
        # optional mode with the reference's `q += q_lora` rounding (delta rounded, then a 16-bit add)
        "delta_then_add_mode": {"achieved": pass_bytes / (ms_dta * 1e-3) / 1e9,
                                "frac": pass_bytes / (ms_dta * 1e-3) / 1e9 / peak, "us_per_launch": ms_dta * 1e3 / n_launch},
        "whole_pass": {"bytes": pass_bytes, "achieved": pass_bytes / (ms * 1e-3) / 1e9,
                       "frac": pass_bytes / (ms * 1e-3) / 1e9 / peak},
    }
    if world > 1:
        fr = torch.tensor([roofline["frac"]], device=dev)
        dist.all_reduce(fr, op=dist.ReduceOp.MIN)
        roofline["frac_min_over_ranks"] = float(fr.item())

    # ---- end to end from pinned host buffers through the public ops -----------------------------
    e2e = None
    if not args.no_e2e:
        # One host->device copy per layer (its two activations sit side by side in one buffer) and one
        # device->host copy per group of layers (eight groups per pass) (a layer's four outputs are column ranges of its
        # [T, sum(h_out)] block; the kernels take the row pitch).
        h_in0 = wl.projections[0].h_in
        widths = [p.h_out for p in wl.projections]
        offs = [sum(widths[:i]) for i in range(len(widths))]
        nl = layers_per_step
        # Two sets of device buffers alternate from step to step, as a serving loop would have them: a step's
        # uploads wait only for the compute of the step before last (which read the same x buffers), its
        # compute only for the download of the step before last (which read the same y buffers), so the
        # downloads, the slowest part, run back to back.
        dxs = [torch.empty(nl, 2, T, h_in0, dtype=dt, device=dev) for _ in range(2)]
        for d in dxs:
            d[:, 0].copy_(x_qkv[:nl]); d[:, 1].copy_(x_o[:nl])
        hx = torch.empty(dxs[0].shape, dtype=dt).pin_memory().copy_(dxs[0].cpu())
        y_alls = [torch.zeros(nl, T, sum(widths), dtype=dt, device=dev) for _ in range(2)]
        yvs = [{n: ya[:, :, o:o + w] for n, o, w in zip(names, offs, widths)} for ya in y_alls]
        hy = torch.empty(y_alls[0].shape, dtype=dt).pin_memory()
        copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        group = max(1, nl // 8)
        x_free = [None, None]          # recorded on `stream` when a step's compute is done with its x buffers
        y_free = [None, None]          # recorded on `copy_out` when a step's downloads are done with its y buffers
        step_no = [0]

        def e2e_step():
            b = step_no[0] & 1
            step_no[0] += 1
            dx, y_all, yv = dxs[b], y_alls[b], yvs[b]
            with torch.cuda.stream(stream):
                ids.copy_(ids_host, non_blocking=True)
                batch.set_ids(ids, pools["q"], tiles=use_tiles)
                if y_free[b] is not None:
                    stream.wait_event(y_free[b])
            ev_in, ev_done = [], {}
            with torch.cuda.stream(copy_in):
                if x_free[b] is not None:
                    copy_in.wait_event(x_free[b])
                for l in range(nl):
                    dx[l].copy_(hx[l], non_blocking=True)
                    ev = torch.cuda.Event(); ev.record(copy_in); ev_in.append(ev)
            with torch.cuda.stream(stream):
                for l in range(nl):
                    stream.wait_event(ev_in[l])
                    batch.apply([(dx[l, 0], yv[n][l], pools[n]) for n in names if n != "o"], l)
                    batch.apply([(dx[l, 1], yv["o"][l], pools["o"])], l)
                    if (l + 1) % group == 0 or l == nl - 1:
                        ev = torch.cuda.Event(); ev.record(stream); ev_done[l] = ev
                x_free[b] = torch.cuda.Event(); x_free[b].record(stream)
            with torch.cuda.stream(copy_out):
                lo = 0
                for l in sorted(ev_done):
                    copy_out.wait_event(ev_done[l])
                    hy[lo:l + 1].copy_(y_all[lo:l + 1], non_blocking=True)
                    lo = l + 1
                y_free[b] = torch.cuda.Event(); y_free[b].record(copy_out)

        for _ in range(2):
            e2e_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        k = max(3, args.steps // 4)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(stream)
        for _ in range(k):
            e2e_step()
        stream.wait_stream(copy_out)                      # the last step's result has reached the host
        e1.record(stream)
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) / k * 1e3
        ms_e2e = max(e0.elapsed_time(e1) / k, wall)
        if world > 1:
            tms = torch.tensor([ms_e2e], device=dev)
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
            ms_e2e = float(tms.item())
        # the two directions alone, for the record: what the host side of this box sustains
        def copy_rate(fn, nbytes):
            fn(); torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            return nbytes * 3 / (time.perf_counter() - t0) / 1e9
        h2d = hx.numel() * 2 + ids_host.numel() * 4
        d2h = hy.numel() * 2
        e2e = {"value": total_tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e,
               "h2d_alone_gbs": copy_rate(lambda: dxs[0].copy_(hx, non_blocking=True), h2d),
               "d2h_alone_gbs": copy_rate(lambda: hy.copy_(y_alls[0], non_blocking=True), d2h),
               "d2h_copies_per_step": -(-nl // group), "device_buffer_sets": 2, "numa": numa}
        del dxs, hx, y_alls, yvs, hy

    gpu_ref = None
    if rank == 0 and world == 1 and not args.no_gpu_reference:
        gpu_ref = gpu_reference_leg(wl, dev, stream, timer, n_layers, x_qkv, x_o, pools, args.steps, cycle)
        if gpu_ref.get("value"):
            gpu_ref["ours_over_gpu_reference"] = (T / (ms * 1e-3)) / gpu_ref["value"]
    pool_gb = round(sum(p.nbytes() for p in pools.values()) / 1e9, 3)
    del x_qkv, x_o, pools, ys, batch
    torch.cuda.empty_cache()
    dropin = None
    if rank == 0 and world == 1 and not args.no_dropin and not use_tiles:
        p0 = wl.projections[0]
        need = 3 * 2 * wl.n_adapters * (wl.n_layers if wl.cfg != 0 else 32) * 16 * p0.h_in * 2 * 3.5     # its pools + the mirror's
        if need < torch.cuda.mem_get_info()[0] * 0.8:
            dropin = dropin_leg(wl, dev, stream, timer, args.steps)
        else:
            dropin = {"note": "not run: its dense pools do not fit this GPU"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu, _ = cpu_legs(wl, steps=2, warmup=1)

    step_bytes = pass_bytes
    l2 = ("inputs larger than L2: a step touches %.0f MB of a %.2f GB pool" % (step_bytes / 1e6, pool_gb)) if step_bytes > 1.5 * L2_BYTES \
        else ("a step touches %.1f MB; consecutive steps use different layers of a %.0f MB pool (%d-step cycle), larger than L2"
              % (step_bytes / 1e6, pool_gb * 1e3, cycle))
    tp_rec = None
    if world > 1 and base.cfg == 1 and not args.no_tp:
        tp_rec = {}
        for c in (3, 4):
            try:
                tp_rec[f"cfg{c}"] = tensor_parallel_leg(args, make_workload(c), rank, local, world, dev)
            except Exception as ex:                      # keep the headline line even if a TP leg fails
                tp_rec[f"cfg{c}"] = {"error": repr(ex)[:300]}
                torch.cuda.empty_cache()

    if rank == 0:
        out = {
            "metric": "lora_shrink_expand_tokens_per_s", "value": total_tokens / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "spread_ms": spread(ms_all), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32-accumulate/" + wl.dtype, "data": "synthetic",
            "config": {"workload": f"cfg{base.cfg}:{base.name}", "tokens_per_gpu": base.n_tokens, "layers": layers_per_step,
                       "adapters": base.n_adapters, "distinct_adapters": int(len(used)), "projections": "q,k,v,o",
                       "pool_gb": pool_gb, "l2": l2, "timing": f"median of {N_PAIRS} CUDA-event pairs of {args.steps} graph replays",
                       "parallelism": "1 GPU" if world == 1 else f"{world} GPUs, batch placed by adapter, no collective",
                       "placement": placement, "note": depth_note},
            "roofline": roofline, "gpu_reference": gpu_ref, "cpu_baseline": cpu, "e2e": e2e, "dropin": dropin, "tp": tp_rec,
            "gpu_launches": launches_per_step * args.steps * N_PAIRS, "gpu_launches_per_step": launches_per_step,
            "clocks": clk.summary(),
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
