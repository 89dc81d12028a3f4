"""Benchmark of the multi-LoRA delta path: one step = one full-model pass (every layer, q/k/v/o).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C] [--impl ours|reference]

Prints ONE JSON line (rank 0).  `value` is tokens/s with inputs resident in HBM (CUDA-graph
replay of the whole pass, CUDA-event timed, max over ranks); `e2e` is the same pass driven
from pinned host buffers through the public ops, host<->device copies inside the timed
region; `roofline` is the shrink + expand kernel pair (the pass without the plan kernel);
`cpu_baseline` is the reference's CPU LoRA arithmetic timed on this host's cores.
With N > 1 each rank holds its own adapters and batch (placement by adapter, no collective).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# DRAM bytes per kernel launch of workload 1, from the ncu capture summarised in
# profiles/bgmv_cfg1_ncu.md: mean of dram__bytes_read.sum + dram__bytes_write.sum over the four
# launches of one layer
TRAFFIC_PER_LAUNCH = 41.2e6


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
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
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


def reference_arm(args, rank, world):
    """The reference's CPU LoRA arithmetic on this host's cores (oracle port), all cores."""
    if rank != 0:
        return
    from ae296_b200.workloads import make_workload
    from oracle.cpu_baseline import time_cpu_lora
    wl = make_workload(args.workload)
    res = time_cpu_lora(wl, sample_layers=1, reps=max(2, args.steps // 4 + 1))
    out = {
        "impl": "reference", "metric": "lora_shrink_expand_tokens_per_s", "value": res["tokens_per_s"],
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": res["seconds_per_layer"] * wl.n_layers * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"cfg{wl.cfg}:{wl.name}", "tokens": wl.n_tokens, "layers": wl.n_layers},
        "cpu_baseline": {"value": res["tokens_per_s"], "unit": "tokens/s", "cores": res["cores"],
                         "kind": "port", "sample": res["sample"]},
        "e2e": {"value": res["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out), flush=True)


def tensor_parallel_arm(args, wl, rank, local, world, dev):
    """Workloads 3 and 4 on N GPUs: A sharded along hidden, B along output, NCCL all-reduce of the
    fp32 shrink partials between the two halves.  Total work is fixed: strong scaling."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from ae296_b200.pool import AdapterPool
    from ae296_b200.tp import TPLora
    from ae296_b200.workloads import SEED_BASE, torch_dtype

    tp = world
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
    pools, xs, ys = {}, {}, {}
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
    eng = TPLora(T, wl.n_adapters, hi, 3, tp, rank, None, dev)
    names = [p.name for p in wl.projections]
    stream = torch.cuda.Stream(dev)

    def one_pass():
        eng.set_ids(ids, pools["q"], tiles=wl.seq_lens is not None)
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
        except Exception:                       # NCCL inside a graph refused: time eager launches
            mode = "eager"
            run = one_pass
        for _ in range(max(args.warmup, 3)):
            run()
        stream.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clk:
            e0.record(stream)
            for _ in range(args.steps):
                run()
            e1.record(stream)
            stream.synchronize()
        torch.cuda.synchronize()
        dist.barrier()
    ms = e0.elapsed_time(e1) / args.steps
    tms = torch.tensor([ms], device=dev)
    dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms = float(tms.item())
    eng.batch.workspace.check()
    if rank == 0:
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        peak = json.load(open(peaks_path))["hbm_gbs"] if os.path.exists(peaks_path) else 6650.0
        per_gpu = wl.bytes_per_layer(tp=tp) * n_layers + 2 * 4 * T * 64 * 4 * 2 * n_layers
        out = {
            "metric": "lora_shrink_expand_tokens_per_s", "value": T / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32-accumulate/" + wl.dtype, "data": "synthetic",
            "config": {"workload": f"cfg{wl.cfg}:{wl.name}", "tokens": T, "layers": n_layers,
                       "adapters": wl.n_adapters, "parallelism": f"tp{tp}: A row-sharded, B column-sharded, "
                       "NCCL all-reduce of fp32 [T,64] shrink partials", "timing": mode,
                       "l2": "inputs larger than L2", "note": note},
            "roofline": {"bound": "hbm", "kernel": "whole pass per GPU (shrink + all-reduce + expand)",
                         "achieved": per_gpu / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": per_gpu / (ms * 1e-3) / 1e9 / peak, "traffic": None},
            "cpu_baseline": None, "e2e": None,
            # per layer two applies, each shrink + fold + expand, and with tiles one tile launch per half
            "gpu_launches": (1 + n_layers * 2 * (3 + (2 if wl.seq_lens is not None else 0))) * args.steps,
            "clocks": clk.summary(),
        }
        print(json.dumps(out), flush=True)


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
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    wl = make_workload(args.workload)
    if wl.cfg in (3, 4) and world > 1:
        tensor_parallel_arm(args, wl, rank, local, world, dev)
        dist.destroy_process_group()
        return
    n_layers = args.layers or wl.n_layers
    # keep the resident pool within one GPU: trim depth if the full pool would not fit
    free_b, _ = torch.cuda.mem_get_info()
    per_layer_pool = wl.pool_bytes() // wl.n_layers
    fit_layers = int((free_b * 0.8) // (per_layer_pool + 1))
    depth_note = None
    if n_layers > fit_layers:
        depth_note = f"pool trimmed to {fit_layers} of {n_layers} layers to fit one GPU"
        n_layers = fit_layers
    T = wl.n_tokens
    x_qkv, x_o, pools = materialize_device(wl, dev, layers=n_layers)
    dt = x_qkv.dtype
    names = [p.name for p in wl.projections]
    ys = {p.name: torch.zeros(n_layers, T, p.h_out, dtype=dt, device=dev) for p in wl.projections}
    ids_host = torch.from_numpy(wl.ids).pin_memory()
    ids = ids_host.to(dev)
    batch = L.LoraBatch(T, wl.n_adapters, wl.projections[0].h_in, 3, dev)
    stream = torch.cuda.Stream(dev)

    # prompts (runs of >= 32 rows of one adapter) go to the tcgen05 tile kernel
    use_tiles = wl.seq_lens is not None

    def one_pass(flags=0, plan=True):
        if plan:
            batch.set_ids(ids, pools["q"], tiles=use_tiles)
        for l in range(n_layers):
            batch.apply([(x_qkv[l], ys[n][l], pools[n]) for n in names if n != "o"], l, flags)
            batch.apply([(x_o[l], ys["o"][l], pools["o"])], l, flags)

    # per layer two applies (q/k/v, o), each a shrink and an expand launch, plus with tiles the tile
    # kernel: one launch, or two when the batch can hold fewer (tile, projection) pairs than the GPU
    # has SMs (the library's own rule)
    n_sm = torch.cuda.get_device_properties(dev).multi_processor_count

    def tile_launches(n_proj):
        return 0 if not use_tiles else (2 if (T // 128 + 1) * n_proj < n_sm else 1)

    launches_per_pass = 1 + n_layers * (4 + tile_launches(3) + tile_launches(1))

    def capture(flags=0, plan=True):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            one_pass(flags, plan)
            stream.synchronize()
            with torch.cuda.graph(g, stream=stream):
                one_pass(flags, plan)
        return g

    def capture_plan_only():
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(g, stream=stream):
                for _ in range(8):
                    batch.set_ids(ids, pools["q"], tiles=use_tiles)
        return g

    def timed(graph, steps, warmup):
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                graph.replay()
            stream.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
        return e0.elapsed_time(e1) / steps       # ms per step

    g_full = capture(0)
    with ClockSampler(local) as clk:
        ms = timed(g_full, args.steps, max(args.warmup, 3))
    if world > 1:
        tms = torch.tensor([ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())

    # roofline of the dominant kernel (expand) and of the shrink, each timed alone
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = json.load(open(peaks_path))["hbm_gbs"], "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    used = wl.distinct()
    rsum = int(wl.ranks[used].sum())
    e = 2
    exp_bytes = sum(rsum * p.h_out * e + 2 * T * p.h_out * e for p in wl.projections) * n_layers
    shr_bytes = sum(rsum * p.h_in * e + T * p.h_in * e + 4 * T for p in wl.projections) * n_layers
    # dominant kernels: the shrink and the expand BGMV kernel, one launch of each per apply; timed
    # together as the whole pass without the plan kernel, and each half alone (the lone shrink half
    # also runs the small kernel that writes the intermediate out for tensor-parallel callers).
    ms_noplan = timed(capture(0, plan=False), args.steps, 3)
    ms_exp = timed(capture(_lib.ONLY_EXPAND, plan=False), args.steps, 3)
    ms_shr = timed(capture(_lib.ONLY_SHRINK, plan=False), args.steps, 3)
    us_plan = timed(capture_plan_only(), args.steps, 3) * 1e3 / 8
    ms_dta = timed(capture(_lib.DELTA_THEN_ADD, plan=False), args.steps, 3)
    n_apply = n_layers * 2
    n_launch = n_apply * 2
    pass_bytes = wl.bytes_per_layer() * n_layers
    # DRAM bytes per launch from the ncu capture summarised in profiles/bgmv_cfg1_ncu.md
    # (dram__bytes_read.sum + dram__bytes_write.sum, mean over the four launches of one layer)
    traffic = TRAFFIC_PER_LAUNCH if (wl.cfg == 1 and not use_tiles) else None
    ach = pass_bytes / (ms_noplan * 1e-3) / 1e9
    roofline = {
        "bound": "hbm",
        "kernel": ("" if not use_tiles else "sgmv_tile_kernel + ") + "bgmv_shrink_tma_kernel + bgmv_expand_tma_kernel",
        "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": traffic,
        "peak_source": peak_src, "bytes_per_launch": pass_bytes / n_launch,
        "us_per_launch": ms_noplan * 1e3 / n_launch, "frac_of_8TBs_nominal": ach / 8000.0,
        "expand_half": {"achieved": exp_bytes / (ms_exp * 1e-3) / 1e9, "frac": exp_bytes / (ms_exp * 1e-3) / 1e9 / peak,
                        "us_per_launch": ms_exp * 1e3 / n_apply},
        "shrink_half": {"achieved": shr_bytes / (ms_shr * 1e-3) / 1e9, "frac": shr_bytes / (ms_shr * 1e-3) / 1e9 / peak,
                        "us_per_launch": ms_shr * 1e3 / n_apply},
        "plan_us": us_plan,
        # optional mode with the reference's `q += q_lora` rounding (delta rounded, then a 16-bit add)
        "delta_then_add_mode": {"achieved": pass_bytes / (ms_dta * 1e-3) / 1e9,
                                "frac": pass_bytes / (ms_dta * 1e-3) / 1e9 / peak, "us_per_launch": ms_dta * 1e3 / n_launch},
        "whole_pass": {"bytes": pass_bytes, "achieved": pass_bytes / (ms * 1e-3) / 1e9,
                       "frac": pass_bytes / (ms * 1e-3) / 1e9 / peak},
    }

    # end to end from pinned host buffers through the public ops
    e2e = None
    if not args.no_e2e:
        # One host->device copy and one device->host copy per layer: the layer's two activations sit
        # side by side in one buffer, and so do its four outputs (each projection's y is a column
        # range of the layer's [T, sum(h_out)] block; the kernels take the row pitch).
        h_in0 = wl.projections[0].h_in
        widths = [p.h_out for p in wl.projections]
        offs = [sum(widths[:i]) for i in range(len(widths))]
        dx = torch.empty(n_layers, 2, T, h_in0, dtype=dt, device=dev)
        dx[:, 0].copy_(x_qkv); dx[:, 1].copy_(x_o)
        hx = torch.empty(dx.shape, dtype=dt).pin_memory().copy_(dx.cpu())
        y_all = torch.zeros(n_layers, T, sum(widths), dtype=dt, device=dev)
        yv = {n: y_all[:, :, o:o + w] for n, o, w in zip(names, offs, widths)}
        hy = torch.empty(y_all.shape, dtype=dt).pin_memory()
        copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

        def e2e_step():
            with torch.cuda.stream(stream):
                ids.copy_(ids_host, non_blocking=True)
                batch.set_ids(ids, pools["q"], tiles=use_tiles)
            ev_in, ev_done = [], []
            with torch.cuda.stream(copy_in):
                for l in range(n_layers):
                    dx[l].copy_(hx[l], non_blocking=True)
                    ev = torch.cuda.Event(); ev.record(copy_in); ev_in.append(ev)
            with torch.cuda.stream(stream):
                for l in range(n_layers):
                    stream.wait_event(ev_in[l])
                    batch.apply([(dx[l, 0], yv[n][l], pools[n]) for n in names if n != "o"], l)
                    batch.apply([(dx[l, 1], yv["o"][l], pools["o"])], l)
                    ev = torch.cuda.Event(); ev.record(stream); ev_done.append(ev)
            with torch.cuda.stream(copy_out):
                for l in range(n_layers):
                    copy_out.wait_event(ev_done[l])
                    hy[l].copy_(y_all[l], non_blocking=True)
            stream.wait_stream(copy_out)

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
        e1.record(stream)
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) / k * 1e3
        ms_e2e = max(e0.elapsed_time(e1) / k, wall)
        if world > 1:
            tms = torch.tensor([ms_e2e], device=dev)
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
            ms_e2e = float(tms.item())
        h2d = hx.numel() * 2 + ids_host.numel() * 4
        d2h = hy.numel() * 2
        e2e = {"value": world * T / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle.cpu_baseline import time_cpu_lora
        res = time_cpu_lora(wl, sample_layers=1, reps=4)
        cpu = {"value": res["tokens_per_s"], "unit": "tokens/s", "cores": res["cores"], "kind": "port",
               "sample": res["sample"]}

    if rank == 0:
        out = {
            "metric": "lora_shrink_expand_tokens_per_s", "value": world * T / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32-accumulate/" + wl.dtype, "data": "synthetic",
            "config": {"workload": f"cfg{wl.cfg}:{wl.name}", "tokens_per_gpu": T, "layers": n_layers,
                       "adapters": wl.n_adapters, "distinct_adapters": int(len(used)), "projections": "q,k,v,o",
                       "pool_gb": round(sum(p.nbytes() for p in pools.values()) / 1e9, 3),
                       "l2": "inputs larger than L2 (per-step working set >> 126 MB)",
                       "parallelism": "1 GPU" if world == 1 else f"{world} replicas placed by adapter, no collective",
                       "note": depth_note},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": launches_per_pass * args.steps, "clocks": clk.summary(),
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
