"""CPU baseline made of the reference's OWN worker processes.  TEST/BENCH INFRASTRUCTURE ONLY.

Drives unmodified ``LoRAapp.run`` loops (lora_cpu/lora_shm_op/app.py:102-154, fetched to
``oracle/_ref/app.py`` by ``oracle/fetch_ref.py``) the way the reference's host side does
(lightllm/models/lora_cpu.py:160-185,218-276), minus the GPU copies:

* the seven POSIX shared-memory segments and their ``<tag>-<name>.shm`` name files
  (create_shm.py:97-127, parsed at app.py:71-75);
* one worker process per core, pinned (the reference pins with numactl, runServerCPULoRA.py:83),
  each holding one adapter's fp32 ``down [H, r]`` / ``up [r, H]`` weights (app.py:38-45);
* a doorbell per job: the int16 value ``2 + row`` (q), ``202 + row`` (k) or ``402 + row`` (v) written
  into the worker's signal slot (lora_cpu.py:181-185; decoded at app.py:108-128); the worker computes
  ``(x.float() @ down @ up).half()`` for that row of the input segment, stores it in the output
  segment and writes 0 back (app.py:133-143); the host polls for the zeros (lora_cpu.py:219).

The doorbell value, not the slot, names the row, so W persistent workers serve any number of rows:
rows are dealt to the workers of their adapter's rank class, 200 rows of the signal space at a time.
The worker has no o-projection branch (app.py:111-128); the o delta has q's shapes and is timed
through the q doorbell.  A worker keeps one set of weights for every layer, as in the reference
(the worker has no layer argument), so a pass of L layers is L rounds over the same workers.
"""
from __future__ import annotations

import importlib.util
import multiprocessing as mp
import os
import sys
import tempfile
import time
import types
from multiprocessing import shared_memory
from typing import Dict, List

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
APP = os.path.join(HERE, "_ref", "app.py")
SEGMENTS = ["shm_array", "shm_out_q", "shm_out_k", "shm_out_v", "shm_out_o"]
ROWS_MAX = 200                 # rows one projection's doorbell range can name (app.py:111-128)
ROW_TOKENS_MAX = 200           # tokens of one row (the worker sees the count through one byte)
BASES = {"q": 2, "k": 202, "v": 402, "o": 2}


def available() -> bool:
    return os.path.isfile(APP)


def _worker_main(folder, ns, core, seed):
    import torch
    try:
        os.sched_setaffinity(0, {core})
    except (AttributeError, OSError):
        pass
    torch.set_num_threads(1)
    spec = importlib.util.spec_from_file_location("ref_lora_app", APP)
    app = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(app)
    app.args = ns                                   # module global read by init_shm (app.py:81-89)
    sys.stdout = open(os.devnull, "w")
    torch.manual_seed(seed)
    w = app.LoRAapp(ns, folder)
    # the workload's value distributions instead of the reference's randn * 0.001 (app.py:38-45)
    g = torch.Generator().manual_seed(seed)
    for nm in "qkvo":
        setattr(w, f"{nm}_down_LoRA", torch.randn(ns.in_size, ns.rank, generator=g) / np.sqrt(ns.in_size))
        setattr(w, f"{nm}_up_LoRA", torch.randn(ns.rank, ns.out_size, generator=g) / np.sqrt(ns.rank))
    w.run()


class ReferenceWorkerPool:
    """Shared-memory segments plus W reference worker processes."""

    def __init__(self, hidden: int, max_len: int, ranks_of_worker: List[int], seed: int = 2960):
        self.hidden, self.max_len = hidden, max_len
        self.folder = tempfile.mkdtemp(prefix="shmnames")
        self.shms: Dict[str, shared_memory.SharedMemory] = {}
        nbytes = 2 * ROWS_MAX * max_len * hidden
        for name in SEGMENTS:
            self._make(name, nbytes)
        self._make("shm_tkn_len", 8)
        self._make("lock", 8)                       # layer hand-shake of the host side (create_shm.py), unused by workers
        n_workers = len(ranks_of_worker)
        self._make("shm_signal", 2 * max(n_workers, 1))
        self.arr = {n: np.ndarray((ROWS_MAX, max_len, hidden), np.float16, buffer=self.shms[n].buf) for n in SEGMENTS}
        self.signal = np.ndarray((n_workers,), np.int16, buffer=self.shms["shm_signal"].buf)
        self.signal[:] = 1
        self.tkn_len = np.ndarray((1,), np.int64, buffer=self.shms["shm_tkn_len"].buf)
        cores = sorted(os.sched_getaffinity(0))
        ctx = mp.get_context("fork")
        self.procs = []
        for i, r in enumerate(ranks_of_worker):
            ns = types.SimpleNamespace(in_size=hidden, out_size=hidden, batch_size=ROWS_MAX, signal_name=None, rank=int(r),
                                       prompt_max_length=max_len, signal_index=i, offset=max_len)
            # core 0 is left to the dispatcher when there are cores to spare
            core = cores[(i + 1) % len(cores)] if len(cores) > n_workers else cores[i % len(cores)]
            p = ctx.Process(target=_worker_main, args=(self.folder, ns, core, seed + i), daemon=True)
            p.start()
            self.procs.append(p)
        self.ranks_of_worker = list(ranks_of_worker)

    def _make(self, name, nbytes):
        s = shared_memory.SharedMemory(create=True, size=nbytes)
        self.shms[name] = s
        with open(os.path.join(self.folder, f"{name}-{s.name}.shm"), "w") as f:
            f.write(f"{name},{s.name}\n")

    def wait_ready(self, timeout=120.0):
        """Rings every worker once (row 0, q) and waits for the acks: all loops are up."""
        self.tkn_len[0] = 1
        t0 = time.time()
        self.signal[:] = 2
        while (self.signal != 0).any():
            if time.time() - t0 > timeout or any(not p.is_alive() for p in self.procs):
                raise TimeoutError("a reference worker did not come up")
            time.sleep(0.001)
        self.signal[:] = 1

    def run_jobs(self, jobs_of_worker: List[List[int]], timeout=120.0) -> float:
        """``jobs_of_worker[w]`` = doorbell values for worker ``w``, in order.  Rings each worker's
        next doorbell as soon as it has acknowledged the previous one; returns the wall time from
        the first doorbell to the last acknowledgement."""
        sig = self.signal
        nxt = [0] * len(jobs_of_worker)
        left = sum(len(j) for j in jobs_of_worker)
        busy = [False] * len(jobs_of_worker)
        t0 = time.perf_counter()
        while left:
            for w, jobs in enumerate(jobs_of_worker):
                if busy[w]:
                    if sig[w] != 0:
                        continue
                    busy[w] = False
                    left -= 1
                if nxt[w] < len(jobs):
                    sig[w] = jobs[nxt[w]]
                    nxt[w] += 1
                    busy[w] = True
            if time.perf_counter() - t0 > timeout:
                raise TimeoutError("reference workers did not finish")
        dt = time.perf_counter() - t0
        sig[:] = 1
        return dt

    def close(self):
        for p in self.procs:
            p.terminate()
        for p in self.procs:
            p.join(timeout=10)
        del self.arr, self.signal, self.tkn_len
        for s in self.shms.values():
            s.close()
            s.unlink()
        for f in os.listdir(self.folder):
            os.remove(os.path.join(self.folder, f))
        os.rmdir(self.folder)


def time_reference_workers(wl, layers: int = 0, steps: int = 2, warmup: int = 1, n_workers: int = 0, seed: int = 2960):
    """Times passes (``layers`` rounds of q/k/v/o, default the workload's depth; the result is scaled
    to the full depth, every round being the same work on the same workers) of workload
    ``wl`` on the reference's worker processes.  One request row per token for decode tokens
    and one row per prompt for prefill requests (a worker takes a whole row, app.py:133-141).

    Returns ``dict(seconds_per_pass, tokens_per_s, cores, workers, sample)``.
    """
    import torch  # noqa: F401  (workers fork with torch already imported)
    if not available():
        raise FileNotFoundError(APP)
    layers = layers or wl.n_layers
    cores = len(os.sched_getaffinity(0))
    W = n_workers or max(1, cores - 1)
    hidden = wl.projections[0].h_in
    # rows: (tokens in the row, adapter)
    if wl.seq_lens is not None:
        nd = wl.n_decode
        rows = [(1, int(a)) for a in wl.ids[:nd]]
        pos = nd
        for ln in wl.seq_lens:
            # the worker reads the row's token count as ONE byte of the shared word (app.py:99,130), and
            # the reference caps prompts at 256 tokens (lightllm/models/lora_cpu.py:14): a longer prompt is
            # served as several rows of at most ROW_TOKENS_MAX tokens
            for c0 in range(0, int(ln), ROW_TOKENS_MAX):
                rows.append((min(ROW_TOKENS_MAX, int(ln) - c0), int(wl.ids[pos])))
            pos += int(ln)
    else:
        rows = [(1, int(a)) for a in wl.ids]
    max_len = max(r[0] for r in rows)
    # the worker reads ONE token count for every row (app.py:130), so rows are served in groups of
    # equal length; workers are split over the rank classes in proportion to their work
    classes = sorted({int(wl.ranks[a]) for _, a in rows})
    cost = {c: sum(n * c for n, a in rows if int(wl.ranks[a]) == c) for c in classes}
    tot = float(sum(cost.values()))
    W = max(W, len(classes))
    share = {c: max(1, int(round(W * cost[c] / tot))) for c in classes}
    while sum(share.values()) > W:
        share[max(share, key=lambda c: share[c])] -= 1
    ranks_of_worker = [c for c in classes for _ in range(share[c])]
    workers_of = {c: [i for i, r in enumerate(ranks_of_worker) if r == c] for c in classes}
    pool = ReferenceWorkerPool(hidden, max_len, ranks_of_worker, seed)
    try:
        pool.wait_ready()
        rng = np.random.default_rng(seed)
        pool.arr["shm_array"][:] = rng.standard_normal((ROWS_MAX, max_len, hidden), dtype=np.float32).astype(np.float16)
        # groups of rows with one token count, at most ROWS_MAX rows each
        by_len: Dict[int, List[int]] = {}
        for i, (n, _) in enumerate(rows):
            by_len.setdefault(n, []).append(i)
        groups = []
        for n, idx in by_len.items():
            for s in range(0, len(idx), ROWS_MAX):
                groups.append((n, idx[s:s + ROWS_MAX]))

        def one_pass():
            t = 0.0
            for _layer in range(layers):
                for n, idx in groups:
                    pool.tkn_len[0] = n
                    jobs = [[] for _ in ranks_of_worker]
                    rr = {c: 0 for c in classes}
                    for proj in "qkvo":
                        for slot, i in enumerate(idx):
                            c = int(wl.ranks[rows[i][1]])
                            ws = workers_of[c]
                            jobs[ws[rr[c] % len(ws)]].append(BASES[proj] + slot)
                            rr[c] += 1
                    t += pool.run_jobs(jobs)
            return t

        for _ in range(warmup):
            one_pass()
        times = [one_pass() for _ in range(steps)]
    finally:
        pool.close()
    sec = float(np.median(times)) * wl.n_layers / layers          # scaled to the workload's depth
    return {
        "seconds_per_pass": sec, "tokens_per_s": wl.n_tokens / sec, "cores": cores, "workers": len(ranks_of_worker),
        "sample": f"{steps} passes of {layers} of {wl.n_layers} layers (x q/k/v/o, {len(rows)} request rows, {len(groups)} doorbell wave(s) per layer) "
                  f"after {warmup} warm-up; {len(ranks_of_worker)} unmodified LoRAapp.run workers, one pinned core each "
                  f"(rank classes {dict(share)}), doorbells over POSIX shared memory, os.cpu_count()={os.cpu_count()}",
    }
