"""Shared helpers of the GPU parity tests: seeded cases, the oracle's answer, the CUDA answer."""
from __future__ import annotations

import numpy as np
import torch

import ae296_b200 as L
from ae296_b200.pool import AdapterPool
from oracle import lora_oracle as O

TOL = 2e-3          # max-abs-error bound relative to the RMS of the exact output


class Case:
    def __init__(self, T, N, h_in, h_out, ranks, dtype="fp16", dense=False, seed=0, n_layers=2,
                 ids=None, zipf=None, device="cuda"):
        rng = np.random.default_rng(seed)
        g = torch.Generator().manual_seed(seed)
        self.dtype = dtype
        self.tdt = {"fp16": torch.float16, "bf16": torch.bfloat16}[dtype]
        ranks = np.broadcast_to(np.asarray(ranks, np.int32), (N,)).copy() if np.ndim(ranks) == 0 else np.asarray(ranks, np.int32)
        if ranks.shape != (N,):
            ranks = rng.choice(ranks, N).astype(np.int32)
        self.ranks = ranks
        self.scalings = (32.0 / ranks).astype(np.float32)
        if ids is None:
            if zipf:
                p = 1.0 / np.arange(1, N + 1) ** zipf
                ids = rng.choice(N, T, p=p / p.sum())
            else:
                ids = rng.integers(0, N, T)
        self.ids = np.asarray(ids, np.int32)
        self.T, self.N, self.h_in, self.h_out, self.n_layers = T, N, h_in, h_out, n_layers
        self.x_cpu = torch.randn(T, h_in, generator=g).to(self.tdt)
        self.pool = AdapterPool.empty(N, n_layers, h_in, h_out, ranks, self.scalings, dtype=self.tdt,
                                      device=device, dense=dense)
        self.A, self.B = [], []
        for a in range(N):
            r = int(ranks[a])
            A = (torch.randn(n_layers, r, h_in, generator=g) / np.sqrt(h_in)).to(self.tdt)
            B = (torch.randn(n_layers, h_out, r, generator=g) / np.sqrt(r)).to(self.tdt)
            self.A.append(A)
            self.B.append(B)
            self.pool.set_adapter(a, A.to(device), B.to(device))
        self.x = self.x_cpu.to(device)
        self.ids_dev = torch.from_numpy(self.ids).to(device)
        self.device = device

    def oracle_delta(self, layer, mid_round=None):
        return O.lora_delta(self.x_cpu.double().numpy(),
                            lambda a: self.A[a][layer].double().numpy(),
                            lambda a: self.B[a][layer].double().numpy(),
                            self.ids, self.scalings.astype(np.float64), mid_round)

    def run(self, layer, y0=None, y_dtype=None, flags=0, ids_dtype=torch.int32, batch=None):
        y_dtype = self.tdt if y_dtype is None else y_dtype
        y = torch.zeros(self.T, self.h_out, dtype=y_dtype, device=self.device) if y0 is None else y0.clone()
        if batch is None:
            batch = L.LoraBatch(self.T, self.N, self.h_in, 1, self.device)
            batch.set_ids(self.ids_dev.to(ids_dtype), self.pool)
        batch.apply([(self.x, y, self.pool)], layer, flags)
        torch.cuda.synchronize()
        batch.workspace.check()          # no bounded device-side wait expired
        return y


def rel_err(got64: np.ndarray, want64: np.ndarray) -> float:
    rms = float(np.sqrt((want64 ** 2).mean()))
    return float(np.abs(got64 - want64).max() / max(rms, 1e-30))


def shared_x_cases(T, N, h_in, h_outs, ranks, dtype, ids, seed, n_layers=1, dense=False):
    """One Case per output width, all with the same activation, ids and ranks (the q/k/v
    projections of one layer share x)."""
    first = Case(T, N, h_in, h_outs[0], ranks, dtype, dense=dense, seed=seed, n_layers=n_layers, ids=ids)
    cases = [first] + [Case(T, N, h_in, h, first.ranks, dtype, dense=dense, seed=seed + i, n_layers=n_layers, ids=ids)
                       for i, h in enumerate(h_outs[1:], 1)]     # one adapter table (ranks) for all of them
    for c in cases[1:]:
        c.x, c.x_cpu = cases[0].x, cases[0].x_cpu
    return cases


def raw_apply(projs, plan, layer, workspace, n_tokens, flags=0, adapters=None):
    """``b200_lora_apply`` called directly with an explicit ``n_tokens`` (the Python wrapper
    refuses a row count that differs from the plan's before the library sees it)."""
    import ctypes as C
    from ae296_b200 import _lib
    from ae296_b200.ops import _DT, adapters_of
    arr = (_lib.Proj * len(projs))()
    for i, (x, y, pool) in enumerate(projs):
        arr[i] = _lib.Proj(x.data_ptr(), y.data_ptr(), pool.wa.data_ptr(), pool.wb.data_ptr(),
                           x.stride(0), y.stride(0), pool.h_in, pool.h_out)
    ad = adapters if adapters is not None else adapters_of(projs[0][2])
    x0, y0 = projs[0][0], projs[0][1]
    return _lib.lib().b200_lora_apply(arr, len(projs), C.byref(ad), plan.buf.data_ptr(), plan.max_tokens, n_tokens,
                                      layer, _DT[x0.dtype], _DT[y0.dtype], flags, workspace.buf.data_ptr(),
                                      workspace.nbytes, torch.cuda.current_stream().cuda_stream)
