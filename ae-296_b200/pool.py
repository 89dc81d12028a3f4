"""Stacked adapter weight pools held in HBM.

Two layouts describe the same logical content (``A_a[layer]`` is ``[r_a, h_in]``
with ``h_in`` contiguous, ``B_a[layer]`` is ``[h_out, r_a]`` with ``r``
contiguous):

* **dense** - the layout the reference allocates
  (lightllm/models/lora_gpu.py:33-40): ``wa_T_all [N, L, R, h_in]`` and
  ``wb_T_all [N, L, h_out, R]``; an adapter of rank ``r_a < R`` uses the first
  ``r_a`` rows of A and the first ``r_a`` columns of B.
* **packed** - ragged ranks without padding: adapter ``a`` owns rows
  ``[L*cum[a], L*cum[a+1])`` of a ``[L*sum(r), h]`` matrix, layer ``l`` at
  ``L*cum[a] + l*r_a``; B's block for (a, l) is a contiguous ``[h_out, r_a]``.
  Every byte the kernels read is a byte of a used adapter, so the algorithmic
  byte count is reachable with mixed ranks.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

MAX_RANK = 64


@dataclass
class AdapterPool:
    wa: torch.Tensor                 # dense: [N,L,R,h_in]; packed: flat
    wb: torch.Tensor                 # dense: [N,L,h_out,R]; packed: flat
    ranks: torch.Tensor              # int32 [N] on device
    scalings: torch.Tensor           # fp32 [N] on device
    cum_ranks: Optional[torch.Tensor]  # int64 [N+1] on device when packed
    n_adapters: int
    n_layers: int
    h_in: int
    h_out: int
    r_pool: int                      # R of the dense layout == max rank
    packed: bool
    ranks_host: np.ndarray
    cum_host: np.ndarray

    @staticmethod
    def empty(n_adapters, n_layers, h_in, h_out, ranks, scalings, dtype=torch.float16,
              device="cuda", dense=False) -> "AdapterPool":
        ranks = np.asarray(ranks, np.int32)
        assert ranks.shape == (n_adapters,)
        if ranks.min() < 1 or ranks.max() > MAX_RANK:
            raise ValueError(f"adapter ranks must lie in [1, {MAX_RANK}]")
        r_pool = int(ranks.max())
        cum = np.zeros(n_adapters + 1, np.int64)
        np.cumsum(ranks, out=cum[1:])
        if dense:
            if r_pool % 8:
                raise ValueError("dense pools need R to be a multiple of 8")
            wa = torch.zeros(n_adapters, n_layers, r_pool, h_in, dtype=dtype, device=device)
            wb = torch.zeros(n_adapters, n_layers, h_out, r_pool, dtype=dtype, device=device)
            cum_t = None
        else:
            if (ranks % 8).any():
                raise ValueError("packed pools need every rank to be a multiple of 8")
            tot = int(cum[-1]) * n_layers
            wa = torch.zeros(tot * h_in, dtype=dtype, device=device)
            wb = torch.zeros(tot * h_out, dtype=dtype, device=device)
            cum_t = torch.from_numpy(cum).to(device)
        return AdapterPool(
            wa, wb,
            torch.from_numpy(ranks.copy()).to(device),
            torch.as_tensor(np.asarray(scalings, np.float32)).to(device),
            cum_t, n_adapters, n_layers, h_in, h_out, r_pool, not dense, ranks, cum)

    # views of one adapter: A [L, r, h_in], B [L, h_out, r]
    def a_block(self, a: int) -> torch.Tensor:
        r = int(self.ranks_host[a])
        if not self.packed:
            return self.wa[a, :, :r, :]
        off = int(self.cum_host[a]) * self.n_layers * self.h_in
        return self.wa[off: off + self.n_layers * r * self.h_in].view(self.n_layers, r, self.h_in)

    def b_block(self, a: int) -> torch.Tensor:
        r = int(self.ranks_host[a])
        if not self.packed:
            return self.wb[a, :, :, :r]
        off = int(self.cum_host[a]) * self.n_layers * self.h_out
        return self.wb[off: off + self.n_layers * r * self.h_out].view(self.n_layers, self.h_out, r)

    def set_adapter(self, a: int, A: torch.Tensor, B: torch.Tensor) -> None:
        self.a_block(a).copy_(A)
        self.b_block(a).copy_(B)

    def load_adapter_async(self, a: int, A_host: torch.Tensor, B_host: torch.Tensor,
                           stream: Optional["torch.cuda.Stream"] = None) -> "torch.cuda.Event":
        """Host -> HBM copy of one adapter's weights into slot ``a`` on ``stream`` (a side stream,
        so that the swap overlaps the running batch); returns the event the compute stream has to
        wait for before the slot is used.  ``A_host [L, r, h_in]`` and ``B_host [L, h_out, r]``
        should be pinned, otherwise the copies are synchronous.  The slot keeps its rank: a packed
        pool cannot grow an adapter in place.  Counterpart of the reference's swapper copies
        (csrc/cuda_ops.hpp:215-229 ``cudaHtoD2DAsyncLora``, lightllm/models/lora_gpu.py:298-321)."""
        r = int(self.ranks_host[a])
        if tuple(A_host.shape) != (self.n_layers, r, self.h_in) or tuple(B_host.shape) != (self.n_layers, self.h_out, r):
            raise ValueError(f"slot {a} holds rank {r}: expected A [L,{r},{self.h_in}] and B [L,{self.h_out},{r}]")
        stream = stream if stream is not None else torch.cuda.current_stream(self.wa.device)
        with torch.cuda.stream(stream):
            self.a_block(a).copy_(A_host, non_blocking=True)
            self.b_block(a).copy_(B_host, non_blocking=True)
            done = torch.cuda.Event()
            done.record(stream)
        return done

    def nbytes(self) -> int:
        return self.wa.numel() * self.wa.element_size() + self.wb.numel() * self.wb.element_size()

    def shard(self, tp: int, rank: int) -> "AdapterPool":
        """Tensor-parallel shard: A split along ``h_in`` (rows of the hidden
        dimension), B split along ``h_out`` (output columns)."""
        assert self.h_in % tp == 0 and self.h_out % tp == 0
        hi, ho = self.h_in // tp, self.h_out // tp
        out = AdapterPool.empty(self.n_adapters, self.n_layers, hi, ho, self.ranks_host,
                                self.scalings.cpu().numpy(), dtype=self.wa.dtype,
                                device=self.wa.device, dense=not self.packed)
        for a in range(self.n_adapters):
            out.set_adapter(a, self.a_block(a)[:, :, rank * hi:(rank + 1) * hi],
                            self.b_block(a)[:, rank * ho:(rank + 1) * ho, :])
        return out
