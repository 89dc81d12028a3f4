"""Tensor-parallel LoRA delta: A sharded along the hidden (input) dimension, B along the output.

Rank ``g`` of ``tp`` holds ``A[..., g*h_in/tp:(g+1)*h_in/tp]`` and ``B[g*h_out/tp:(g+1)*h_out/tp, :]``,
consumes the matching column slice of ``x`` and produces the matching column slice of ``y``
(the base model's q/k/v column split, lightllm/models/llama/layer_weights/transformer_layer_weight.py:45-56).
The only exchange is the sum of the small fp32 shrink partials ``[T, 64]`` per projection:

    shrink (ONLY_SHRINK)  ->  all_reduce(v, SUM) over NCCL/NVLink  ->  expand (ONLY_EXPAND)

or, with ``exchange="peer"``, one library call per apply (``b200_lora_apply_tp``) that sums the partials with
the library's own kernels over peer memory.

The reference instead replicates A and needs no collective (lightllm/models/lora_gpu.py:25-26,33-34)
at the price of reading A ``tp`` times; that scheme is ``LoraBatch.apply`` with the full ``x``.
One process per GPU; ``torch.distributed`` supplies the process group.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _lib
from .ops import LoraBatch
from .pool import AdapterPool


def column_slice(t: torch.Tensor, tp: int, rank: int) -> torch.Tensor:
    """Columns ``[rank*w, (rank+1)*w)`` of a ``[T, tp*w]`` tensor (a strided view, no copy)."""
    w = t.shape[-1] // tp
    if w * tp != t.shape[-1]:
        raise ValueError("width not divisible by the tensor-parallel degree")
    return t[..., rank * w:(rank + 1) * w]


def allreduce_partials(v: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Sum of the ranks' shrink partials, in place (NCCL on GPU tensors, gloo on CPU tensors)."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(v, op=dist.ReduceOp.SUM, group=group)
    return v


class PeerExchange:
    """The ranks' landing buffers for ``b200_lora_tp_exchange``: allocated by the library (so that they can be
    exported), handles handed round through the process group, every peer's buffer mapped into this process."""

    def __init__(self, max_tokens: int, n_proj: int, tp: int, rank: int, group: Optional[dist.ProcessGroup] = None):
        import ctypes as C
        L = _lib.lib()
        self._C, self._L = C, L
        self.tp, self.rank, self.max_tokens, self.n_proj = tp, rank, max_tokens, n_proj
        nbytes = L.b200_lora_tp_bytes(max_tokens, n_proj, tp)
        if nbytes == 0:
            raise ValueError("bad tensor-parallel exchange dimensions (2..8 ranks)")
        base = C.c_void_p(0)
        _lib.check(L.b200_lora_tp_alloc(C.byref(base), nbytes), "tp_alloc")
        self.base = base.value
        handle = (C.c_ubyte * 64)()
        _lib.check(L.b200_lora_tp_export(self.base, handle), "tp_export")
        handles = [None] * tp
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.ctx = _lib.TpContext()
        self.ctx.tp, self.ctx.rank = tp, rank
        self._mapped = []
        for r in range(tp):
            if r == rank:
                ptr = self.base
            else:
                m = C.c_void_p(0)
                buf = (C.c_ubyte * 64).from_buffer_copy(handles[r])
                _lib.check(L.b200_lora_tp_open(buf, C.byref(m)), f"tp_open(rank {r})")
                ptr = m.value
                self._mapped.append(ptr)
            _lib.check(L.b200_lora_tp_layout(C.byref(self.ctx), r, ptr, max_tokens, n_proj), "tp_layout")
        dist.barrier(group=group)                  # every rank has mapped every buffer before anyone pushes

    def exchange(self, workspace, n_tokens: int, n_proj: int, skip_arrival: bool = False) -> None:
        """Sums ``v [n_proj][max_tokens][64]`` of ``workspace`` over the ranks in place (``n_proj`` of this
        apply, at most the number the buffers were sized for; the same on every rank)."""
        if not 1 <= n_proj <= self.n_proj:
            raise ValueError("more projections than the exchange buffers were sized for")
        _lib.check(self._L.b200_lora_tp_exchange(
            self._C.byref(self.ctx), workspace.buf.data_ptr(), self.max_tokens, int(n_tokens), int(n_proj),
            1 if skip_arrival else 0, torch.cuda.current_stream(workspace.buf.device).cuda_stream), "tp_exchange")

    def close(self) -> None:
        for m in self._mapped:
            self._L.b200_lora_tp_close(m)
        self._mapped = []
        if self.base:
            self._L.b200_lora_tp_free(self.base)
            self.base = None


class TPLora:
    """One rank's view of a tensor-parallel LoRA batch.

    ``exchange="nccl"`` sums the shrink partials with ``torch.distributed.all_reduce``;
    ``exchange="peer"`` with the library's own one-kernel exchange over peer memory (NVLink), which needs
    the ranks to be processes on one node with peer access between their GPUs."""

    def __init__(self, max_tokens: int, n_adapters: int, h_in_shard: int, n_proj: int, tp: int, rank: int,
                 group: Optional[dist.ProcessGroup] = None, device="cuda", exchange: str = "nccl"):
        self.tp, self.rank, self.group = tp, rank, group
        self.batch = LoraBatch(max_tokens, n_adapters, h_in_shard, n_proj, device)
        self._v = self.batch.workspace.v_view()
        self.n_proj = n_proj
        if exchange not in ("nccl", "peer"):
            raise ValueError("exchange is 'nccl' or 'peer'")
        self.peer = PeerExchange(max_tokens, n_proj, tp, rank, group) if (exchange == "peer" and tp > 1) else None

    def set_ids(self, ids: torch.Tensor, pool_shard: AdapterPool, tiles: bool = False) -> "TPLora":
        """``tiles=True`` sends tall contiguous runs (prompts) to the tcgen05 tile kernel, which
        then runs as two halves too (shrink half publishes v, expand half reads the summed v)."""
        self.batch.set_ids(ids, pool_shard, tiles=tiles)
        return self

    def apply(self, projs: Sequence[Tuple[torch.Tensor, torch.Tensor, AdapterPool]], layer: int,
              skip_arrival: bool = False) -> None:
        """``projs``: ``(x_shard [T, h_in/tp], y_shard [T, h_out/tp], pool_shard)`` per projection.
        ``skip_arrival`` (peer exchange only) withholds this rank's packets: a failure made on the
        host, with which tests check that the peers give up instead of hanging."""
        n = len(projs)
        t = projs[0][0].shape[0]
        if self.peer is not None:
            # one library call: both halves and, between them, the exchange of the rows each kernel chain
            # owns (tall runs on the tile kernels' side stream, the rest beside the BGMV kernels)
            if n > self.peer.n_proj:
                raise ValueError("more projections than the exchange buffers were sized for")
            self.batch.apply(projs, layer, 0, tp_ctx=self.peer.ctx, skip_arrival=skip_arrival)
            return
        self.batch.apply(projs, layer, _lib.ONLY_SHRINK)
        allreduce_partials(self._v[:n, :t] if t == self._v.shape[1] else self._v[:n], self.group)
        self.batch.apply(projs, layer, _lib.ONLY_EXPAND)

    def close(self) -> None:
        if self.peer is not None:
            self.peer.close()
            self.peer = None
