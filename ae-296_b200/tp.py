"""Tensor-parallel LoRA delta: A sharded along the hidden (input) dimension, B along the output.

Rank ``g`` of ``tp`` holds ``A[..., g*h_in/tp:(g+1)*h_in/tp]`` and ``B[g*h_out/tp:(g+1)*h_out/tp, :]``,
consumes the matching column slice of ``x`` and produces the matching column slice of ``y``
(the base model's q/k/v column split, lightllm/models/llama/layer_weights/transformer_layer_weight.py:45-56).
The only exchange is the sum of the small fp32 shrink partials ``[T, 64]`` per projection:

    shrink (ONLY_SHRINK)  ->  all_reduce(v, SUM) over NCCL/NVLink  ->  expand (ONLY_EXPAND)

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


class TPLora:
    """One rank's view of a tensor-parallel LoRA batch."""

    def __init__(self, max_tokens: int, n_adapters: int, h_in_shard: int, n_proj: int, tp: int, rank: int,
                 group: Optional[dist.ProcessGroup] = None, device="cuda"):
        self.tp, self.rank, self.group = tp, rank, group
        self.batch = LoraBatch(max_tokens, n_adapters, h_in_shard, n_proj, device)
        self._v = self.batch.workspace.v_view()

    def set_ids(self, ids: torch.Tensor, pool_shard: AdapterPool, tiles: bool = False) -> "TPLora":
        """``tiles=True`` sends tall contiguous runs (prompts) to the tcgen05 tile kernel, which
        then runs as two halves too (shrink half publishes v, expand half reads the summed v)."""
        self.batch.set_ids(ids, pool_shard, tiles=tiles)
        return self

    def apply(self, projs: Sequence[Tuple[torch.Tensor, torch.Tensor, AdapterPool]], layer: int) -> None:
        """``projs``: ``(x_shard [T, h_in/tp], y_shard [T, h_out/tp], pool_shard)`` per projection."""
        n = len(projs)
        t = projs[0][0].shape[0]
        self.batch.apply(projs, layer, _lib.ONLY_SHRINK)
        allreduce_partials(self._v[:n, :t] if t == self._v.shape[1] else self._v[:n], self.group)
        self.batch.apply(projs, layer, _lib.ONLY_EXPAND)
