"""Adapter-aware batching: from the router's per-request adapter ids to the kernels' plan.

The reference builds ``lora_ids`` (one int32 per request) next to ``b_start_loc`` / ``b_seq_len`` for every
batch (lightllm/server/router/model_infer/pre_process.py:17,38,50 and :80,92,100), stores them in the infer
state (lightllm/common/basemodel/basemodel.py:200,227) and then never reads them: its LoRA op indexes with a
random tensor (lightllm/models/lora_gpu.py:120,124).  Here they drive the op:

* ``order_by_adapter``   the order in which a router should lay out the requests of a batch so that requests
                          of one adapter are neighbours (stable: arrival order is kept inside an adapter);
* ``plan_for_requests``   the plan of a batch given exactly the three tensors the reference prepares;
* ``delta_cost_us``       a cost estimate of the LoRA delta of a candidate batch for schedulers that compare
                          placements (the role ``cost_model.get_latency(n, rank_func(ranks))`` plays in
                          scheduler/scheduler/manager.py:52-98).
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from .ops import LoraBatch
from .pool import AdapterPool


def order_by_adapter(lora_ids: Sequence[int]) -> np.ndarray:
    """Indices that sort the requests by adapter id, arrival order kept inside one adapter."""
    return np.argsort(np.asarray(lora_ids, np.int64), kind="stable")


def plan_for_requests(batch: LoraBatch, pool: AdapterPool, lora_ids: torch.Tensor, b_start_loc: torch.Tensor,
                      b_seq_len: torch.Tensor, total_token_num: int, prefill: bool) -> LoraBatch:
    """Builds ``batch``'s plan from the tensors of ``prepare_prefill_inputs`` / ``prepare_decode_inputs``.

    Prefill: the rows of request ``b`` are ``[b_start_loc[b], b_start_loc[b] + b_seq_len[b])`` of the un-padded
    token matrix, so every request is one segment of adapter ``lora_ids[b]`` and long prompts go to the
    tensor-core tiles.  Decode: one row per request, ``lora_ids`` is the per-token id vector itself.
    All three are int32 CUDA tensors, as the reference makes them."""
    if lora_ids.dtype != torch.int32 or b_start_loc.dtype != torch.int32 or b_seq_len.dtype != torch.int32:
        raise ValueError("lora_ids, b_start_loc and b_seq_len are int32 tensors")
    n_req = lora_ids.numel()
    if b_start_loc.numel() != n_req or b_seq_len.numel() != n_req:
        raise ValueError("one entry per request expected")
    if not prefill:
        if total_token_num != n_req:
            raise ValueError("a decode batch has one token per request")
        return batch.set_ids(lora_ids.contiguous(), pool, tiles=False)
    starts = torch.empty(n_req + 1, dtype=torch.int32, device=lora_ids.device)
    starts[:n_req] = b_start_loc
    starts[n_req] = int(total_token_num)
    return batch.set_segments(starts, lora_ids.contiguous(), int(total_token_num), pool, tiles=True)


def delta_cost_us(ranks_of_requests: Sequence[int], tokens_of_requests: Sequence[int], adapters_of_requests: Sequence[int],
                  h_in: int, h_out: int, n_projections: int = 4, n_layers: int = 32, hbm_gbs: float = 6540.0,
                  efficiency: float = 0.6, launch_us: float = 4.0, launches_per_layer: int = 4) -> float:
    """Estimated time of the LoRA delta of one step for a candidate batch: the algorithmic bytes (every
    distinct adapter's A and B once, x once, y read and written) at ``efficiency`` x the HBM bandwidth, plus a
    per-launch floor.  A model, not a measurement: schedulers use it to rank placements."""
    ranks = np.asarray(ranks_of_requests, np.int64)
    toks = np.asarray(tokens_of_requests, np.int64)
    ads = np.asarray(adapters_of_requests, np.int64)
    if not (len(ranks) == len(toks) == len(ads)):
        raise ValueError("one entry per request expected")
    _, first = np.unique(ads, return_index=True)
    weight_bytes = int(ranks[first].sum()) * (h_in + h_out) * 2
    t = int(toks.sum())
    per_proj = weight_bytes + t * h_in * 2 + 2 * t * h_out * 2 + 4 * t
    stream_us = per_proj * n_projections * n_layers / (hbm_gbs * 1e3 * efficiency)
    return max(stream_us, launch_us * launches_per_layer * n_layers * 0.5)
