"""Placement of independent requests on several GPUs by adapter (no collective on the data path).

Every adapter lives on exactly one GPU and a token is served where its adapter lives, so each
GPU runs the single-GPU kernels on its own sub-batch against its own, smaller pool.  The
reference keeps one pool per model process and never routes by adapter (its index tensor is
random, lightllm/models/lora_gpu.py:120); its cluster-level counterpart is the request router of
the scheduler simulator (scheduler/scheduler/manager.py:52-98).

Two policies:

* ``"mod"``       adapter ``a`` lives on GPU ``a % G`` (stateless, what a router can compute alone);
* ``"balanced"``  adapters are dealt to GPUs by decreasing load, each to the GPU with the least
                  load so far (longest-processing-time-first), so that a skewed popularity (a few
                  hot adapters) does not overload one GPU.  The load of an adapter is its token
                  count, or, when the adapters' ranks are given, an estimate of the bytes its
                  tokens make the kernels move: the delta path is bound by memory traffic, an
                  adapter's weights are read once per work segment of eight tokens, and a rank-64
                  adapter costs eight times a rank-8 one.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np


@dataclass
class Placement:
    gpu_of_adapter: np.ndarray          # int32 [N]   GPU that holds each adapter (-1: unused under "balanced")
    local_id: np.ndarray                # int32 [N]   slot of the adapter in its GPU's pool
    adapters: List[np.ndarray]          # per GPU: global adapter ids in slot order
    tokens: List[np.ndarray]            # per GPU: indices into the global batch, original order kept
    local_ids: List[np.ndarray]         # per GPU: the sub-batch's adapter ids as pool slots (int32)

    @property
    def n_gpus(self) -> int:
        return len(self.adapters)

    def scatter(self, rows_per_gpu: Sequence[np.ndarray], width: int, dtype=np.float32) -> np.ndarray:
        """Puts per-GPU results ``[T_g, width]`` back into global token order."""
        total = sum(len(t) for t in self.tokens)
        out = np.zeros((total, width), dtype)
        for t, r in zip(self.tokens, rows_per_gpu):
            out[t] = r
        return out


WORK_SEGMENT_TOKENS = 8      # the kernels read an adapter's weights once per this many of its tokens
TOKEN_COST_IN_RANK_ROWS = 1.5  # bytes of one token's x and y (read, read + write) relative to one rank row of A and B


def adapter_load(counts: np.ndarray, ranks: Optional[Sequence[int]] = None) -> np.ndarray:
    """Per-adapter load of a batch with ``counts[a]`` tokens of adapter ``a``: the token count, or with
    ``ranks`` an estimate of the memory traffic in units of one rank row of A and B."""
    counts = np.asarray(counts, np.int64)
    if ranks is None:
        return counts.astype(np.float64)
    r = np.asarray(ranks, np.float64)
    if r.shape != counts.shape:
        raise ValueError("one rank per adapter")
    segments = -(-counts // WORK_SEGMENT_TOKENS)
    return segments * r + TOKEN_COST_IN_RANK_ROWS * counts


def place_by_adapter(ids: Sequence[int], n_gpus: int, n_adapters: int, policy: str = "balanced",
                     resident_all: bool = True, ranks: Optional[Sequence[int]] = None) -> Placement:
    """Splits a batch with per-token adapter ``ids`` over ``n_gpus`` GPUs.

    ``resident_all=True`` places every one of the ``n_adapters`` adapters (a serving pool holds
    adapters that the current batch does not use); otherwise only the batch's adapters.
    ``ranks`` (one per adapter) makes the ``"balanced"`` policy balance estimated bytes instead of tokens.
    """
    ids = np.asarray(ids, np.int64)
    if n_gpus < 1:
        raise ValueError("n_gpus must be positive")
    if ids.size and (ids.min() < 0 or ids.max() >= n_adapters):
        raise ValueError("adapter id out of range")
    counts = np.bincount(ids, minlength=n_adapters)
    gpu_of = np.full(n_adapters, -1, np.int32)
    if policy == "mod":
        gpu_of[:] = np.arange(n_adapters) % n_gpus
        if not resident_all:
            gpu_of[counts == 0] = -1
    elif policy == "balanced":
        cost = adapter_load(counts, ranks)
        load = np.zeros(n_gpus, np.float64)
        held = np.zeros(n_gpus, np.int64)
        order = np.argsort(-cost, kind="stable")             # heaviest first; ties by adapter id
        for a in order:
            if counts[a] == 0 and not resident_all:
                continue
            # least load first, then fewest adapters, then lowest GPU index: deterministic
            g = int(np.lexsort((np.arange(n_gpus), held, load))[0])
            gpu_of[a] = g
            load[g] += cost[a]
            held[g] += 1
    else:
        raise ValueError(f"unknown policy {policy!r}")
    local = np.full(n_adapters, -1, np.int32)
    adapters, tokens, local_ids = [], [], []
    for g in range(n_gpus):
        mine = np.nonzero(gpu_of == g)[0].astype(np.int32)
        local[mine] = np.arange(len(mine), dtype=np.int32)
        adapters.append(mine)
    tok_gpu = gpu_of[ids] if ids.size else np.zeros(0, np.int32)
    for g in range(n_gpus):
        t = np.nonzero(tok_gpu == g)[0].astype(np.int64)
        tokens.append(t)
        local_ids.append(local[ids[t]].astype(np.int32))
    return Placement(gpu_of, local, adapters, tokens, local_ids)
