"""Host-side mirror of the reference's GPU LoRA layer object.

``Lora_GPU`` keeps the constructor keys, attribute names and the three
``invoke_one_layer_{q,k,v}(x, layer_id, prefill=False)`` methods of
lightllm/models/lora_gpu.py:16-163, so the layer-infer code
(lightllm/models/llama/layer_infer/transformer_layer_infer.py:101-111) can call it
unchanged.  Differences, all on purpose:

* the decode op is this package's CUDA BGMV instead of ``punica.ops.add_lora_bgmv``, with one
  plan per batch size (built once, not per call) and q/k/v of a layer computed in one fused pass;
* prefill uses the same kernels on request-aligned segments (slot ``b`` <-> request ``b``)
  instead of two ``torch.bmm`` calls and two transposed copies; ``prefill_mid_round``
  reproduces that op's fp16 rounding of the ``[B, L, r]`` intermediate;
* adapter ids come from ``set_indices`` (the reference draws random ids once,
  lora_gpu.py:120, reading past its pool when ``batch_size < 32``);
* no sockets, no swapper, no process exit on error: errors raise.
"""
from __future__ import annotations

from typing import Optional

import torch

import numpy as np

from . import _lib
from .ops import LoraBatch, _adapters_struct, apply
from .pool import AdapterPool


class Lora_GPU:
    def __init__(self, configJson, shared: bool = False, dtype=torch.float16, prefill_mid_round: bool = True):
        self.device = torch.cuda.current_device()
        self.n_layers = configJson["n_layers"]
        self.batch_size = configJson["batch_size"]
        self.lora_rank = configJson["lora_rank"]
        self.in_size = configJson["hidden_dim"]
        self.tp_degree = configJson["tp_degree"]
        self.output_size = configJson["hidden_dim"] // self.tp_degree
        self.max_prefill_batch_size = configJson["max_prefill_batch_size"]
        self.prefill_mid_round = prefill_mid_round
        dev = f"cuda:{self.device}"

        def pool(n, scale):
            down = (torch.randn(n, self.n_layers, self.lora_rank, self.in_size, device=dev) * scale).to(dtype)
            up = (torch.randn(n, self.n_layers, self.output_size, self.lora_rank, device=dev) * scale).to(dtype)
            return down, up

        # decode pools: [N, L, r, H] and [N, L, H/tp, r]   (lora_gpu.py:33-40)
        self.q_down, self.q_up = pool(self.batch_size, 0.001)
        self.k_down, self.k_up = pool(self.batch_size, 0.001)
        self.v_down, self.v_up = pool(self.batch_size, 0.001)
        # prefill slots (lora_gpu.py:54-72)
        self.q_down_prefill, self.q_up_prefill = pool(self.max_prefill_batch_size, 0.001)
        self.k_down_prefill, self.k_up_prefill = pool(self.max_prefill_batch_size, 0.001)
        self.v_down_prefill, self.v_up_prefill = pool(self.max_prefill_batch_size, 0.001)
        g = torch.Generator(device=dev).manual_seed(0)
        self.select_inds = [torch.randint(0, self.batch_size, (i + 1,), device=dev, generator=g)
                            for i in range(self.batch_size)]

        def view(down, up, n):       # the reference's tensors described as a dense pool of uniform rank
            return AdapterPool(down, up, None, None, None, n, self.n_layers, self.in_size, self.output_size,
                               self.lora_rank, False, np.full(n, self.lora_rank, np.int32),
                               np.arange(n + 1, dtype=np.int64) * self.lora_rank)

        self._decode_pools = [view(d, u, self.batch_size) for d, u in
                              ((self.q_down, self.q_up), (self.k_down, self.k_up), (self.v_down, self.v_up))]
        self._prefill_pools = [view(d, u, self.max_prefill_batch_size) for d, u in
                               ((self.q_down_prefill, self.q_up_prefill), (self.k_down_prefill, self.k_up_prefill),
                                (self.v_down_prefill, self.v_up_prefill))]
        self._ad_decode = _adapters_struct(self.batch_size, self.n_layers, self.lora_rank, scale=1.0)
        self._ad_prefill = _adapters_struct(self.max_prefill_batch_size, self.n_layers, self.lora_rank, scale=1.0)
        # one plan + workspace per decode batch size in use (built by the first call or by
        # set_indices), one for prefill that grows to the largest batch seen
        self._decode_batch = {}
        self._prefill_batch = None
        self._prefill_shape = None
        self._fused = None               # (x identity, layer, prefill) -> the k and v deltas computed with q

    def set_indices(self, indices: torch.Tensor) -> None:
        """Adapter slot of each decode token for batches of ``len(indices)`` tokens."""
        bsz = indices.numel()
        self.select_inds[bsz - 1] = indices.to(device=f"cuda:{self.device}")
        self._decode_batch.pop(bsz, None)

    # ---- the three calls the layer code makes ------------------------------------------
    # The layer code asks for q, k and v of one layer in that order with the same input
    # (lightllm/models/llama/layer_infer/transformer_layer_infer.py:108-111).  The q call computes
    # all three deltas in one fused pass (x is read once, one shrink and one expand launch instead
    # of three each) and the k and v calls hand out their parts; a k or v call that does not follow
    # such a q call computes its own.
    def _fused_key(self, x, layer_id, prefill):
        return (x.data_ptr(), x._version, tuple(x.shape), int(layer_id), bool(prefill))

    def _invoke(self, which, x, layer_id, prefill):
        key = self._fused_key(x, layer_id, prefill)
        if which > 0 and self._fused is not None and self._fused[0] == key:
            out = self._fused[1][which]
            if which == 2:
                self._fused = None
            return out
        projs = (0, 1, 2) if which == 0 else (which,)
        ys = self._prefill(x, layer_id, projs) if prefill else self._decode(x, layer_id, projs)
        if which == 0:
            self._fused = (key, ys)
        return ys[which]

    def invoke_one_layer_q(self, x, layer_id, prefill=False):
        return self._invoke(0, x, layer_id, prefill)

    def invoke_one_layer_k(self, x, layer_id, prefill=False):
        return self._invoke(1, x, layer_id, prefill)

    def invoke_one_layer_v(self, x, layer_id, prefill=False):
        return self._invoke(2, x, layer_id, prefill)

    def _decode(self, x, layer_id, projs):
        """x ``[bsz, H]``; token ``t`` uses slot ``select_inds[bsz-1][t]`` (lora_gpu.py:137-138)."""
        bsz = x.shape[0]
        batch = self._decode_batch.get(bsz)
        if batch is None:
            batch = LoraBatch(bsz, self.batch_size, self.in_size, 3, x.device)
            batch.plan.build(self.select_inds[bsz - 1], self._ad_decode)
            self._decode_batch[bsz] = batch
        y = torch.zeros(3, bsz, self.output_size, device=x.device, dtype=x.dtype)
        apply([(x, y[i], self._decode_pools[i]) for i in projs], batch.plan, layer_id, batch.workspace,
              _lib.NO_TENSOR, self._ad_decode)
        return {i: y[i] for i in projs}

    def _prefill(self, x, layer_id, projs):
        """x ``[B, L, H]``: request ``b`` uses prefill slot ``b`` (lora_gpu.py:125-128).  One plan +
        workspace serves every shape: it grows to the largest batch seen and the segment table is
        rebuilt (one small kernel) when ``(B, L)`` changes, so nothing accumulates per shape."""
        bsz, seqlen, hidden = x.shape
        rows = bsz * seqlen
        if self._prefill_batch is None or rows > self._prefill_batch.plan.max_tokens:
            self._prefill_batch = LoraBatch(rows, self.max_prefill_batch_size, self.in_size, 3, x.device)
            self._prefill_shape = None
        batch = self._prefill_batch
        if self._prefill_shape != (bsz, seqlen):
            starts = torch.arange(0, (bsz + 1) * seqlen, seqlen, dtype=torch.int32, device=x.device)
            slots = torch.arange(bsz, dtype=torch.int32, device=x.device)
            batch.plan.from_segments(starts, slots, rows, self._ad_prefill)
            self._prefill_shape = (bsz, seqlen)
        y = torch.zeros(3, rows, self.output_size, device=x.device, dtype=x.dtype)
        flags = _lib.MID_ROUND if self.prefill_mid_round else 0
        x2 = x.reshape(rows, hidden)
        apply([(x2, y[i], self._prefill_pools[i]) for i in projs], batch.plan, layer_id, batch.workspace, flags,
              self._ad_prefill)
        return {i: y[i].view(bsz, seqlen, self.output_size) for i in projs}
