"""Host-side mirror of the reference's GPU LoRA layer object.

``Lora_GPU`` keeps the constructor keys, attribute names and the three
``invoke_one_layer_{q,k,v}(x, layer_id, prefill=False)`` methods of
lightllm/models/lora_gpu.py:16-163, so the layer-infer code
(lightllm/models/llama/layer_infer/transformer_layer_infer.py:101-111) can call it
unchanged.  Differences, all on purpose:

* the decode op is this package's CUDA BGMV instead of ``punica.ops.add_lora_bgmv``;
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

from . import _lib
from .ops import LoraBatch, add_lora_bgmv
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
        self._prefill_batch = {}

    def set_indices(self, indices: torch.Tensor) -> None:
        """Adapter slot of each decode token for batches of ``len(indices)`` tokens."""
        self.select_inds[indices.numel() - 1] = indices.to(device=f"cuda:{self.device}")

    # ---- the three calls the layer code makes ------------------------------------------
    def _invoke(self, x, layer_id, prefill, down, up, down_p, up_p):
        if prefill:
            return self._prefill(x, layer_id, down_p, up_p)
        bsz = x.shape[0]
        y = torch.zeros(bsz, self.output_size, device=x.device, dtype=x.dtype)
        add_lora_bgmv(y, x, down, up, self.select_inds[bsz - 1], layer_id, 1)
        return y

    def invoke_one_layer_q(self, x, layer_id, prefill=False):
        return self._invoke(x, layer_id, prefill, self.q_down, self.q_up, self.q_down_prefill, self.q_up_prefill)

    def invoke_one_layer_k(self, x, layer_id, prefill=False):
        return self._invoke(x, layer_id, prefill, self.k_down, self.k_up, self.k_down_prefill, self.k_up_prefill)

    def invoke_one_layer_v(self, x, layer_id, prefill=False):
        return self._invoke(x, layer_id, prefill, self.v_down, self.v_up, self.v_down_prefill, self.v_up_prefill)

    def _prefill(self, x, layer_id, down_p, up_p):
        """x ``[B, L, H]``: request ``b`` uses prefill slot ``b`` (lora_gpu.py:125-128)."""
        bsz, seqlen, hidden = x.shape
        key = (bsz, seqlen)
        st = self._prefill_batch.get(key)
        if st is None:
            pool = AdapterPool(down_p, up_p, None, None, None, self.max_prefill_batch_size, self.n_layers,
                               self.in_size, self.output_size, self.lora_rank, False, None, None)
            batch = LoraBatch(bsz * seqlen, self.max_prefill_batch_size, self.in_size, 1, x.device)
            starts = torch.arange(0, (bsz + 1) * seqlen, seqlen, dtype=torch.int32, device=x.device)
            slots = torch.arange(bsz, dtype=torch.int32, device=x.device)
            from .ops import _adapters_struct
            ad = _adapters_struct(self.max_prefill_batch_size, self.n_layers, self.lora_rank)
            batch.plan.from_segments(starts, slots, bsz * seqlen, ad)
            st = (batch, ad)
            self._prefill_batch[key] = st
        batch, ad = st
        pool = AdapterPool(down_p, up_p, None, None, None, self.max_prefill_batch_size, self.n_layers,
                           self.in_size, self.output_size, self.lora_rank, False, None, None)
        y = torch.zeros(bsz * seqlen, self.output_size, device=x.device, dtype=x.dtype)
        from .ops import apply
        flags = _lib.MID_ROUND if self.prefill_mid_round else 0
        apply([(x.reshape(bsz * seqlen, hidden), y, pool)], batch.plan, layer_id, batch.workspace, flags, ad)
        return y.view(bsz, seqlen, self.output_size)
