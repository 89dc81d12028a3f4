"""CPU oracle for the multi-LoRA delta path.  TEST INFRASTRUCTURE ONLY.

This file restates, in numpy (float64 unless noted), the arithmetic of the
reference's LoRA path so that the CUDA kernels can be checked against it.  It
is imported only by the test-suite, the smoke check and the CPU-baseline leg
of the benchmark; the product never routes through it.

What is pinned and what is not
------------------------------
* The CPU-assisted worker (``cpu_worker``) and the prefill batched-matmul op
  (``prefill_bmm``) are pinned: ``tests/golden`` holds vectors produced by the
  reference's own worker loop and by its literal ``torch.bmm`` expression.
* The decode BGMV op is computed by the third-party module ``punica``
  (pinned ``punica==0.2.0`` in the reference's requirements.txt:75) whose
  source is not part of the reference tree.  PARITY UNPINNED at that boundary:
  ``bgmv`` follows the call sites and pool layout
  (lightllm/models/lora_gpu.py:33-40,137-138) and the dense statement the
  reference left beside the call (lightllm/models/lora_gpu.py:136).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import numpy as np


# --------------------------------------------------------------------------------
# rounding helpers
# --------------------------------------------------------------------------------

def round_bf16(a: np.ndarray) -> np.ndarray:
    """Round float values to bfloat16 (nearest-even), returned as float32."""
    f = np.ascontiguousarray(a, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16) << 16
    out = r.astype(np.uint32).view(np.float32).reshape(f.shape)
    return np.where(np.isnan(f), f, out)


def round_to(a: np.ndarray, dtype: str) -> np.ndarray:
    """Round float64 values once to ``dtype`` and return them as float64."""
    if dtype == "fp16":
        return np.asarray(a, np.float64).astype(np.float16).astype(np.float64)
    if dtype == "bf16":
        # float64 -> float32 -> bf16 would round twice; go through an exact
        # sticky-bit narrowing instead.
        a = np.asarray(a, np.float64)
        f = a.astype(np.float32)
        # make f the truncation-toward-zero of a with a sticky low bit, so the
        # second rounding sees on which side of a tie the true value lies
        u = f.view(np.uint32).copy()
        inexact = f.astype(np.float64) != a
        away = np.abs(f.astype(np.float64)) > np.abs(a)
        u = np.where(inexact & away, u - 1, u)        # back to truncation
        u = np.where(inexact, u | 1, u)               # sticky bit
        return round_bf16(u.astype(np.uint32).view(np.float32)).astype(np.float64)
    if dtype == "fp32":
        return np.asarray(a, np.float64).astype(np.float32).astype(np.float64)
    if dtype == "fp64":
        return np.asarray(a, np.float64)
    raise ValueError(dtype)


# --------------------------------------------------------------------------------
# segment bookkeeping (bit-exact integer work)
# --------------------------------------------------------------------------------

def stable_segments(ids: Sequence[int], n_adapters: int) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Stable counting sort of token -> adapter ids.

    Returns ``perm`` (token positions ordered by adapter id, original order
    kept inside one adapter), ``seg_starts`` (S+1 offsets into ``perm``) and
    ``seg_adapter`` (the adapter of each of the S non-empty segments, in
    ascending order).  Restated with explicit loops so that it does not share
    code with ``numpy.argsort``, against which the tests compare it.
    """
    ids = np.asarray(ids, np.int64)
    counts = np.zeros(n_adapters, np.int64)
    for a in ids:
        if a < 0 or a >= n_adapters:
            raise ValueError("adapter id out of range")
        counts[a] += 1
    offs = np.zeros(n_adapters + 1, np.int64)
    for a in range(n_adapters):
        offs[a + 1] = offs[a] + counts[a]
    cursor = offs[:-1].copy()
    perm = np.zeros(len(ids), np.int32)
    for t, a in enumerate(ids):
        perm[cursor[a]] = t
        cursor[a] += 1
    seg_adapter = np.array([a for a in range(n_adapters) if counts[a] > 0], np.int32)
    seg_starts = np.array([offs[a] for a in seg_adapter] + [len(ids)], np.int32)
    return perm, seg_starts, seg_adapter


# --------------------------------------------------------------------------------
# the delta itself
# --------------------------------------------------------------------------------

def lora_delta(x: np.ndarray, a_of, b_of, ids: Sequence[int], scalings: Sequence[float],
               mid_round: Optional[str] = None) -> np.ndarray:
    """``delta[t] = scale_a * (x[t] @ A_a^T) @ B_a^T`` with ``a = ids[t]``, float64.

    ``a_of(a)`` returns A_a as ``[r, h_in]`` and ``b_of(a)`` B_a as
    ``[h_out, r]`` (the transposed storage of lightllm/models/lora_gpu.py:33-34),
    both already holding the rounded I/O-dtype values.  ``mid_round`` rounds
    the ``[T, r]`` intermediate once to that dtype, as the reference's batched
    matmul pair does on fp16 tensors (lightllm/models/lora_gpu.py:127-128);
    ``None`` keeps it exact (the fp32-accumulate BGMV and the CPU worker keep
    at least fp32 there, lora_cpu/lora_shm_op/app.py:136-137).
    """
    x = np.asarray(x, np.float64)
    ids = np.asarray(ids, np.int64)
    out = None
    for a in np.unique(ids):
        A = np.asarray(a_of(int(a)), np.float64)
        B = np.asarray(b_of(int(a)), np.float64)
        if out is None:
            out = np.zeros((x.shape[0], B.shape[0]), np.float64)
        rows = np.nonzero(ids == a)[0]
        v = x[rows] @ A.T
        if mid_round is not None:
            v = round_to(v, mid_round)
        out[rows] = float(scalings[int(a)]) * (v @ B.T)
    if out is None:
        raise ValueError("empty batch: output width unknown")
    return out


def bgmv(y: np.ndarray, x: np.ndarray, a_of, b_of, ids, scalings, out_dtype: str,
         mid_round: Optional[str] = None) -> np.ndarray:
    """Accumulating op: ``round(y + delta)`` with one rounding to ``out_dtype``.

    Call shape of ``punica.ops.add_lora_bgmv(y, x, wa_T_all, wb_T_all, indicies,
    layer_idx, scale)`` at lightllm/models/lora_gpu.py:138,150,162 (y passed as
    zeros at :137).
    """
    return round_to(np.asarray(y, np.float64) + lora_delta(x, a_of, b_of, ids, scalings, mid_round), out_dtype)


def delta_then_add(base: np.ndarray, delta_lowp: np.ndarray, dtype: str) -> np.ndarray:
    """``q += q_lora`` on low-precision tensors: a second rounding
    (lightllm/models/llama/layer_infer/transformer_layer_infer.py:160-170)."""
    return round_to(np.asarray(base, np.float64) + np.asarray(delta_lowp, np.float64), dtype)


def tp_column_slice(full: np.ndarray, tp: int, rank: int) -> np.ndarray:
    """The columns of a full-width delta one tensor-parallel rank collects
    (lightllm/models/lora_cpu.py:43-45,224-232)."""
    w = full.shape[-1] // tp
    return full[..., rank * w:(rank + 1) * w]


# --------------------------------------------------------------------------------
# restatements of the two reference code paths that run without a GPU
# --------------------------------------------------------------------------------

def cpu_worker(x_half, down_f32, up_f32, threads: int = 1):
    """One CPU worker's arithmetic: ``(x.float() @ down @ up).half()``
    (lora_cpu/lora_shm_op/app.py:136-141).  torch CPU tensors in and out, the
    same three operators as the reference.  The reference pins every worker to
    one core (runServerCPULoRA.py:83), so the default runs on one thread; with
    that, results are bit-identical to the reference worker on the same host
    (the fp32 summation order of the matmul depends on the thread count)."""
    import torch
    old = torch.get_num_threads()
    if threads and threads != old:
        torch.set_num_threads(threads)
    try:
        with torch.no_grad():
            return (x_half.float() @ down_f32 @ up_f32).half()
    finally:
        if threads and threads != old:
            torch.set_num_threads(old)


def prefill_bmm(x, wa_T, wb_T):
    """The reference's GPU prefill op as written: two batched matmuls on
    fp16/bf16 tensors, the ``[B, L, r]`` intermediate materialised in the I/O
    dtype (lightllm/models/lora_gpu.py:127-128).  ``x [B,L,H]``, ``wa_T
    [B,r,H]``, ``wb_T [B,H_out,r]`` torch tensors (any device)."""
    import torch
    with torch.no_grad():
        return torch.bmm(torch.bmm(x, wa_T.transpose(-1, -2).contiguous()),
                         wb_T.transpose(-1, -2).contiguous())
