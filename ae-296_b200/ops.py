"""Python-facing multi-LoRA ops: thin wrappers that pass tensor addresses to the C ABI.

``add_lora_bgmv`` keeps the positional signature the reference's layer code calls
(``punica.ops.add_lora_bgmv(y, x, wa_T_all, wb_T_all, indicies, layer_idx, scale)``,
lightllm/models/lora_gpu.py:138,150,162).  The generalised ops add per-adapter ranks and
scalings, packed pools, adapter-sorted segments and fused q/k/v application.

PyTorch is used for device memory and streams only; all arithmetic runs in the CUDA
library, and there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import Adapters, LoraError, Proj, check
from .pool import AdapterPool

_DT = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise ValueError("LoRA ops need CUDA tensors (no CPU path exists)")


def _adapters_struct(n_adapters, n_layers, r_pool, ranks=None, scalings=None, cum_ranks=None,
                     packed=False, scale=1.0, ranks_pow2=False, total_rank=0) -> Adapters:
    return Adapters(
        ranks.data_ptr() if ranks is not None else None,
        scalings.data_ptr() if scalings is not None else None,
        cum_ranks.data_ptr() if cum_ranks is not None else None,
        n_adapters, n_layers, r_pool, 1 if packed else 0, float(scale), 1 if ranks_pow2 else 0,
        int(total_rank))


def adapters_of(pool: AdapterPool) -> Adapters:
    """The pool's adapter table; promises power-of-two ranks to the library when the host
    copy of the ranks shows it (which selects the TMA kernels)."""
    rh = pool.ranks_host
    if pool.packed:
        pow2 = bool(np.isin(rh, (8, 16, 32, 64)).all())
    else:
        pow2 = bool((rh == pool.r_pool).all()) and pool.r_pool in (8, 16, 32, 64)
    return _adapters_struct(pool.n_adapters, pool.n_layers, pool.r_pool, pool.ranks, pool.scalings,
                            pool.cum_ranks, pool.packed, 1.0, pow2, int(pool.cum_host[-1]))


class LoraPlan:
    """Device-resident segment table of one batch (see ``b200_lora_plan_build``)."""

    def __init__(self, max_tokens: int, n_adapters: int, device="cuda"):
        self.max_tokens, self.n_adapters = int(max_tokens), int(n_adapters)
        nbytes = _lib.lib().b200_lora_plan_bytes(self.max_tokens, self.n_adapters)
        if nbytes == 0:
            raise ValueError("bad plan dimensions")
        self.buf = torch.zeros((nbytes + 15) // 16 * 2, dtype=torch.int64, device=device)
        self.nbytes = self.buf.numel() * 8
        self._keep = None
        self.n_tokens = 0            # rows of the batch the plan was last built for

    def build(self, ids: torch.Tensor, adapters: Adapters) -> "LoraPlan":
        _require_cuda(ids)
        if ids.dtype not in (torch.int32, torch.int64) or not ids.is_contiguous():
            raise ValueError("ids must be a contiguous int32/int64 tensor")
        self.n_tokens = int(ids.numel())
        check(_lib.lib().b200_lora_plan_build(
            self.buf.data_ptr(), self.nbytes, self.max_tokens, ids.data_ptr(),
            1 if ids.dtype == torch.int64 else 0, ids.numel(), C.byref(adapters), _stream(ids.device)),
            "plan_build")
        return self

    def from_segments(self, seg_starts: torch.Tensor, seg_adapter: torch.Tensor, n_tokens: int,
                      adapters: Adapters) -> "LoraPlan":
        _require_cuda(seg_starts, seg_adapter)
        if seg_starts.dtype != torch.int32 or seg_adapter.dtype != torch.int32:
            raise ValueError("segment tables must be int32")
        self._keep = (seg_starts, seg_adapter)
        self.n_tokens = int(n_tokens)
        check(_lib.lib().b200_lora_plan_from_segments(
            self.buf.data_ptr(), self.nbytes, self.max_tokens, seg_starts.data_ptr(), seg_adapter.data_ptr(),
            seg_adapter.numel(), int(n_tokens), C.byref(adapters), _stream(seg_starts.device)),
            "plan_from_segments")
        return self

    def read(self) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
        """(perm, seg_starts, seg_adapter) as host arrays; raises on a bad id or segment table."""
        perm = np.zeros(self.max_tokens, np.int32)
        starts = np.zeros(self.max_tokens + 1, np.int32)
        adapter = np.zeros(self.max_tokens, np.int32)
        ns, nt = C.c_int32(0), C.c_int32(0)
        check(_lib.lib().b200_lora_plan_read(
            self.buf.data_ptr(), perm.ctypes.data, starts.ctypes.data, adapter.ctypes.data,
            C.byref(ns), C.byref(nt), _stream(self.buf.device)), "plan_read")
        return perm[:nt.value], starts[:ns.value + 1], adapter[:ns.value]


class LoraWorkspace:
    """Scratch for the ``[T, r]`` intermediate and the split-K partial sums."""

    def check(self) -> None:
        """Synchronises and raises if a kernel recorded a device-side error (expired wait)."""
        check(_lib.lib().b200_lora_workspace_status(self.buf.data_ptr(), _stream(self.buf.device)),
              "workspace_status")

    def __init__(self, max_tokens: int, n_proj: int, max_h_in: int, device="cuda"):
        self.max_tokens, self.n_proj, self.max_h_in = int(max_tokens), int(n_proj), int(max_h_in)
        nbytes = _lib.lib().b200_lora_workspace_bytes(self.max_tokens, self.n_proj, self.max_h_in)
        if nbytes == 0:
            raise ValueError("bad workspace dimensions")
        # 128-byte aligned base: the library's layout aligns v relative to the base address
        raw = torch.zeros(nbytes + 128, dtype=torch.uint8, device=device)                   # zero-filled once
        skew = (-raw.data_ptr()) % 128
        self._raw = raw
        self.buf = raw[skew: skew + nbytes]
        self.nbytes = nbytes

    def v_view(self) -> torch.Tensor:
        """The fp32 shrink result ``v [n_proj, max_tokens, 64]`` inside the workspace
        (what tensor-parallel ranks sum between the shrink and the expand half)."""
        off, size = C.c_size_t(0), C.c_size_t(0)
        check(_lib.lib().b200_lora_workspace_v_region(self.max_tokens, self.n_proj, C.byref(off), C.byref(size)),
              "workspace_v_region")
        return self.buf[off.value: off.value + size.value].view(torch.float32).view(self.n_proj, self.max_tokens, 64)


def apply(projs: Sequence[Tuple[torch.Tensor, torch.Tensor, AdapterPool]], plan: LoraPlan, layer: int,
          workspace: LoraWorkspace, flags: int = 0, adapters: Optional[Adapters] = None, tp_ctx=None,
          skip_arrival: bool = False) -> None:
    """``y += scale_a * (x @ A_a^T) @ B_a^T`` for up to four projections ``(x, y, pool)`` of one layer.

    All pools must share one adapter table (ranks, scalings, layout).  With ``tp_ctx`` (the library's
    peer-exchange context of a tensor-parallel rank) the call is ``b200_lora_apply_tp``: ``x``, ``y`` and the
    pools are this rank's shards and the shrink result is summed over the ranks inside the call."""
    if not 1 <= len(projs) <= _lib.MAX_PROJ:
        raise ValueError("1..4 projections per call")
    arr = (Proj * len(projs))()
    io = None
    ydt = None
    for i, (x, y, pool) in enumerate(projs):
        _require_cuda(x, y, pool.wa)
        if x.dim() != 2 or y.dim() != 2 or x.shape[0] != y.shape[0]:
            raise ValueError("x and y must be [T, h] with the same T")
        if x.stride(1) != 1 or y.stride(1) != 1:
            raise ValueError("x and y rows must be contiguous")
        if x.shape[1] != pool.h_in or y.shape[1] != pool.h_out:
            raise ValueError("x/y widths do not match the pool")
        if x.dtype != pool.wa.dtype or x.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("x and the pool must both be fp16 or both bf16")
        if io is None:
            io, ydt = x.dtype, y.dtype
        if x.dtype != io or y.dtype != ydt or ydt not in (io, torch.float32):
            raise ValueError("all projections share the I/O dtype; y is that dtype or fp32")
        if x.shape[0] != plan.n_tokens:
            raise ValueError(f"the plan was built for {plan.n_tokens} rows, x has {x.shape[0]}")
        arr[i] = Proj(x.data_ptr(), y.data_ptr(), pool.wa.data_ptr(), pool.wb.data_ptr(),
                      x.stride(0), y.stride(0), pool.h_in, pool.h_out)
    ad = adapters if adapters is not None else adapters_of(projs[0][2])
    if tp_ctx is not None:
        check(_lib.lib().b200_lora_apply_tp(
            arr, len(projs), C.byref(ad), plan.buf.data_ptr(), plan.max_tokens, int(projs[0][0].shape[0]), int(layer),
            _DT[io], _DT[ydt], int(flags), workspace.buf.data_ptr(), workspace.nbytes, C.byref(tp_ctx),
            1 if skip_arrival else 0, _stream(projs[0][0].device)), "apply_tp")
        return
    check(_lib.lib().b200_lora_apply(
        arr, len(projs), C.byref(ad), plan.buf.data_ptr(), plan.max_tokens, int(projs[0][0].shape[0]), int(layer),
        _DT[io], _DT[ydt],
        int(flags), workspace.buf.data_ptr(), workspace.nbytes, _stream(projs[0][0].device)), "apply")


# ---- the reference's operator call ---------------------------------------------------------------
class _OpState:
    """Plan + workspace behind :func:`add_lora_bgmv` for one (device, stream), and what the plan
    was built from."""

    def __init__(self):
        self.batch: Optional[LoraBatch] = None
        self.dims = (0, 0, 0)            # capacity: tokens, adapters, h_in
        self.key = None
        self.ids_ref = None


_OP_STATE = {}


def invalidate_plan_cache() -> None:
    """Forget the plans :func:`add_lora_bgmv` keeps.  Needed only after the contents of an index
    tensor were changed behind torch's back (a custom kernel or a raw pointer write, which do not
    bump the tensor's version counter)."""
    for st in _OP_STATE.values():
        st.key, st.ids_ref = None, None


def _plan_for(ids: torch.Tensor, t: int, n: int, r: int, h_in: int, scale: float, ad: Adapters) -> LoraBatch:
    """The plan of ``ids``, rebuilt only when it can have changed.

    The reference's decode loop calls the op 3 x n_layers times per step with the SAME index tensor
    (lightllm/models/lora_gpu.py:138,150,162 with ``select_inds[bsz-1]``).  The plan depends on
    the ids, N, r and the scale only, so it is kept while the very same tensor object is passed
    again unmodified (torch's version counter) and rebuilt otherwise.  A plan built outside a
    CUDA-graph capture is never used inside one, nor one capture's plan in another: the capture's
    identifier is part of the key, so every graph contains the build of the plan it applies (its
    first call) and replays rebuild it from the index tensor's contents of the moment."""
    dev = ids.device
    skey = (dev.index, _stream(dev))
    st = _OP_STATE.get(skey)
    if st is None:
        st = _OP_STATE[skey] = _OpState()
    if st.batch is None or t > st.dims[0] or n > st.dims[1] or h_in > st.dims[2]:
        st.dims = (max(t, st.dims[0]), max(n, st.dims[1]), max(h_in, st.dims[2]))
        st.batch = LoraBatch(st.dims[0], st.dims[1], st.dims[2], 1, dev)
        st.key = None
    cap = C.c_ulonglong(0)
    check(_lib.lib().b200_lora_stream_capture_id(_stream(dev), C.byref(cap)), "stream_capture_id")
    key = (ids.data_ptr(), ids._version, ids.dtype, t, n, r, float(scale), cap.value)
    same = st.key == key and st.ids_ref is not None and st.ids_ref() is ids
    if not same:
        st.batch.plan.build(ids, ad)
        st.key = key
        st.ids_ref = weakref.ref(ids)
    return st.batch


def add_lora_bgmv(y: torch.Tensor, x: torch.Tensor, wa_T_all: torch.Tensor, wb_T_all: torch.Tensor,
                  indicies: torch.Tensor, layer_idx: int, scale: float) -> None:
    """In place ``y[t] += scale * (x[t] @ wa_T_all[i_t, layer]^T) @ wb_T_all[i_t, layer]^T``.

    Same arguments as the reference's decode op: ``y [T, h_out]``, ``x [T, h_in]``,
    ``wa_T_all [N, L, r, h_in]``, ``wb_T_all [N, L, h_out, r]`` contiguous fp16/bf16 CUDA
    tensors, ``indicies [T]`` int64 (or int32) CUDA tensor.  Returns ``None``.

    Two launches (shrink, expand) when the index tensor is the one of the previous call on this
    stream, unmodified; one more (the plan kernel) when it is new.
    """
    _require_cuda(y, x, wa_T_all, wb_T_all, indicies)
    if wa_T_all.dim() != 4 or wb_T_all.dim() != 4:
        raise ValueError("weight pools must be [N, L, r, h_in] and [N, L, h_out, r]")
    n, l, r, h_in = wa_T_all.shape
    h_out = wb_T_all.shape[2]
    if tuple(wb_T_all.shape) != (n, l, h_out, r):
        raise ValueError("wa_T_all / wb_T_all shapes disagree")
    t = x.shape[0]
    if tuple(x.shape) != (t, h_in) or tuple(y.shape) != (t, h_out) or indicies.numel() != t:
        raise ValueError("x, y, indicies shapes disagree with the pools")
    for ten in (y, x, wa_T_all, wb_T_all, indicies):
        if not ten.is_contiguous():
            raise ValueError("add_lora_bgmv needs contiguous tensors")
    if not (y.dtype == x.dtype == wa_T_all.dtype == wb_T_all.dtype) or x.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("fp16 or bf16 tensors of one dtype expected")
    if indicies.dtype not in (torch.int32, torch.int64):
        raise ValueError("indicies must be int32 or int64")
    ad = _adapters_struct(n, l, r, scale=scale)
    batch = _plan_for(indicies, t, n, r, h_in, scale, ad)
    arr = (Proj * 1)(Proj(x.data_ptr(), y.data_ptr(), wa_T_all.data_ptr(), wb_T_all.data_ptr(), h_in, h_out, h_in, h_out))
    check(_lib.lib().b200_lora_apply(
        arr, 1, C.byref(ad), batch.plan.buf.data_ptr(), batch.plan.max_tokens, t, int(layer_idx), _DT[x.dtype],
        _DT[x.dtype], _lib.NO_TENSOR, batch.workspace.buf.data_ptr(), batch.workspace.nbytes, _stream(x.device)),
        "add_lora_bgmv")


def add_lora_bgmv_once(y: torch.Tensor, x: torch.Tensor, wa_T_all: torch.Tensor, wb_T_all: torch.Tensor,
                       indicies: torch.Tensor, layer_idx: int, scale: float, workspace: torch.Tensor) -> None:
    """The same op as ONE C-ABI call (``b200_add_lora_bgmv``): plan and scratch live in the
    caller's ``workspace`` (any dtype, ``b200_add_lora_bgmv_workspace_bytes`` bytes or more, no
    preparation needed) and the plan is rebuilt by every call.  For bindings that cannot keep
    state between calls; tensors as for :func:`add_lora_bgmv`, shapes are not re-validated."""
    _require_cuda(y, x, wa_T_all, wb_T_all, indicies, workspace)
    n, l, r, h_in = wa_T_all.shape
    h_out = wb_T_all.shape[2]
    t = x.shape[0]
    check(_lib.lib().b200_add_lora_bgmv(
        y.data_ptr(), x.data_ptr(), wa_T_all.data_ptr(), wb_T_all.data_ptr(), indicies.data_ptr(),
        1 if indicies.dtype == torch.int64 else 0, t, h_in, h_out, n, l, r, int(layer_idx), float(scale),
        _DT[x.dtype], workspace.data_ptr(), workspace.numel() * workspace.element_size(), _stream(x.device)),
        "add_lora_bgmv")


def add_lora_bgmv_workspace_bytes(n_tokens: int, n_adapters: int, h_in: int) -> int:
    return int(_lib.lib().b200_add_lora_bgmv_workspace_bytes(n_tokens, n_adapters, h_in))


def add_lora_bgmv_static(y: torch.Tensor, x: torch.Tensor, wa_T_all: torch.Tensor, wb_T_all: torch.Tensor,
                         indicies: torch.Tensor, layer_idx: int, scale: float) -> None:
    """``add_lora_bgmv`` for callers that must not allocate device memory.

    Same arguments and result as :func:`add_lora_bgmv`, but the library's built-in scratch
    array is used instead of a workspace tensor, so nothing is allocated - not by this wrapper
    either.  Meant for processes that have given all of HBM to their KV cache or that may not
    call ``cudaMalloc`` after start-up.  Accepts at most 64 tokens, 1024 adapters and
    ``h_in <= 8192`` (larger calls raise).  All calls on a GPU share that one array: issue them
    on one stream, or order the streams, because overlapping calls race.  Make the first call
    on a device outside stream capture (it performs a one-time address lookup)."""
    _require_cuda(y, x, wa_T_all, wb_T_all, indicies)
    n, l, r, h_in = wa_T_all.shape
    h_out = wb_T_all.shape[2]
    t = x.shape[0]
    if tuple(wb_T_all.shape) != (n, l, h_out, r) or tuple(x.shape) != (t, h_in) or tuple(y.shape) != (t, h_out) \
            or indicies.numel() != t:
        raise ValueError("x, y, indicies shapes disagree with the pools")
    for ten in (y, x, wa_T_all, wb_T_all, indicies):
        if not ten.is_contiguous():
            raise ValueError("add_lora_bgmv_static needs contiguous tensors")
    if not (y.dtype == x.dtype == wa_T_all.dtype == wb_T_all.dtype) or x.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("fp16 or bf16 tensors of one dtype expected")
    if indicies.dtype not in (torch.int32, torch.int64):
        raise ValueError("indicies must be int32 or int64")
    check(_lib.lib().b200_add_lora_bgmv_static(
        y.data_ptr(), x.data_ptr(), wa_T_all.data_ptr(), wb_T_all.data_ptr(), indicies.data_ptr(),
        1 if indicies.dtype == torch.int64 else 0, t, h_in, h_out, n, l, r, int(layer_idx), float(scale),
        _DT[x.dtype], _stream(x.device)), "add_lora_bgmv_static")


def add_lora_bgmv_static_status(device=None) -> None:
    """Synchronises and raises if the last :func:`add_lora_bgmv_static` call on ``device`` saw an
    adapter id out of range (that call left ``y`` unchanged) or an expired device-side wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        check(_lib.lib().b200_add_lora_bgmv_static_status(_stream(dev)), "add_lora_bgmv_static_status")


class LoraBatch:
    """Plan + workspace of one batch, reused across layers and projections."""

    def __init__(self, max_tokens: int, n_adapters: int, max_h_in: int, n_proj: int = 4, device="cuda"):
        self.plan = LoraPlan(max_tokens, n_adapters, device)
        self.workspace = LoraWorkspace(max_tokens, n_proj, max_h_in, device)
        self.tiles = False

    def set_ids(self, ids: torch.Tensor, pool: AdapterPool, tiles: bool = False) -> "LoraBatch":
        """Per-token adapter ids.  ``tiles=True`` also launches the tcgen05 tile kernel for
        tall contiguous runs (mixed prefill + decode batches); decode batches leave it off."""
        self.plan.build(ids, adapters_of(pool))
        self.tiles = tiles
        return self

    def set_segments(self, seg_starts, seg_adapter, n_tokens, pool: AdapterPool, tiles: bool = True) -> "LoraBatch":
        self.plan.from_segments(seg_starts, seg_adapter, n_tokens, adapters_of(pool))
        self.tiles = tiles
        return self

    def apply(self, projs, layer: int, flags: int = 0, tp_ctx=None, skip_arrival: bool = False) -> None:
        if not self.tiles:
            flags |= _lib.NO_TENSOR
        apply(projs, self.plan, layer, self.workspace, flags, tp_ctx=tp_ctx, skip_arrival=skip_arrival)


def add_lora_bgmv_v2(y, x, pool: AdapterPool, indicies, layer_idx: int, flags: int = 0) -> None:
    """BGMV with per-adapter ranks and scalings taken from ``pool`` (dense or packed)."""
    b = LoraBatch(x.shape[0], pool.n_adapters, pool.h_in, 1, x.device).set_ids(indicies, pool)
    b.apply([(x, y, pool)], layer_idx, flags)


def add_lora_sgmv(y, x, pool: AdapterPool, seg_starts, seg_adapter, layer_idx: int, flags: int = 0) -> None:
    """SGMV on adapter-sorted rows: segment ``s`` = rows ``[seg_starts[s], seg_starts[s+1])``."""
    b = LoraBatch(x.shape[0], pool.n_adapters, pool.h_in, 1, x.device)
    b.set_segments(seg_starts, seg_adapter, x.shape[0], pool)
    b.apply([(x, y, pool)], layer_idx, flags)
