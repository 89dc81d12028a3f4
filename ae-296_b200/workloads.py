"""Seeded synthetic workloads for the multi-LoRA delta path.

Five named workloads follow the shapes of a Llama-2 serving deployment that
applies a per-token LoRA delta to the q/k/v/o projections.  Only shapes, value
distributions and adapter-popularity skew are modelled; no dataset is used.

Generation rule (identical for every workload ``c``):

* integer draws use ``numpy.random.default_rng(2960 + c)`` in the order
  ranks -> adapter ids -> prompt lengths;
* tensors are drawn in fp32 as x, then per projection A then B, scaled to
  ``x ~ N(0,1)``, ``A ~ N(0, 1/h_in)``, ``B ~ N(0, 1/r)`` and cast to the I/O
  dtype; ``scaling = 32 / r``.

The weight pools use the *packed* layout of :mod:`pool` unless ``dense=True``.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np

SEED_BASE = 2960
LORA_ALPHA = 32.0


@dataclass
class Projection:
    name: str
    h_in: int
    h_out: int


@dataclass
class Workload:
    """Integer-level description of one batch; tensors come from ``materialize``."""

    cfg: int
    name: str
    dtype: str                      # "fp16" | "bf16"
    n_layers: int
    n_adapters: int
    ranks: np.ndarray               # int32 [N]
    ids: np.ndarray                 # int32 [T], adapter id per token
    projections: List[Projection]
    seq_lens: Optional[np.ndarray] = None   # prefill request lengths, if any
    n_decode: int = 0               # leading decode tokens (rest are prefill rows)
    description: str = ""

    @property
    def n_tokens(self) -> int:
        return int(self.ids.shape[0])

    @property
    def scalings(self) -> np.ndarray:
        return (LORA_ALPHA / self.ranks.astype(np.float64)).astype(np.float32)

    @property
    def r_max(self) -> int:
        return int(self.ranks.max())

    def distinct(self) -> np.ndarray:
        return np.unique(self.ids)

    # ---- algorithmic cost model -------------------------------------------------
    def bytes_per_layer(self, elem: int = 2, tp: int = 1, projs: Optional[Sequence[str]] = None) -> int:
        """Algorithmic HBM bytes of one layer over the selected projections.

        Per projection: every *used* adapter's A and B once, x once, y read and
        written (the op accumulates), ids as int32.  The ``[T, r]`` intermediate
        stays on chip and counts zero.  Under tensor parallelism the figure is
        per GPU: weights/tp, x columns/tp, y columns/tp.
        """
        used = self.distinct()
        rsum = int(self.ranks[used].sum())
        t = self.n_tokens
        total = 0
        for p in self.projections:
            if projs is not None and p.name not in projs:
                continue
            total += rsum * (p.h_in + p.h_out) * elem // tp
            total += t * p.h_in * elem // tp
            total += 2 * t * p.h_out * elem // tp
            total += 4 * t
        return total

    def flops_per_layer(self, projs: Optional[Sequence[str]] = None) -> int:
        r_tok = self.ranks[self.ids].astype(np.int64)
        total = 0
        for p in self.projections:
            if projs is not None and p.name not in projs:
                continue
            total += int((2 * r_tok * (p.h_in + p.h_out)).sum())
        return total

    def pool_bytes(self, elem: int = 2) -> int:
        rs = int(self.ranks.astype(np.int64).sum())
        return sum(rs * self.n_layers * (p.h_in + p.h_out) * elem for p in self.projections)

    def scaled(self, hidden_div: int = 1, n_layers: Optional[int] = None,
               max_tokens: Optional[int] = None) -> "Workload":
        """Same draws with smaller dims; used by parity tests that run the oracle."""
        projs = [Projection(p.name, max(p.h_in // hidden_div, 64), max(p.h_out // hidden_div, 64))
                 for p in self.projections]
        ids = self.ids if max_tokens is None else self.ids[:max_tokens]
        return dataclasses.replace(
            self, projections=projs, ids=ids.copy(),
            n_layers=self.n_layers if n_layers is None else n_layers,
            name=f"{self.name}/div{hidden_div}")


def zipf_probs(n: int, alpha: float) -> np.ndarray:
    p = 1.0 / np.arange(1, n + 1, dtype=np.float64) ** alpha
    return p / p.sum()


def _qkvo(h: int, kv: Optional[int] = None) -> List[Projection]:
    kv = h if kv is None else kv
    return [Projection("q", h, h), Projection("k", h, kv), Projection("v", h, kv), Projection("o", h, h)]


def make_workload(cfg: int) -> Workload:
    rng = np.random.default_rng(SEED_BASE + cfg)
    if cfg == 0:
        n, t = 8, 32
        ranks = np.full(n, 16, np.int32)
        ids = rng.integers(0, n, t).astype(np.int32)
        return Workload(0, "decode-7b-1layer", "fp16", 1, n, ranks, ids, _qkvo(4096), n_decode=t,
                        description="Llama-2-7B shapes, one layer, 32 decode tokens, 8 adapters rank 16")
    if cfg == 1:
        n, t = 128, 256
        ranks = rng.choice([8, 16, 32, 64], n).astype(np.int32)
        ids = rng.choice(n, t, p=zipf_probs(n, 1.0)).astype(np.int32)
        return Workload(1, "decode-7b-full", "fp16", 32, n, ranks, ids, _qkvo(4096), n_decode=t,
                        description="Llama-2-7B shapes, 32 layers, 256 decode tokens, 128 adapters ranks {8,16,32,64}, Zipf(1.0)")
    if cfg == 2:
        n = 16
        ranks = np.full(n, 32, np.int32)
        lens = rng.integers(128, 1025, n)
        ids = np.repeat(np.arange(n, dtype=np.int32), lens)
        return Workload(2, "prefill-7b-sgmv", "fp16", 32, n, ranks, ids, _qkvo(4096), seq_lens=lens,
                        description="Llama-2-7B shapes, 16 prompts U[128,1024] sorted by adapter, rank 32")
    if cfg == 3:
        n, nd, npf, lp = 256, 448, 4, 512
        ranks = rng.choice([16, 32, 64], n).astype(np.int32)
        draw = rng.choice(n, nd + npf, p=zipf_probs(n, 1.0)).astype(np.int32)
        ids = np.concatenate([draw[:nd], np.repeat(draw[nd:], lp)]).astype(np.int32)
        return Workload(3, "mixed-13b-tp", "bf16", 40, n, ranks, ids, _qkvo(5120),
                        seq_lens=np.full(npf, lp), n_decode=nd,
                        description="Llama-2-13B shapes, 448 decode tokens + 4x512 prefill, 256 adapters ranks {16,32,64}, Zipf(1.0)")
    if cfg == 4:
        n, t = 512, 512
        ranks = np.full(n, 64, np.int32)
        ids = rng.choice(n, t, p=zipf_probs(n, 1.2)).astype(np.int32)
        return Workload(4, "decode-70b-tp8", "bf16", 80, n, ranks, ids, _qkvo(8192, 1024), n_decode=t,
                        description="Llama-2-70B GQA shapes, 512 decode tokens, 512 adapters rank 64, Zipf(1.2)")
    raise ValueError(f"unknown workload {cfg}")


# ---- tensors ---------------------------------------------------------------------

def torch_dtype(name: str):
    import torch
    return {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}[name]


def materialize(wl: Workload, device="cpu", layers: Optional[int] = None, dense: bool = False,
                device_rng: bool = False, projs: Optional[Sequence[str]] = None):
    """Draw x and the A/B pools of ``wl``.

    Returns ``(xs, pools)``: ``xs[name]`` is the ``[T, h_in]`` activation of a
    projection (q/k/v share one tensor, o has its own) and ``pools[name]`` an
    :class:`~pool.AdapterPool`.  ``device_rng=True`` draws on ``device`` (used
    at full size where a CPU draw of tens of GB would dominate the run); the
    CPU draw is the pinned one used for parity fixtures.
    """
    import torch
    from .pool import AdapterPool

    dt = torch_dtype(wl.dtype)
    n_layers = wl.n_layers if layers is None else layers
    gen_dev = device if device_rng else "cpu"
    g = torch.Generator(device=gen_dev)
    g.manual_seed(SEED_BASE + wl.cfg)
    t = wl.n_tokens

    def randn(*shape):
        return torch.randn(*shape, generator=g, device=gen_dev, dtype=torch.float32)

    xs = {}
    x_qkv = randn(t, wl.projections[0].h_in).to(dt).to(device)
    pools = {}
    for p in wl.projections:
        if projs is not None and p.name not in projs:
            continue
        if p.name == "o":
            xs[p.name] = randn(t, p.h_in).to(dt).to(device)
        else:
            xs[p.name] = x_qkv
        pool = AdapterPool.empty(wl.n_adapters, n_layers, p.h_in, p.h_out, wl.ranks, wl.scalings,
                                 dtype=dt, device=device, dense=dense)
        for a in range(wl.n_adapters):
            r = int(wl.ranks[a])
            A = randn(n_layers, r, p.h_in) * (1.0 / np.sqrt(p.h_in))
            B = randn(n_layers, p.h_out, r) * (1.0 / np.sqrt(r))
            pool.set_adapter(a, A.to(dt), B.to(dt))
        pools[p.name] = pool
    return xs, pools


def materialize_device(wl: Workload, device, layers: Optional[int] = None, projs: Optional[Sequence[str]] = None,
                       per_layer_x: bool = True):
    """Full-size pools drawn directly on ``device`` (seeded), for the benchmark.

    One ``normal_`` fills each flat packed pool, then every adapter's B block is scaled to
    ``N(0, 1/r_a)``.  Returns ``(x_qkv [L,T,h], x_o [L,T,h], pools)``; ``per_layer_x=False``
    gives ``L = 1``.
    """
    import torch
    from .pool import AdapterPool

    dt = torch_dtype(wl.dtype)
    n_layers = wl.n_layers if layers is None else layers
    g = torch.Generator(device=device)
    g.manual_seed(SEED_BASE + wl.cfg)
    t = wl.n_tokens
    lx = n_layers if per_layer_x else 1
    h = wl.projections[0].h_in
    x_qkv = torch.empty(lx, t, h, dtype=dt, device=device).normal_(0, 1, generator=g)
    x_o = torch.empty(lx, t, h, dtype=dt, device=device).normal_(0, 1, generator=g)
    pools = {}
    for p in wl.projections:
        if projs is not None and p.name not in projs:
            continue
        pool = AdapterPool.empty(wl.n_adapters, n_layers, p.h_in, p.h_out, wl.ranks, wl.scalings,
                                 dtype=dt, device=device, dense=False)
        pool.wa.normal_(0, 1.0 / float(np.sqrt(p.h_in)), generator=g)
        pool.wb.normal_(0, 1.0, generator=g)
        for a in range(wl.n_adapters):
            pool.b_block(a).mul_(1.0 / float(np.sqrt(wl.ranks[a])))
        pools[p.name] = pool
    return x_qkv, x_o, pools
