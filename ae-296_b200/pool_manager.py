"""Adapter residency: which adapter sits in which slot of the HBM pools, and how it gets there.

Counterpart of the pool handling spread over the reference's ``Lora_GPU`` and its swapper sidecar:

* ``load_lora_prefill`` (lightllm/models/lora_gpu.py:165-188): adapters of a prefill batch copied host -> HBM
  into the prefill slots on demand;
* the swapper's pipelined copy (shared_tensor.py:111-152): an adapter arrives layer group by layer group,
  groups 1, 2, 3 first and group 0 last, and publishes ``progress`` 1 (started) -> 2 -> 3 -> 4 -> 0 (all
  there), which ``use_gpu_pipeline(layer_id)`` (lora_gpu.py:298-321) turns into "may this layer already take
  the GPU path";
* ``merge_lora_prefill`` (lora_gpu.py:202-217): prefill slots copied into decode slots once the prompt is done
  (the reference picks the decode slots at random; here an allocator hands out free slots and evicts the least
  recently used adapter that no running request holds);
* ``remove_lora`` (lora_gpu.py:229-242): the reference compacts the pool by shifting every later slot down one;
  here a slot is simply returned to the allocator, no bytes move.

One manager drives several pools (q, k, v, o ...) that share the slot numbering and the adapter table.
Copies are plain ``copy_`` calls: host -> device from pinned memory on the stream the caller names,
device -> device for the merge.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .pool import AdapterPool


class PoolFull(RuntimeError):
    """Every slot that could take the adapter is held by a running request."""


@dataclass
class _Load:
    events: List[Optional["torch.cuda.Event"]]      # one per layer group, in copy order
    order: List[int]                                # group index of each event
    done_groups: int = 0


class SlotAllocator:
    """Adapter uid <-> slot, with reference counts of running requests and LRU eviction."""

    def __init__(self, slot_ranks: Sequence[int], any_rank: bool):
        self.slot_ranks = [int(r) for r in slot_ranks]
        self.any_rank = any_rank                     # dense pools: a slot takes any rank up to the pool's R
        self.slot_of: Dict[Hashable, int] = {}
        self.uid_of: Dict[int, Hashable] = {}
        self.refs: Dict[Hashable, int] = {}
        self.lru: "OrderedDict[Hashable, None]" = OrderedDict()      # resident and unreferenced, oldest first
        self.free: List[int] = list(range(len(self.slot_ranks)))

    def lookup(self, uid) -> Optional[int]:
        return self.slot_of.get(uid)

    def _fits(self, slot: int, rank: int) -> bool:
        return rank <= self.slot_ranks[slot] if self.any_rank else rank == self.slot_ranks[slot]

    def acquire(self, uid, rank: int) -> Tuple[int, bool, Optional[Hashable]]:
        """Returns ``(slot, resident, evicted_uid)``.  ``resident`` says the adapter was already there
        (nothing to load); otherwise the caller loads it into ``slot``."""
        if uid in self.slot_of:
            self.refs[uid] = self.refs.get(uid, 0) + 1
            self.lru.pop(uid, None)
            return self.slot_of[uid], True, None
        slot, evicted = None, None
        for i, s in enumerate(self.free):
            if self._fits(s, rank):
                slot = self.free.pop(i)
                break
        if slot is None:
            for victim in self.lru:                  # least recently used first
                if self._fits(self.slot_of[victim], rank):
                    evicted = victim
                    break
            if evicted is None:
                raise PoolFull(f"no free or evictable slot for an adapter of rank {rank}")
            slot = self.slot_of.pop(evicted)
            del self.uid_of[slot]
            del self.lru[evicted]
            self.refs.pop(evicted, None)
        self.slot_of[uid] = slot
        self.uid_of[slot] = uid
        self.refs[uid] = 1
        return slot, False, evicted

    def release(self, uid) -> None:
        """A request that used the adapter has finished; the adapter stays resident until evicted."""
        n = self.refs.get(uid, 0) - 1
        if n < 0:
            raise KeyError(f"adapter {uid!r} is not held")
        self.refs[uid] = n
        if n == 0:
            self.lru[uid] = None
            self.lru.move_to_end(uid)

    def remove(self, uid) -> int:
        """Drops the adapter and frees its slot at once."""
        if self.refs.get(uid, 0) > 0:
            raise RuntimeError(f"adapter {uid!r} is held by a running request")
        slot = self.slot_of.pop(uid)
        del self.uid_of[slot]
        self.lru.pop(uid, None)
        self.refs.pop(uid, None)
        self.free.append(slot)
        return slot


def layer_groups(n_layers: int, n_groups: int = 4) -> List[range]:
    """The swapper's groups: ``n_groups`` equal runs of layers (8 each for 32 layers)."""
    per = -(-n_layers // n_groups)
    return [range(g * per, min(n_layers, (g + 1) * per)) for g in range(n_groups) if g * per < n_layers]


class AdapterPoolManager:
    def __init__(self, decode_pools: Dict[str, AdapterPool], prefill_pools: Optional[Dict[str, AdapterPool]] = None,
                 n_groups: int = 4):
        self.decode = decode_pools
        self.prefill = prefill_pools or {}
        first = next(iter(decode_pools.values()))
        self.n_layers = first.n_layers
        self.groups = layer_groups(self.n_layers, n_groups)
        # the swapper copies groups 1.. first and group 0 last (shared_tensor.py:111-152)
        self.group_order = list(range(1, len(self.groups))) + [0]
        self.slots = SlotAllocator(first.ranks_host, any_rank=not first.packed)
        self._loads: Dict[Tuple[str, int], _Load] = {}

    # ---- loading ------------------------------------------------------------------------------------
    def _copy_group(self, pool: AdapterPool, slot: int, A: torch.Tensor, B: torch.Tensor, layers: range, rank: int):
        a_dst, b_dst = pool.a_block(slot), pool.b_block(slot)
        if not pool.packed:                           # dense slot: the adapter's rows / columns, zero beyond its rank
            a_dst, b_dst = pool.wa[slot], pool.wb[slot]
            if rank < pool.r_pool:
                a_dst[layers.start:layers.stop, rank:].zero_()
                b_dst[layers.start:layers.stop, :, rank:].zero_()
            a_dst, b_dst = a_dst[:, :rank], b_dst[:, :, :rank]
        a_dst[layers.start:layers.stop].copy_(A[layers.start:layers.stop], non_blocking=True)
        b_dst[layers.start:layers.stop].copy_(B[layers.start:layers.stop], non_blocking=True)

    def load(self, which: str, slot: int, weights: Dict[str, Tuple[torch.Tensor, torch.Tensor]],
             stream: Optional["torch.cuda.Stream"] = None, pipelined: bool = True) -> None:
        """Copies one adapter (``weights[name] = (A [L, r, h_in], B [L, h_out, r])``, pinned host tensors for an
        asynchronous copy) into ``slot`` of the ``which`` ("decode" | "prefill") pools, layer group by layer
        group in the swapper's order, and records an event after each group."""
        pools = self.decode if which == "decode" else self.prefill
        rank = int(next(iter(weights.values()))[0].shape[1])
        on_gpu = next(iter(pools.values())).wa.is_cuda
        order = self.group_order if pipelined else list(range(len(self.groups)))
        load = _Load(events=[], order=order)
        ctx = torch.cuda.stream(stream) if (on_gpu and stream is not None) else _null()
        with ctx:
            for g in order:
                for name, (A, B) in weights.items():
                    self._copy_group(pools[name], slot, A, B, self.groups[g], rank)
                if on_gpu:
                    ev = torch.cuda.Event()
                    ev.record(stream if stream is not None else torch.cuda.current_stream())
                    load.events.append(ev)
                else:
                    load.events.append(None)
        for pool in pools.values():
            if not pool.packed and int(pool.ranks_host[slot]) != rank:
                pool.ranks_host[slot] = rank
                pool.ranks[slot] = rank
        self._loads[(which, slot)] = load

    def progress(self, which: str, slot: int) -> int:
        """The swapper's progress word for a slot: 1 started, 2 / 3 / 4 after the second / third / fourth
        layer group, 0 when the whole adapter is there (or nothing is being loaded)."""
        load = self._loads.get((which, slot))
        if load is None:
            return 0
        while load.done_groups < len(load.events):
            ev = load.events[load.done_groups]
            if ev is not None and not ev.query():
                break
            load.done_groups += 1
        if load.done_groups == len(load.events):
            del self._loads[(which, slot)]
            return 0
        return 1 + load.done_groups

    def use_gpu_pipeline(self, layer_id: int, which: str = "prefill", slot: int = 0) -> bool:
        """May ``layer_id`` take the GPU path for this slot yet (lightllm/models/lora_gpu.py:298-321)."""
        load = self._loads.get((which, slot))
        p = self.progress(which, slot)
        if p == 0:
            return True
        done = set(load.order[:load.done_groups])
        for g, layers in enumerate(self.groups):
            if layer_id in layers:
                return g in done
        raise IndexError("layer out of range")

    def wait(self, which: str, slot: int, stream: Optional["torch.cuda.Stream"] = None) -> None:
        """Makes ``stream`` (default: the current one) wait for the slot's outstanding copies."""
        load = self._loads.get((which, slot))
        if load is None:
            return
        for ev in load.events[load.done_groups:]:
            if ev is not None:
                (stream or torch.cuda.current_stream()).wait_event(ev)

    # ---- the reference's calls ----------------------------------------------------------------------
    def load_lora_prefill(self, adapters: Sequence[Dict[str, Tuple[torch.Tensor, torch.Tensor]]],
                          stream: Optional["torch.cuda.Stream"] = None) -> None:
        """Request ``b`` of the prefill batch gets prefill slot ``b`` (lightllm/models/lora_gpu.py:165-188)."""
        for b, w in enumerate(adapters):
            self.load("prefill", b, w, stream)

    def merge_lora_prefill(self, uids: Sequence[Hashable], ranks: Optional[Sequence[int]] = None) -> List[int]:
        """Prefill slot ``i`` becomes resident as adapter ``uids[i]`` in a decode slot; returns the decode slots
        (lightllm/models/lora_gpu.py:202-217).  An adapter that is resident already is not copied again."""
        out = []
        for i, uid in enumerate(uids):
            pool0 = next(iter(self.prefill.values()))
            rank = int(ranks[i]) if ranks is not None else int(pool0.ranks_host[i])
            slot, resident, _ = self.slots.acquire(uid, rank)
            if not resident:
                self.wait("prefill", i)
                for name, dst in self.decode.items():
                    src = self.prefill[name]
                    if dst.packed:
                        dst.a_block(slot).copy_(src.a_block(i))
                        dst.b_block(slot).copy_(src.b_block(i))
                    else:
                        dst.wa[slot].copy_(src.wa[i])
                        dst.wb[slot].copy_(src.wb[i])
                        if int(dst.ranks_host[slot]) != rank:
                            dst.ranks_host[slot] = rank
                            dst.ranks[slot] = rank
            out.append(slot)
        return out

    def acquire(self, uid, rank: int, weights=None, stream=None) -> int:
        """Decode slot of adapter ``uid`` for one more running request; loads it when it is not resident."""
        if weights is None and self.slots.lookup(uid) is None:
            raise KeyError(f"adapter {uid!r} is not resident and no weights were given")
        slot, resident, _ = self.slots.acquire(uid, rank)
        if not resident:
            self.load("decode", slot, weights, stream)
        return slot

    def release(self, uid) -> None:
        self.slots.release(uid)

    def remove_lora(self, rm_uids: Sequence[Hashable]) -> List[int]:
        """Frees the slots of finished adapters (lightllm/models/lora_gpu.py:229-242)."""
        return [self.slots.remove(u) for u in rm_uids]


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
