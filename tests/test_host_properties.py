"""Property tests (hypothesis) of the host-side bookkeeping: the slot allocator of the adapter pool manager, the
placement of a batch over GPUs and the request order by adapter.  No GPU."""
import numpy as np
from hypothesis import given, settings, strategies as st

from ae296_b200.batching import order_by_adapter
from ae296_b200.placement import adapter_load, place_by_adapter
from ae296_b200.pool_manager import PoolFull, SlotAllocator, layer_groups

RANKS = [8, 16, 32, 64]


@settings(max_examples=150, deadline=None)
@given(slot_ranks=st.lists(st.sampled_from(RANKS), min_size=1, max_size=6), any_rank=st.booleans(),
       ops=st.lists(st.tuples(st.sampled_from(["acquire", "release", "remove"]), st.integers(0, 9), st.sampled_from(RANKS)),
                    max_size=60))
def test_slot_allocator_keeps_its_books(slot_ranks, any_rank, ops):
    """Whatever the sequence of calls: a slot has at most one adapter and an adapter one slot, the slot fits the
    adapter's rank, held adapters are never evicted, and free + used slots are all the slots."""
    al = SlotAllocator(slot_ranks, any_rank)
    held, rank_of = {}, {}
    for op, uid, rank in ops:
        if op == "acquire":
            rank = rank_of.get(uid, rank)                    # an adapter keeps its rank
            try:
                slot, resident, evicted = al.acquire(uid, rank)
            except PoolFull:
                assert al.lookup(uid) is None
                continue
            assert resident == (uid in rank_of)               # resident iff it was there before the call
            rank_of[uid] = rank
            assert not (resident and evicted is not None)    # a resident adapter evicts nobody
            assert (rank <= slot_ranks[slot]) if any_rank else (rank == slot_ranks[slot])
            if evicted is not None:
                assert held.get(evicted, 0) == 0 and al.lookup(evicted) is None
                rank_of.pop(evicted, None)
            held[uid] = held.get(uid, 0) + 1
        elif op == "release":
            if held.get(uid, 0) > 0:
                al.release(uid)
                held[uid] -= 1
            else:
                try:
                    al.release(uid)
                    assert False, "released an adapter nobody holds"
                except KeyError:
                    pass
        else:
            if al.lookup(uid) is not None and held.get(uid, 0) == 0:
                al.remove(uid)
                rank_of.pop(uid, None)
        # the books
        assert len(set(al.slot_of.values())) == len(al.slot_of)
        assert {al.uid_of[s] for s in al.slot_of.values()} == set(al.slot_of)
        assert sorted(list(al.slot_of.values()) + al.free) == list(range(len(slot_ranks)))
        for u, n in held.items():
            if n > 0:
                assert al.lookup(u) is not None and u not in al.lru
        assert all(al.refs.get(u, 0) == 0 for u in al.lru)


@settings(max_examples=100, deadline=None)
@given(n=st.integers(1, 40), g=st.integers(1, 8), t=st.integers(0, 300), seed=st.integers(0, 2 ** 16),
       policy=st.sampled_from(["mod", "balanced"]), with_ranks=st.booleans(), resident_all=st.booleans())
def test_placement_places_every_token_where_its_adapter_lives(n, g, t, seed, policy, with_ranks, resident_all):
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, n, t).astype(np.int32)
    ranks = rng.choice(RANKS, n).astype(np.int32) if with_ranks else None
    pl = place_by_adapter(ids, g, n, policy, resident_all=resident_all, ranks=ranks)
    assert pl.n_gpus == g
    seen = np.concatenate(pl.tokens) if t else np.zeros(0, np.int64)
    assert sorted(seen.tolist()) == list(range(t))                              # every token exactly once
    for gpu in range(g):
        toks, loc, mine = pl.tokens[gpu], pl.local_ids[gpu], pl.adapters[gpu]
        assert np.all(np.diff(toks) > 0)                                        # arrival order kept
        assert np.array_equal(mine[loc], ids[toks])                             # slot -> global adapter id
        assert np.all(pl.gpu_of_adapter[mine] == gpu)
    used = np.unique(ids)
    assert np.all(pl.gpu_of_adapter[used] >= 0)
    if resident_all:
        assert np.all(pl.gpu_of_adapter >= 0)
    if policy == "balanced" and t:
        cost = adapter_load(np.bincount(ids, minlength=n), ranks)
        loads = np.array([cost[a].sum() for a in pl.adapters])
        assert loads.max() - loads.min() <= cost.max() + 1e-9                   # longest-processing-time-first bound


@settings(max_examples=100, deadline=None)
@given(ids=st.lists(st.integers(0, 12), max_size=80))
def test_order_by_adapter_is_a_stable_sort(ids):
    order = order_by_adapter(ids)
    a = np.asarray(ids, np.int64)[order]
    assert sorted(order.tolist()) == list(range(len(ids)))
    assert np.all(np.diff(a) >= 0)
    for x in set(ids):
        pos = order[a == x]
        assert np.all(np.diff(pos) > 0)                                          # arrival order inside an adapter


@given(n_layers=st.integers(1, 100), n_groups=st.integers(1, 8))
def test_layer_groups_cover_the_layers_once(n_layers, n_groups):
    groups = layer_groups(n_layers, n_groups)
    flat = [l for gr in groups for l in gr]
    assert sorted(flat) == list(range(n_layers))
