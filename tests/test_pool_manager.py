"""Adapter residency: slot allocation, eviction, pipelined loading, merge and remove.
CPU tests use CPU pools (copies are immediate); one GPU test loads on a side stream and runs the op."""
import numpy as np
import pytest
import torch

from ae296_b200.pool import AdapterPool
from ae296_b200.pool_manager import AdapterPoolManager, PoolFull, SlotAllocator, layer_groups


def host_adapter(L, r, h_in, h_out, seed, names=("q", "k"), dtype=torch.float16, pin=False):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for n in names:
        A = (torch.randn(L, r, h_in, generator=g) / np.sqrt(h_in)).to(dtype)
        B = (torch.randn(L, h_out, r, generator=g) / np.sqrt(r)).to(dtype)
        out[n] = (A.pin_memory(), B.pin_memory()) if pin else (A, B)
    return out


def dense_pools(n, L, h, R, device="cpu", names=("q", "k")):
    return {nm: AdapterPool.empty(n, L, h, h, np.full(n, R, np.int32), np.ones(n, np.float32), device=device, dense=True)
            for nm in names}


def test_allocator_hits_evicts_lru_and_respects_running_requests():
    al = SlotAllocator([16, 16, 16], any_rank=True)
    s = [al.acquire(u, 8)[0] for u in "abc"]
    assert sorted(s) == [0, 1, 2]
    with pytest.raises(PoolFull):
        al.acquire("d", 8)                               # all three are held
    al.release("b"); al.release("a")                     # b became idle first
    slot, resident, evicted = al.acquire("d", 8)
    assert (slot, resident, evicted) == (s[1], False, "b")
    assert al.acquire("a", 8) == (s[0], True, None)      # a hit revives an idle adapter
    al.release("a")
    assert al.remove("a") == s[0] and al.lookup("a") is None
    with pytest.raises(RuntimeError):
        al.remove("c")                                   # still running
    packed = SlotAllocator([8, 64], any_rank=False)      # packed pools: a slot keeps its rank
    assert packed.acquire("x", 64)[0] == 1
    with pytest.raises(PoolFull):
        packed.acquire("y", 64)


def test_layer_groups_match_the_swappers_for_32_layers():
    assert [list(g)[0:1] + list(g)[-1:] for g in layer_groups(32)] == [[0, 7], [8, 15], [16, 23], [24, 31]]
    assert [len(g) for g in layer_groups(40)] == [10, 10, 10, 10]
    assert [len(g) for g in layer_groups(2)] == [1, 1]


def test_load_merge_remove_on_cpu_pools():
    L, h, R = 8, 32, 16
    mgr = AdapterPoolManager(dense_pools(4, L, h, R), dense_pools(2, L, h, R))
    ads = [host_adapter(L, 16, h, h, 1), host_adapter(L, 8, h, h, 2)]          # the second has a smaller rank
    mgr.load_lora_prefill(ads)
    assert mgr.progress("prefill", 0) == 0 and mgr.use_gpu_pipeline(3)
    for b, w in enumerate(ads):
        for nm, (A, B) in w.items():
            r = A.shape[1]
            assert torch.equal(mgr.prefill[nm].wa[b, :, :r], A) and torch.equal(mgr.prefill[nm].wb[b, :, :, :r], B)
            assert not mgr.prefill[nm].wa[b, :, r:].any()                        # padding rows are zero
    assert [int(v) for v in mgr.prefill["q"].ranks_host] == [16, 8]
    slots = mgr.merge_lora_prefill(["u0", "u1"])
    assert len(set(slots)) == 2
    for b, s in enumerate(slots):
        assert torch.equal(mgr.decode["k"].wa[s], mgr.prefill["k"].wa[b])
        assert int(mgr.decode["k"].ranks_host[s]) == [16, 8][b] and int(mgr.decode["k"].ranks[s]) == [16, 8][b]
    assert mgr.merge_lora_prefill(["u0"]) == [slots[0]]                         # resident: same slot, one more reference
    mgr.release("u0"); mgr.release("u0"); mgr.release("u1")
    assert mgr.remove_lora(["u1"]) == [slots[1]]
    # four more adapters fill the pool and push the idle one out
    for i in range(3):
        mgr.acquire(f"n{i}", 16, host_adapter(L, 16, h, h, 10 + i))
    assert mgr.slots.lookup("u0") is not None
    mgr.acquire("n3", 16, host_adapter(L, 16, h, h, 20))
    assert mgr.slots.lookup("u0") is None
    with pytest.raises(KeyError):
        mgr.acquire("unknown", 16)                                              # not resident, nothing to load


@pytest.mark.gpu
def test_pipelined_load_on_a_side_stream_then_decode_matches_oracle():
    import ae296_b200 as Lb
    from lora_testlib import TOL, rel_err
    from oracle import lora_oracle as O
    L, h, R, N = 8, 512, 16, 6
    pools = dense_pools(N, L, h, R, device="cuda", names=("q",))
    mgr = AdapterPoolManager(pools)
    side = torch.cuda.Stream()
    held = {}
    for i in range(N):
        held[i] = host_adapter(L, 16, h, h, 100 + i, names=("q",), pin=True)
        slot = mgr.acquire(f"a{i}", 16, held[i], stream=side)
        assert slot == mgr.slots.lookup(f"a{i}")
        assert mgr.progress("decode", slot) in (0, 1, 2, 3, 4)
        mgr.wait("decode", slot)                       # the compute stream waits for the copies
    torch.cuda.synchronize()
    for i in range(N):
        s = mgr.slots.lookup(f"a{i}")
        assert mgr.progress("decode", s) == 0 and all(mgr.use_gpu_pipeline(l, "decode", s) for l in range(L))
    T = 40
    ids = np.random.default_rng(0).integers(0, N, T)
    slot_ids = torch.tensor([mgr.slots.lookup(f"a{i}") for i in ids], device="cuda")
    x = torch.randn(T, h, generator=torch.Generator().manual_seed(1)).half()
    y = torch.zeros(T, h, dtype=torch.float16, device="cuda")
    Lb.add_lora_bgmv(y, x.cuda(), pools["q"].wa, pools["q"].wb, slot_ids, 5, 1.0)
    torch.cuda.synchronize()
    want = O.lora_delta(x.double().numpy(), lambda a: held[a]["q"][0][5].double().numpy(),
                        lambda a: held[a]["q"][1][5].double().numpy(), ids, np.ones(N))
    rms = np.sqrt((want ** 2).mean())
    assert np.abs(y.double().cpu().numpy() - want).max() <= TOL * rms + np.abs(want).max() * 2.0 ** -10
