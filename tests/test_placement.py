"""CPU: placement by adapter - every token lands where its adapter lives, nothing is lost or
duplicated, and the oracle's delta of the re-assembled sub-batches equals the unsplit one."""
import os

import numpy as np
import pytest

from ae296_b200.placement import place_by_adapter
from ae296_b200.workloads import zipf_probs
from oracle import lora_oracle as O


@pytest.mark.parametrize("policy", ["mod", "balanced"])
@pytest.mark.parametrize("G", [1, 2, 4, 8])
def test_partition_is_exact(policy, G):
    rng = np.random.default_rng(G)
    N, T = 96, 700
    ids = rng.choice(N, T, p=zipf_probs(N, 1.0))
    pl = place_by_adapter(ids, G, N, policy)
    assert sorted(np.concatenate(pl.tokens).tolist()) == list(range(T))        # a partition of the batch
    assert sorted(np.concatenate(pl.adapters).tolist()) == list(range(N))      # and of the pool
    for g in range(G):
        assert np.all(np.diff(pl.tokens[g]) > 0)                                # original order kept
        assert np.array_equal(pl.adapters[g][pl.local_ids[g]], ids[pl.tokens[g]])
        assert np.all(pl.gpu_of_adapter[pl.adapters[g]] == g)
    if policy == "mod":
        assert np.array_equal(pl.gpu_of_adapter, np.arange(N) % G)


def test_balanced_beats_mod_on_skewed_popularity():
    rng = np.random.default_rng(0)
    N, T, G = 256, 4096, 8
    ids = rng.choice(N, T, p=zipf_probs(N, 1.2))
    worst = lambda pl: max(len(t) for t in pl.tokens)
    bal, mod = place_by_adapter(ids, G, N, "balanced"), place_by_adapter(ids, G, N, "mod")
    hottest = np.bincount(ids).max()
    assert worst(bal) <= worst(mod)
    assert worst(bal) <= max(hottest, int(np.ceil(T / G * 1.05)))              # within 5 % of even, or one hot adapter


def test_popularity_shapes_of_the_reference_traces():
    """Popularity vectors with the skew of the reference's trace files (maximum / minimum
    probability 0.14 / 2e-5 at 128 adapters ... 0.042 / 5e-6 at 512): placement stays balanced."""
    for n, pmax, pmin in ((128, 0.14, 2e-5), (256, 0.079, 1e-5), (512, 0.042, 5e-6)):
        p = np.geomspace(pmax, pmin, n)
        p /= p.sum()
        ids = np.random.default_rng(n).choice(n, 8192, p=p)
        pl = place_by_adapter(ids, 8, n, "balanced")
        loads = np.array([len(t) for t in pl.tokens])
        assert loads.max() <= max(np.bincount(ids).max(), 1.05 * 8192 / 8)


def test_sub_batches_reassemble_to_the_unsplit_delta():
    rng = np.random.default_rng(3)
    N, T, H, G = 12, 40, 32, 3
    ranks = rng.choice([4, 8], N)
    A = [rng.standard_normal((r, H)) for r in ranks]
    B = [rng.standard_normal((H, r)) for r in ranks]
    x = rng.standard_normal((T, H))
    ids = rng.integers(0, N, T)
    scal = 32.0 / ranks
    full = O.lora_delta(x, lambda a: A[a], lambda a: B[a], ids, scal)
    pl = place_by_adapter(ids, G, N, "balanced", resident_all=False)
    parts = []
    for g in range(G):
        ad = pl.adapters[g]
        if len(pl.tokens[g]) == 0:
            parts.append(np.zeros((0, H)))
            continue
        parts.append(O.lora_delta(x[pl.tokens[g]], lambda a: A[ad[a]], lambda a: B[ad[a]], pl.local_ids[g], scal[ad]))
    assert np.allclose(pl.scatter(parts, H, np.float64), full, rtol=0, atol=1e-12)
    with pytest.raises(ValueError):
        place_by_adapter([0, 12], 2, 12)


def test_balanced_by_bytes_evens_out_ragged_ranks():
    """With ranks given the policy balances what the kernels move: an adapter's weights once per work
    segment of eight tokens, a rank-64 adapter eight times a rank-8 one."""
    from ae296_b200.placement import adapter_load
    rng = np.random.default_rng(5)
    n, t, g = 512, 2048, 8
    ranks = rng.choice([8, 16, 32, 64], n).astype(np.int32)
    p = 1.0 / np.arange(1, n + 1)
    ids = rng.choice(n, t, p=p / p.sum()).astype(np.int32)
    cost = adapter_load(np.bincount(ids, minlength=n), ranks)
    spread = {}
    for name, kw in (("tokens", {}), ("bytes", {"ranks": ranks})):
        pl = place_by_adapter(ids, g, n, "balanced", **kw)
        loads = np.array([cost[a].sum() for a in pl.adapters])
        spread[name] = loads.max() / loads.mean()
        assert sorted(np.concatenate(pl.tokens).tolist()) == list(range(t))          # every token placed once
        again = place_by_adapter(ids, g, n, "balanced", **kw)
        assert np.array_equal(pl.gpu_of_adapter, again.gpu_of_adapter)               # deterministic
    assert spread["bytes"] <= 1.02 and spread["bytes"] < spread["tokens"]
    # an adapter with 9 tokens is two work segments; unused adapters cost nothing
    assert adapter_load(np.array([9, 0, 1]), [64, 64, 8]).tolist() == [2 * 64 + 1.5 * 9, 0.0, 8 + 1.5]
    with pytest.raises(ValueError):
        adapter_load(np.array([1, 2]), [8])
