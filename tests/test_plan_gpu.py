"""GPU: the device-built segment table is bit-exact against the oracle's stable counting sort."""
import numpy as np
import pytest
import torch

import ae296_b200 as L
from ae296_b200.ops import _adapters_struct
from oracle import lora_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,N,seed", [(1, 1, 0), (2, 8, 1), (31, 8, 2), (33, 8, 3), (256, 128, 4), (1024, 7, 5),
                                      (1025, 3000, 6), (5000, 64, 7), (9336, 16, 8)])
@pytest.mark.parametrize("idt", [torch.int32, torch.int64])
def test_plan_matches_stable_sort(T, N, seed, idt):
    rng = np.random.default_rng(seed)
    p = 1.0 / np.arange(1, N + 1)
    ids = rng.choice(N, T, p=p / p.sum())
    plan = L.LoraPlan(T + 5, N)          # capacity larger than the batch
    plan.build(torch.from_numpy(ids).to("cuda", idt), _adapters_struct(N, 1, 16))
    perm, starts, adapters = plan.read()
    operm, ostarts, oadapters = O.stable_segments(ids, N)
    assert np.array_equal(perm, operm)
    assert np.array_equal(starts, ostarts)
    assert np.array_equal(adapters, oadapters)
    assert np.array_equal(perm, np.argsort(ids, kind="stable").astype(np.int32))


def test_plan_from_segments_round_trip_and_validation():
    lens = np.array([5, 1, 40, 200, 3])
    starts = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    adapters = np.array([4, 2, 9, 0, 7], np.int32)      # need not be sorted
    T = int(starts[-1])
    plan = L.LoraPlan(T, 10)
    ad = _adapters_struct(10, 1, 16)
    plan.from_segments(torch.from_numpy(starts).cuda(), torch.from_numpy(adapters).cuda(), T, ad)
    perm, s, a = plan.read()
    assert np.array_equal(perm, np.arange(T)) and np.array_equal(s, starts) and np.array_equal(a, adapters)
    bad = starts.copy()
    bad[2] = bad[1]                                       # empty segment
    plan.from_segments(torch.from_numpy(bad).cuda(), torch.from_numpy(adapters).cuda(), T, ad)
    with pytest.raises(L.LoraError) as e:
        plan.read()
    assert e.value.code == -10
