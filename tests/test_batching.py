"""Adapter-aware batching: request order, cost model (CPU) and the plan built from the router's tensors (GPU)."""
import numpy as np
import pytest
import torch

from ae296_b200.batching import delta_cost_us, order_by_adapter, plan_for_requests


def test_order_is_stable_and_groups_adapters():
    ids = [5, 2, 5, 0, 2, 5]
    o = order_by_adapter(ids)
    assert list(o) == [3, 1, 4, 0, 2, 5]
    assert list(np.asarray(ids)[o]) == [0, 2, 2, 5, 5, 5]


def test_cost_grows_with_distinct_adapters_and_ranks_not_with_repeats():
    base = delta_cost_us([16] * 128, [1] * 128, list(range(128)), 4096, 4096)
    same = delta_cost_us([16] * 128, [1] * 128, [0] * 128, 4096, 4096)
    big = delta_cost_us([64] * 128, [1] * 128, list(range(128)), 4096, 4096)
    assert same < base < big
    assert delta_cost_us([16], [1], [0], 4096, 4096) >= 4.0 * 4 * 32 * 0.5 - 1e-9      # the launch floor
    with pytest.raises(ValueError):
        delta_cost_us([16], [1, 2], [0], 64, 64)


@pytest.mark.gpu
def test_plan_from_router_tensors_prefill_and_decode():
    import ae296_b200 as L
    from lora_testlib import TOL, Case, rel_err
    lens = np.array([40, 5, 130, 33])
    lora_ids = np.array([3, 0, 3, 1], np.int32)                    # two requests share adapter 3
    ids_tok = np.repeat(lora_ids, lens)
    c = Case(int(lens.sum()), 4, 256, 256, [16, 32, 64, 16], "fp16", seed=4, ids=ids_tok)
    start = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)
    dev = lambda a: torch.from_numpy(np.asarray(a, np.int32)).cuda()
    batch = L.LoraBatch(c.T, 4, 256, 1)
    plan_for_requests(batch, c.pool, dev(lora_ids), dev(start), dev(lens), c.T, prefill=True)
    perm, s, a = batch.plan.read()
    assert np.array_equal(perm, np.arange(c.T)) and np.array_equal(a, lora_ids)
    assert np.array_equal(s, np.concatenate([start, [c.T]]))
    y = torch.zeros(c.T, 256, dtype=torch.float32, device="cuda")
    batch.apply([(c.x, y, c.pool)], 0)
    torch.cuda.synchronize()
    batch.workspace.check()
    assert rel_err(y.double().cpu().numpy(), c.oracle_delta(0)) <= TOL
    # decode: one token per request
    d = Case(4, 4, 256, 256, c.ranks, "fp16", seed=5, ids=lora_ids)
    b2 = L.LoraBatch(4, 4, 256, 1)
    plan_for_requests(b2, d.pool, dev(lora_ids), dev([0, 1, 2, 3]), dev([9, 9, 9, 9]), 4, prefill=False)
    assert rel_err(d.run(0, y_dtype=torch.float32, batch=b2).double().cpu().numpy(), d.oracle_delta(0)) <= TOL
    with pytest.raises(ValueError):
        plan_for_requests(b2, d.pool, dev(lora_ids).long(), dev([0, 1, 2, 3]), dev([1] * 4), 4, prefill=False)
