"""CPU: the seeded workloads reproduce the figures the roofline arithmetic is based on."""
import numpy as np
import torch

from ae296_b200.workloads import make_workload, materialize
from ae296_b200.pool import AdapterPool
from oracle import lora_oracle as O


def test_pinned_draws():
    w1 = make_workload(1)
    assert w1.n_tokens == 256 and len(w1.distinct()) == 69 and int(w1.ranks[w1.distinct()].sum()) == 2280
    assert w1.bytes_per_layer() == 174_592_000          # 174.6 MB per layer, all four projections
    assert w1.bytes_per_layer() * 32 == 5_586_944_000
    w2 = make_workload(2)
    assert w2.seq_lens.tolist() == [537, 824, 517, 341, 399, 247, 211, 845, 932, 822, 305, 334, 379, 996, 658, 989]
    assert w2.n_tokens == 9336
    assert len(make_workload(3).distinct()) == 130 and make_workload(3).n_tokens == 2496
    w4 = make_workload(4)
    assert len(w4.distinct()) == 119 and [p.h_out for p in w4.projections] == [8192, 1024, 1024, 8192]
    assert abs(make_workload(0).bytes_per_layer() - 11_535_000) < 2000


def test_pool_layouts_hold_the_same_adapters_and_shard_consistently():
    wl = make_workload(1).scaled(hidden_div=32, n_layers=2, max_tokens=16)
    xs, packed = materialize(wl, "cpu", projs=["q"])
    _, dense = materialize(wl, "cpu", dense=True, projs=["q"])
    p, d = packed["q"], dense["q"]
    for a in (0, 5, 127):
        assert torch.equal(p.a_block(a), d.a_block(a)) and torch.equal(p.b_block(a), d.b_block(a))
    # tensor-parallel shards: A along h_in, B along h_out; partial sums add up to the whole
    x = xs["q"].double().numpy()
    ids = wl.ids
    full = O.lora_delta(x, lambda a: p.a_block(a)[1].double().numpy(), lambda a: p.b_block(a)[1].double().numpy(),
                        ids, wl.scalings.astype(np.float64))
    tp = 2
    shards = [p.shard(tp, g) for g in range(tp)]
    hi, ho = p.h_in // tp, p.h_out // tp
    for a in np.unique(ids):
        rows = np.nonzero(ids == a)[0]
        v = sum(x[rows][:, g * hi:(g + 1) * hi] @ shards[g].a_block(int(a))[1].double().numpy().T for g in range(tp))
        for g in range(tp):
            y = wl.scalings[a] * (v @ shards[g].b_block(int(a))[1].double().numpy().T)
            assert np.allclose(y, O.tp_column_slice(full[rows], tp, g), rtol=1e-12, atol=1e-12)
