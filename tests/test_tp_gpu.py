"""GPU (one device): the split shrink -> sum -> expand sequence of the tensor-parallel path.

Both ranks' shards are run one after the other on the same GPU (kernels of different ranks
never wait on one another); their shrink partials are added where NCCL would sum them."""
import numpy as np
import pytest
import torch

import ae296_b200 as L
from ae296_b200 import _lib
from ae296_b200.tp import column_slice
from lora_testlib import TOL, Case, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tp", [2, 4])
def test_sharded_shrink_sum_expand_matches_oracle(tp):
    c = Case(50, 10, 2048, 1024, [16, 32, 64], "bf16", seed=31, zipf=1.0)
    shards = [c.pool.shard(tp, g) for g in range(tp)]
    batches = [L.LoraBatch(c.T, c.N, c.h_in // tp, 1).set_ids(c.ids_dev, shards[g]) for g in range(tp)]
    y = torch.zeros(c.T, c.h_out, dtype=torch.float32, device="cuda")
    for g in range(tp):
        batches[g].apply([(column_slice(c.x, tp, g), column_slice(y, tp, g), shards[g])], 1, _lib.ONLY_SHRINK)
    total = sum(b.workspace.v_view() for b in batches)       # what all_reduce(SUM) leaves on every rank
    for g in range(tp):
        batches[g].workspace.v_view().copy_(total)
        batches[g].apply([(column_slice(c.x, tp, g), column_slice(y, tp, g), shards[g])], 1, _lib.ONLY_EXPAND)
    torch.cuda.synchronize()
    for b in batches:
        b.workspace.check()
    assert rel_err(y.double().cpu().numpy(), c.oracle_delta(1)) <= TOL


def test_sharded_halves_with_tcgen05_tiles():
    """Prompts (tall runs) on the tile kernel, run as shrink half / sum / expand half."""
    tp = 2
    rng = np.random.default_rng(5)
    ids = np.concatenate([rng.integers(0, 6, 40), np.repeat([7, 3], [200, 90])]).astype(np.int32)
    c = Case(len(ids), 8, 1024, 512, [16, 32, 64], "fp16", seed=41, ids=ids)
    shards = [c.pool.shard(tp, g) for g in range(tp)]
    batches = [L.LoraBatch(c.T, c.N, c.h_in // tp, 1).set_ids(c.ids_dev, shards[g], tiles=True) for g in range(tp)]
    y = torch.zeros(c.T, c.h_out, dtype=torch.float32, device="cuda")
    for g in range(tp):
        batches[g].apply([(column_slice(c.x, tp, g), column_slice(y, tp, g), shards[g])], 0, _lib.ONLY_SHRINK)
    total = sum(b.workspace.v_view() for b in batches)
    for g in range(tp):
        batches[g].workspace.v_view().copy_(total)
        batches[g].apply([(column_slice(c.x, tp, g), column_slice(y, tp, g), shards[g])], 0, _lib.ONLY_EXPAND)
    torch.cuda.synchronize()
    for b in batches:
        b.workspace.check()
    assert rel_err(y.double().cpu().numpy(), c.oracle_delta(0)) <= TOL
