"""CPU: the timed CPU baseline really is the reference's worker, and it computes the oracle's answer.

Needs ``oracle/_ref/app.py`` (``python oracle/fetch_ref.py`` where the reference checkout is mounted);
skipped elsewhere."""
import numpy as np
import pytest
import torch

from oracle import lora_oracle as O
from oracle import ref_worker_baseline as RW

pytestmark = pytest.mark.skipif(not RW.available(), reason="oracle/_ref/app.py not fetched")


def test_reference_workers_answer_doorbells_with_the_oracles_result():
    hidden, max_len, ranks = 256, 4, [8, 16]
    pool = RW.ReferenceWorkerPool(hidden, max_len, ranks, seed=77)
    try:
        pool.wait_ready()
        rng = np.random.default_rng(0)
        x = rng.standard_normal((RW.ROWS_MAX, max_len, hidden)).astype(np.float16)
        pool.arr["shm_array"][:] = x
        pool.tkn_len[0] = 3
        # worker 0 (rank 8): rows 5 (q) and 7 (v); worker 1 (rank 16): row 2 (k)
        pool.run_jobs([[2 + 5, 402 + 7], [202 + 2]])
        for w, nm, row in ((0, "q", 5), (0, "v", 7), (1, "k", 2)):
            g = torch.Generator().manual_seed(77 + w)
            weights = {}
            for p in "qkvo":
                weights[p] = (torch.randn(hidden, ranks[w], generator=g) / np.sqrt(hidden),
                              torch.randn(ranks[w], hidden, generator=g) / np.sqrt(ranks[w]))
            want = O.cpu_worker(torch.from_numpy(x[row, :3]), *weights[nm])
            got = pool.arr[f"shm_out_{nm}"][row, :3]
            assert np.array_equal(got.view(np.uint16), want.numpy().view(np.uint16))
    finally:
        pool.close()


def test_timing_leg_reports_cores_and_scales_to_full_depth():
    from ae296_b200.workloads import make_workload
    wl = make_workload(0)
    res = RW.time_reference_workers(wl, layers=1, steps=2, warmup=1, n_workers=2)
    assert res["workers"] == 2 and res["cores"] >= 1
    assert res["tokens_per_s"] > 0 and "LoRAapp.run" in res["sample"]
