"""GPU, two ranks over NCCL: ``TPLora`` itself (shrink half, all-reduce of the fp32 partials, expand
half) against the oracle's column slice, one process per GPU.  Skipped where fewer than two GPUs
are visible; the single-GPU tests cover the same kernels with the ranks run one after the other."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, q, exchange="nccl", fail_rank=-1):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [root, os.path.join(root, "tests")]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from ae296_b200.tp import TPLora, column_slice
        from lora_testlib import TOL, rel_err, shared_x_cases
        from oracle import lora_oracle as O
        rng = np.random.default_rng(9)
        ids = np.concatenate([rng.integers(0, 10, 60), np.repeat([3, 8], [160, 70])]).astype(np.int32)
        dev = f"cuda:{rank}"
        cases = shared_x_cases(len(ids), 12, 2048, (2048, 512, 512), [16, 32, 64], "bf16", ids, seed=55)
        for c in cases:                        # Case puts its tensors on the current device
            assert c.x.device.index == rank
        shards = [c.pool.shard(world, rank) for c in cases]
        errs = []
        if fail_rank >= 0:
            # rank `fail_rank` withholds its arrival signal in the second apply: its peers' bounded wait runs
            # out and shows as a status; nobody hangs, and the process group is torn down normally afterwards
            import ae296_b200 as L
            eng = TPLora(len(ids), 12, 2048 // world, 3, world, rank, None, dev, exchange="peer").set_ids(cases[0].ids_dev, shards[0])
            ys = [torch.zeros(len(ids), c.h_out // world, dtype=torch.float32, device=dev) for c in cases]
            xs = column_slice(cases[0].x, world, rank)
            eng.apply([(xs, y, sh) for y, sh in zip(ys, shards)], 0)
            torch.cuda.synchronize()
            eng.batch.workspace.check()
            dist.barrier()
            eng.apply([(xs, y, sh) for y, sh in zip(ys, shards)], 0, skip_arrival=(rank == fail_rank))
            torch.cuda.synchronize()
            code = 0
            try:
                eng.batch.workspace.check()
            except L.LoraError as e:
                code = e.code
            q.put((rank, code))
            dist.barrier()
            eng.close()
            return
        for tiles in (False, True):
            eng = TPLora(len(ids), 12, 2048 // world, 3, world, rank, None, dev, exchange=exchange).set_ids(cases[0].ids_dev, shards[0], tiles=tiles)
            ys = [torch.zeros(len(ids), c.h_out // world, dtype=torch.float32, device=dev) for c in cases]
            xs = column_slice(cases[0].x, world, rank)
            for _ in range(2):                 # a second apply accumulates: y = 2 * delta
                eng.apply([(xs, y, sh) for y, sh in zip(ys, shards)], 0)
            torch.cuda.synchronize()
            eng.batch.workspace.check()
            for c, y in zip(cases, ys):
                want = O.tp_column_slice(2 * c.oracle_delta(0), world, rank)
                full_rms = float(np.sqrt(((2 * c.oracle_delta(0)) ** 2).mean()))
                errs.append(float(np.abs(y.double().cpu().numpy() - want).max() / full_rms))
            eng.close()
        if exchange == "peer":
            # the exchange as a call of its own between the two halves (b200_lora_tp_exchange: every row, all 64 columns)
            from ae296_b200 import _lib
            eng = TPLora(len(ids), 12, 2048 // world, 3, world, rank, None, dev, exchange="peer").set_ids(cases[0].ids_dev, shards[0])
            ys = [torch.zeros(len(ids), c.h_out // world, dtype=torch.float32, device=dev) for c in cases]
            xs = column_slice(cases[0].x, world, rank)
            projs = [(xs, y, sh) for y, sh in zip(ys, shards)]
            eng.batch.apply(projs, 0, _lib.ONLY_SHRINK)
            eng.peer.exchange(eng.batch.workspace, len(ids), len(projs))
            eng.batch.apply(projs, 0, _lib.ONLY_EXPAND)
            torch.cuda.synchronize()
            eng.batch.workspace.check()
            for c, y in zip(cases, ys):
                want = O.tp_column_slice(c.oracle_delta(0), world, rank)
                full_rms = float(np.sqrt((c.oracle_delta(0) ** 2).mean()))
                errs.append(float(np.abs(y.double().cpu().numpy() - want).max() / full_rms))
            eng.close()
        q.put((rank, max(errs)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tplora_two_nccl_ranks_match_oracle_column_slices():
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert set(res) == {0, 1} and max(res.values()) <= 2e-3, res


def _spawn(world, **kw):
    import torch.multiprocessing as mp
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q), kwargs=kw) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    return res


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("via_owner", ["0", "1"])
def test_tplora_peer_exchange_matches_oracle_column_slices(via_owner, monkeypatch):
    """The library's own exchange over peer memory instead of the NCCL all-reduce: every rank sending to every
    rank, and the route through an owning rank that large exchanges take from four ranks on (forced here)."""
    monkeypatch.setenv("B200_LORA_TP_VIA_OWNER", via_owner)     # read once per process: the spawned ranks inherit it
    res = _spawn(2, exchange="peer")
    assert set(res) == {0, 1} and max(res.values()) <= 2e-3, res


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_that_never_arrives_is_a_timeout_status_not_a_hang():
    res = _spawn(2, fail_rank=1)
    assert res[0] == -11, res            # rank 0 waited for rank 1's signal and gave up
    assert res[1] == 0, res              # rank 1 itself saw rank 0 arrive
