"""CPU, 2 gloo ranks: the tensor-parallel decomposition and its one collective.

Each rank computes its shrink partial with the oracle's arithmetic on its own shard of A and x,
the partials are summed with the same helper the GPU path uses, and each rank's expand with its
shard of B must reproduce its column slice of the unsharded answer."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ae296_b200.tp import allreduce_partials, column_slice
from ae296_b200.workloads import make_workload, materialize
from oracle import lora_oracle as O


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    wl = make_workload(3).scaled(hidden_div=40, n_layers=1, max_tokens=48)      # bf16, mixed ranks
    xs, pools = materialize(wl, "cpu", projs=["q"])
    pool = pools["q"]
    shard = pool.shard(world, rank)
    x = column_slice(xs["q"], world, rank).double().numpy()
    ids, t = wl.ids, wl.n_tokens
    v = torch.zeros(t, 64, dtype=torch.float64)
    for a in np.unique(ids):
        rows = np.nonzero(ids == a)[0]
        r = int(wl.ranks[a])
        v[rows, :r] = torch.from_numpy(x[rows] @ shard.a_block(int(a))[0].double().numpy().T)
    allreduce_partials(v)                                   # the one exchange of the path
    y = np.zeros((t, shard.h_out))
    for a in np.unique(ids):
        rows = np.nonzero(ids == a)[0]
        r = int(wl.ranks[a])
        y[rows] = wl.scalings[a] * (v[rows, :r].numpy() @ shard.b_block(int(a))[0].double().numpy().T)
    full = O.lora_delta(xs["q"].double().numpy(), lambda a: pool.a_block(a)[0].double().numpy(),
                        lambda a: pool.b_block(a)[0].double().numpy(), ids, wl.scalings.astype(np.float64))
    err = float(np.abs(y - O.tp_column_slice(full, world, rank)).max())
    q.put((rank, err))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_tensor_parallel_decomposition():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert set(res) == {0, 1} and max(res.values()) < 1e-9
