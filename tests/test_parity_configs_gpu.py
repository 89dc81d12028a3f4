"""GPU parity at the shapes of the five benchmark workloads that the smaller tests do not reach,
against the float64 oracle and against vectors made by the reference's own CPU worker.

Every case goes through the C ABI.  fp32 outputs are compared with the oracle (max-abs-error
<= 2e-3 x RMS of the exact output), 16-bit outputs must be the single rounding of the fp32 result,
and a second run must be bit-identical."""
import ctypes as C
import os
import sys

import numpy as np
import pytest
import torch

import ae296_b200 as L
from ae296_b200 import _lib
from ae296_b200.tp import column_slice
from ae296_b200.workloads import make_workload
from lora_testlib import TOL, Case, raw_apply, rel_err, shared_x_cases
from oracle import lora_oracle as O

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def apply_all(cases, batch, layer, y_dtype, flags=0):
    ys = [torch.zeros(c.T, c.h_out, dtype=y_dtype, device="cuda") for c in cases]
    batch.apply([(c.x, y, c.pool) for c, y in zip(cases, ys)], layer, flags)
    torch.cuda.synchronize()
    batch.workspace.check()
    return ys


def test_mixed_13b_batch_full_width_three_projections():
    """Workload 3 as drawn: hidden 5120 (2.5 super-chunks of 2048 columns), bf16, ranks {16, 32, 64},
    448 decode tokens followed by four 512-token prompts, per-token ids; prompts on the tcgen05
    tiles, decode tokens on the BGMV kernels, q/k/v in one apply."""
    wl = make_workload(3)
    cases = shared_x_cases(wl.n_tokens, wl.n_adapters, 5120, (5120, 5120, 5120), wl.ranks, "bf16", wl.ids, seed=2963)
    batch = L.LoraBatch(wl.n_tokens, wl.n_adapters, 5120, 3).set_ids(cases[0].ids_dev, cases[0].pool, tiles=True)
    y32 = apply_all(cases, batch, 0, torch.float32)
    y16 = apply_all(cases, batch, 0, torch.bfloat16)
    for c, a, b in zip(cases, y32, y16):
        assert rel_err(a.double().cpu().numpy(), c.oracle_delta(0)) <= TOL
        assert torch.equal(b, a.to(torch.bfloat16))
    for a, b in zip(apply_all(cases, batch, 0, torch.bfloat16), y16):
        assert torch.equal(a, b)
    # the same batch with everything on the BGMV kernels
    batch.tiles = False
    for c, a in zip(cases, apply_all(cases, batch, 0, torch.float32)):
        assert rel_err(a.double().cpu().numpy(), c.oracle_delta(0)) <= TOL


def test_prefill_7b_full_size_three_projections_one_apply():
    """Workload 2 as drawn (16 prompts, 9336 rows, rank 32, hidden 4096) with q/k/v in one apply:
    219 (tile, projection) pairs, more than there are SMs, so one launch runs both phases."""
    wl = make_workload(2)
    assert wl.n_tokens == 9336
    cases = shared_x_cases(wl.n_tokens, 16, 4096, (4096, 4096, 4096), wl.ranks, "fp16", wl.ids, seed=2962)
    starts = torch.from_numpy(np.concatenate([[0], np.cumsum(wl.seq_lens)]).astype(np.int32)).cuda()
    segs = torch.arange(16, dtype=torch.int32, device="cuda")
    batch = L.LoraBatch(wl.n_tokens, 16, 4096, 3).set_segments(starts, segs, wl.n_tokens, cases[0].pool, tiles=True)
    y32 = apply_all(cases, batch, 0, torch.float32)
    y16 = apply_all(cases, batch, 0, torch.float16)
    for c, a, b in zip(cases, y32, y16):
        assert rel_err(a.double().cpu().numpy(), c.oracle_delta(0)) <= TOL
        assert torch.equal(b, a.to(torch.float16))
    for a, b in zip(apply_all(cases, batch, 0, torch.float16), y16):
        assert torch.equal(a, b)
    # the reference's prefill op rounds the [T, r] intermediate to fp16 (lightllm/models/lora_gpu.py:127-128)
    ymid = apply_all(cases[:1], L.LoraBatch(wl.n_tokens, 16, 4096, 1).set_segments(starts, segs, wl.n_tokens, cases[0].pool),
                     0, torch.float32, L.MID_ROUND)[0]
    assert rel_err(ymid.double().cpu().numpy(), cases[0].oracle_delta(0, mid_round="fp16")) <= TOL


@pytest.mark.parametrize("name,h_in,h_outs,ranks,dtype,T,N,zipf", [
    ("13b-tp8", 5120, (5120, 5120, 5120), [16, 32, 64], "bf16", 96, 40, 1.0),      # shards 640 -> 640
    ("70b-tp8-qkv", 8192, (8192, 1024, 1024), 64, "bf16", 64, 24, 1.2),            # shards 1024 -> 1024 | 128 | 128
    ("odd-widths", 2560, (2560, 320 * 8, 192 * 8), [16, 32, 64], "fp16", 70, 20, 1.0),   # shards 320 -> 320 | 320 | 192: general kernels
])
def test_eight_way_shards_shrink_sum_expand(name, h_in, h_outs, ranks, dtype, T, N, zipf):
    """The shard widths of eight-way tensor parallelism (A cut along the hidden dimension, B along
    the output), run rank after rank on one GPU: shrink halves, the sum NCCL would form, expand
    halves.  640 and 128 are whole 128-column blocks (the TMA kernels take them); 320 and 192 are not
    (the general kernels' two halves)."""
    tp = 8
    rng = np.random.default_rng(5)
    p = 1.0 / np.arange(1, N + 1) ** zipf
    ids = rng.choice(N, T, p=p / p.sum()).astype(np.int32)
    cases = shared_x_cases(T, N, h_in, h_outs, ranks, dtype, ids, seed=71)
    n = len(cases)
    shards = [[c.pool.shard(tp, g) for c in cases] for g in range(tp)]
    batches = [L.LoraBatch(T, N, h_in // tp, n).set_ids(cases[0].ids_dev, shards[g][0]) for g in range(tp)]
    ys = [torch.zeros(T, h, dtype=torch.float32, device="cuda") for h in h_outs]

    def projs(g):
        return [(column_slice(c.x, tp, g), column_slice(y, tp, g), sh) for c, y, sh in zip(cases, ys, shards[g])]

    for g in range(tp):
        batches[g].apply(projs(g), 0, _lib.ONLY_SHRINK)
    total = sum(b.workspace.v_view() for b in batches)
    for g in range(tp):
        batches[g].workspace.v_view().copy_(total)
        batches[g].apply(projs(g), 0, _lib.ONLY_EXPAND)
    torch.cuda.synchronize()
    for b in batches:
        b.workspace.check()
    for c, y in zip(cases, ys):
        assert rel_err(y.double().cpu().numpy(), c.oracle_delta(0)) <= TOL


def _golden_check(got16, ref16, delta64):
    """CUDA output against the reference worker's fp16 output: both round once to fp16 from
    (at least) fp32 sums, so they may differ by one fp16 step of the larger magnitude plus the
    fp32 summation error."""
    rms = np.sqrt((delta64 ** 2).mean())
    got, ref = got16.astype(np.float64), ref16.astype(np.float64)
    assert np.abs(got - ref).max() <= TOL * rms + np.abs(ref).max() * 2.0 ** -10


def test_cuda_matches_reference_cpu_worker_small_vectors():
    """The reference's unmodified CPU worker (lora_cpu/lora_shm_op/app.py:133-141) on 5 requests of
    24 tokens, 3 adapters of rank 8, hidden 256: its stored q/k/v outputs against this library's."""
    g = np.load(os.path.join(GOLD, "worker_small.npz"))
    B, Lr, H, N, r = [int(v) for v in g["dims"]]
    x = torch.from_numpy(g["x"]).reshape(B * Lr, H).cuda()
    ids = torch.from_numpy(np.repeat(g["ids"], Lr).astype(np.int64)).cuda()
    for nm in "qkv":
        wa = torch.from_numpy(g[f"wa_{nm}"]).unsqueeze(1).contiguous().cuda()       # [N, 1, r, H]
        wb = torch.from_numpy(g[f"wb_{nm}"]).unsqueeze(1).contiguous().cuda()       # [N, 1, H, r]
        y = torch.zeros(B * Lr, H, dtype=torch.float16, device="cuda")
        L.add_lora_bgmv(y, x, wa, wb, ids, 0, 1.0)
        torch.cuda.synchronize()
        d = O.lora_delta(g["x"].astype(np.float64).reshape(B * Lr, H), lambda a: g[f"wa_{nm}"][a].astype(np.float64),
                         lambda a: g[f"wb_{nm}"][a].astype(np.float64), np.repeat(g["ids"], Lr), np.ones(N))
        _golden_check(y.cpu().numpy(), g[f"out_{nm}"].reshape(B * Lr, H), d)


def test_cuda_matches_reference_cpu_worker_decode_4096():
    """Workload 0's decode batch (32 tokens, 8 adapters of rank 16, hidden 4096) as the reference's CPU
    workers computed it: inputs regenerated from the seed (digests checked), outputs compared on the
    stored column sample."""
    sys.path.insert(0, GOLD)
    import make_golden
    g = np.load(os.path.join(GOLD, "worker_decode4096.npz"))
    B, Lr, H, N, r = [int(v) for v in g["dims"]]
    x, wa, wb = make_golden.regenerate_worker_inputs(int(g["seed"]), B, Lr, H, N, r)
    import hashlib
    assert hashlib.sha256(np.ascontiguousarray(x.numpy()).tobytes()).hexdigest() == str(g["x_sha"])
    xd = x.reshape(B * Lr, H).cuda()
    ids64 = torch.from_numpy(g["ids"].astype(np.int64)).cuda()
    for nm in "qkv":
        wad = wa[nm].unsqueeze(1).contiguous().cuda()
        wbd = wb[nm].unsqueeze(1).contiguous().cuda()
        y = torch.zeros(B, H, dtype=torch.float16, device="cuda")
        L.add_lora_bgmv(y, xd, wad, wbd, ids64, 0, 1.0)
        torch.cuda.synchronize()
        d = O.lora_delta(x.double().numpy().reshape(B, H), lambda a: wa[nm][a].double().numpy(),
                         lambda a: wb[nm][a].double().numpy(), g["ids"], np.ones(N))
        _golden_check(y.cpu().numpy()[:, ::64], g[f"out_{nm}_cols"].reshape(B, -1), d)


def test_one_call_op_reuses_a_workspace_across_shapes():
    """``b200_add_lora_bgmv`` on ONE caller buffer with growing, then shrinking token counts and a
    changing adapter count, on a shape that takes the general kernels (rank 24; their arrival
    counters and the control block must be clear whatever an earlier call left in those bytes)."""
    nbytes = L.add_lora_bgmv_workspace_bytes(96, 40, 640)
    ws = torch.full((nbytes // 4 + 1,), -1, dtype=torch.int32, device="cuda")        # starts full of ones
    for T, N, seed in [(8, 5, 0), (96, 40, 1), (33, 12, 2), (96, 40, 3), (2, 40, 4)]:
        c = Case(T, N, 640, 384, 24, "fp16", dense=True, seed=seed, zipf=1.0)
        y = torch.zeros(T, 384, dtype=torch.float16, device="cuda")
        L.add_lora_bgmv_once(y, c.x, c.pool.wa, c.pool.wb, c.ids_dev.long(), 1, 0.5, ws)
        torch.cuda.synchronize()
        want = O.lora_delta(c.x_cpu.double().numpy(), lambda a: c.A[a][1].double().numpy(),
                            lambda a: c.B[a][1].double().numpy(), c.ids, np.full(N, 0.5))
        rms = np.sqrt((want ** 2).mean())
        assert np.abs(y.double().cpu().numpy() - want).max() <= TOL * rms + np.abs(want).max() * 2.0 ** -11


def test_drop_in_op_keeps_the_plan_while_the_index_tensor_is_unchanged():
    """``add_lora_bgmv`` rebuilds its plan only when the index tensor may have changed."""
    c = Case(40, 9, 512, 768, 16, "fp16", dense=True, seed=5)
    ids = c.ids_dev.long()

    def run(index):
        y = torch.zeros(c.T, c.h_out, dtype=torch.float16, device="cuda")
        L.add_lora_bgmv(y, c.x, c.pool.wa, c.pool.wb, index, 0, 1.0)
        torch.cuda.synchronize()
        return y

    def want(index_np):
        d = O.lora_delta(c.x_cpu.double().numpy(), lambda a: c.A[a][0].double().numpy(),
                         lambda a: c.B[a][0].double().numpy(), index_np, np.ones(c.N))
        return d, np.sqrt((d ** 2).mean())

    first = run(ids)
    assert torch.equal(run(ids), first)                       # plan reused
    d, rms = want(c.ids)
    assert np.abs(first.double().cpu().numpy() - d).max() <= TOL * rms + np.abs(d).max() * 2.0 ** -11
    ids[3] = (int(ids[3]) + 1) % c.N                          # in-place change: the plan must follow
    changed = c.ids.copy(); changed[3] = int(ids[3])
    d2, rms2 = want(changed)
    assert np.abs(run(ids).double().cpu().numpy() - d2).max() <= TOL * rms2 + np.abs(d2).max() * 2.0 ** -11
    other = torch.from_numpy(c.ids[::-1].copy()).cuda().long()  # another tensor of the same shape
    d3, rms3 = want(c.ids[::-1])
    assert np.abs(run(other).double().cpu().numpy() - d3).max() <= TOL * rms3 + np.abs(d3).max() * 2.0 ** -11


@pytest.mark.parametrize("shape", ["tma", "general"])
def test_plan_of_another_batch_size_is_refused_on_the_device(shape):
    """An apply whose row count differs from the plan's must not index x and y with the plan's token
    rows: it changes nothing and the workspace reports the mismatch."""
    h, r = (512, 16) if shape == "tma" else (640, 24)
    c = Case(64, 6, h, h, r, "fp16", dense=True, seed=8)
    batch = L.LoraBatch(64, 6, h, 1).set_ids(c.ids_dev, c.pool)
    x_small = c.x[:32].contiguous()
    y = torch.zeros(32, h, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        batch.apply([(x_small, y, c.pool)], 0)                # the Python wrapper notices first
    assert raw_apply([(x_small, y, c.pool)], batch.plan, 0, batch.workspace, 32, _lib.NO_TENSOR) == 0
    torch.cuda.synchronize()
    assert not y.any()
    with pytest.raises(L.LoraError) as e:
        batch.workspace.check()
    assert e.value.code == -2
    # the workspace is usable again once its error word is cleared
    _lib.check(_lib.lib().b200_lora_workspace_init(batch.workspace.buf.data_ptr(), 64, torch.cuda.current_stream().cuda_stream))
    got = c.run(0, batch=batch)
    assert rel_err(got.double().cpu().numpy(), c.oracle_delta(0)) <= TOL + 2.0 ** -9
