"""GPU parity of the prefill SGMV path (tcgen05 tiles for tall segments + BGMV for the rest)."""
import os

import numpy as np
import pytest
import torch

import ae296_b200 as L
from lora_testlib import TOL, Case, rel_err
from oracle import lora_oracle as O

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def seg_case(lens, adapters, ranks, n_adapters, h_in, h_out, dtype="fp16", dense=False, seed=0):
    ids = np.repeat(np.asarray(adapters, np.int32), lens)
    c = Case(int(np.sum(lens)), n_adapters, h_in, h_out, np.asarray(ranks, np.int32), dtype, dense=dense, seed=seed, ids=ids)
    starts = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    c.seg_starts = torch.from_numpy(starts).cuda()
    c.seg_adapter = torch.from_numpy(np.asarray(adapters, np.int32)).cuda()
    return c


def run_segments(c, layer, y_dtype=None, flags=0, tiles=True):
    y = torch.zeros(c.T, c.h_out, dtype=c.tdt if y_dtype is None else y_dtype, device="cuda")
    batch = L.LoraBatch(c.T, c.N, c.h_in, 1)
    batch.set_segments(c.seg_starts, c.seg_adapter, c.T, c.pool, tiles=tiles)
    batch.apply([(c.x, y, c.pool)], layer, flags)
    torch.cuda.synchronize()
    batch.workspace.check()
    return y


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_tall_and_short_segments_mixed_ranks(dtype):
    # tall tiles: ranks 16/32/64 with >= 32 rows (one spans two tiles, one ends mid-tile);
    # BGMV: the rank-8 segment, the 5-row and the 31-row segments
    lens = [5, 200, 37, 130, 31, 64, 128, 40]
    adapters = [0, 1, 2, 3, 4, 5, 6, 7]
    ranks = [16, 64, 32, 16, 64, 8, 32, 64]
    c = seg_case(lens, adapters, ranks, 8, 512, 384, dtype, seed=17)
    for layer in (0, 1):
        want = c.oracle_delta(layer)
        y32 = run_segments(c, layer, y_dtype=torch.float32)
        assert rel_err(y32.double().cpu().numpy(), want) <= TOL
        # the same batch entirely on the BGMV kernels agrees too
        y32b = run_segments(c, layer, y_dtype=torch.float32, tiles=False)
        assert rel_err(y32b.double().cpu().numpy(), want) <= TOL
        # 16-bit output: one rounding of the fp32 result
        y16 = run_segments(c, layer)
        assert torch.equal(y16, y32.to(c.tdt))
        assert torch.equal(run_segments(c, layer, y_dtype=torch.float32), y32)      # reproducible


def test_mid_round_matches_rounded_intermediate():
    c = seg_case([96, 33, 140], [2, 0, 1], [32, 16, 64], 3, 256, 256, "fp16", seed=5)
    y32 = run_segments(c, 1, y_dtype=torch.float32, flags=L.MID_ROUND)
    assert rel_err(y32.double().cpu().numpy(), c.oracle_delta(1, mid_round="fp16")) <= TOL


def test_reference_prefill_golden():
    """The reference's own prefill method (two fp16 batched matmuls) on its own inputs."""
    g = np.load(os.path.join(GOLD, "prefill_bmm_small.npz"))
    B, Lp, H, r, nl, layer = [int(v) for v in g["dims"]]
    x = torch.from_numpy(g["x"]).cuda().reshape(B * Lp, H)
    wa, wb = torch.from_numpy(g["wa"]).cuda(), torch.from_numpy(g["wb"]).cuda()
    pool = L.AdapterPool(wa, wb, None, None, None, B, nl, H, H, r, False, np.full(B, r, np.int32),
                         np.arange(B + 1, dtype=np.int64) * r)
    ad = L.ops._adapters_struct(B, nl, r)
    batch = L.LoraBatch(B * Lp, B, H, 1)
    starts = torch.arange(0, (B + 1) * Lp, Lp, dtype=torch.int32, device="cuda")
    batch.plan.from_segments(starts, torch.arange(B, dtype=torch.int32, device="cuda"), B * Lp, ad)
    y = torch.zeros(B * Lp, H, dtype=torch.float16, device="cuda")
    L.apply([(x, y, pool)], batch.plan, layer, batch.workspace, L.MID_ROUND, ad)
    torch.cuda.synchronize()
    batch.workspace.check()
    ref = g["y"].astype(np.float64).reshape(B * Lp, H)
    got = y.double().cpu().numpy()
    rms = np.sqrt((ref ** 2).mean())
    # both sides round the intermediate and the output to fp16: allow one output ulp on top
    assert np.abs(got - ref).max() <= TOL * rms + np.abs(ref).max() * 2 ** -10


def test_lora_gpu_mirror_prefill_and_decode():
    cfg = {"n_layers": 2, "batch_size": 8, "lora_rank": 16, "hidden_dim": 256, "tp_degree": 1,
           "max_prefill_batch_size": 3, "mode": "aaas-cached"}
    torch.manual_seed(0)
    obj = L.Lora_GPU(cfg)
    x = torch.randn(3, 40, 256, device="cuda").half()
    y = obj.invoke_one_layer_q(x, 1, prefill=True)
    ref = O.prefill_bmm(x, obj.q_down_prefill[:3, 1], obj.q_up_prefill[:3, 1])
    rms = float(ref.float().pow(2).mean().sqrt())
    assert float((y.float() - ref.float()).abs().max()) <= TOL * rms + float(ref.abs().max()) * 2 ** -10
    xd = torch.randn(5, 256, device="cuda").half()
    idx = torch.tensor([3, 0, 7, 3, 1], device="cuda")
    obj.set_indices(idx)
    yd = obj.invoke_one_layer_k(xd, 0)
    want = torch.stack([(xd[i].float() @ obj.k_down[idx[i], 0].float().t()) @ obj.k_up[idx[i], 0].float().t()
                        for i in range(5)])
    rms = float(want.pow(2).mean().sqrt())
    assert float((yd.float() - want).abs().max()) <= TOL * rms + float(want.abs().max()) * 2 ** -10


def test_mixed_decode_and_prefill_from_ids():
    """Per-token ids: decode tokens in random order followed by contiguous prompts."""
    rng = np.random.default_rng(3)
    n = 12
    ranks = rng.choice([16, 32, 64], n).astype(np.int32)
    dec = rng.integers(0, n, 70)
    ids = np.concatenate([dec, np.repeat([11, 4], [150, 64])]).astype(np.int32)   # adapter 4 may also decode
    c = Case(len(ids), n, 512, 512, ranks, "bf16", seed=23, ids=ids)
    y = torch.zeros(c.T, c.h_out, dtype=torch.float32, device="cuda")
    batch = L.LoraBatch(c.T, n, 512, 1).set_ids(c.ids_dev, c.pool, tiles=True)
    batch.apply([(c.x, y, c.pool)], 0)
    torch.cuda.synchronize()
    batch.workspace.check()
    assert rel_err(y.double().cpu().numpy(), c.oracle_delta(0)) <= TOL


def test_full_size_prefill_batch():
    """The prefill workload at full size (16 prompts of 128..1024 tokens, rank 32, hidden 4096), one
    projection: 73 tiles, so phase 1 is cut in two along k and phase 2 by output columns."""
    lens = [537, 824, 517, 341, 399, 247, 211, 845, 932, 822, 305, 334, 379, 996, 658, 989]
    c = seg_case(lens, list(range(16)), [32] * 16, 16, 4096, 4096, "fp16", seed=2962)
    want = c.oracle_delta(0)
    y32 = run_segments(c, 0, y_dtype=torch.float32)
    assert rel_err(y32.double().cpu().numpy(), want) <= TOL
    y16 = run_segments(c, 0)
    assert torch.equal(y16, y32.to(c.tdt))                 # one rounding of the fp32 result
    assert torch.equal(run_segments(c, 0), y16)            # reproducible
    # the reference's rounding of the intermediate (its prefill op keeps fp16 tensors)
    y_mid = run_segments(c, 0, y_dtype=torch.float32, flags=L.MID_ROUND)
    assert rel_err(y_mid.double().cpu().numpy(), c.oracle_delta(0, mid_round="fp16")) <= TOL


def test_few_whole_tiles_three_projections_cut_along_k():
    """Few tiles (two launches: phase 1 cut eight ways along k, then phase 2 by columns), three projections
    of different widths in one call, runs of whole 128-row tiles (their y leaves by tensor store) next to a
    partial one, and an output width that ends in half a 128-column slice."""
    lens, adapters, ranks = [256, 128, 100, 384], [3, 0, 2, 1], [64, 16, 32, 32]
    cases = [seg_case(lens, adapters, ranks, 4, 1024, h_out, "bf16", seed=40 + i) for i, h_out in enumerate((320, 128, 576))]
    T = cases[0].T
    batch = L.LoraBatch(T, 4, 1024, 3)
    batch.set_segments(cases[0].seg_starts, cases[0].seg_adapter, T, cases[0].pool, tiles=True)

    def run(y_dtype):
        ys = [torch.zeros(T, c.h_out, dtype=y_dtype, device="cuda") for c in cases]
        batch.apply([(c.x, y, c.pool) for c, y in zip(cases, ys)], 1)
        torch.cuda.synchronize()
        batch.workspace.check()
        return ys

    y32, y16 = run(torch.float32), run(torch.bfloat16)
    for c, a, b in zip(cases, y32, y16):
        assert rel_err(a.double().cpu().numpy(), c.oracle_delta(1)) <= TOL
        assert torch.equal(b, a.to(torch.bfloat16))            # one rounding of the fp32 result
    for a, b in zip(run(torch.bfloat16), y16):
        assert torch.equal(a, b)                               # reproducible whichever CTA adds the k parts
    # y that is not zero: the update adds to what is there
    base = [torch.randn(T, c.h_out, device="cuda").to(torch.bfloat16) for c in cases]
    ys = [b.clone() for b in base]
    batch.apply([(c.x, y, c.pool) for c, y in zip(cases, ys)], 1)
    torch.cuda.synchronize()
    for b, y, d in zip(base, ys, y32):
        want = b.float() + d
        # bf16 output of a fused multiply-add: within one bf16 step of the separately rounded sum
        assert float((y.float() - want).abs().max()) <= float(want.abs().max()) * 2.0 ** -7


def test_more_pairs_than_sms_single_launch():
    """Enough tiles that both phases run in one launch per apply (at least as many (tile, projection)
    pairs as SMs): full rounds of whole pairs, then a last round cut by output columns."""
    rng = np.random.default_rng(77)
    lens = [int(v) for v in rng.integers(300, 700, 14)]          # about 7000 rows: over 50 tiles, three projections
    ranks = [int(v) for v in rng.choice([16, 32, 64], 14)]
    cases = [seg_case(lens, list(range(14)), ranks, 14, 1024, h_out, "fp16", seed=60 + i) for i, h_out in enumerate((1024, 256, 1024))]
    T = cases[0].T
    n_sm = torch.cuda.get_device_properties(0).multi_processor_count
    assert (T // 128 + 1) * 3 >= n_sm
    batch = L.LoraBatch(T, 14, 1024, 3)
    batch.set_segments(cases[0].seg_starts, cases[0].seg_adapter, T, cases[0].pool, tiles=True)

    def run(y_dtype):
        ys = [torch.zeros(T, c.h_out, dtype=y_dtype, device="cuda") for c in cases]
        batch.apply([(c.x, y, c.pool) for c, y in zip(cases, ys)], 0)
        torch.cuda.synchronize()
        batch.workspace.check()
        return ys

    y32, y16 = run(torch.float32), run(torch.float16)
    for c, a, b in zip(cases, y32, y16):
        assert rel_err(a.double().cpu().numpy(), c.oracle_delta(0)) <= TOL
        assert torch.equal(b, a.to(torch.float16))
    for a, b in zip(run(torch.float16), y16):
        assert torch.equal(a, b)


def test_mixed_apply_in_a_cuda_graph_forks_and_joins():
    """An apply with tall runs and other rows runs its tile launches on a side stream inside the call; captured
    into a CUDA graph that is a fork and a join.  Replays must accumulate the oracle's delta once each, bit for
    bit the same as the eager call, and work that follows on the caller's stream must see the tiles' rows."""
    rng = np.random.default_rng(31)
    n = 10
    ranks = rng.choice([16, 32, 64], n).astype(np.int32)
    ids = np.concatenate([rng.integers(0, n, 90), np.repeat([7, 2], [200, 130])]).astype(np.int32)
    c = Case(len(ids), n, 1024, 768, ranks, "bf16", seed=29, ids=ids)
    batch = L.LoraBatch(c.T, n, 1024, 1).set_ids(c.ids_dev, c.pool, tiles=True)
    y_eager = torch.zeros(c.T, c.h_out, dtype=torch.float32, device="cuda")
    batch.apply([(c.x, y_eager, c.pool)], 0)              # also the first call on this device: made outside capture
    torch.cuda.synchronize()
    y = torch.zeros_like(y_eager)
    total = torch.zeros(1, dtype=torch.float64, device="cuda")
    s = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            batch.apply([(c.x, y, c.pool)], 0)
            total.copy_(y.double().sum().reshape(1))       # ordered after the join: sees tall and short rows
    y.zero_()
    g.replay()
    torch.cuda.synchronize()
    batch.workspace.check()
    assert torch.equal(y, y_eager)
    assert abs(float(total) - float(y_eager.double().sum())) <= 1e-6 * float(y_eager.double().abs().sum())
    g.replay()
    torch.cuda.synchronize()
    assert rel_err(y.double().cpu().numpy(), 2 * c.oracle_delta(0)) <= TOL


def test_serial_tiles_switch_gives_the_same_bits(tmp_path):
    """B200_LORA_SERIAL_TILES=1 keeps the tile launches on the caller's stream; the result is the same, bit for bit."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = f"""
import sys
sys.path[:0] = [{root!r}, {os.path.join(root, 'tests')!r}]
import numpy as np, torch
import ae296_b200 as L
from lora_testlib import Case
rng = np.random.default_rng(41)
ranks = rng.choice([16, 32, 64], 9).astype(np.int32)
ids = np.concatenate([rng.integers(0, 9, 80), np.repeat([5, 1], [140, 260])]).astype(np.int32)
c = Case(len(ids), 9, 768, 1024, ranks, "fp16", seed=43, ids=ids)
y = torch.zeros(c.T, c.h_out, dtype=c.tdt, device="cuda")
b = L.LoraBatch(c.T, 9, 768, 1).set_ids(c.ids_dev, c.pool, tiles=True)
for _ in range(3):
    b.apply([(c.x, y, c.pool)], 0)
torch.cuda.synchronize()
b.workspace.check()
np.save(sys.argv[1], y.float().cpu().numpy())
"""
    outs = []
    for name, extra in (("fork", {}), ("serial", {"B200_LORA_SERIAL_TILES": "1"})):
        path = str(tmp_path / f"{name}.npy")
        env = dict(os.environ, **extra)
        env.pop("B200_LORA_SERIAL_TILES", None) if not extra else None
        subprocess.run([sys.executable, "-c", script, path], check=True, env=env, timeout=300)
        outs.append(np.load(path))
    assert np.abs(outs[0]).max() > 0 and np.array_equal(outs[0], outs[1])
