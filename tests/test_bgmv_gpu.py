"""GPU parity of the decode BGMV path against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import ae296_b200 as L
from lora_testlib import TOL, Case, rel_err
from oracle import lora_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T", [1, 2, 31, 33])
@pytest.mark.parametrize("r", [8, 16, 64])
@pytest.mark.parametrize("H", [128, 4096])
def test_tiny_exhaustive(T, r, H):
    c = Case(T, 5, H, H, r, "fp16", dense=False, seed=T * 100 + r + H)
    want = c.oracle_delta(1)
    y32 = c.run(1, y_dtype=torch.float32)
    assert rel_err(y32.double().cpu().numpy(), want) <= TOL
    y16 = c.run(1)
    # the low-precision output is the single rounding of the fp32 result
    assert torch.equal(y16, y32.to(torch.float16))
    # a second run is bit-identical (fixed-order split-K reduction, no float atomics)
    assert torch.equal(c.run(1, y_dtype=torch.float32), y32)


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("dense", [False, True])
def test_mixed_ranks_both_layouts(dtype, dense):
    c = Case(96, 24, 1024, 768, [8, 16, 32, 64], dtype, dense=dense, seed=7, zipf=1.0)
    for layer in (0, 1):
        want = c.oracle_delta(layer)
        y32 = c.run(layer, y_dtype=torch.float32)
        assert rel_err(y32.double().cpu().numpy(), want) <= TOL
        assert torch.equal(c.run(layer), y32.to(c.tdt))


def test_dense_pool_ranks_not_multiple_of_8_and_garbage_padding():
    c = Case(40, 6, 512, 512, np.array([3, 12, 20, 33, 50, 64], np.int32), "fp16", dense=True, seed=3)
    # poison the unused rows/columns of the dense pool: they must never be read into the result
    for a in range(c.N):
        r = int(c.ranks[a])
        c.pool.wa[a, :, r:, :] = float("nan")
        c.pool.wb[a, :, :, r:] = float("nan")
    y32 = c.run(0, y_dtype=torch.float32)
    assert rel_err(y32.double().cpu().numpy(), c.oracle_delta(0)) <= TOL


def test_accumulates_into_y_with_strides_and_canaries():
    c = Case(37, 9, 640, 384, [16, 32], "bf16", seed=11)
    g = torch.Generator().manual_seed(5)
    pad = 16
    ybig = torch.randn(c.T + 2, c.h_out + 2 * pad, generator=g).to(torch.bfloat16).cuda()
    before = ybig.clone()
    xbig = torch.full((c.T, c.h_in + 24), 7.0, dtype=torch.bfloat16, device="cuda")
    xbig[:, :c.h_in] = c.x
    yv = ybig[1:-1, pad:pad + c.h_out]
    batch = L.LoraBatch(c.T, c.N, c.h_in, 1).set_ids(c.ids_dev, c.pool)
    batch.apply([(xbig[:, :c.h_in], yv, c.pool)], 1)
    torch.cuda.synchronize()
    want = O.round_to(before[1:-1, pad:pad + c.h_out].double().cpu().numpy() + c.oracle_delta(1), "bf16")
    got = yv.double().cpu().numpy()
    rms = np.sqrt((want ** 2).mean())
    # one bf16 rounding of (y + delta): within half an ulp of the exact sum plus the fp32 error
    assert np.abs(got - want).max() <= np.abs(want).max() * 2 ** -8 + TOL * rms
    mask = torch.ones_like(ybig, dtype=torch.bool)
    mask[1:-1, pad:pad + c.h_out] = False
    assert torch.equal(ybig[mask], before[mask]), "bytes outside the y view were written"


def test_reference_call_signature_int64_ids():
    c = Case(32, 8, 4096, 4096, 16, "fp16", dense=True, seed=2960)
    y = torch.zeros(c.T, c.h_out, dtype=torch.float16, device="cuda")
    ret = L.add_lora_bgmv(y, c.x, c.pool.wa, c.pool.wb, c.ids_dev.long(), 1, 2.0)
    torch.cuda.synchronize()
    assert ret is None
    want = O.lora_delta(c.x_cpu.double().numpy(), lambda a: c.A[a][1].double().numpy(),
                        lambda a: c.B[a][1].double().numpy(), c.ids, np.full(c.N, 2.0))
    got = y.double().cpu().numpy()
    rms = np.sqrt((want ** 2).mean())
    assert np.abs(got - want).max() <= TOL * rms + np.abs(want).max() * 2 ** -11


def test_mid_round_flag_matches_bmm_rounding():
    c = Case(64, 4, 512, 512, 32, "fp16", seed=9, ids=np.repeat(np.arange(4), 16))
    y32 = c.run(0, y_dtype=torch.float32, flags=L.MID_ROUND)
    assert rel_err(y32.double().cpu().numpy(), c.oracle_delta(0, mid_round="fp16")) <= TOL


def test_fused_qkv_equals_separate_calls():
    c = Case(48, 12, 1024, 1024, [8, 64], "fp16", seed=21, zipf=1.0)
    k = Case(48, 12, 1024, 256, c.ranks, "fp16", seed=22, ids=c.ids)
    ys = [torch.zeros(48, h, dtype=torch.float16, device="cuda") for h in (1024, 256, 1024)]
    batch = L.LoraBatch(48, 12, 1024, 3).set_ids(c.ids_dev, c.pool)
    batch.apply([(c.x, ys[0], c.pool), (c.x, ys[1], k.pool), (c.x, ys[2], c.pool)], 1)
    torch.cuda.synchronize()
    batch.workspace.check()

    def close(a, b):
        # the fused call cuts the split-K sums at other places than a single-projection call,
        # so the fp32 sums may differ in their last bits: allow one fp16 ulp of the result
        a, b = a.float(), b.float()
        return bool(((a - b).abs() <= 2.0 ** -10 * b.abs().clamp_min(2.0 ** -6)).all())

    assert close(ys[0], c.run(1))
    assert close(ys[2], ys[0])
    k.x, k.x_cpu = c.x, c.x_cpu
    assert close(ys[1], k.run(1))


def test_outputs_side_by_side_in_one_buffer():
    """q | k | v as column ranges of one [T, sum(h_out)] block (row pitch larger than the width), x as
    one of two activations that share a buffer: same bits as separate contiguous tensors, nothing
    written outside the ranges.  Decode kernels and, with tall runs, the tile kernel."""
    for tiles, ids in ((False, None), (True, np.concatenate([np.arange(40) % 6, np.repeat([7, 2], [128, 70])]).astype(np.int32))):
        T = 48 if ids is None else len(ids)
        c = Case(T, 12, 1024, 1024, [16, 64], "bf16", seed=31, zipf=1.0 if ids is None else None, ids=ids)
        k = Case(T, 12, 1024, 256, c.ranks, "bf16", seed=32, ids=c.ids)
        pools, widths = [c.pool, k.pool, c.pool], [1024, 256, 1024]
        xx = torch.zeros(2, T, 1024, dtype=torch.bfloat16, device="cuda")
        xx[1].copy_(c.x)
        g = torch.Generator().manual_seed(9)
        block = torch.randn(T, sum(widths) + 64, generator=g).to(torch.bfloat16).cuda()     # 64 canary columns
        sep = [block[:, o:o + w].clone() for o, w in zip((0, 1024, 1280), widths)]
        before = block.clone()
        views = [block[:, o:o + w] for o, w in zip((0, 1024, 1280), widths)]
        batch = L.LoraBatch(T, 12, 1024, 3).set_ids(c.ids_dev, c.pool, tiles=tiles)
        batch.apply([(xx[1], v, p) for v, p in zip(views, pools)], 1)
        batch.apply([(c.x, y, p) for y, p in zip(sep, pools)], 1)
        torch.cuda.synchronize()
        batch.workspace.check()
        for v, y in zip(views, sep):
            assert torch.equal(v, y)
        assert torch.equal(block[:, sum(widths):], before[:, sum(widths):])
        assert not torch.equal(views[0], before[:, :1024])


def test_errors_are_raised_not_swallowed():
    c = Case(8, 4, 128, 128, 8, "fp16", seed=1)
    bad = c.ids_dev.clone()
    bad[3] = 4                      # == N: out of range
    batch = L.LoraBatch(8, 4, 128, 1)
    batch.plan.build(bad, L.adapters_of(c.pool))
    with pytest.raises(L.LoraError) as e:
        batch.plan.read()
    assert e.value.code == -8
    # such a plan applies nothing
    y = torch.zeros(8, 128, dtype=torch.float16, device="cuda")
    batch.apply([(c.x, y, c.pool)], 0)
    torch.cuda.synchronize()
    assert not y.any()
    with pytest.raises(L.LoraError):
        batch.set_ids(c.ids_dev, c.pool).apply([(c.x, y, c.pool)], 5)       # layer out of range
    with pytest.raises(ValueError):
        L.add_lora_bgmv(y.cpu(), c.x.cpu(), c.pool.wa.cpu(), c.pool.wb.cpu(), c.ids_dev.cpu(), 0, 1.0)


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_delta_then_add_mode(dtype):
    """The reference adds the 16-bit delta to the projection in 16-bit arithmetic (q += q_lora)."""
    c = Case(70, 12, 1024, 768, [8, 16, 32, 64], dtype, seed=77, zipf=1.0)
    # y starting at zero (how the reference calls the op): identical to the default mode
    assert torch.equal(c.run(1, flags=L.DELTA_THEN_ADD), c.run(1))
    # y starting elsewhere: round(delta) added in the I/O type, the oracle's delta_then_add
    g = torch.Generator().manual_seed(3)
    y0 = torch.randn(c.T, c.h_out, generator=g).to(c.tdt).cuda()
    got = c.run(1, y0=y0, flags=L.DELTA_THEN_ADD).double().cpu().numpy()
    delta = O.round_to(c.oracle_delta(1), dtype)
    want = O.delta_then_add(y0.double().cpu().numpy(), delta, dtype)
    ulp = 2.0 ** (-10 if dtype == "fp16" else -7)
    assert np.abs(got - want).max() <= ulp * np.abs(want).max()
    assert (got != want).mean() < 0.02          # only ties of the delta's own rounding may differ


@pytest.mark.parametrize("T,N,h_in,h_out,ranks,zipf,dtype", [
    (256, 128, 4096, 4096, [8, 16, 32, 64], 1.0, "fp16"),      # decode batch of the 7B workload
    (512, 96, 8192, 1024, 64, 1.2, "bf16"),                    # GQA k/v shapes of the 70B workload
    (512, 96, 8192, 8192, 64, 1.2, "bf16"),                    # its q/o shapes: 64 units per segment
])
def test_full_size_decode_segments_spanning_many_ctas(T, N, h_in, h_out, ranks, zipf, dtype):
    """At these sizes a work segment's units are spread over several CTAs, so its intermediate is
    the sum of several split-K slots that the expand kernel's producers add up themselves."""
    c = Case(T, N, h_in, h_out, ranks, dtype, seed=11, zipf=zipf, n_layers=1)
    want = c.oracle_delta(0)
    got32 = c.run(0, y_dtype=torch.float32)
    assert rel_err(got32.double().cpu().numpy(), want) <= TOL
    # 16-bit output: the single rounding of the fp32 result; a second run is bit-identical
    got16 = c.run(0)
    assert torch.equal(got16, got32.to(c.tdt))
    assert torch.equal(c.run(0), got16)
    # linearity in x: doubling x doubles the delta; exactly so in bf16 (powers of two commute with
    # every rounding), up to the fp16 subnormals of the intermediate's lo halves in fp16
    c.x = (c.x_cpu * 2).to(c.device)
    twice = c.run(0, y_dtype=torch.float32)
    if dtype == "bf16":
        assert torch.equal(twice, got32 * 2)
    else:
        assert rel_err(twice.double().cpu().numpy(), 2 * got32.double().cpu().numpy()) <= 1e-5


def test_adapter_swapped_in_on_a_side_stream():
    """An adapter slot reloaded from pinned host memory on a side stream while the batch runs."""
    c = Case(24, 6, 512, 768, [16, 32], "fp16", seed=21)
    before = c.run(0, y_dtype=torch.float32)
    a = int(c.ids[0])
    g = torch.Generator().manual_seed(5)
    r = int(c.ranks[a])
    A_new = (torch.randn(c.n_layers, r, c.h_in, generator=g) / np.sqrt(c.h_in)).to(c.tdt).pin_memory()
    B_new = (torch.randn(c.n_layers, c.h_out, r, generator=g) / np.sqrt(r)).to(c.tdt).pin_memory()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())          # the running batch still reads the slot
    done = c.pool.load_adapter_async(a, A_new, B_new, side)
    torch.cuda.current_stream().wait_event(done)
    c.A[a], c.B[a] = A_new, B_new
    after = c.run(0, y_dtype=torch.float32)
    assert rel_err(after.double().cpu().numpy(), c.oracle_delta(0)) <= TOL
    rows = torch.from_numpy(c.ids != a).cuda()
    assert torch.equal(after[rows], before[rows])           # other adapters' tokens are untouched
    with pytest.raises(ValueError):
        c.pool.load_adapter_async(a, A_new[:, :8], B_new, side)
