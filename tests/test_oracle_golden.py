"""CPU: the oracle against the golden vectors made by the reference's own code."""
import hashlib
import os
import sys

import numpy as np
import pytest
import torch

from oracle import lora_oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")
sys.path.insert(0, GOLD)
import make_golden  # noqa: E402  (only its input regeneration helper is used)


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_cpu_worker_matches_reference_worker_small():
    g = np.load(os.path.join(GOLD, "worker_small.npz"))
    B, L, H, N, r = g["dims"]
    x = torch.from_numpy(g["x"])
    for nm in "qkv":
        wa, wb = torch.from_numpy(g[f"wa_{nm}"]), torch.from_numpy(g[f"wb_{nm}"])
        for b in range(B):
            a = int(g["ids"][b])
            out = O.cpu_worker(x[b], wa[a].float().t().contiguous(), wb[a].float().t().contiguous())
            assert np.array_equal(out.numpy().view(np.uint16), g[f"out_{nm}"][b].view(np.uint16))


def test_cpu_worker_matches_reference_decode4096():
    g = np.load(os.path.join(GOLD, "worker_decode4096.npz"))
    B, L, H, N, r = [int(v) for v in g["dims"]]
    x, wa, wb = make_golden.regenerate_worker_inputs(int(g["seed"]), B, L, H, N, r)
    assert sha(x.numpy()) == str(g["x_sha"]), "torch's seeded CPU normal draw changed; regenerate the fixtures"
    for nm in "qkv":
        assert sha(wa[nm].numpy()) == str(g[f"wa_{nm}_sha"])
        out = np.zeros((B, L, H), np.float16)
        for b in range(B):
            a = int(g["ids"][b])
            out[b] = O.cpu_worker(x[b], wa[nm][a].float().t().contiguous(),
                                  wb[nm][a].float().t().contiguous()).numpy()
        assert sha(out) == str(g[f"out_{nm}_sha"])
        assert np.array_equal(out[:, :, ::64], g[f"out_{nm}_cols"])


def test_fp64_delta_agrees_with_reference_worker():
    """The float64 statement and the reference's fp32 worker agree to fp16 rounding."""
    g = np.load(os.path.join(GOLD, "worker_small.npz"))
    B, L, H, N, r = [int(v) for v in g["dims"]]
    x = g["x"].astype(np.float64).reshape(B * L, H)
    ids = np.repeat(g["ids"], L)
    for nm in "qkv":
        wa, wb = g[f"wa_{nm}"].astype(np.float64), g[f"wb_{nm}"].astype(np.float64)
        d = O.lora_delta(x, lambda a: wa[a], lambda a: wb[a], ids, np.ones(N))
        ref = g[f"out_{nm}"].astype(np.float64).reshape(B * L, H)
        rms = np.sqrt((d ** 2).mean())
        assert np.abs(O.round_to(d, "fp16") - ref).max() <= 2e-3 * rms + np.abs(ref).max() * 2 ** -11


def test_prefill_bmm_matches_reference_method():
    g = np.load(os.path.join(GOLD, "prefill_bmm_small.npz"))
    B, L, H, r, nl, layer = [int(v) for v in g["dims"]]
    x, wa, wb = (torch.from_numpy(g[k]) for k in ("x", "wa", "wb"))
    y = O.prefill_bmm(x, wa[:B, layer], wb[:B, layer])
    assert np.array_equal(y.numpy().view(np.uint16), g["y"].view(np.uint16))
    # the float64 statement with an fp16-rounded intermediate lands within fp16 rounding of it
    ids = np.repeat(np.arange(B), L)
    d = O.lora_delta(g["x"].astype(np.float64).reshape(B * L, H), lambda a: g["wa"][a, layer].astype(np.float64),
                     lambda a: g["wb"][a, layer].astype(np.float64), ids, np.ones(B), mid_round="fp16")
    ref = g["y"].astype(np.float64).reshape(B * L, H)
    rms = np.sqrt((d ** 2).mean())
    assert np.abs(d - ref).max() <= 2e-3 * rms + np.abs(ref).max() * 2 ** -10


@pytest.mark.parametrize("t,n,seed", [(1, 1, 0), (7, 3, 1), (256, 128, 2), (1000, 17, 3), (33, 512, 4)])
def test_stable_segments_is_a_stable_argsort(t, n, seed):
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, n, t)
    perm, starts, adapters = O.stable_segments(ids, n)
    assert np.array_equal(perm, np.argsort(ids, kind="stable").astype(np.int32))
    uniq, counts = np.unique(ids, return_counts=True)
    assert np.array_equal(adapters, uniq.astype(np.int32))
    assert np.array_equal(np.diff(starts), counts)
    assert starts[0] == 0 and starts[-1] == t


def test_stable_segments_rejects_bad_id():
    with pytest.raises(ValueError):
        O.stable_segments([0, 5], 5)


def test_rounding_helpers_match_torch():
    rng = np.random.default_rng(0)
    a = (rng.standard_normal(20000) * np.exp(rng.uniform(-12, 10, 20000))).astype(np.float32).astype(np.float64)
    t = torch.from_numpy(a.astype(np.float32))         # fp32-representable: torch rounds once too
    assert np.array_equal(O.round_to(a, "fp16"), t.to(torch.float16).double().numpy())
    assert np.array_equal(O.round_to(a, "bf16"), t.to(torch.bfloat16).double().numpy())
    # values a float32 cannot hold: one rounding from float64, no double rounding through fp32
    tie = 1.0 + 2.0 ** -8                                # midpoint of two bf16 neighbours
    trap = np.array([tie, tie + 2.0 ** -30, tie - 2.0 ** -30, 1.0 + 3 * 2.0 ** -8])
    want = np.array([1.0, 1.0 + 2.0 ** -7, 1.0, 1.0 + 2.0 ** -6])
    assert np.array_equal(O.round_to(trap, "bf16"), want)


def test_delta_then_add_and_tp_slice():
    rng = np.random.default_rng(1)
    base = rng.standard_normal((4, 16))
    delta = rng.standard_normal((4, 16))
    out = O.delta_then_add(O.round_to(base, "fp16"), O.round_to(delta, "fp16"), "fp16")
    ref = (torch.from_numpy(base).half() + torch.from_numpy(delta).half()).double().numpy()
    assert np.array_equal(out, ref)
    assert np.array_equal(O.tp_column_slice(delta, 4, 2), delta[:, 8:12])
