"""GPU: the allocation-free entry point agrees with the workspace-taking one.

Some users of this library cannot allocate device memory when they call it (all of HBM is
already committed to a KV cache, or allocation after start-up is forbidden).
``b200_add_lora_bgmv_static`` serves them from a scratch array built into the library.  This
test calls it through the C ABI twice in a row - the second call finds the array holding the
first call's leftovers - and compares each result with the ordinary entry point on the same
inputs.  It is collected last so that a stop-at-first-failure run has seen every other test.
"""
import numpy as np
import pytest
import torch

import ae296_b200 as L
from lora_testlib import TOL
from oracle import lora_oracle as O

pytestmark = pytest.mark.gpu


def _inputs(seed, t, n, h_in, h_out, r, dtype):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(t, h_in, generator=g).to(dtype).cuda()
    wa = (torch.randn(n, 2, r, h_in, generator=g) / np.sqrt(h_in)).to(dtype).cuda()
    wb = (torch.randn(n, 2, h_out, r, generator=g) / np.sqrt(r)).to(dtype).cuda()
    ids = torch.randint(0, n, (t,), generator=g).cuda()
    y0 = torch.randn(t, h_out, generator=g).to(dtype).cuda()
    return x, wa, wb, ids, y0


def test_static_scratch_entry_point_matches_workspace_entry_point_twice():
    cases = [(101, 33, 6, 1024, 768, 16, torch.float16), (202, 64, 40, 4096, 4096, 64, torch.bfloat16)]
    for seed, t, n, h_in, h_out, r, dtype in cases:        # two calls in a row, different shapes
        x, wa, wb, ids, y0 = _inputs(seed, t, n, h_in, h_out, r, dtype)
        want = y0.clone()
        ws = torch.empty(L.add_lora_bgmv_workspace_bytes(t, n, h_in), dtype=torch.uint8, device="cuda")
        L.add_lora_bgmv_once(want, x, wa, wb, ids, 1, 0.5, ws)          # b200_add_lora_bgmv, caller's workspace
        got = y0.clone()
        before = torch.cuda.memory_allocated()
        L.add_lora_bgmv_static(got, x, wa, wb, ids, 1, 0.5)
        assert torch.cuda.memory_allocated() == before, "the static entry point must not allocate"
        torch.cuda.synchronize()
        L.add_lora_bgmv_static_status()
        # same kernels, same launch geometry, same summation order: the same bits
        assert torch.equal(got, want)
        # and the answer itself, against the float64 oracle: y0 + 0.5 * delta rounded once
        idn = ids.cpu().numpy()
        d = O.lora_delta(x.double().cpu().numpy(), lambda a: wa[a, 1].double().cpu().numpy(),
                         lambda a: wb[a, 1].double().cpu().numpy(), idn, np.full(n, 0.5))
        exact = y0.double().cpu().numpy() + d
        ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)
        assert np.abs(got.double().cpu().numpy() - exact).max() <= TOL * np.sqrt((d ** 2).mean()) + ulp * np.abs(exact).max()
    # a call beyond the stated limits is refused, not attempted
    x, wa, wb, ids, y0 = _inputs(303, 65, 4, 256, 256, 8, torch.float16)
    with pytest.raises(L.LoraError) as e:
        L.add_lora_bgmv_static(y0.clone(), x, wa, wb, ids, 0, 1.0)
    assert e.value.code == -6
    # an adapter id outside the pool: y stays as it was and the status call says why
    x, wa, wb, ids, y0 = _inputs(404, 16, 4, 256, 256, 8, torch.float16)
    ids[5] = 4
    y = y0.clone()
    L.add_lora_bgmv_static(y, x, wa, wb, ids, 0, 1.0)
    torch.cuda.synchronize()
    assert torch.equal(y, y0)
    with pytest.raises(L.LoraError) as e:
        L.add_lora_bgmv_static_status()
    assert e.value.code == -8
