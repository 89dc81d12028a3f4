"""CPU: the C-ABI library loads, exports every declared symbol and validates its arguments.

No kernel is launched here; argument checks happen before any CUDA call."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = "".join(open(os.path.join(ROOT, "include", h)).read() for h in sorted(os.listdir(os.path.join(ROOT, "include"))))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    names = declared_symbols()
    assert len(names) >= 12
    from ae296_b200 import _lib
    assert sorted(_lib.SYMBOLS) == names, "ctypes table and header disagree"
    for n in names:
        assert getattr(lib, n) is not None


def test_sizes_and_identification(lib):
    assert lib.b200_lora_arch() == 100
    assert lib.b200_lora_plan_bytes(256, 128) > 256 * 4 * 16
    assert lib.b200_lora_plan_bytes(0, 4) == 0
    assert lib.b200_lora_workspace_bytes(256, 3, 4096) > 3 * 256 * 64 * 4
    assert lib.b200_lora_workspace_bytes(256, 5, 4096) == 0          # more than 4 projections
    off, size = C.c_size_t(0), C.c_size_t(0)
    assert lib.b200_lora_workspace_v_region(256, 3, C.byref(off), C.byref(size)) == 0
    assert off.value % 128 == 0 and size.value == 3 * 256 * 64 * 4
    assert off.value + size.value <= lib.b200_lora_workspace_bytes(256, 3, 4096)


def test_argument_errors_come_back_as_status_codes(lib):
    from ae296_b200._lib import Adapters, Proj
    ad = Adapters(None, None, None, 4, 2, 16, 0, 1.0, 0, 0)
    assert lib.b200_lora_plan_build(None, 0, 8, None, 0, 8, C.byref(ad), None) == -1          # null
    bad = Adapters(None, None, None, 4, 2, 80, 0, 1.0, 0, 0)
    assert lib.b200_lora_plan_build(C.c_void_p(256), 1 << 20, 8, C.c_void_p(256), 0, 8, C.byref(bad), None) == -5
    assert lib.b200_lora_plan_build(C.c_void_p(256), 16, 8, C.c_void_p(256), 0, 8, C.byref(ad), None) == -6
    assert lib.b200_lora_plan_build(C.c_void_p(256), 1 << 20, 8, C.c_void_p(256), 0, 9, C.byref(ad), None) == -2
    pj = (Proj * 1)(Proj(256, 256, 256, 256, 128, 128, 128, 128))
    big = 1 << 30
    args = (pj, 1, C.byref(ad), C.c_void_p(256), 8, 8)
    assert lib.b200_lora_apply(*args, 2, 0, 0, 0, C.c_void_p(256), big, None) == -9           # layer >= L
    assert lib.b200_lora_apply(*args, 0, 2, 0, 0, C.c_void_p(256), big, None) == -3           # fp32 inputs
    assert lib.b200_lora_apply(*args, 0, 0, 0, 0, C.c_void_p(256), 64, None) == -6            # workspace too small
    odd = (Proj * 1)(Proj(256, 256, 256, 256, 132, 128, 132, 128))
    assert lib.b200_lora_apply(odd, 1, C.byref(ad), C.c_void_p(256), 8, 8, 0, 0, 0, 0, C.c_void_p(256), big, None) == -2
    mis = (Proj * 1)(Proj(260, 256, 256, 256, 128, 128, 128, 128))
    assert lib.b200_lora_apply(mis, 1, C.byref(ad), C.c_void_p(256), 8, 8, 0, 0, 0, 0, C.c_void_p(256), big, None) == -4
    # the allocation-free entry point refuses sizes beyond its static scratch
    assert lib.b200_add_lora_bgmv_static(None, None, None, None, None, 0, 65, 256, 256, 4, 1, 8, 0, 1.0, 0, None) == -6


def test_missing_library_fails_loudly(monkeypatch):
    from ae296_b200 import _lib
    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libb200lora.so")
    with pytest.raises(ImportError):
        _lib.lib()


def test_tensor_parallel_entry_points_check_their_arguments(lib):
    """Host-only parts of the tensor-parallel ABI: buffer size, layout arithmetic, argument checks."""
    from ae296_b200._lib import Adapters, Proj, TpContext
    assert lib.b200_lora_tp_bytes(256, 3, 1) == 0 and lib.b200_lora_tp_bytes(256, 3, 9) == 0      # 2..8 ranks
    assert lib.b200_lora_tp_bytes(256, 5, 2) == 0
    # two sets of two landing buffers of (tp + 1) slots of 8-byte packets, then the counter block
    slot = 3 * 256 * 64 * 8
    assert lib.b200_lora_tp_bytes(256, 3, 4) == 4 * 5 * slot + 24576
    ctx = TpContext()
    ctx.tp, ctx.rank = 4, 1
    base = 1 << 30
    for r in range(4):
        assert lib.b200_lora_tp_layout(C.byref(ctx), r, C.c_void_p(base * (r + 1)), 256, 3) == 0
        assert ctx.landing[r][0] == base * (r + 1) and ctx.landing[r][1] == base * (r + 1) + 5 * slot
        assert ctx.flags[r] == base * (r + 1) + 4 * 5 * slot
    assert ctx.set_stride == 2 * 5 * slot
    assert lib.b200_lora_tp_layout(C.byref(ctx), 8, C.c_void_p(base), 256, 3) == -2
    assert lib.b200_lora_tp_layout(None, 0, C.c_void_p(base), 256, 3) == -1
    ad = Adapters(None, None, None, 4, 2, 16, 0, 1.0, 0, 0)
    pj = (Proj * 1)(Proj(256, 256, 256, 256, 128, 128, 128, 128))
    big = 1 << 30
    args = (pj, 1, C.byref(ad), C.c_void_p(256), 8, 8, 0, 0, 0)
    assert lib.b200_lora_apply_tp(*args, 0, C.c_void_p(256), big, None, 0, None) == -1          # no context
    from ae296_b200 import _lib
    for half in (_lib.ONLY_SHRINK, _lib.ONLY_EXPAND):                                               # the call runs both halves itself
        assert lib.b200_lora_apply_tp(*args, half, C.c_void_p(256), big, C.byref(ctx), 0, None) == -2
    one = TpContext()
    one.tp, one.rank = 1, 0
    assert lib.b200_lora_apply_tp(*args, 0, C.c_void_p(256), big, C.byref(one), 0, None) == -2    # fewer than two ranks
    hole = TpContext()
    hole.tp, hole.rank, hole.set_stride = 2, 0, 1024
    assert lib.b200_lora_apply_tp(*args, 0, C.c_void_p(256), big, C.byref(hole), 0, None) == -2   # unmapped peers
    assert lib.b200_lora_tp_exchange(C.byref(hole), C.c_void_p(256), 8, 8, 1, 0, None) == -1
