"""ctypes binding of ``libb200lora.so`` (the C ABI declared in ``include/b200_lora.h``).

There is no fallback: if the library is missing or fails to load, importing the
ops raises.  Nothing here touches the GPU; loading the library and resolving
its symbols works on a machine without one.
"""
from __future__ import annotations

import ctypes as C
import os

from .build import LIB_PATH

F16, BF16, F32 = 0, 1, 2
MID_ROUND, NO_TENSOR, ONLY_SHRINK, ONLY_EXPAND, DELTA_THEN_ADD, KEEP_PARTIALS = 1, 2, 4, 8, 32, 64
MAX_RANK, MAX_PROJ = 64, 4

STATUS = {
    0: "ok", -1: "null pointer", -2: "bad dimension", -3: "unsupported dtype", -4: "misaligned pointer",
    -5: "rank out of range", -6: "plan/workspace too small", -7: "CUDA error", -8: "adapter id out of range",
    -9: "layer out of range", -10: "bad segment table", -11: "device wait timed out", -12: "unsupported",
}


class LoraError(RuntimeError):
    def __init__(self, code: int, what: str = ""):
        self.code = code
        detail = STATUS.get(code, "unknown")
        if code == -7:
            detail += ": " + lib().b200_lora_last_cuda_error().decode()
        super().__init__(f"b200_lora status {code} ({detail}) {what}".strip())


class Adapters(C.Structure):
    _fields_ = [("ranks", C.c_void_p), ("scalings", C.c_void_p), ("cum_ranks", C.c_void_p),
                ("n_adapters", C.c_int32), ("n_layers", C.c_int32), ("r_pool", C.c_int32),
                ("packed", C.c_int32), ("scale", C.c_float), ("ranks_pow2", C.c_int32), ("total_rank", C.c_int64)]


class TpContext(C.Structure):
    _fields_ = [("landing", (C.c_void_p * 2) * 8), ("flags", C.c_void_p * 8), ("tp", C.c_int32), ("rank", C.c_int32),
                ("set_stride", C.c_size_t)]


class Proj(C.Structure):
    _fields_ = [("x", C.c_void_p), ("y", C.c_void_p), ("wa", C.c_void_p), ("wb", C.c_void_p),
                ("ldx", C.c_int64), ("ldy", C.c_int64), ("h_in", C.c_int32), ("h_out", C.c_int32)]


# name -> (restype, argtypes); every symbol the headers under include/ declare
SYMBOLS = {
    "b200_lora_arch": (C.c_int, []),
    "b200_lora_last_cuda_error": (C.c_char_p, []),
    "b200_lora_stream_capture_id": (C.c_int, [C.c_void_p, C.POINTER(C.c_ulonglong)]),
    "b200_lora_plan_bytes": (C.c_size_t, [C.c_int32, C.c_int32]),
    "b200_lora_plan_build": (C.c_int, [C.c_void_p, C.c_size_t, C.c_int32, C.c_void_p, C.c_int32, C.c_int32,
                                       C.POINTER(Adapters), C.c_void_p]),
    "b200_lora_plan_from_segments": (C.c_int, [C.c_void_p, C.c_size_t, C.c_int32, C.c_void_p, C.c_void_p,
                                               C.c_int32, C.c_int32, C.POINTER(Adapters), C.c_void_p]),
    "b200_lora_plan_read": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.c_void_p]),
    "b200_lora_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    "b200_lora_workspace_init": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200_lora_workspace_v_region": (C.c_int, [C.c_int32, C.c_int32, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "b200_lora_workspace_status": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_lora_apply": (C.c_int, [C.POINTER(Proj), C.c_int32, C.POINTER(Adapters), C.c_void_p, C.c_int32,
                                  C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                  C.c_size_t, C.c_void_p]),
    "b200_add_lora_bgmv_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    "b200_add_lora_bgmv": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                     C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                     C.c_int32, C.c_float, C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200_add_lora_bgmv_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                            C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                            C.c_int32, C.c_float, C.c_int32, C.c_void_p]),
    "b200_add_lora_bgmv_static_status": (C.c_int, [C.c_void_p]),
    "b200_lora_tp_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    "b200_lora_tp_alloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "b200_lora_tp_free": (C.c_int, [C.c_void_p]),
    "b200_lora_tp_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200_lora_tp_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "b200_lora_tp_close": (C.c_int, [C.c_void_p]),
    "b200_lora_tp_layout": (C.c_int, [C.POINTER(TpContext), C.c_int32, C.c_void_p, C.c_int32, C.c_int32]),
    "b200_lora_tp_exchange": (C.c_int, [C.POINTER(TpContext), C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                        C.c_void_p]),
    "b200_lora_apply_tp": (C.c_int, [C.POINTER(Proj), C.c_int32, C.POINTER(Adapters), C.c_void_p, C.c_int32,
                                     C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                     C.c_size_t, C.POINTER(TpContext), C.c_int32, C.c_void_p]),
    # include/b200_cpu_assist.h
    "b200_xfer_register_pinned": (C.c_int, [C.c_void_p, C.c_size_t]),
    "b200_xfer_unregister_pinned": (C.c_int, [C.c_void_p]),
    "b200_xfer_d2h_async": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200_xfer_signal_d2h_async": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200_xfer_d2h_with_signal_async": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t,
                                                  C.c_void_p, C.c_void_p]),
    "b200_xfer_h2d_async": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]),
    "b200_xfer_h2d_2d_async": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                         C.c_size_t, C.c_void_p]),
    "b200_xfer_stream_synchronize": (C.c_int, [C.c_void_p]),
    "b200_cpu_assist_invoke": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_void_p]),
    "b200_cpu_assist_collect_qkv": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                              C.c_int64, C.POINTER(C.c_int32), C.c_void_p]),
}

_LIB = None


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m ae296_b200.build` "
                "(there is no CPU or PyTorch fallback for the LoRA kernels)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)      # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = res, args
        _LIB = handle
    return _LIB


def check(code: int, what: str = "") -> None:
    if code != 0:
        raise LoraError(code, what)
