"""B200-native (sm_100a) multi-LoRA delta ``y += scale_a * (x @ A_a^T) @ B_a^T``.

The arithmetic lives in ``lib/libb200lora.so`` (hand-written CUDA behind the C ABI of
``include/b200_lora.h``); this package is the Python host side that mirrors the
interface of the reference's LoRA layer objects.
"""
from . import workloads                                      # noqa: F401
from .pool import AdapterPool, MAX_RANK                      # noqa: F401
from ._lib import LoraError, MID_ROUND, NO_TENSOR, DELTA_THEN_ADD   # noqa: F401
from .ops import (LoraBatch, LoraPlan, LoraWorkspace, add_lora_bgmv, add_lora_bgmv_once,   # noqa: F401
                  add_lora_bgmv_static, add_lora_bgmv_static_status, add_lora_bgmv_v2, add_lora_sgmv,
                  add_lora_bgmv_workspace_bytes, adapters_of, apply, invalidate_plan_cache)
from . import ops                                            # noqa: F401
from .lora_gpu import Lora_GPU                               # noqa: F401
from .lora_cpu import Lora_CPU, ShmSegments                  # noqa: F401
from .placement import place_by_adapter                      # noqa: F401
