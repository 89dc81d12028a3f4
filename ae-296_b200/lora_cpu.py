"""Host-side mirror of the reference's CPU-assisted LoRA object, on the native transport.

``Lora_CPU`` keeps the constructor keys and the two calls the layer code makes
(``invoke_lora_async(hidden_states, tkn_num, layer_id, lora_inds=None, is_o=False)`` and
``collect_qkv(tkn_num, batch_size, lora_inds=None) -> (q, k, v)``; lightllm/models/lora_cpu.py:138,187,
called from lightllm/models/llama/layer_infer/transformer_layer_infer.py:122-135).  The work those
methods do in Python in the reference - per-request device->host copies, three doorbell copies,
polling the signal table and pitched host->device copies of this rank's columns - runs in the C++
library (``b200_cpu_assist_invoke`` / ``b200_cpu_assist_collect_qkv``) with checked CUDA calls,
the caller's stream and a time limit on every wait.

``ShmSegments`` creates the shared-memory segments and their ``<tag>-<name>.shm`` name files the
way the reference's ``create_shm.py:38-130`` does, for tests and for the benchmark; a deployment
attaches to existing ones through ``shm_name_folder``.
"""
from __future__ import annotations

import ctypes as C
import os
import tempfile
from multiprocessing import shared_memory
from typing import Dict, Optional

import numpy as np
import torch

from . import _lib
from ._lib import LoraError, check

PROMPT_MAX_LENGTH = 256          # lightllm/models/lora_cpu.py:14
SEGMENTS = ["shm_array", "shm_out_q", "shm_out_k", "shm_out_v", "shm_out_o"]


class CpuAssist(C.Structure):
    _fields_ = [("shm_x", C.c_void_p), ("shm_out", C.c_void_p * 3), ("shm_signal", C.c_void_p),
                ("shm_tkn_len", C.c_void_p), ("lock", C.c_void_p), ("dev_numbers", C.c_void_p),
                ("lora_num", C.c_int32), ("prompt_max", C.c_int32), ("hidden", C.c_int32),
                ("tp_degree", C.c_int32), ("gpu_id", C.c_int32), ("n_layers", C.c_int32),
                ("token_per_lora", C.c_int32), ("host_copies", C.c_int32)]


class ShmSegments:
    """Owner of the seven segments (x, four outputs, token count, signals) and the lock."""

    def __init__(self, lora_num: int, hidden: int, prompt_max: int = PROMPT_MAX_LENGTH, folder: Optional[str] = None):
        self.folder = folder or tempfile.mkdtemp(prefix="shmnames")
        self.lora_num, self.hidden, self.prompt_max = lora_num, hidden, prompt_max
        self.shms: Dict[str, shared_memory.SharedMemory] = {}
        for name in SEGMENTS:
            self._make(name, 2 * lora_num * prompt_max * hidden)
        self._make("shm_tkn_len", 8)
        self._make("shm_signal", 2 * 3 * lora_num)
        self._make("lock", 8)
        sig = np.ndarray((3, lora_num), np.int16, buffer=self.shms["shm_signal"].buf)
        sig[:] = 1
        np.ndarray((1,), np.int64, buffer=self.shms["shm_tkn_len"].buf)[0] = 1
        del sig

    def _make(self, name, nbytes):
        s = shared_memory.SharedMemory(create=True, size=nbytes)
        self.shms[name] = s
        with open(os.path.join(self.folder, f"{name}-{s.name}.shm"), "w") as f:
            f.write(f"{name},{s.name}\n")

    def close(self):
        for s in self.shms.values():
            s.close()
            s.unlink()
        for f in os.listdir(self.folder):
            os.remove(os.path.join(self.folder, f))
        os.rmdir(self.folder)


def _attach(folder: str, tag: str) -> shared_memory.SharedMemory:
    files = [f for f in os.listdir(folder) if f.endswith(".shm") and tag in f]
    if len(files) != 1:
        raise FileNotFoundError(f"expected one '{tag}' name file in {folder}, found {len(files)}")
    return shared_memory.SharedMemory(name=files[0][:-4].split("-")[1])


class Lora_CPU:
    def __init__(self, configJson, gpu_id: int, shm_name_folder: Optional[str] = None, device=None,
                 timeout_s: float = 10.0, host_copies: bool = False):
        self.batch_size = configJson["batch_size"]
        self.lora_num = configJson["lora_num"]
        self.tp_degree = configJson["tp_degree"]
        self.hidden_dim = configJson["hidden_dim"]
        self.lora_rank = configJson["lora_rank"]
        self.cpu_capacity = configJson["token_per_lora"]
        self.n_layers = configJson["n_layers"]
        self.gpu_id = gpu_id
        self.out_size = self.hidden_dim // self.tp_degree
        self.timeout_us = int(timeout_s * 1e6)
        self.host_copies = bool(host_copies)
        self.prompt_max = int(configJson.get("prompt_max_length", PROMPT_MAX_LENGTH))
        folder = shm_name_folder or os.getenv("shm_name_folder")
        if not folder:
            raise ValueError("shm_name_folder (argument or environment variable) names the shared-memory segments")
        self._shms = {tag: _attach(folder, tag) for tag in ("shm_array", "shm_out_q", "shm_out_k", "shm_out_v",
                                                            "shm_signal", "shm_tkn_len", "lock")}
        self._np = {tag: np.ndarray((len(s.buf),), np.uint8, buffer=s.buf) for tag, s in self._shms.items()}
        ptr = {tag: a.ctypes.data for tag, a in self._np.items()}
        self.shm_signal = np.ndarray((3, self.lora_num), np.int16, buffer=self._shms["shm_signal"].buf)
        self._pinned = []
        if host_copies:
            self.device = torch.device("cpu")
            self.numbers = None
        else:
            self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
            # source of the doorbell values (lora_cpu.py:71-72)
            self.numbers = torch.arange(0, 1025, dtype=torch.int16, device=self.device)
            L = _lib.lib()
            for tag in ("shm_array", "shm_out_q", "shm_out_k", "shm_out_v", "shm_signal"):
                check(L.b200_xfer_register_pinned(ptr[tag], len(self._np[tag])), f"register_pinned({tag})")
                self._pinned.append(ptr[tag])
        self._c = CpuAssist(ptr["shm_array"], (C.c_void_p * 3)(ptr["shm_out_q"], ptr["shm_out_k"], ptr["shm_out_v"]),
                            ptr["shm_signal"], ptr["shm_tkn_len"], ptr["lock"],
                            self.numbers.data_ptr() if self.numbers is not None else None,
                            self.lora_num, self.prompt_max, self.hidden_dim, self.tp_degree, gpu_id, self.n_layers,
                            self.cpu_capacity, 1 if host_copies else 0)
        self.active_cpu = 0

    def _stream(self):
        return None if self.host_copies else torch.cuda.current_stream(self.device).cuda_stream

    def invoke_lora_async(self, hidden_states, tkn_num, layer_id, lora_inds=None, is_o=False):
        """``hidden_states [B * L, H]`` fp16 on this object's device, ``tkn_num = L``."""
        if hidden_states.dtype != torch.float16 or not hidden_states.is_contiguous():
            raise ValueError("hidden_states must be a contiguous fp16 tensor")
        if hidden_states.device.type != self.device.type:
            raise ValueError("hidden_states is not on this object's device")
        rows = hidden_states.numel() // self.hidden_dim
        batch = rows // tkn_num
        self.active_cpu = batch * ((tkn_num - 1) // self.cpu_capacity + 1)
        check(_lib.lib().b200_cpu_assist_invoke(C.byref(self._c), hidden_states.data_ptr(), rows, int(tkn_num), int(layer_id),
                                                self.timeout_us, self._stream()), "cpu_assist_invoke")

    def collect_qkv(self, tkn_num, batch_size, lora_inds=None):
        """Returns ``(q, k, v)``, each ``[batch_size, tkn_num, hidden/tp]`` fp16.  Raises ``LoraError``
        (code -11) when a worker did not answer within the time limit."""
        shape = (batch_size, tkn_num, self.out_size)
        q, k, v = (torch.zeros(shape, dtype=torch.float16, device=self.device) for _ in range(3))
        missing = C.c_int32(0)
        rc = _lib.lib().b200_cpu_assist_collect_qkv(C.byref(self._c), q.data_ptr(), k.data_ptr(), v.data_ptr(), int(tkn_num),
                                                    int(batch_size), self.timeout_us, C.byref(missing), self._stream())
        if rc != 0:
            raise LoraError(rc, f"cpu_assist_collect_qkv: {missing.value} worker job(s) did not answer")
        return q, k, v

    def close(self):
        L = _lib.lib()
        for p in self._pinned:
            L.b200_xfer_unregister_pinned(p)
        self._pinned = []
        self._np = {}
        self.shm_signal = None
        for s in self._shms.values():
            s.close()
        self._shms = {}
