"""Regenerates the golden vectors under tests/golden/ from the reference itself.

Run where the reference tree is mounted:

    python tests/golden/make_golden.py --reference <path of the reference checkout>

Two reference code paths run without a GPU and are executed UNMODIFIED here:

* ``LoRAapp.run`` (lora_cpu/lora_shm_op/app.py:102-154): real worker
  processes attached to real POSIX shared memory, woken by the int16 doorbell
  values the host side writes (lightllm/models/lora_cpu.py:181-185).  Only the
  eight weight attributes are overwritten with seeded weights, and the GPU
  copies of the host side are replaced by host writes.
* ``Lora_GPU.invoke_one_layer_q(x, layer, prefill=True)``
  (lightllm/models/lora_gpu.py:122-128): the object is created without its
  constructor (which needs a GPU, zmq ports and the absent ``punica`` module)
  and given CPU pools, so the method's own ``torch.bmm`` pair produces the
  vector.

The decode BGMV op lives in ``punica`` (not in the tree): nothing here pins it.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
import multiprocessing as mp
import os
import sys
import tempfile
import time
import types
from multiprocessing import shared_memory

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


# ---------------------------------------------------------------------------------
# reference worker harness
# ---------------------------------------------------------------------------------

SEGMENTS = ["shm_array", "shm_out_q", "shm_out_k", "shm_out_v", "shm_out_o"]


def _worker_main(ref_root, folder, ns, weights):
    sys.path.insert(0, os.path.join(ref_root, "lora_cpu", "lora_shm_op"))
    spec = importlib.util.spec_from_file_location(
        "ref_lora_app", os.path.join(ref_root, "lora_cpu", "lora_shm_op", "app.py"))
    app = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(app)
    app.args = ns                       # module global read by init_shm
    sys.stdout = open(os.devnull, "w")
    torch.set_num_threads(1)
    w = app.LoRAapp(ns, folder)
    for k, v in weights.items():
        setattr(w, k, v)
    w.run()


class ReferenceWorkers:
    """Owns the shared-memory segments and a set of reference worker processes."""

    def __init__(self, ref_root, n_rows, max_len, hidden, rank, offset):
        self.ref_root, self.n_rows, self.max_len, self.hidden = ref_root, n_rows, max_len, hidden
        self.rank, self.offset = rank, offset
        self.folder = tempfile.mkdtemp(prefix="shmnames")
        self.shms = {}
        nbytes = 2 * n_rows * max_len * hidden
        for name in SEGMENTS:
            self._make(name, nbytes)
        self._make("shm_tkn_len", 8)
        self._make("shm_signal", 2 * 3 * n_rows)
        self.arr = {n: np.ndarray((n_rows, max_len, hidden), np.float16, buffer=self.shms[n].buf)
                    for n in SEGMENTS}
        self.signal = np.ndarray((3 * n_rows,), np.int16, buffer=self.shms["shm_signal"].buf)
        self.signal[:] = 1
        self.tkn_len = np.ndarray((1,), np.int64, buffer=self.shms["shm_tkn_len"].buf)
        self.procs = []

    def _make(self, name, nbytes):
        s = shared_memory.SharedMemory(create=True, size=nbytes)
        self.shms[name] = s
        with open(os.path.join(self.folder, f"{name}-{s.name}.shm"), "w") as f:
            f.write(f"{name},{s.name}\n")

    def spawn(self, row, weights):
        ns = types.SimpleNamespace(
            in_size=self.hidden, out_size=self.hidden, batch_size=self.n_rows, signal_name=None,
            rank=self.rank, prompt_max_length=self.max_len, signal_index=row, offset=self.offset)
        p = mp.get_context("fork").Process(target=_worker_main,
                                            args=(self.ref_root, self.folder, ns, weights), daemon=True)
        p.start()
        self.procs.append(p)

    def ring(self, row, base, timeout=60.0):
        """Doorbell value ``base + row`` into slot ``row``; wait for the ack (0)."""
        self.signal[row] = base + row
        t0 = time.time()
        while self.signal[row] != 0:
            if time.time() - t0 > timeout:
                raise TimeoutError("reference worker did not acknowledge")
        self.signal[row] = 1

    def close(self):
        for p in self.procs:
            p.terminate()
        for p in self.procs:
            p.join()
        del self.arr, self.signal, self.tkn_len
        for s in self.shms.values():
            s.close()
            s.unlink()
        for f in os.listdir(self.folder):
            os.remove(os.path.join(self.folder, f))
        os.rmdir(self.folder)


def run_reference_workers(ref_root, x_req, adapters_of_row, weights_of_adapter, rank, wave=6):
    """x_req [B, L, H] fp16; returns dict q/k/v -> [B, L, H] fp16 computed by the
    reference's worker processes, ``wave`` rows at a time."""
    B, L, H = x_req.shape
    rw = ReferenceWorkers(ref_root, B, max(L, 1), H, rank, offset=max(L, 1))
    out = {}
    try:
        rw.tkn_len[0] = L
        rw.arr["shm_array"][:, :L, :] = x_req
        for r0 in range(0, B, wave):
            rows = list(range(r0, min(B, r0 + wave)))
            for row in rows:
                wq = weights_of_adapter(adapters_of_row[row])
                rw.spawn(row, wq)
            for base in (2, 202, 402):
                for row in rows:
                    rw.ring(row, base)
            for p in rw.procs:
                p.terminate()
            for p in rw.procs:
                p.join()
            rw.procs = []
        for nm, seg in (("q", "shm_out_q"), ("k", "shm_out_k"), ("v", "shm_out_v")):
            out[nm] = rw.arr[seg][:, :L, :].copy()
    finally:
        rw.close()
    return out


# ---------------------------------------------------------------------------------
# cases
# ---------------------------------------------------------------------------------

def worker_case(ref_root, seed, B, L, H, n_adapters, rank, store_inputs):
    g = torch.Generator().manual_seed(seed)
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, n_adapters, B).astype(np.int32)
    x = torch.randn(B, L, H, generator=g).half()
    W = {}
    for a in range(n_adapters):
        for nm in "qkv":
            down = (torch.randn(rank, H, generator=g) / np.sqrt(H)).half()      # A_a  [r, H]
            up = (torch.randn(H, rank, generator=g) / np.sqrt(rank)).half()     # B_a  [H, r]
            W[(a, nm)] = (down, up)

    def weights_of(a):
        d = {}
        for nm in "qkv":
            down, up = W[(int(a), nm)]
            d[f"{nm}_down_LoRA"] = down.float().t().contiguous()     # [H, r] fp32
            d[f"{nm}_up_LoRA"] = up.float().t().contiguous()         # [r, H] fp32
        return d

    out = run_reference_workers(ref_root, x.numpy(), ids, weights_of, rank)
    rec = {"seed": np.int64(seed), "ids": ids, "dims": np.array([B, L, H, n_adapters, rank], np.int64),
           "x_sha": sha(x.numpy())}
    for nm in "qkv":
        rec[f"out_{nm}_sha"] = sha(out[nm])
        wa = torch.stack([W[(a, nm)][0] for a in range(n_adapters)]).numpy()
        wb = torch.stack([W[(a, nm)][1] for a in range(n_adapters)]).numpy()
        rec[f"wa_{nm}_sha"], rec[f"wb_{nm}_sha"] = sha(wa), sha(wb)
        if store_inputs:
            rec[f"wa_{nm}"], rec[f"wb_{nm}"] = wa, wb
            rec[f"out_{nm}"] = out[nm]
        else:
            rec[f"out_{nm}_cols"] = out[nm][:, :, ::64].copy()       # every 64th column
    if store_inputs:
        rec["x"] = x.numpy()
    return rec


def regenerate_worker_inputs(seed, B, L, H, n_adapters, rank):
    """Same draws as ``worker_case``; used by tests for the seed-only fixture."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, L, H, generator=g).half()
    wa = {nm: [] for nm in "qkv"}
    wb = {nm: [] for nm in "qkv"}
    for a in range(n_adapters):
        for nm in "qkv":
            wa[nm].append((torch.randn(rank, H, generator=g) / np.sqrt(H)).half())
            wb[nm].append((torch.randn(H, rank, generator=g) / np.sqrt(rank)).half())
    return x, {k: torch.stack(v) for k, v in wa.items()}, {k: torch.stack(v) for k, v in wb.items()}


def bmm_case(ref_root, seed, B, L, H, rank, n_layers, layer):
    sys.modules.setdefault("punica", types.ModuleType("punica"))       # absent third-party module
    spec = importlib.util.spec_from_file_location(
        "ref_lora_gpu", os.path.join(ref_root, "lightllm", "models", "lora_gpu.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, L, H, generator=g).half()
    wa = (torch.randn(B, n_layers, rank, H, generator=g) / np.sqrt(H)).half()
    wb = (torch.randn(B, n_layers, H, rank, generator=g) / np.sqrt(rank)).half()
    obj = mod.Lora_GPU.__new__(mod.Lora_GPU)
    obj.q_down_prefill, obj.q_up_prefill = wa, wb
    obj.select_inds = [torch.zeros(i + 1, dtype=torch.int64) for i in range(B)]
    y = obj.invoke_one_layer_q(x, layer, prefill=True)
    return {"seed": np.int64(seed), "dims": np.array([B, L, H, rank, n_layers, layer], np.int64),
            "x": x.numpy(), "wa": wa.numpy(), "wb": wb.numpy(), "y": y.numpy()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    args = ap.parse_args()
    torch.manual_seed(0)

    small = worker_case(args.reference, seed=29600, B=5, L=24, H=256, n_adapters=3, rank=8, store_inputs=True)
    np.savez_compressed(os.path.join(HERE, "worker_small.npz"), **small)

    # decode workload 0 at full width: 32 one-token requests, 8 adapters, rank 16;
    # inputs are regenerated from the seed, outputs kept as digests + a column sample
    cfg0 = worker_case(args.reference, seed=2960, B=32, L=1, H=4096, n_adapters=8, rank=16, store_inputs=False)
    np.savez_compressed(os.path.join(HERE, "worker_decode4096.npz"), **cfg0)

    bmm = bmm_case(args.reference, seed=29601, B=3, L=40, H=256, rank=16, n_layers=2, layer=1)
    np.savez_compressed(os.path.join(HERE, "prefill_bmm_small.npz"), **bmm)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
