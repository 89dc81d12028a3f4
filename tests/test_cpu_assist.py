"""The CPU-assisted transport (include/b200_cpu_assist.h) and its Python mirror ``Lora_CPU``.

CPU tests drive the whole protocol with memcpy copies (``host_copies``) against worker processes - the
reference's unmodified ``LoRAapp.run`` where ``oracle/_ref/app.py`` has been fetched, else threads that
restate it with the oracle - and make failures on the host (a worker that never answers, a rank that never
publishes its layer).  GPU tests run the same protocol with CUDA copies and check the raw copy entry points
byte for byte."""
import ctypes as C
import threading
import time

import numpy as np
import pytest
import torch

import ae296_b200 as L
from ae296_b200 import _lib
from ae296_b200.lora_cpu import CpuAssist, Lora_CPU, ShmSegments
from oracle import lora_oracle as O
from oracle import ref_worker_baseline as RW


def weights_of(seed, hidden, rank):
    """The draw of ``oracle/ref_worker_baseline._worker_main`` for one worker."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for nm in "qkvo":
        w[nm] = (torch.randn(hidden, rank, generator=g) / np.sqrt(hidden), torch.randn(rank, hidden, generator=g) / np.sqrt(rank))
    return w


class PortWorkers:
    """Threads that restate the reference's worker loop (lora_cpu/lora_shm_op/app.py:102-143) with the
    oracle's arithmetic; worker ``i`` listens on signal slot ``i`` of the flat [3 * n] table."""

    def __init__(self, segs: ShmSegments, n, hidden, rank, seed, dead=()):
        self.stop = False
        sig = np.ndarray((3 * n,), np.int16, buffer=segs.shms["shm_signal"].buf)
        tkn = np.ndarray((1,), np.int64, buffer=segs.shms["shm_tkn_len"].buf)
        x = np.ndarray((n, segs.prompt_max, hidden), np.float16, buffer=segs.shms["shm_array"].buf)
        outs = {nm: np.ndarray((n, segs.prompt_max, hidden), np.float16, buffer=segs.shms[f"shm_out_{nm}"].buf) for nm in "qkv"}
        self.views = (sig, tkn, x, outs)

        def loop(i):
            w = weights_of(seed + i, hidden, rank)
            while not self.stop:
                s = int(sig[i])
                if s > 1:
                    nm, row = ("q", s - 2) if s < 202 else ("k", s - 202) if s < 402 else ("v", s - 402)
                    t = int(tkn[0])
                    res = O.cpu_worker(torch.from_numpy(x[row, :t].copy()), *w[nm])
                    outs[nm][row, :t] = res.numpy()
                    sig[i] = 0
                else:
                    time.sleep(0.0002)

        self.threads = [threading.Thread(target=loop, args=(i,), daemon=True) for i in range(3 * n) if i not in dead]
        for t in self.threads:
            t.start()

    def close(self):
        self.stop = True
        for t in self.threads:
            t.join(timeout=5)
        self.views = None


def cfg(n, hidden, tp=1, cap=8, prompt_max=16, n_layers=4):
    return {"batch_size": n, "lora_num": n, "tp_degree": tp, "hidden_dim": hidden, "lora_rank": 8, "token_per_lora": cap,
            "n_layers": n_layers, "prompt_max_length": prompt_max}


def expected(x, n, tkn, hidden, rank, seed, nm, tp, gpu_id):
    p = "qkv".index(nm)
    out = torch.stack([O.cpu_worker(x[b], *weights_of(seed + p * n + b, hidden, rank)[nm]) for b in range(n)])
    w = hidden // tp
    return out[:, :, gpu_id * w:(gpu_id + 1) * w]


@pytest.mark.parametrize("tp", [1, 2, 4])
def test_protocol_round_trip_with_host_copies_against_port_workers(tp):
    n, hidden, rank, tkn, seed = 3, 64, 8, 5, 900
    segs = ShmSegments(n, hidden, prompt_max=16)
    workers = PortWorkers(segs, n, hidden, rank, seed)
    try:
        ranks = [Lora_CPU(cfg(n, hidden, tp), g, shm_name_folder=segs.folder, host_copies=True, timeout_s=20) for g in range(tp)]
        x = torch.randn(n * tkn, hidden, generator=torch.Generator().manual_seed(1)).half()
        for layer in (0, 1):
            for r in ranks:                                   # rank 0 ships x and rings; the others wait for the layer
                r.invoke_lora_async(x, tkn, layer)
            for g, r in enumerate(ranks):
                q, k, v = r.collect_qkv(tkn, n)
                for nm, got in zip("qkv", (q, k, v)):
                    want = expected(x.view(n, tkn, hidden), n, tkn, hidden, rank, seed, nm, tp, g)
                    assert got.shape == (n, tkn, hidden // tp)
                    assert torch.equal(got, want), (nm, g)    # copies are byte-exact
        for r in ranks:
            r.close()
    finally:
        workers.close()
        segs.close()


@pytest.mark.skipif(not RW.available(), reason="oracle/_ref/app.py not fetched")
def test_protocol_round_trip_against_the_reference_worker_processes():
    n, hidden, rank, tkn, seed = 2, 128, 8, 3, 300
    pool = RW.ReferenceWorkerPool(hidden, 4, [rank] * (3 * n), seed=seed)
    try:
        pool.wait_ready()
        lc = Lora_CPU({"batch_size": n, "lora_num": n, "tp_degree": 1, "hidden_dim": hidden, "lora_rank": rank,
                       "token_per_lora": 4, "n_layers": 2, "prompt_max_length": 4}, 0, shm_name_folder=pool.folder,
                      host_copies=True, timeout_s=30)
        x = torch.randn(n * tkn, hidden, generator=torch.Generator().manual_seed(2)).half()
        lc.invoke_lora_async(x, tkn, 0)
        q, k, v = lc.collect_qkv(tkn, n)
        for nm, got in zip("qkv", (q, k, v)):
            assert torch.equal(got, expected(x.view(n, tkn, hidden), n, tkn, hidden, rank, seed, nm, 1, 0)), nm
        lc.close()
    finally:
        pool.close()


def test_dead_worker_is_a_status_not_a_hang():
    n, hidden, rank, tkn = 2, 64, 8, 2
    segs = ShmSegments(n, hidden, prompt_max=8)
    workers = PortWorkers(segs, n, hidden, rank, 5, dead={1, 4})          # q of request 1 and v of request 0 never answer
    try:
        lc = Lora_CPU(cfg(n, hidden, prompt_max=8), 0, shm_name_folder=segs.folder, host_copies=True, timeout_s=0.3)
        lc.invoke_lora_async(torch.zeros(n * tkn, hidden, dtype=torch.float16), tkn, 0)
        t0 = time.time()
        with pytest.raises(L.LoraError) as e:
            lc.collect_qkv(tkn, n)
        assert e.value.code == -11 and "2 worker job" in str(e.value)
        assert time.time() - t0 < 5
        lc.close()
    finally:
        workers.close()
        segs.close()


def test_rank_that_never_sees_its_layer_times_out_and_bad_shapes_are_refused():
    n, hidden = 2, 64
    segs = ShmSegments(n, hidden, prompt_max=8)
    try:
        r1 = Lora_CPU(cfg(n, hidden, tp=2, prompt_max=8), 1, shm_name_folder=segs.folder, host_copies=True, timeout_s=0.2)
        x = torch.zeros(n * 2, hidden, dtype=torch.float16)
        with pytest.raises(L.LoraError) as e:
            r1.invoke_lora_async(x, 2, 3)                      # rank 0 never published layer 3
        assert e.value.code == -11
        r0 = Lora_CPU(cfg(n, hidden, tp=2, prompt_max=8), 0, shm_name_folder=segs.folder, host_copies=True, timeout_s=0.2)
        r0.invoke_lora_async(x, 2, 3)
        r1.invoke_lora_async(x, 2, 3)                          # now it returns
        with pytest.raises(L.LoraError) as e:
            r0.invoke_lora_async(torch.zeros(3 * 9, hidden, dtype=torch.float16), 9, 0)   # longer than the segment's rows
        assert e.value.code == -2
        with pytest.raises(L.LoraError) as e:
            r0.invoke_lora_async(torch.zeros(3 * 2, hidden, dtype=torch.float16), 2, 0)   # more requests than worker slots
        assert e.value.code == -2
        c = CpuAssist()
        assert _lib.lib().b200_cpu_assist_invoke(C.byref(c), None, 2, 2, 0, 0, None) == -1
        r0.close(); r1.close()
    finally:
        segs.close()


# ---- GPU ------------------------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("tp", [1, 2, 4])
def test_gpu_protocol_round_trip_and_column_slices(tp):
    n, hidden, rank, tkn, seed = 3, 256, 8, 6, 40
    segs = ShmSegments(n, hidden, prompt_max=8)
    workers = PortWorkers(segs, n, hidden, rank, seed)
    try:
        ranks = [Lora_CPU(cfg(n, hidden, tp, prompt_max=8), g, shm_name_folder=segs.folder, timeout_s=30) for g in range(tp)]
        x = torch.randn(n * tkn, hidden, generator=torch.Generator().manual_seed(3)).half()
        xd = x.cuda()
        for r in ranks:
            r.invoke_lora_async(xd, tkn, 1)
        for g, r in enumerate(ranks):
            q, k, v = r.collect_qkv(tkn, n)
            torch.cuda.synchronize()
            for nm, got in zip("qkv", (q, k, v)):
                assert torch.equal(got.cpu(), expected(x.view(n, tkn, hidden), n, tkn, hidden, rank, seed, nm, tp, g)), (nm, g)
        # the CPU-assisted delta and the GPU op agree on the same inputs (fp16 output of fp32-or-better sums)
        w = [weights_of(seed + b, hidden, rank)["q"] for b in range(n)]
        wa = torch.stack([d.t().contiguous().half() for d, _ in w]).unsqueeze(1).cuda()           # [n, 1, r, H]
        wb = torch.stack([u.t().contiguous().half() for _, u in w]).unsqueeze(1).cuda()           # [n, 1, H, r]
        y = torch.zeros(n * tkn, hidden, dtype=torch.float16, device="cuda")
        L.add_lora_bgmv(y, xd, wa, wb, torch.arange(n, device="cuda").repeat_interleave(tkn), 0, 1.0)
        torch.cuda.synchronize()
        ref = expected(x.view(n, tkn, hidden), n, tkn, hidden, rank, seed, "q", 1, 0).reshape(n * tkn, hidden).float()
        rms = float(ref.pow(2).mean().sqrt())
        # the worker's weights are fp32, the GPU pool holds their fp16 roundings: one input rounding apart
        assert float((y.cpu().float() - ref).abs().max()) <= 2e-3 * rms + float(ref.abs().max()) * 2 ** -9
        for r in ranks:
            r.close()
    finally:
        workers.close()
        segs.close()


@pytest.mark.gpu
def test_gpu_raw_copies_are_byte_exact_and_the_doorbell_follows_the_data():
    lib = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    rows, width, pitch = 37, 96, 160                              # elements
    host = torch.arange(rows * pitch, dtype=torch.int16).view(rows, pitch).pin_memory()
    dev = torch.zeros(4 + rows * width, dtype=torch.int16, device="cuda")
    assert lib.b200_xfer_h2d_2d_async(host.data_ptr() + 2 * 11, dev.data_ptr(), 2 * pitch, 2 * width, 2 * width, rows, 4, stream) == 0
    assert lib.b200_xfer_stream_synchronize(stream) == 0
    assert torch.equal(dev[4:].view(rows, width).cpu(), host[:, 11:11 + width])
    assert not dev[:4].any()
    assert lib.b200_xfer_h2d_2d_async(host.data_ptr(), dev.data_ptr(), 2 * width, 2 * width, 2 * pitch, rows, 0, stream) == -2   # wider than the pitch
    # a large device -> host copy, then the doorbell: when the doorbell is seen, the data is all there
    big = torch.randint(-30000, 30000, (64 << 20,), dtype=torch.int16, device="cuda")
    out = torch.zeros(big.numel() - 8, dtype=torch.int16).pin_memory()
    sig = torch.ones(4, dtype=torch.int16).pin_memory()
    numbers = torch.arange(0, 1025, dtype=torch.int16, device="cuda")
    torch.cuda.synchronize()
    assert lib.b200_xfer_d2h_async(big.data_ptr(), 8, out.data_ptr(), 2 * out.numel(), stream) == 0
    assert lib.b200_xfer_signal_d2h_async(numbers.data_ptr(), 402, sig.data_ptr() + 2, 4, stream) == 0
    t0 = time.time()
    while int(sig[1]) != 402 and time.time() - t0 < 30:
        pass
    assert [int(v) for v in sig] == [1, 402, 403, 1]
    assert torch.equal(out[-4096:], big[-4096:].cpu()) and torch.equal(out[:4096], big[8:8 + 4096].cpu())
    torch.cuda.synchronize()
    assert torch.equal(out, big[8:].cpu())
    # pinning a plain host buffer and the combined data + signal copy
    buf = np.zeros(1 << 16, np.int16)
    assert lib.b200_xfer_register_pinned(buf.ctypes.data, buf.nbytes) == 0
    one = np.zeros(1, np.uint8)
    assert lib.b200_xfer_register_pinned(one.ctypes.data, 1) == 0
    flags = torch.tensor([7, 9], dtype=torch.uint8, device="cuda")
    assert lib.b200_xfer_d2h_with_signal_async(big.data_ptr(), 0, buf.ctypes.data, buf.nbytes, flags.data_ptr(), 1,
                                               one.ctypes.data, stream) == 0
    assert lib.b200_xfer_stream_synchronize(stream) == 0
    assert int(one[0]) == 9 and np.array_equal(buf, big[:1 << 16].cpu().numpy())
    assert lib.b200_xfer_unregister_pinned(buf.ctypes.data) == 0 and lib.b200_xfer_unregister_pinned(one.ctypes.data) == 0
    assert lib.b200_xfer_d2h_async(None, 0, buf.ctypes.data, 4, stream) == -1
