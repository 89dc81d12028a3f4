// CPU-assisted LoRA transport: checked copies, stream-ordered doorbells and the host protocol
// declared in include/b200_cpu_assist.h.  Host code only; the arithmetic runs in the CPU workers.
#include <string.h>

#include <atomic>
#include <chrono>
#include <vector>

#include <cuda_runtime.h>

#include "b200_cpu_assist.h"
#include "b200_lora.h"

namespace {

int status_of(cudaError_t e) { return e == cudaSuccess ? B200_LORA_OK : B200_LORA_ERR_CUDA; }

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

using Clock = std::chrono::steady_clock;

inline bool expired(const Clock::time_point& t0, int64_t timeout_us) {
    return timeout_us >= 0 && std::chrono::duration_cast<std::chrono::microseconds>(Clock::now() - t0).count() > timeout_us;
}

// signal words are written by other processes: read them as such
inline int16_t load_signal(const int16_t* p) { return *reinterpret_cast<const volatile int16_t*>(p); }

// one copy of the protocol, by CUDA or (host_copies) by memcpy
int copy_d2h(const b200_cpu_assist* c, const void* dev, size_t elem_offset, void* host, size_t nbytes, void* stream) {
    const char* src = static_cast<const char*>(dev) + 2 * elem_offset;
    if (c->host_copies) { memcpy(host, src, nbytes); return B200_LORA_OK; }
    return status_of(cudaMemcpyAsync(host, src, nbytes, cudaMemcpyDeviceToHost, as_stream(stream)));
}

int copy_h2d_2d(const b200_cpu_assist* c, const void* host, void* dev, size_t src_pitch, size_t dst_pitch, size_t width,
                size_t height, size_t elem_offset, void* stream) {
    char* dst = static_cast<char*>(dev) + 2 * elem_offset;
    if (c->host_copies) {
        for (size_t r = 0; r < height; ++r) memcpy(dst + r * dst_pitch, static_cast<const char*>(host) + r * src_pitch, width);
        return B200_LORA_OK;
    }
    return status_of(cudaMemcpy2DAsync(dst, dst_pitch, host, src_pitch, width, height, cudaMemcpyHostToDevice, as_stream(stream)));
}

int check_layout(const b200_cpu_assist* c) {
    if (!c || !c->shm_x || !c->shm_out[0] || !c->shm_out[1] || !c->shm_out[2] || !c->shm_signal || !c->shm_tkn_len || !c->lock)
        return B200_LORA_ERR_NULL;
    if (c->lora_num < 1 || c->prompt_max < 1 || c->hidden < 1 || c->tp_degree < 1 || c->gpu_id < 0 ||
        c->gpu_id >= c->tp_degree || c->hidden % c->tp_degree || c->n_layers < 1 || c->token_per_lora < 1)
        return B200_LORA_ERR_DIM;
    return B200_LORA_OK;
}

}  // namespace

extern "C" {

int b200_xfer_register_pinned(void* host, size_t nbytes) {
    if (!host) return B200_LORA_ERR_NULL;
    return status_of(cudaHostRegister(host, nbytes, cudaHostRegisterPortable));
}

int b200_xfer_unregister_pinned(void* host) {
    if (!host) return B200_LORA_ERR_NULL;
    return status_of(cudaHostUnregister(host));
}

int b200_xfer_d2h_async(const void* dev, size_t elem_offset, void* host_dst, size_t nbytes, void* stream) {
    if (!dev || !host_dst) return B200_LORA_ERR_NULL;
    return status_of(cudaMemcpyAsync(host_dst, static_cast<const char*>(dev) + 2 * elem_offset, nbytes, cudaMemcpyDeviceToHost,
                                     as_stream(stream)));
}

int b200_xfer_signal_d2h_async(const void* dev_numbers, size_t elem_offset, void* host_signals, size_t nbytes, void* stream) {
    return b200_xfer_d2h_async(dev_numbers, elem_offset, host_signals, nbytes, stream);
}

int b200_xfer_d2h_with_signal_async(const void* dev, size_t elem_offset, void* host_dst, size_t nbytes,
                                    const void* dev_signals, size_t index, void* host_signal_dst, void* stream) {
    if (!dev_signals || !host_signal_dst) return B200_LORA_ERR_NULL;
    int rc = b200_xfer_d2h_async(dev, elem_offset, host_dst, nbytes, stream);
    if (rc) return rc;
    return status_of(cudaMemcpyAsync(host_signal_dst, static_cast<const char*>(dev_signals) + index, 1, cudaMemcpyDeviceToHost,
                                     as_stream(stream)));
}

int b200_xfer_h2d_async(const void* host_src, void* dev, size_t elem_offset, size_t nbytes, void* stream) {
    if (!dev || !host_src) return B200_LORA_ERR_NULL;
    return status_of(cudaMemcpyAsync(static_cast<char*>(dev) + 2 * elem_offset, host_src, nbytes, cudaMemcpyHostToDevice,
                                     as_stream(stream)));
}

int b200_xfer_h2d_2d_async(const void* host_src, void* dev, size_t src_pitch, size_t dst_pitch, size_t width,
                           size_t height, size_t elem_offset, void* stream) {
    if (!dev || !host_src) return B200_LORA_ERR_NULL;
    if (width > src_pitch || width > dst_pitch) return B200_LORA_ERR_DIM;
    if (height == 0 || width == 0) return B200_LORA_OK;
    return status_of(cudaMemcpy2DAsync(static_cast<char*>(dev) + 2 * elem_offset, dst_pitch, host_src, src_pitch, width, height,
                                       cudaMemcpyHostToDevice, as_stream(stream)));
}

int b200_xfer_stream_synchronize(void* stream) { return status_of(cudaStreamSynchronize(as_stream(stream))); }

int b200_cpu_assist_invoke(const b200_cpu_assist* c, const void* hidden_states, int32_t n_rows, int32_t tkn_num,
                           int32_t layer_id, int64_t timeout_us, void* stream) {
    int rc = check_layout(c);
    if (rc) return rc;
    if (!hidden_states || (!c->host_copies && !c->dev_numbers)) return B200_LORA_ERR_NULL;
    if (tkn_num < 1 || tkn_num > c->prompt_max || n_rows < tkn_num || n_rows % tkn_num || layer_id < 0) return B200_LORA_ERR_DIM;
    const int batch = n_rows / tkn_num;
    const int per_request = (tkn_num - 1) / c->token_per_lora + 1;
    const int jobs = batch * per_request;                       // worker jobs per projection
    // doorbell values 2.. / 202.. / 402.. leave room for 200 jobs per projection (lora_cpu/lora_shm_op/app.py:111-128)
    if (jobs > c->lora_num || jobs > 200 || batch > c->lora_num) return B200_LORA_ERR_DIM;

    if (c->gpu_id == 0) {
        for (int i = 0; i < 3 * c->lora_num; ++i) c->shm_signal[i] = 1;
        std::atomic_thread_fence(std::memory_order_release);
        *c->lock = (uint8_t)(layer_id % c->n_layers + 1);
    } else {
        const auto t0 = Clock::now();
        while (*c->lock != (uint8_t)(layer_id + 1))
            if (expired(t0, timeout_us)) return B200_LORA_ERR_TIMEOUT;
        return B200_LORA_OK;                                    // rank 0 alone ships x (lora_cpu.py:169-170)
    }
    *c->shm_tkn_len = tkn_num < c->token_per_lora ? tkn_num : c->token_per_lora;
    std::atomic_thread_fence(std::memory_order_release);
    const size_t row_bytes = 2 * (size_t)c->hidden;
    for (int b = 0; b < batch; ++b) {
        rc = copy_d2h(c, hidden_states, (size_t)b * tkn_num * c->hidden,
                      static_cast<char*>(c->shm_x) + (size_t)b * c->prompt_max * row_bytes, (size_t)tkn_num * row_bytes, stream);
        if (rc) return rc;
    }
    // three doorbell copies, ordered after the data on the same stream
    const int base[3] = {2, 202, 402};
    for (int p = 0; p < 3; ++p) {
        int16_t* dst = c->shm_signal + (size_t)p * c->lora_num;
        if (c->host_copies) {
            std::atomic_thread_fence(std::memory_order_release);
            for (int i = 0; i < jobs; ++i) reinterpret_cast<volatile int16_t*>(dst)[i] = (int16_t)(base[p] + i);
        } else {
            rc = status_of(cudaMemcpyAsync(dst, c->dev_numbers + base[p], 2 * (size_t)jobs, cudaMemcpyDeviceToHost, as_stream(stream)));
            if (rc) return rc;
        }
    }
    return B200_LORA_OK;
}

int b200_cpu_assist_collect_qkv(const b200_cpu_assist* c, void* q, void* k, void* v, int32_t tkn_num,
                                int32_t batch_size, int64_t timeout_us, int32_t* missing, void* stream) {
    if (missing) *missing = 0;
    int rc = check_layout(c);
    if (rc) return rc;
    if (!q || !k || !v) return B200_LORA_ERR_NULL;
    if (tkn_num < 1 || tkn_num > c->prompt_max || batch_size < 1) return B200_LORA_ERR_DIM;
    const int cap = c->token_per_lora;
    const int per_request = (tkn_num - 1) / cap + 1;
    const int jobs = batch_size * per_request;
    if (jobs > c->lora_num || jobs > 200) return B200_LORA_ERR_DIM;
    const int last_rows = tkn_num % cap > 0 ? tkn_num % cap : cap;
    const size_t out_size = (size_t)c->hidden / c->tp_degree;
    void* res[3] = {q, k, v};
    std::vector<char> done((size_t)3 * jobs, 0);
    int left = 3 * jobs;
    const auto t0 = Clock::now();
    while (left > 0) {
        for (int b = 0; b < batch_size; ++b)
            for (int off = 0; off < per_request; ++off) {
                const int i = b * per_request + off;
                for (int p = 0; p < 3; ++p) {
                    if (done[(size_t)p * jobs + i] || load_signal(c->shm_signal + (size_t)p * c->lora_num + i) != 0) continue;
                    std::atomic_thread_fence(std::memory_order_acquire);
                    // this rank's columns of the job's rows (lora_cpu.py:224-232)
                    const char* src = static_cast<const char*>(c->shm_out[p]) +
                                      2 * (size_t)c->hidden * ((size_t)off * cap + (size_t)b * c->prompt_max) + 2 * out_size * c->gpu_id;
                    rc = copy_h2d_2d(c, src, res[p], 2 * (size_t)c->hidden, 2 * out_size, 2 * out_size,
                                     off == per_request - 1 ? last_rows : cap,
                                     out_size * ((size_t)off * cap + (size_t)b * tkn_num), stream);
                    if (rc) return rc;
                    done[(size_t)p * jobs + i] = 1;
                    --left;
                }
            }
        if (left > 0 && expired(t0, timeout_us)) {
            if (missing) *missing = left;
            return B200_LORA_ERR_TIMEOUT;
        }
    }
    return B200_LORA_OK;
}

}  // extern "C"
