/*
 * b200_cpu_assist.h - C ABI of the CPU-assisted LoRA transport: the copies and doorbells that carry
 * activations from the GPU to CPU worker processes over pinned shared memory and bring the deltas
 * back.  Native counterpart of the reference's `tensor_cp` extension (csrc/cuda_ops.hpp,
 * csrc/interface.cpp) and of the host protocol built on it (lightllm/models/lora_cpu.py:138-276).
 *
 * Differences from the reference, all on purpose: every CUDA return code is checked and comes back
 * as a status; the stream is an argument (the reference uses file-scope global streams and the
 * legacy default stream); nothing here is global state; every wait has a time limit.
 *
 * Status codes are those of b200_lora.h (B200_LORA_OK, _ERR_NULL, _ERR_DIM, _ERR_CUDA, _ERR_TIMEOUT).
 */
#ifndef B200_CPU_ASSIST_H
#define B200_CPU_ASSIST_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- copies (csrc/cuda_ops.hpp).  Offsets are in 2-byte ELEMENTS, sizes and pitches in bytes, as in the
 * reference; host addresses are plain pointers (the reference passes them as uint64). ------------------- */

/* cudaHostRegister(..., cudaHostRegisterPortable): register_pinned_memory (cuda_ops.hpp:109). */
int b200_xfer_register_pinned(void* host, size_t nbytes);
int b200_xfer_unregister_pinned(void* host);
/* device -> host of nbytes from dev + offset elements: cudaDtoHAsync (:122); the synchronous form (:115)
 * is this call followed by b200_xfer_stream_synchronize. */
int b200_xfer_d2h_async(const void* dev, size_t elem_offset, void* host_dst, size_t nbytes, void* stream);
/* the doorbell copy: a slice of a device int16 `arange` lands in the workers' signal row, stream-ordered
 * after the data copies: cudaSignalDtoHAsync (:128). */
int b200_xfer_signal_d2h_async(const void* dev_numbers, size_t elem_offset, void* host_signals, size_t nbytes, void* stream);
/* data copy followed by a one-byte signal copy on the same stream: cudaDtoHAsyncWithSignal (:134). */
int b200_xfer_d2h_with_signal_async(const void* dev, size_t elem_offset, void* host_dst, size_t nbytes,
                                    const void* dev_signals, size_t index, void* host_signal_dst, void* stream);
/* host -> device into dev + offset elements: cudaHtoDAsync (:159); cudaHtoD (:151) is this + synchronize. */
int b200_xfer_h2d_async(const void* host_src, void* dev, size_t elem_offset, size_t nbytes, void* stream);
/* pitched host -> device copy (a rank's column slice of the workers' full-width output):
 * cudaHtoD2D / cudaHtoD2DAsync / cudaHtoD2DAsyncLora (:173, :199, :215); the caller picks the stream. */
int b200_xfer_h2d_2d_async(const void* host_src, void* dev, size_t src_pitch, size_t dst_pitch, size_t width,
                           size_t height, size_t elem_offset, void* stream);
/* stream_synchronize (:43). */
int b200_xfer_stream_synchronize(void* stream);

/* ---- the host protocol (lightllm/models/lora_cpu.py) --------------------------------------------------- */

/* The shared-memory segments a model process attaches to (created by the reference's create_shm.py:38-130;
 * attributes of Lora_CPU, lora_cpu.py:30-117).  All host pointers; x/out segments are [lora_num,
 * prompt_max, hidden] fp16. */
typedef struct b200_cpu_assist {
    void*    shm_x;             /* activations for the workers              (shm_array)   */
    void*    shm_out[3];        /* the workers' q, k, v deltas              (shm_out_q/k/v) */
    int16_t* shm_signal;        /* [3, lora_num] doorbells: > 1 work, 0 done, 1 idle        */
    int64_t* shm_tkn_len;       /* [1] rows per worker job                                  */
    volatile uint8_t* lock;     /* [1] layer hand-shake between tensor-parallel ranks       */
    const int16_t* dev_numbers; /* device int16 arange(0, >= 602): source of the doorbell values */
    int32_t lora_num;           /* rows of the signal table = worker slots per projection   */
    int32_t prompt_max;         /* PROMPT_MAX_LENGTH (lora_cpu.py:14)                       */
    int32_t hidden;             /* hidden_dim                                               */
    int32_t tp_degree, gpu_id;  /* this rank collects columns [gpu_id * hidden/tp, +hidden/tp) */
    int32_t n_layers;
    int32_t token_per_lora;     /* rows one worker takes (cpu_capacity)                     */
    int32_t host_copies;        /* 0: CUDA copies.  1: the "device" pointers are host memory and every copy
                                   is an immediate memcpy - lets the protocol run against real worker
                                   processes on a machine without a GPU */
} b200_cpu_assist;

/* Lora_CPU.invoke_lora_async(hidden_states, tkn_num, layer_id) (lora_cpu.py:138-185).
 * hidden_states: device [batch * tkn_num, hidden] fp16.  Rank 0 arms the signal table, publishes the layer
 * in `lock`, copies every request's rows to the x segment and rings 3 * n doorbells with three copies of
 * consecutive values starting at 2, 202 and 402; other ranks only wait (at most timeout_us) for the layer. */
int b200_cpu_assist_invoke(const b200_cpu_assist* c, const void* hidden_states, int32_t n_rows, int32_t tkn_num,
                           int32_t layer_id, int64_t timeout_us, void* stream);

/* Lora_CPU.collect_qkv(tkn_num, batch_size) (lora_cpu.py:187-276).  q/k/v: device [batch, tkn_num, hidden/tp]
 * fp16, zero-filled by the caller.  Polls the doorbells; each finished (request, chunk, projection) is copied,
 * this rank's columns only, into place.  Gives up after timeout_us: returns B200_LORA_ERR_TIMEOUT and sets
 * *missing (if not NULL) to the number of worker jobs that never answered - a dead worker is a status, not a
 * hang.  The copies are enqueued on `stream`; results are complete when the stream reaches that point. */
int b200_cpu_assist_collect_qkv(const b200_cpu_assist* c, void* q, void* k, void* v, int32_t tkn_num,
                                int32_t batch_size, int64_t timeout_us, int32_t* missing, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_CPU_ASSIST_H */
