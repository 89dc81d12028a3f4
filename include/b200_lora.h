/*
 * b200_lora.h - C ABI of the B200 (sm_100a) multi-LoRA delta library.
 *
 *     y[t, :] += scale_a * (x[t, :] . A_a^T) . B_a^T        a = adapter of token t
 *
 * Plain pointers and sizes only.  Every pointer named "device" is a CUDA device
 * address on the current device; the caller owns all memory.  No entry point
 * allocates device memory (except where a comment says it owns a static
 * array), synchronises the stream, or throws: each returns a b200_lora_status.
 * All work is enqueued on the `stream` argument (a cudaStream_t passed as
 * void*), so calls are stream-ordered and re-entrant across streams as long
 * as plans and workspaces are not shared between streams.
 *
 * Weight layout (the reference's stacked pools, lightllm/models/lora_gpu.py:33-40):
 *   dense  : wa [N, L, R, h_in]  (h_in contiguous),  wb [N, L, h_out, R] (R contiguous)
 *   packed : adapter a owns rows [L*cum[a], L*cum[a+1]) of a [L*sum(r), h] matrix,
 *            layer l at row L*cum[a] + l*r_a; wb's (a,l) block is a contiguous [h_out, r_a].
 */
#ifndef B200_LORA_H
#define B200_LORA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum b200_lora_status {
    B200_LORA_OK = 0,
    B200_LORA_ERR_NULL = -1,       /* a required pointer is NULL */
    B200_LORA_ERR_DIM = -2,        /* a dimension is zero, negative, or not a multiple of 8 */
    B200_LORA_ERR_DTYPE = -3,      /* unsupported element type */
    B200_LORA_ERR_ALIGN = -4,      /* a pointer or leading dimension is not 16-byte aligned */
    B200_LORA_ERR_RANK = -5,       /* rank outside [1, B200_LORA_MAX_RANK] */
    B200_LORA_ERR_WORKSPACE = -6,  /* plan or workspace buffer too small */
    B200_LORA_ERR_CUDA = -7,       /* a CUDA runtime call failed; see b200_lora_last_cuda_error */
    B200_LORA_ERR_ID_RANGE = -8,   /* plan build saw an adapter id outside [0, N) */
    B200_LORA_ERR_LAYER = -9,      /* layer index outside [0, L) */
    B200_LORA_ERR_SEGMENTS = -10,  /* segment offsets not monotone or not covering [0, T] */
    B200_LORA_ERR_TIMEOUT = -11,   /* a bounded device-side wait expired */
    B200_LORA_ERR_UNSUPPORTED = -12
} b200_lora_status;

enum { B200_LORA_F16 = 0, B200_LORA_BF16 = 1, B200_LORA_F32 = 2 };
enum { B200_LORA_MAX_RANK = 64, B200_LORA_MAX_PROJ = 4 };

/* flags of b200_lora_apply */
enum {
    B200_LORA_MID_ROUND = 1,   /* round the [T, r] intermediate to the I/O type, as the reference's
                                  batched-matmul prefill op does (lightllm/models/lora_gpu.py:127-128) */
    B200_LORA_NO_TENSOR = 2,   /* keep tall segments on the BGMV kernels too (no tcgen05 tiles) */
    B200_LORA_ONLY_SHRINK = 4, /* tensor parallel: run only the shrink half; the intermediate v is left in the
                                  workspace (b200_lora_workspace_v_region) for the caller to sum over ranks */
    B200_LORA_ONLY_EXPAND = 8, /* tensor parallel: run only the expand half on the workspace's current v */
    B200_LORA_KEEP_PARTIALS = 64, /* with B200_LORA_ONLY_SHRINK on the TMA kernels: leave the split-K partial sums
                                   as they are instead of adding them up into v (a caller that reduces them
                                   itself, or that times the shrink kernel alone) */
    B200_LORA_DELTA_THEN_ADD = 32 /* 16-bit y only: round the delta to the I/O type and add it to y in that
                                   type, as the reference's `q += q_lora` does
                                   (lightllm/models/llama/layer_infer/transformer_layer_infer.py:160-170).
                                   Identical to the default when y starts at zero, which is how the
                                   reference calls the op (lora_gpu.py:137); otherwise a second rounding.
                                   Applies to the TMA BGMV kernels; other paths ignore it. */
};

/* The adapter table shared by the projections of one layer.
 * Mirrors the pool attributes of Lora_GPU (lightllm/models/lora_gpu.py:24-40) and adds
 * per-adapter ranks and scalings, which the reference fixes to one rank and scale 1. */
typedef struct b200_lora_adapters {
    const int32_t* ranks;      /* device [N]; NULL: every adapter has rank r_pool */
    const float*   scalings;   /* device [N]; NULL: every adapter uses `scale` */
    const int64_t* cum_ranks;  /* device [N+1] exclusive prefix of ranks; required when packed */
    int32_t n_adapters;        /* N */
    int32_t n_layers;          /* L */
    int32_t r_pool;            /* R of the dense layout; upper bound of every rank */
    int32_t packed;            /* 0 dense, 1 packed */
    float   scale;
    int32_t ranks_pow2;        /* caller's promise that every rank is 8, 16, 32 or 64 (and equals r_pool
                                  when dense); selects the TMA kernels.  Checked on the device when a
                                  plan is built: a broken promise yields B200_LORA_ERR_RANK from
                                  b200_lora_plan_read and a plan that applies nothing. */
    int64_t total_rank;        /* sum of all ranks (packed pools); 0 = not known */
} b200_lora_adapters;

/* One projection (q, k, v or o): replaces one (x, pool pair, y) triple of
 * Lora_GPU.invoke_one_layer_{q,k,v} (lightllm/models/lora_gpu.py:122-163). */
typedef struct b200_lora_proj {
    const void* x;   /* device [T, h_in], row stride ldx elements */
    void*       y;   /* device [T, h_out], row stride ldy elements; accumulated in place */
    const void* wa;  /* device A pool */
    const void* wb;  /* device B pool */
    int64_t ldx, ldy;
    int32_t h_in, h_out;
} b200_lora_proj;

/* Library / build identification: returns the compiled-for architecture (100). */
int b200_lora_arch(void);
/* Text of the last CUDA error this thread's calls observed ("" if none). */
const char* b200_lora_last_cuda_error(void);
/* *id = the identifier of the CUDA-graph capture `stream` is part of, 0 when it is not capturing.
 * Host code that keeps a plan between calls (the reference's loop passes the same index tensor
 * 3 x n_layers times, lightllm/models/lora_gpu.py:138,150,162) uses it to keep a plan only within
 * one capture: a graph must contain the build of every plan it applies. */
int b200_lora_stream_capture_id(void* stream, unsigned long long* id);

/* ---- plan: adapter-index gather and segment bookkeeping -----------------------------
 * The plan is a device-resident table built from the per-token adapter ids: a stable
 * counting sort (token order kept inside one adapter), the segment list, and the work
 * units the kernels walk.  One plan serves every layer and projection of a step.
 * Replaces the reference's per-call index tensor `select_inds[bsz-1]`
 * (lightllm/models/lora_gpu.py:120,124). */
size_t b200_lora_plan_bytes(int32_t max_tokens, int32_t n_adapters);

/* `max_tokens` is the capacity the plan buffer was sized for (n_tokens <= max_tokens); the
 * same value is passed to b200_lora_apply and sizes the workspace. */
/* ids: device [T], int32 (ids_are_i64 == 0) or int64.  ranks as in b200_lora_adapters. */
int b200_lora_plan_build(void* plan, size_t plan_bytes, int32_t max_tokens, const void* ids,
                         int32_t ids_are_i64, int32_t n_tokens, const b200_lora_adapters* adapters,
                         void* stream);

/* Rows of x are already grouped: segment s covers rows [seg_starts[s], seg_starts[s+1]) and
 * uses adapter seg_adapter[s].  Both arrays are device int32; n_segs is a host value. */
int b200_lora_plan_from_segments(void* plan, size_t plan_bytes, int32_t max_tokens,
                                 const int32_t* seg_starts, const int32_t* seg_adapter, int32_t n_segs,
                                 int32_t n_tokens, const b200_lora_adapters* adapters, void* stream);

/* Copies the plan's tables to host arrays (synchronises `stream`): perm [T], seg_starts
 * [T+1], seg_adapter [T]; *n_segs receives S.  Returns B200_LORA_ERR_ID_RANGE if the build
 * saw an id outside [0, N) (such a plan applies nothing). */
int b200_lora_plan_read(const void* plan, int32_t* perm, int32_t* seg_starts, int32_t* seg_adapter,
                        int32_t* n_segs, int32_t* n_tokens, void* stream);

/* ---- apply ---------------------------------------------------------------------------- */
size_t b200_lora_workspace_bytes(int32_t max_tokens, int32_t n_proj, int32_t max_h_in);
/* Zero-fills a fresh workspace; call once per allocation, before its first use.  The
 * kernels leave the control words zero again when they finish. */
int b200_lora_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/* Applies the delta of `layer` to up to B200_LORA_MAX_PROJ projections in one pass.
 * io_dtype: type of x, wa, wb (F16 | BF16).  y_dtype: io_dtype or F32.  n_tokens: rows of x
 * and y (the value the plan was built with).  Unless B200_LORA_NO_TENSOR is set, tall
 * contiguous segments of rank 16/32/64 run on the tcgen05 tile kernel, the rest on the BGMV
 * kernels; decode-only batches should set the flag and save that kernel's launch.  The two
 * kinds touch disjoint rows, and the tile launches run on a side stream inside the call (forked
 * from `stream` and joined to it again before the call returns, so the call stays ordered on
 * `stream` and captures into a CUDA graph as a fork and a join).  The side stream is created by
 * the first such call of a host thread on a device, which should be made outside stream capture
 * (inside one it runs the launches one after the other); B200_LORA_SERIAL_TILES=1 in the
 * environment keeps everything on `stream`. */
int b200_lora_apply(const b200_lora_proj* projs, int32_t n_proj, const b200_lora_adapters* adapters,
                    const void* plan, int32_t max_tokens, int32_t n_tokens, int32_t layer,
                    int32_t io_dtype, int32_t y_dtype, int32_t flags, void* workspace,
                    size_t workspace_bytes, void* stream);

/* Where the fp32 shrink result v [n_proj][max_tokens][64] sits inside a workspace: byte offset
 * and size.  Tensor-parallel callers all-reduce this region between a B200_LORA_ONLY_SHRINK
 * and a B200_LORA_ONLY_EXPAND call (A sharded along h_in, B along h_out); the reference
 * replicates A instead and needs no exchange (lightllm/models/lora_gpu.py:25-26,33-34). */
int b200_lora_workspace_v_region(int32_t max_tokens, int32_t n_proj, size_t* offset_bytes, size_t* size_bytes);

/* ---- tensor-parallel exchange over peer memory (no counterpart in the reference, which replicates A) -----
 * Sums the fp32 shrink result v over the tensor-parallel ranks between a B200_LORA_ONLY_SHRINK and a
 * B200_LORA_ONLY_EXPAND apply with ONE kernel per rank: every rank stores its partial into a landing
 * buffer in every peer's memory (plain 8-byte stores over NVLink, each carrying a value and the number of
 * the exchange), polls - with a bound - its own landing buffer until its peers' packets show that number
 * and adds the values up in rank order (all ranks obtain the same bits).  No flag, fence or barrier stands
 * between data and consumer.  Takes the place of an NCCL all-reduce of b200_lora_workspace_v_region.
 *
 * Set-up, once per process: b200_lora_tp_alloc a buffer of b200_lora_tp_bytes, b200_lora_tp_export its
 * 64-byte handle, hand the handles round (any host channel), b200_lora_tp_open every peer's handle and
 * fill b200_lora_tp with b200_lora_tp_layout.  Every rank must issue the same sequence of exchanges.
 * A rank whose peer never arrives gives up after a second or two: the exchange leaves v incomplete and
 * b200_lora_workspace_status returns B200_LORA_ERR_TIMEOUT; nothing hangs. */
enum { B200_LORA_TP_MAX_RANKS = 8, B200_LORA_TP_COUNTER_BYTES = 24576 };
typedef struct b200_lora_tp {
    void* landing[B200_LORA_TP_MAX_RANKS][2];  /* [r][b]: landing buffer b of rank r as mapped into this process */
    void* flags[B200_LORA_TP_MAX_RANKS];       /* [r]: rank r's counters and hint words (peers write the hints) */
    int32_t tp, rank;
    size_t set_stride;                         /* bytes from the landing buffers of set 0 to those of set 1 */
} b200_lora_tp;
size_t b200_lora_tp_bytes(int32_t max_tokens, int32_t n_proj, int32_t tp);
int b200_lora_tp_alloc(void** base, size_t bytes);                 /* cudaMalloc + zero fill (IPC-exportable) */
int b200_lora_tp_free(void* base);
int b200_lora_tp_export(void* base, void* handle64);              /* cudaIpcGetMemHandle */
int b200_lora_tp_open(const void* handle64, void** mapped);       /* cudaIpcOpenMemHandle, enables peer access */
int b200_lora_tp_close(void* mapped);
/* Fills tp->landing[r] / tp->flags[r] from rank r's buffer base (own base for r == rank, mapped bases else). */
int b200_lora_tp_layout(b200_lora_tp* tp, int32_t r, void* base, int32_t max_tokens, int32_t n_proj);
/* The exchange on `workspace`'s v region.  skip_arrival != 0 withholds this rank's packets (a failure
 * made on the host, for tests of the peers' bounded wait). */
int b200_lora_tp_exchange(const b200_lora_tp* tp, void* workspace, int32_t max_tokens, int32_t n_tokens,
                          int32_t n_proj, int32_t skip_arrival, void* stream);
/* b200_lora_apply for a tensor-parallel rank in ONE call: shrink half, exchange, expand half.  `flags` as
 * for b200_lora_apply, without the ONLY_* bits.  Two exchanges run per apply, each with its own landing
 * buffers and counters: that of the rows of tall runs between the two tile launches (on a side stream
 * inside the call), that of all other rows between the BGMV halves; each moves only the rank columns of its
 * rows, and each hides behind the other chain's kernels.  With B200_LORA_NO_TENSOR there is one exchange.
 * From four ranks on the tall rows' exchange goes through an owning rank per group of rows (partials to the
 * owner, its sum to everybody); B200_LORA_TP_VIA_OWNER=0/1 in the environment forces either route.
 * All ranks must make the same calls with the same flags on the same plan contents. */
int b200_lora_apply_tp(const b200_lora_proj* projs, int32_t n_proj, const b200_lora_adapters* adapters,
                       const void* plan, int32_t max_tokens, int32_t n_tokens, int32_t layer, int32_t io_dtype,
                       int32_t y_dtype, int32_t flags, void* workspace, size_t workspace_bytes,
                       const b200_lora_tp* tp, int32_t skip_arrival, void* stream);

/* Reads the workspace's sticky device-side error word (synchronises `stream`):
 * B200_LORA_OK, B200_LORA_ERR_TIMEOUT if a bounded wait inside a kernel expired, or
 * B200_LORA_ERR_DIM if an apply was given a plan built for another max_tokens or n_tokens
 * (such an apply changes nothing: the plan's token rows would not fit x and y). */
int b200_lora_workspace_status(const void* workspace, void* stream);

/* ---- the reference's operator call -------------------------------------------------------
 * Same arguments as punica.ops.add_lora_bgmv(y, x, wa_T_all, wb_T_all, indicies, layer_idx,
 * scale) at lightllm/models/lora_gpu.py:138,150,162, flattened to pointers and sizes.
 * Builds a plan inside `workspace` and applies one projection.  `workspace` needs no
 * preparation and may be reused by calls of any shape that fit it: every call clears the
 * control words of its own layout. */
size_t b200_add_lora_bgmv_workspace_bytes(int32_t n_tokens, int32_t n_adapters, int32_t h_in);
int b200_add_lora_bgmv(void* y, const void* x, const void* wa_T_all, const void* wb_T_all,
                       const void* indicies, int32_t indicies_are_i64, int32_t n_tokens,
                       int32_t h_in, int32_t h_out, int32_t n_adapters, int32_t n_layers, int32_t r,
                       int32_t layer_idx, float scale, int32_t dtype,
                       void* workspace, size_t workspace_bytes, void* stream);

/* ---- allocation-free variant of the operator call ------------------------------------------
 * No counterpart in the reference.  Some callers may not allocate device memory at all: a
 * serving process that has already handed every free byte of HBM to its KV cache (a late
 * cudaMalloc would fail or evict), a decode loop that cannot afford the device-wide
 * synchronisation cudaMalloc/cudaFree imply, or a host whose policy forbids allocation after
 * start-up.  For them this entry point takes only inputs and outputs; the
 * plan and the split-K scratch that b200_add_lora_bgmv keeps in a caller-provided workspace
 * live in a fixed array inside the library (B200_LORA_STATIC_SCRATCH_BYTES, present on every
 * GPU that loads the library, for the life of the process).  It calls no cudaMalloc, cudaFree
 * or allocating library routine.
 *
 * Limits: n_tokens <= B200_LORA_STATIC_MAX_TOKENS, n_adapters <= B200_LORA_STATIC_MAX_ADAPTERS,
 * h_in <= B200_LORA_STATIC_MAX_H_IN; anything larger returns B200_LORA_ERR_WORKSPACE and does
 * nothing.  The first call on a device looks up the array's device address (one-time set-up),
 * so make that first call outside any stream capture.  All calls on one GPU share the one
 * array: calls that may overlap on the GPU (different streams without an ordering between
 * them) race on it and give wrong results; calls ordered on one stream are fine. */
enum {
    B200_LORA_STATIC_MAX_TOKENS = 64,
    B200_LORA_STATIC_MAX_ADAPTERS = 1024,
    B200_LORA_STATIC_MAX_H_IN = 8192,
    B200_LORA_STATIC_SCRATCH_BYTES = 3 * 512 * 1024
};
int b200_add_lora_bgmv_static(void* y, const void* x, const void* wa_T_all, const void* wb_T_all,
                              const void* indicies, int32_t indicies_are_i64, int32_t n_tokens,
                              int32_t h_in, int32_t h_out, int32_t n_adapters, int32_t n_layers, int32_t r,
                              int32_t layer_idx, float scale, int32_t dtype, void* stream);
/* Outcome of the last b200_add_lora_bgmv_static call on the current device, read back from the
 * built-in array (synchronises `stream`; no counterpart in the reference): B200_LORA_OK, or
 * what b200_lora_plan_read / b200_lora_workspace_status would report for that call
 * (an adapter id outside [0, N) leaves y unchanged; an expired device wait).  The next
 * static call overwrites it. */
int b200_add_lora_bgmv_static_status(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_LORA_H */
