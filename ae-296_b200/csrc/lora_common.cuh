// Shared device/host definitions of the multi-LoRA delta kernels (sm_100a).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "b200_lora.h"

namespace b200lora {

constexpr int kMaxRank = B200_LORA_MAX_RANK;   // 64
constexpr int kMaxProj = B200_LORA_MAX_PROJ;   // 4
constexpr int kMaxSub = 16;                    // most sub-ranges of one super-chunk (rank 64)
constexpr int kSuper = 2048;                   // columns (shrink) / rows (expand) per super-chunk
constexpr int kCtaThreads = 512;
constexpr int kChunkTok = 8;                   // BGMV work segments hold at most this many tokens
constexpr int kTallMin = 32;                   // a contiguous segment at least this long is "tall"
constexpr int kTileM = 128;                    // token rows of one tensor-core tile

// ---- plan layout --------------------------------------------------------------------------
// All fields are int32.  `cap` is the token capacity the buffer was sized for.
struct PlanHeader {
    int n_tokens;
    int n_segs;
    int n_units;      // sum over short segments of r_pad/8
    int error;        // 0 ok, 1 adapter id out of range, 2 bad segment table, 3 rank promise broken
    int n_tiles;      // 128-row tiles of tall segments
    int cap;
    int n_adapters;
    int identity;     // 1: perm is the identity (rows pre-grouped)
    int n_units_short;  // units of short segments; they come first in unit_tab
    int n_wsegs;        // work segments
    int pad[6];
};
static_assert(sizeof(PlanHeader) == 64, "plan header is 16 words");

// One BGMV work unit: a work segment (<= 8 tokens of one adapter) times one sub-range of
// columns (shrink) or rows (expand).  Everything a CTA needs to start loading, in 64 bytes.
struct UnitRec {
    int adapter;
    int rank;
    short sub;        // index of the sub-range inside a 2048-wide super-chunk
    short ntok;
    float scale;      // the adapter's scaling
    int wseg;         // work-segment index (selects the split-K arrival counter)
    int start;        // sorted position of the first token
    int cum_lo, cum_hi;   // cum_ranks[adapter] (packed pools)
    int tok[8];       // token rows
};
static_assert(sizeof(UnitRec) == 64, "unit record is 16 words");

struct PlanView {
    PlanHeader* hdr;
    int* perm;          // [cap]       sorted position -> token row
    int* seg_start;     // [cap + 1]   sorted position of each segment's first token
    int* seg_adapter;   // [cap]
    int* seg_rank;      // [cap]       rank of the segment's adapter
    int* seg_flags;     // [cap]       bit0: tall (handled by the tensor-core tiles)
    int* ws_start;      // [cap + 1]   work segments: adapter segments cut into <= kChunkTok tokens
    int* ws_adapter;    // [cap]
    int* ws_rank;       // [cap]
    int* ws_unit0;      // [cap]       first unit record of the work segment
    int* unit_tab;      // [16 * cap][16]  one record per weight unit (see UnitRec)
    int* tile_tab;      // [cap]       two words per tile of a tall run: first sorted position, (seg << 8) | (rows - 1)
    int* hist;          // [n_adapters + 1]
};

__host__ __device__ inline size_t plan_words(int cap, int n_adapters) {
    // header + perm + seg_start + 3 seg arrays + units + tiles + hist, each padded to 4 words
    auto pad4 = [](size_t w) { return (w + 3) & ~size_t(3); };
    return 16 + pad4(cap) + 2 * pad4(cap + 1) + 6 * pad4(cap) + 16 * kMaxSub * (size_t)cap + pad4(cap) +
           pad4((size_t)n_adapters + 1);
}

__host__ __device__ inline PlanView plan_view(void* base, int cap, int n_adapters) {
    auto pad4 = [](size_t w) { return (w + 3) & ~size_t(3); };
    int* w = reinterpret_cast<int*>(base);
    PlanView v;
    v.hdr = reinterpret_cast<PlanHeader*>(w);      w += 16;
    v.perm = w;                                    w += pad4(cap);
    v.seg_start = w;                               w += pad4(cap + 1);
    v.seg_adapter = w;                             w += pad4(cap);
    v.seg_rank = w;                                w += pad4(cap);
    v.seg_flags = w;                               w += pad4(cap);
    v.ws_start = w;                                w += pad4(cap + 1);
    v.ws_adapter = w;                              w += pad4(cap);
    v.ws_rank = w;                                 w += pad4(cap);
    v.ws_unit0 = w;                                w += pad4(cap);
    v.unit_tab = w;                                w += 16 * kMaxSub * (size_t)cap;
    v.tile_tab = w;                                w += pad4(cap);
    v.hist = w;
    (void)n_adapters;
    return v;
}

// ---- workspace layout ----------------------------------------------------------------------
// control words (zero at rest), then the reduced intermediate v [n_proj][cap][64] fp32, then
// the split-K partials [n_kchunk][n_proj][cap][64] fp32.
struct WorkspaceCtl {
    unsigned reserved0[4];
    unsigned error;           // sticky device-side error word
    unsigned reserved1[11];
};
static_assert(sizeof(WorkspaceCtl) == 64, "control block is 16 words");

__host__ __device__ inline int max_kchunks(int h_in) { return (h_in + 127) / 128; }

__host__ __device__ inline size_t ws_counter_words(int cap) { return (size_t)kMaxProj * cap; }

// control block and arrival counters: what must be zero before the first launch
__host__ __device__ inline size_t ws_ctl_bytes(int cap) { return sizeof(WorkspaceCtl) + 4 * ((ws_counter_words(cap) + 3) & ~size_t(3)); }

__host__ __device__ inline size_t workspace_bytes(int cap, int n_proj, int max_h_in) {
    size_t ctl = ws_ctl_bytes(cap);
    size_t v = (size_t)n_proj * cap * kMaxRank * 4;
    size_t part = (size_t)max_kchunks(max_h_in) * n_proj * cap * kMaxRank * 4;
    return ctl + v + part + 256;
}

struct WorkspaceView {
    WorkspaceCtl* ctl;
    unsigned* counters;   // [kMaxProj][cap]  arrivals per (projection, work segment); general-path kernels only
    float* v;             // [n_proj][cap][64]
    float* partial;       // [kchunk][n_proj][cap][64]
};

__host__ __device__ inline WorkspaceView workspace_view(void* base, int cap, int n_proj) {
    char* p = reinterpret_cast<char*>(base);
    WorkspaceView w;
    w.ctl = reinterpret_cast<WorkspaceCtl*>(p);            p += sizeof(WorkspaceCtl);
    w.counters = reinterpret_cast<unsigned*>(p);           p += 4 * ((ws_counter_words(cap) + 3) & ~size_t(3));
    p = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(p) + 127) & ~uintptr_t(127));
    w.v = reinterpret_cast<float*>(p);                     p += (size_t)n_proj * cap * kMaxRank * 4;
    w.partial = reinterpret_cast<float*>(p);
    return w;
}

// ---- kernel parameters ------------------------------------------------------------------------
struct ProjArgs {
    const void* x;
    void* y;
    const void* wa;
    const void* wb;
    long long ldx, ldy;
    int h_in, h_out;
    int n_super_in, n_super_out;
};

struct ApplyParams {
    alignas(64) CUtensorMap amap[kMaxProj][4];   // 2-D maps over the A pools ([rows, h_in]), box 128 columns x (8, 16, 32, 64) rows
                                              // by rank class: all rank rows of an adapter in one copy; TMA kernels only
    ProjArgs proj[kMaxProj];
    int n_proj;
    int total_super_in, total_super_out;
    const int* ranks;
    const float* scalings;
    const long long* cum_ranks;
    int n_adapters, n_layers, r_pool, packed;
    float scale;
    int layer;
    int flags;
    int y_f32;
    int cap;
    int n_tokens;                        // rows of x and y in this call (<= cap)
    void* plan;
    void* workspace;
};

// Tensor maps of the tcgen05 tile kernel (all over local memory).
struct SgmvParams {
    alignas(64) CUtensorMap xmap[kMaxProj];      // x [T, h_in], box 64 x 128, 128-byte swizzle
    CUtensorMap amap[kMaxProj][3];               // A pool [rows, h_in], box 64 x (16 | 32 | 64), 128-byte swizzle
    CUtensorMap bmap[kMaxProj][3];               // B pool viewed as [rows, 16 | 32 | 64], box rank x 128
    CUtensorMap ymap[kMaxProj];                  // y [T, h_out] (16-bit y only), box 64 x 128, 128-byte swizzle
};

// element offset of adapter a's A block [r, h] for `layer`, and its row count / row pitch
__device__ __forceinline__ long long block_row0(const ApplyParams& p, int a, int r) {
    if (p.packed) return (long long)p.n_layers * p.cum_ranks[a] + (long long)p.layer * r;
    return ((long long)a * p.n_layers + p.layer) * p.r_pool;
}
__device__ __forceinline__ long long block_row0(const ApplyParams& p, const UnitRec& u) {
    if (p.packed)
        return (long long)p.n_layers * (((long long)u.cum_hi << 32) | (unsigned)u.cum_lo) + (long long)p.layer * u.rank;
    return ((long long)u.adapter * p.n_layers + p.layer) * p.r_pool;
}
__device__ __forceinline__ int b_pitch(const ApplyParams& p, int r) { return p.packed ? r : p.r_pool; }

// Values of the workspace's sticky error word: 1..15 name the bounded wait that expired, this one
// says that an apply call was given a plan built for another capacity or another number of rows.
constexpr unsigned kErrPlanMismatch = 64u;

// May this apply walk the plan?  A plan whose build failed applies nothing (its own error word
// tells why); a plan built for other sizes would index x and y out of range, so it applies
// nothing either and the workspace's error word records it.
__device__ __forceinline__ bool plan_usable(const PlanHeader& hdr, const ApplyParams& p, unsigned* err) {
    if (hdr.error) return false;
    if (hdr.cap != p.cap || hdr.n_tokens != p.n_tokens) {
        if (threadIdx.x == 0) atomicMax(err, kErrPlanMismatch);
        return false;
    }
    return true;
}

__host__ __device__ __forceinline__ int pad_rank(int r) { return r <= 8 ? 8 : r <= 16 ? 16 : r <= 32 ? 32 : 64; }
// sub-ranges per 2048-wide super-chunk for a padded rank: 8->4, 16->4, 32->8, 64->16, i.e. a unit is
// 512 / 512 / 256 / 128 columns (shrink) or rows (expand) wide and holds <= 16 KB of weights
__host__ __device__ __forceinline__ int n_sub(int r_pad) { return r_pad <= 16 ? 4 : r_pad / 4; }


// ---- 16-bit -> fp32 helpers ------------------------------------------------------------------
template <typename T> struct Cvt;
template <> struct Cvt<__half> {
    static constexpr bool is_bf16 = false;
    static __device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
    }
    static __device__ __forceinline__ unsigned pack2(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<unsigned*>(&h);
    }
    static __device__ __forceinline__ float round1(float a) { return __half2float(__float2half_rn(a)); }
};
template <> struct Cvt<__nv_bfloat16> {
    static constexpr bool is_bf16 = true;
    static __device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
        const unsigned* w = reinterpret_cast<const unsigned*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
    }
    static __device__ __forceinline__ unsigned pack2(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<unsigned*>(&h);
    }
    static __device__ __forceinline__ float round1(float a) { return __bfloat162float(__float2bfloat16_rn(a)); }
};

__device__ __forceinline__ uint4 ldg_nc16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ldg16(const void* p) { return *reinterpret_cast<const uint4*>(p); }

// ---- programmatic dependent launch -----------------------------------------------------------
// Kernels of this library are launched with programmatic stream serialisation, so a kernel's CTAs
// may start while its predecessor in the stream still runs, and use that to set up and to request
// data that the predecessor does not write.  Two rules keep this safe for chains of any length:
//   1. every CTA waits for the predecessor (griddepcontrol.wait by at least one thread) before it
//      exits, idle CTAs included, so that a kernel's completion implies its predecessor's;
//   2. a CTA lets the successor launch (griddepcontrol.launch_dependents) only after that wait.
// By induction, when any CTA of a kernel runs, every kernel before its predecessor has completed:
// what those wrote (the activations, the y an earlier apply accumulated into) may be read at once,
// and only what the predecessor itself writes has to wait.  Both instructions are no-ops without
// the launch attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_prior() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// ---- launchers implemented by the kernel files ---------------------------------------------
struct PlanAdapters {          // what the plan bakes into its unit records
    const int* ranks;
    const long long* cum_ranks;   // NULL for dense pools
    const float* scalings;        // NULL: uniform `scale`
    float scale;
    int r_pool;
    int n_adapters;
    int ranks_pow2;               // caller's promise: every rank is 8/16/32/64 (dense: == r_pool)
};
cudaError_t launch_plan_build(void* plan, int cap, const void* ids, int ids_i64, int n_tokens,
                              const PlanAdapters& ad, cudaStream_t s);
cudaError_t launch_plan_from_segments(void* plan, int cap, const int* seg_starts, const int* seg_adapter,
                                      int n_segs, int n_tokens, const PlanAdapters& ad, cudaStream_t s);
cudaError_t launch_bgmv(const ApplyParams& p, int io_dtype, int n_sm, cudaStream_t s);
cudaError_t launch_bgmv_tma(const ApplyParams& p, int io_dtype, int n_sm, cudaStream_t s);
int bgmv_tma_shrink_grid(int n_sm);       // CTAs of the TMA shrink kernel (whoever adds up its split-K slots needs it)
cudaError_t launch_tp_exchange(const b200_lora_tp* tp, void* workspace, int n_proj, int cap, int n_tokens, int skip_push,
                               int n_sm, cudaStream_t s);
// one exchange of a tensor-parallel apply: the rows of the plan's tiles (`tall`) or of its BGMV work segments
// (`fold_grid` > 0: the BGMV rows' v is still the split-K slots of a TMA shrink kernel of that many CTAs)
cudaError_t launch_tp_exchange_rows(const b200_lora_tp* tp, int set, bool tall, bool all_units, const ApplyParams& p, int fold_grid,
                                    int io_dtype, int skip_push, int n_sm, cudaStream_t s);
bool sgmv_tiles_supported(const ApplyParams& p);
cudaError_t launch_sgmv_tiles(const ApplyParams& p, const SgmvParams& sp, int io_dtype, int n_sm, cudaStream_t s);

}  // namespace b200lora
