// extern "C" entry points declared in include/b200_lora.h: argument checks and launches only.
#include <string.h>

#include <cstdlib>
#include <mutex>

#include "lora_common.cuh"

using namespace b200lora;

namespace {

thread_local char g_last_error[256] = "";

int cuda_fail(cudaError_t e) {
    strncpy(g_last_error, cudaGetErrorString(e), sizeof(g_last_error) - 1);
    return B200_LORA_ERR_CUDA;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// ---- tensor maps for the TMA kernels --------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
        tried = true;
    }
    return fn;
}

// 2-D map over a row-major 16-bit matrix [rows, inner] with row pitch `pitch` elements;
// cached per (base, shape, box)
bool tensor_map_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows, uint32_t box_inner,
                   uint32_t box_rows, CUtensorMapSwizzle swizzle, uint64_t pitch = 0) {
    if (pitch == 0) pitch = inner;
    // Encoded maps are kept in a hashed, 4-way set-associative table (4096 entries): an eager loop over
    // many layers presents a few hundred (base pointer, shape) keys per step, and a look-up touches one set.
    struct Entry { const void* base; uint64_t inner, rows, pitch; uint32_t bi, br; int sw; bool used; CUtensorMap map; };
    constexpr int kSets = 1024, kWays = 4;
    static Entry cache[kSets][kWays];
    static unsigned char victim[kSets];
    static std::mutex mu;
    uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
    h = (h ^ (inner * 0x9E3779B97F4A7C15ull) ^ (rows * 0xC2B2AE3D27D4EB4Full) ^ (pitch << 21) ^ ((uint64_t)box_inner << 40) ^
         ((uint64_t)box_rows << 48) ^ ((uint64_t)swizzle << 56)) * 0xFF51AFD7ED558CCDull;
    const int set_idx = (int)((h >> 40) % kSets);
    Entry* set = cache[set_idx];
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < kWays; ++i) {
        const Entry& e = set[i];
        if (e.used && e.base == base && e.inner == inner && e.rows == rows && e.pitch == pitch && e.bi == box_inner &&
            e.br == box_rows && e.sw == (int)swizzle) { *out = e.map; return true; }
    }
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    alignas(64) CUtensorMap m;
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {pitch * 2};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    int way = -1;
    for (int i = 0; i < kWays && way < 0; ++i)
        if (!set[i].used) way = i;
    if (way < 0) {                                          // a full set: its ways are replaced in turn
        way = victim[set_idx];
        victim[set_idx] = (unsigned char)((way + 1) % kWays);
    }
    Entry& e = set[way];
    e.base = base; e.inner = inner; e.rows = rows; e.pitch = pitch; e.bi = box_inner; e.br = box_rows; e.sw = (int)swizzle;
    e.used = true; e.map = m;
    *out = m;
    return true;
}

// The tile kernels (tall runs) and the BGMV kernels (everything else) of one apply touch disjoint
// rows of y, v and the split-K partials, so they run as two chains: the tiles on a side stream
// that forks from the caller's stream and joins it again before the call returns.  Each chain is
// a string of short dependent launches whose start-up and tail leave SMs idle; the other chain's
// CTAs fill them.  One side stream per host thread and device, created on first use (outside
// stream capture: a first use inside a capture runs the two chains one after the other).
struct SideStream {
    cudaStream_t stream;
    cudaEvent_t fork, join;
    int state;                // 0 not tried, 1 ready, -1 unavailable
};
SideStream* side_stream(cudaStream_t caller) {
    static const bool serial = [] { const char* v = getenv("B200_LORA_SERIAL_TILES"); return v && v[0] == '1'; }();
    if (serial) return nullptr;
    thread_local SideStream side[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    SideStream& ss = side[dev];
    if (ss.state == 0) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(caller, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
            cudaGetLastError();
            return nullptr;                                  // try again on a later call
        }
        const bool ok = cudaStreamCreateWithFlags(&ss.stream, cudaStreamNonBlocking) == cudaSuccess &&
                        cudaEventCreateWithFlags(&ss.fork, cudaEventDisableTiming) == cudaSuccess &&
                        cudaEventCreateWithFlags(&ss.join, cudaEventDisableTiming) == cudaSuccess;
        if (!ok) cudaGetLastError();
        ss.state = ok ? 1 : -1;
    }
    return ss.state == 1 ? &ss : nullptr;
}

// rows of an A pool viewed as a [rows, h_in] matrix
uint64_t pool_rows(const b200_lora_adapters* ad) {
    if (!ad->packed) return (uint64_t)ad->n_adapters * ad->n_layers * ad->r_pool;
    if (ad->total_rank > 0) return (uint64_t)ad->total_rank * ad->n_layers;
    return (uint64_t)ad->n_adapters * ad->n_layers * kMaxRank;       // upper bound
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_adapters(const b200_lora_adapters* ad) {
    if (!ad) return B200_LORA_ERR_NULL;
    if (ad->n_adapters < 1 || ad->n_layers < 1) return B200_LORA_ERR_DIM;
    if (ad->r_pool < 1 || ad->r_pool > kMaxRank) return B200_LORA_ERR_RANK;
    if (ad->packed) {
        if (!ad->cum_ranks || !ad->ranks) return B200_LORA_ERR_NULL;
    } else if (ad->r_pool % 8) {
        return B200_LORA_ERR_RANK;     // rows of the dense B pool must stay 16-byte aligned
    }
    return B200_LORA_OK;
}

// true when the TMA kernels may be used as far as ranks are concerned
bool fast_ranks(const b200_lora_adapters* ad) {
    const int r = ad->r_pool;
    const bool pow2 = (r == 8 || r == 16 || r == 32 || r == 64);
    if (!ad->packed && !ad->ranks) return pow2;
    return ad->ranks_pow2 != 0 && (ad->packed || pow2);
}

// the workspace's sticky error word as a status code
int status_of_error_word(unsigned word) {
    if (word == 0u) return B200_LORA_OK;
    return word >= kErrPlanMismatch ? B200_LORA_ERR_DIM : B200_LORA_ERR_TIMEOUT;
}

PlanAdapters plan_adapters(const b200_lora_adapters* ad) {
    PlanAdapters pa;
    pa.ranks = ad->ranks;
    pa.cum_ranks = ad->packed ? reinterpret_cast<const long long*>(ad->cum_ranks) : nullptr;
    pa.scalings = ad->scalings;
    pa.scale = ad->scale;
    pa.r_pool = ad->r_pool;
    pa.n_adapters = ad->n_adapters;
    pa.ranks_pow2 = fast_ranks(ad) ? 1 : 0;
    return pa;
}

}  // namespace

// Scratch for b200_add_lora_bgmv_static: plan + workspace of the largest accepted call.  It
// lives in the library image, so every GPU that loads the library carries it until exit.
static __device__ __align__(256) unsigned char g_static_scratch[B200_LORA_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_mu;
void* g_static_ptr[64] = {nullptr};      // device address of the array, per device (guarded by the mutex)
size_t g_static_last_pb[64] = {0};       // plan bytes of the last static call, per device

// One-time set-up per device: in host code `g_static_scratch` is only a stand-in for the device
// array, so its device address has to be asked for, with that device current.
int static_scratch_address(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e);
    if (dev < 0 || dev >= 64) return B200_LORA_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e);
        g_static_ptr[dev] = ptr;
    }
    *out = g_static_ptr[dev];
    return B200_LORA_OK;
}
}  // namespace

extern "C" {

int b200_lora_arch(void) { return 100; }

const char* b200_lora_last_cuda_error(void) { return g_last_error; }

int b200_lora_stream_capture_id(void* stream, unsigned long long* id) {
    if (!id) return B200_LORA_ERR_NULL;
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    unsigned long long cid = 0;
    cudaError_t e = cudaStreamGetCaptureInfo(static_cast<cudaStream_t>(stream), &st, &cid);
    if (e != cudaSuccess) return cuda_fail(e);
    *id = st == cudaStreamCaptureStatusActive ? cid : 0ull;
    return B200_LORA_OK;
}

size_t b200_lora_plan_bytes(int32_t max_tokens, int32_t n_adapters) {
    if (max_tokens < 1 || n_adapters < 1) return 0;
    return plan_words(max_tokens, n_adapters) * 4;
}

int b200_lora_plan_build(void* plan, size_t plan_bytes, int32_t max_tokens, const void* ids,
                         int32_t ids_are_i64, int32_t n_tokens, const b200_lora_adapters* adapters,
                         void* stream) {
    if (!plan || !ids) return B200_LORA_ERR_NULL;
    int rc = check_adapters(adapters);
    if (rc) return rc;
    if (n_tokens < 1 || n_tokens > max_tokens) return B200_LORA_ERR_DIM;
    const int cap = max_tokens;
    if (plan_bytes < b200_lora_plan_bytes(cap, adapters->n_adapters)) return B200_LORA_ERR_WORKSPACE;
    if (!aligned16(plan)) return B200_LORA_ERR_ALIGN;
    cudaError_t e = launch_plan_build(plan, cap, ids, ids_are_i64, n_tokens, plan_adapters(adapters),
                                      static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? B200_LORA_OK : cuda_fail(e);
}

int b200_lora_plan_from_segments(void* plan, size_t plan_bytes, int32_t max_tokens,
                                 const int32_t* seg_starts, const int32_t* seg_adapter, int32_t n_segs,
                                 int32_t n_tokens, const b200_lora_adapters* adapters, void* stream) {
    if (!plan || !seg_starts || !seg_adapter) return B200_LORA_ERR_NULL;
    int rc = check_adapters(adapters);
    if (rc) return rc;
    if (n_tokens < 1 || n_tokens > max_tokens || n_segs < 1 || n_segs > n_tokens) return B200_LORA_ERR_DIM;
    const int cap = max_tokens;
    if (plan_bytes < b200_lora_plan_bytes(cap, adapters->n_adapters)) return B200_LORA_ERR_WORKSPACE;
    if (!aligned16(plan)) return B200_LORA_ERR_ALIGN;
    cudaError_t e = launch_plan_from_segments(plan, cap, seg_starts, seg_adapter, n_segs, n_tokens,
                                              plan_adapters(adapters), static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? B200_LORA_OK : cuda_fail(e);
}

int b200_lora_plan_read(const void* plan, int32_t* perm, int32_t* seg_starts, int32_t* seg_adapter,
                        int32_t* n_segs, int32_t* n_tokens, void* stream) {
    if (!plan || !n_segs || !n_tokens) return B200_LORA_ERR_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    PlanHeader h;
    cudaError_t e = cudaMemcpyAsync(&h, plan, sizeof(h), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return cuda_fail(e);
    *n_segs = h.n_segs;
    *n_tokens = h.n_tokens;
    if (h.error == 1) return B200_LORA_ERR_ID_RANGE;
    if (h.error == 3) return B200_LORA_ERR_RANK;
    if (h.error) return B200_LORA_ERR_SEGMENTS;
    PlanView pv = plan_view(const_cast<void*>(plan), h.cap, h.n_adapters);
    if (perm) e = cudaMemcpyAsync(perm, pv.perm, 4 * (size_t)h.n_tokens, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess && seg_starts)
        e = cudaMemcpyAsync(seg_starts, pv.seg_start, 4 * (size_t)(h.n_segs + 1), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess && seg_adapter)
        e = cudaMemcpyAsync(seg_adapter, pv.seg_adapter, 4 * (size_t)h.n_segs, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    return e == cudaSuccess ? B200_LORA_OK : cuda_fail(e);
}

size_t b200_lora_workspace_bytes(int32_t max_tokens, int32_t n_proj, int32_t max_h_in) {
    if (max_tokens < 1 || n_proj < 1 || n_proj > kMaxProj || max_h_in < 8) return 0;
    return workspace_bytes(max_tokens, n_proj, max_h_in);
}

int b200_lora_workspace_init(void* workspace, size_t bytes, void* stream) {
    if (!workspace) return B200_LORA_ERR_NULL;
    if (bytes < sizeof(WorkspaceCtl)) return B200_LORA_ERR_WORKSPACE;
    cudaError_t e = cudaMemsetAsync(workspace, 0, bytes, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? B200_LORA_OK : cuda_fail(e);
}

static bool tp_usable(const b200_lora_tp* tp) {
    if (tp->tp < 2 || tp->tp > B200_LORA_TP_MAX_RANKS || tp->rank < 0 || tp->rank >= tp->tp || tp->set_stride == 0) return false;
    for (int r = 0; r < tp->tp; ++r)
        if (!tp->landing[r][0] || !tp->landing[r][1] || !tp->flags[r]) return false;
    return true;
}

// One apply.  With `tp` it is the tensor-parallel form: each chain (the tiles on the side stream,
// the BGMV kernels on the caller's) runs its shrink half, the exchange of its own rows of v over
// the ranks, and its expand half.
static int apply_core(const b200_lora_proj* projs, int32_t n_proj, const b200_lora_adapters* adapters,
                      const void* plan, int32_t max_tokens, int32_t n_tokens, int32_t layer, int32_t io_dtype,
                      int32_t y_dtype, int32_t flags, void* workspace, size_t workspace_bytes_, void* stream,
                      const b200_lora_tp* tp, int skip_arrival) {
    if (!projs || !plan || !workspace) return B200_LORA_ERR_NULL;
    if (tp && !tp_usable(tp)) return B200_LORA_ERR_DIM;
    if (tp && (flags & (B200_LORA_ONLY_SHRINK | B200_LORA_ONLY_EXPAND))) return B200_LORA_ERR_DIM;
    int rc = check_adapters(adapters);
    if (rc) return rc;
    if (n_proj < 1 || n_proj > kMaxProj || max_tokens < 1 || n_tokens < 1 || n_tokens > max_tokens) return B200_LORA_ERR_DIM;
    if (io_dtype != B200_LORA_F16 && io_dtype != B200_LORA_BF16) return B200_LORA_ERR_DTYPE;
    if (y_dtype != io_dtype && y_dtype != B200_LORA_F32) return B200_LORA_ERR_DTYPE;
    if (layer < 0 || layer >= adapters->n_layers) return B200_LORA_ERR_LAYER;
    if (!aligned16(plan) || !aligned16(workspace)) return B200_LORA_ERR_ALIGN;

    ApplyParams p;
    memset(&p, 0, sizeof(p));
    int max_h_in = 0;
    for (int i = 0; i < n_proj; ++i) {
        const b200_lora_proj& q = projs[i];
        if (!q.x || !q.y || !q.wa || !q.wb) return B200_LORA_ERR_NULL;
        if (q.h_in < 8 || q.h_out < 8 || (q.h_in % 8) || (q.h_out % 8)) return B200_LORA_ERR_DIM;
        if (q.ldx < q.h_in || q.ldy < q.h_out || (q.ldx % 8) || (q.ldy % 8)) return B200_LORA_ERR_DIM;
        if (!aligned16(q.x) || !aligned16(q.y) || !aligned16(q.wa) || !aligned16(q.wb)) return B200_LORA_ERR_ALIGN;
        ProjArgs& a = p.proj[i];
        a.x = q.x; a.y = q.y; a.wa = q.wa; a.wb = q.wb;
        a.ldx = q.ldx; a.ldy = q.ldy; a.h_in = q.h_in; a.h_out = q.h_out;
        a.n_super_in = (q.h_in + kSuper - 1) / kSuper;
        a.n_super_out = (q.h_out + kSuper - 1) / kSuper;
        p.total_super_in += a.n_super_in;
        p.total_super_out += a.n_super_out;
        if (q.h_in > max_h_in) max_h_in = q.h_in;
    }
    if (workspace_bytes_ < workspace_bytes(max_tokens, n_proj, max_h_in)) return B200_LORA_ERR_WORKSPACE;
    p.n_proj = n_proj;
    p.ranks = adapters->ranks;
    p.scalings = adapters->scalings;
    p.cum_ranks = reinterpret_cast<const long long*>(adapters->cum_ranks);
    p.n_adapters = adapters->n_adapters;
    p.n_layers = adapters->n_layers;
    p.r_pool = adapters->r_pool;
    p.packed = adapters->packed;
    p.scale = adapters->scale;
    p.layer = layer;
    p.flags = flags;
    p.y_f32 = (y_dtype == B200_LORA_F32);
    p.cap = max_tokens;
    p.n_tokens = n_tokens;
    p.plan = const_cast<void*>(plan);
    p.workspace = workspace;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int n_sm = sm_count();
    cudaError_t e = cudaSuccess;
    SideStream* side = nullptr;
    if (!sgmv_tiles_supported(p)) p.flags |= B200_LORA_NO_TENSOR;
    if (!(p.flags & B200_LORA_NO_TENSOR)) {
        SgmvParams sp;
        memset(&sp, 0, sizeof(sp));
        bool ok = true;
        const uint64_t arows = pool_rows(adapters);
        for (int i = 0; i < n_proj && ok; ++i) {
            const b200_lora_proj& q = projs[i];
            ok = tensor_map_2d(&sp.xmap[i], q.x, (uint64_t)q.h_in, (uint64_t)n_tokens, 64, 128,
                               CU_TENSOR_MAP_SWIZZLE_128B, (uint64_t)q.ldx);
            if (ok && !p.y_f32)
                ok = tensor_map_2d(&sp.ymap[i], q.y, (uint64_t)q.h_out, (uint64_t)n_tokens, 64, 128,
                                   CU_TENSOR_MAP_SWIZZLE_128B, (uint64_t)q.ldy);
            for (int c = 0; c < 3 && ok; ++c) {
                const uint64_t rc = 16u << c;
                if (!adapters->packed && rc != (uint64_t)adapters->r_pool) continue;   // dense pools have one rank
                const uint64_t brows = arows * (uint64_t)q.h_out / rc;
                const CUtensorMapSwizzle sw = c == 0 ? CU_TENSOR_MAP_SWIZZLE_32B
                                            : c == 1 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
                ok = tensor_map_2d(&sp.bmap[i][c], q.wb, rc, brows, (uint32_t)rc, 128, sw) &&
                     tensor_map_2d(&sp.amap[i][c], q.wa, (uint64_t)q.h_in, arows, 64, (uint32_t)rc, CU_TENSOR_MAP_SWIZZLE_128B);
            }
        }
        if (!ok) p.flags |= B200_LORA_NO_TENSOR;        // no driver entry point: everything on the BGMV kernels
        else {
            side = side_stream(s);
            if (side && (cudaEventRecord(side->fork, s) != cudaSuccess ||
                         cudaStreamWaitEvent(side->stream, side->fork, 0) != cudaSuccess)) {
                cudaGetLastError();
                side = nullptr;
            }
            cudaStream_t ts = side ? side->stream : s;
            if (!tp) e = launch_sgmv_tiles(p, sp, io_dtype, n_sm, ts);
            else {
                ApplyParams h = p;
                h.flags = p.flags | B200_LORA_ONLY_SHRINK;
                e = launch_sgmv_tiles(h, sp, io_dtype, n_sm, ts);
                if (e == cudaSuccess) e = launch_tp_exchange_rows(tp, 1, true, false, p, 0, io_dtype, skip_arrival, n_sm, ts);
                h.flags = p.flags | B200_LORA_ONLY_EXPAND;
                if (e == cudaSuccess) e = launch_sgmv_tiles(h, sp, io_dtype, n_sm, ts);
            }
        }
    }
    bool fast = fast_ranks(adapters);
    for (int i = 0; i < n_proj; ++i)
        // units are cut at multiples of 128 columns (the shrink kernel's weight box, the widest
        // per-warp column group of the expand kernel), so the last unit of a row may be partial
        if ((projs[i].h_in % 128) || (projs[i].h_out % 128) || projs[i].h_in > 8192) fast = false;
    if (fast) {
        for (int i = 0; i < n_proj && fast; ++i)
            for (int c = 0; c < 4 && fast; ++c) {
                const uint32_t rc = 8u << c;
                if (!adapters->packed && rc != (uint32_t)adapters->r_pool) continue;    // dense pools have one rank
                fast = tensor_map_2d(&p.amap[i][c], projs[i].wa, (uint64_t)projs[i].h_in, pool_rows(adapters), 128, rc,
                                     CU_TENSOR_MAP_SWIZZLE_NONE);
            }
    }
    auto bgmv = [&](const ApplyParams& q) { return fast ? launch_bgmv_tma(q, io_dtype, n_sm, s) : launch_bgmv(q, io_dtype, n_sm, s); };
    if (e == cudaSuccess && !tp) e = bgmv(p);
    if (e == cudaSuccess && tp) {
        // the TMA shrink kernel leaves its split-K slots and the exchange adds them up; the general one leaves v
        ApplyParams h = p;
        h.flags = p.flags | B200_LORA_ONLY_SHRINK | (fast ? B200_LORA_KEEP_PARTIALS : 0);
        e = bgmv(h);
        if (e == cudaSuccess)
            e = launch_tp_exchange_rows(tp, 0, false, (p.flags & B200_LORA_NO_TENSOR) != 0, p, fast ? bgmv_tma_shrink_grid(n_sm) : 0,
                                        io_dtype, skip_arrival, n_sm, s);
        h.flags = p.flags | B200_LORA_ONLY_EXPAND;
        if (e == cudaSuccess) e = bgmv(h);
    }
    if (side) {                                             // the side stream always joins, also after a failed launch
        cudaError_t j = cudaEventRecord(side->join, side->stream);
        if (j == cudaSuccess) j = cudaStreamWaitEvent(s, side->join, 0);
        if (e == cudaSuccess) e = j;
    }
    return e == cudaSuccess ? B200_LORA_OK : cuda_fail(e);
}

int b200_lora_apply(const b200_lora_proj* projs, int32_t n_proj, const b200_lora_adapters* adapters,
                    const void* plan, int32_t max_tokens, int32_t n_tokens, int32_t layer, int32_t io_dtype,
                    int32_t y_dtype, int32_t flags, void* workspace, size_t workspace_bytes_, void* stream) {
    return apply_core(projs, n_proj, adapters, plan, max_tokens, n_tokens, layer, io_dtype, y_dtype, flags, workspace,
                      workspace_bytes_, stream, nullptr, 0);
}

int b200_lora_apply_tp(const b200_lora_proj* projs, int32_t n_proj, const b200_lora_adapters* adapters,
                       const void* plan, int32_t max_tokens, int32_t n_tokens, int32_t layer, int32_t io_dtype,
                       int32_t y_dtype, int32_t flags, void* workspace, size_t workspace_bytes_, const b200_lora_tp* tp,
                       int32_t skip_arrival, void* stream) {
    if (!tp) return B200_LORA_ERR_NULL;
    return apply_core(projs, n_proj, adapters, plan, max_tokens, n_tokens, layer, io_dtype, y_dtype, flags, workspace,
                      workspace_bytes_, stream, tp, skip_arrival);
}

int b200_lora_workspace_v_region(int32_t max_tokens, int32_t n_proj, size_t* offset_bytes, size_t* size_bytes) {
    if (!offset_bytes || !size_bytes) return B200_LORA_ERR_NULL;
    if (max_tokens < 1 || n_proj < 1 || n_proj > kMaxProj) return B200_LORA_ERR_DIM;
    // the view only does address arithmetic: run it on a fictitious 128-byte-aligned base
    WorkspaceView w = workspace_view(reinterpret_cast<void*>(uintptr_t(1) << 20), max_tokens, n_proj);
    *offset_bytes = reinterpret_cast<uintptr_t>(w.v) - (uintptr_t(1) << 20);
    *size_bytes = (size_t)n_proj * max_tokens * kMaxRank * 4;
    return B200_LORA_OK;
}

// ---- tensor-parallel exchange ---------------------------------------------------------------------
// one allocation: two sets of two landing buffers [tp + 1][n_proj][max_tokens][64] of 8-byte packets (value,
// exchange number), then per set the exchange counter and the CTA counter; everything 256-byte aligned
static size_t tp_landing_bytes(int32_t max_tokens, int32_t n_proj, int32_t tp) {
    return (((size_t)(tp + 1) * n_proj * max_tokens * kMaxRank * 8) + 255) & ~size_t(255);     // a slot per rank + one for owners' sums
}

size_t b200_lora_tp_bytes(int32_t max_tokens, int32_t n_proj, int32_t tp) {
    if (max_tokens < 1 || n_proj < 1 || n_proj > kMaxProj || tp < 2 || tp > B200_LORA_TP_MAX_RANKS) return 0;
    return 4 * tp_landing_bytes(max_tokens, n_proj, tp) + B200_LORA_TP_COUNTER_BYTES;
}

int b200_lora_tp_alloc(void** base, size_t bytes) {
    if (!base || bytes == 0) return B200_LORA_ERR_NULL;
    cudaError_t e = cudaMalloc(base, bytes);
    if (e == cudaSuccess) e = cudaMemset(*base, 0, bytes);
    return e == cudaSuccess ? B200_LORA_OK : cuda_fail(e);
}

int b200_lora_tp_free(void* base) {
    cudaError_t e = cudaFree(base);
    return e == cudaSuccess ? B200_LORA_OK : cuda_fail(e);
}

int b200_lora_tp_export(void* base, void* handle64) {
    if (!base || !handle64) return B200_LORA_ERR_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, base);
    if (e != cudaSuccess) return cuda_fail(e);
    memcpy(handle64, &h, 64);
    return B200_LORA_OK;
}

int b200_lora_tp_open(const void* handle64, void** mapped) {
    if (!handle64 || !mapped) return B200_LORA_ERR_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    cudaError_t e = cudaIpcOpenMemHandle(mapped, h, cudaIpcMemLazyEnablePeerAccess);
    return e == cudaSuccess ? B200_LORA_OK : cuda_fail(e);
}

int b200_lora_tp_close(void* mapped) {
    cudaError_t e = cudaIpcCloseMemHandle(mapped);
    return e == cudaSuccess ? B200_LORA_OK : cuda_fail(e);
}

int b200_lora_tp_layout(b200_lora_tp* tp, int32_t r, void* base, int32_t max_tokens, int32_t n_proj) {
    if (!tp || !base) return B200_LORA_ERR_NULL;
    if (r < 0 || r >= B200_LORA_TP_MAX_RANKS || tp->tp < 2 || tp->tp > B200_LORA_TP_MAX_RANKS) return B200_LORA_ERR_DIM;
    const size_t lb = tp_landing_bytes(max_tokens, n_proj, tp->tp);
    char* b = static_cast<char*>(base);
    tp->landing[r][0] = b;
    tp->landing[r][1] = b + lb;
    tp->flags[r] = b + 4 * lb;
    tp->set_stride = 2 * lb;
    return B200_LORA_OK;
}

int b200_lora_tp_exchange(const b200_lora_tp* tp, void* workspace, int32_t max_tokens, int32_t n_tokens,
                          int32_t n_proj, int32_t skip_arrival, void* stream) {
    if (!tp || !workspace) return B200_LORA_ERR_NULL;
    if (tp->tp < 2 || tp->tp > B200_LORA_TP_MAX_RANKS || tp->rank < 0 || tp->rank >= tp->tp) return B200_LORA_ERR_DIM;
    if (max_tokens < 1 || n_tokens < 1 || n_tokens > max_tokens || n_proj < 1 || n_proj > kMaxProj) return B200_LORA_ERR_DIM;
    if (!tp_usable(tp)) return B200_LORA_ERR_NULL;
    cudaError_t e = launch_tp_exchange(tp, workspace, n_proj, max_tokens, n_tokens, skip_arrival, sm_count(),
                                       static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? B200_LORA_OK : cuda_fail(e);
}

int b200_lora_workspace_status(const void* workspace, void* stream) {
    if (!workspace) return B200_LORA_ERR_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    WorkspaceCtl ctl;
    cudaError_t e = cudaMemcpyAsync(&ctl, workspace, sizeof(ctl), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return cuda_fail(e);
    return status_of_error_word(ctl.error);
}

size_t b200_add_lora_bgmv_workspace_bytes(int32_t n_tokens, int32_t n_adapters, int32_t h_in) {
    size_t pb = b200_lora_plan_bytes(n_tokens, n_adapters);
    size_t wb = b200_lora_workspace_bytes(n_tokens, 1, h_in);
    if (!pb || !wb) return 0;
    return ((pb + 255) & ~size_t(255)) + wb;
}

int b200_add_lora_bgmv(void* y, const void* x, const void* wa_T_all, const void* wb_T_all,
                       const void* indicies, int32_t indicies_are_i64, int32_t n_tokens,
                       int32_t h_in, int32_t h_out, int32_t n_adapters, int32_t n_layers, int32_t r,
                       int32_t layer_idx, float scale, int32_t dtype,
                       void* workspace, size_t workspace_bytes_, void* stream) {
    if (!workspace) return B200_LORA_ERR_NULL;
    if (n_tokens < 1 || n_adapters < 1) return B200_LORA_ERR_DIM;
    if (workspace_bytes_ < b200_add_lora_bgmv_workspace_bytes(n_tokens, n_adapters, h_in)) return B200_LORA_ERR_WORKSPACE;
    b200_lora_adapters ad;
    memset(&ad, 0, sizeof(ad));
    ad.n_adapters = n_adapters; ad.n_layers = n_layers; ad.r_pool = r; ad.packed = 0; ad.scale = scale;
    size_t pb = (b200_lora_plan_bytes(n_tokens, n_adapters) + 255) & ~size_t(255);
    char* ws = static_cast<char*>(workspace) + pb;
    // Where the control words sit depends on this call's n_tokens and n_adapters, so a buffer that
    // served a call of another shape holds that call's records or partial sums there: clear them
    // (error word and arrival counters must start at zero) on every call.
    cudaError_t ce = cudaMemsetAsync(ws, 0, ws_ctl_bytes(n_tokens), static_cast<cudaStream_t>(stream));
    if (ce != cudaSuccess) return cuda_fail(ce);
    int rc = b200_lora_plan_build(workspace, pb, n_tokens, indicies, indicies_are_i64, n_tokens, &ad, stream);
    if (rc) return rc;
    b200_lora_proj pj;
    pj.x = x; pj.y = y; pj.wa = wa_T_all; pj.wb = wb_T_all;
    pj.ldx = h_in; pj.ldy = h_out; pj.h_in = h_in; pj.h_out = h_out;
    return b200_lora_apply(&pj, 1, &ad, workspace, n_tokens, n_tokens, layer_idx, dtype, dtype, B200_LORA_NO_TENSOR, ws,
                           workspace_bytes_ - pb, stream);
}

// ---- allocation-free variant ---------------------------------------------------------------
int b200_add_lora_bgmv_static(void* y, const void* x, const void* wa_T_all, const void* wb_T_all,
                              const void* indicies, int32_t indicies_are_i64, int32_t n_tokens,
                              int32_t h_in, int32_t h_out, int32_t n_adapters, int32_t n_layers, int32_t r,
                              int32_t layer_idx, float scale, int32_t dtype, void* stream) {
    if (n_tokens < 1 || n_tokens > B200_LORA_STATIC_MAX_TOKENS || n_adapters < 1 ||
        n_adapters > B200_LORA_STATIC_MAX_ADAPTERS || h_in < 8 || h_in > B200_LORA_STATIC_MAX_H_IN)
        return B200_LORA_ERR_WORKSPACE;          // beyond what the static scratch was sized for
    const size_t need = b200_add_lora_bgmv_workspace_bytes(n_tokens, n_adapters, h_in);
    if (need == 0 || need > (size_t)B200_LORA_STATIC_SCRATCH_BYTES) return B200_LORA_ERR_WORKSPACE;

    void* scratch = nullptr;
    int rc = static_scratch_address(&scratch);       // the first call on a device looks the address up
    if (rc) return rc;
    // The array keeps whatever the previous call left; b200_add_lora_bgmv clears the control
    // words (arrival counters, error word) of this call's layout and rebuilds the plan.
    const size_t pb = (b200_lora_plan_bytes(n_tokens, n_adapters) + 255) & ~size_t(255);
    {
        std::lock_guard<std::mutex> lock(g_static_mu);
        int dev = 0;
        cudaGetDevice(&dev);
        g_static_last_pb[dev] = pb;              // where the last call's workspace part begins
    }
    return b200_add_lora_bgmv(y, x, wa_T_all, wb_T_all, indicies, indicies_are_i64, n_tokens, h_in, h_out,
                              n_adapters, n_layers, r, layer_idx, scale, dtype, scratch,
                              (size_t)B200_LORA_STATIC_SCRATCH_BYTES, stream);
}

int b200_add_lora_bgmv_static_status(void* stream) {
    void* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc) return rc;
    size_t pb;
    {
        std::lock_guard<std::mutex> lock(g_static_mu);
        int dev = 0;
        cudaGetDevice(&dev);
        pb = g_static_last_pb[dev];
    }
    if (pb == 0) return B200_LORA_OK;            // no call yet on this device
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    PlanHeader h;
    WorkspaceCtl ctl;
    cudaError_t e = cudaMemcpyAsync(&h, scratch, sizeof(h), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(&ctl, static_cast<char*>(scratch) + pb, sizeof(ctl), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return cuda_fail(e);
    if (h.error == 1) return B200_LORA_ERR_ID_RANGE;
    if (h.error == 3) return B200_LORA_ERR_RANK;
    if (h.error) return B200_LORA_ERR_SEGMENTS;
    return status_of_error_word(ctl.error);
}

}  // extern "C"
