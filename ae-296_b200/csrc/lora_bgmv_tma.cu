// Decode BGMV, fast path: TMA bulk copies + mbarrier pipeline + mma.sync.
//
// Used when every adapter rank is 8, 16, 32 or 64 and every projection width is a multiple
// of 256, which makes each unit's weight tile a handful of plain contiguous byte ranges:
//   shrink  A rows [r, KC] of one adapter/layer     -> r bulk copies (one per row)
//   expand  B rows [JC, r] of one adapter/layer     -> ONE bulk copy (rows are contiguous)
// A dedicated producer warp walks the unit list and issues `cp.async.bulk` copies (weights,
// the unit's activation rows, the y tile to update) into a 4-stage shared-memory ring; each
// stage's arrival is tracked by an mbarrier transaction count.  The consumer warps never
// compute a load address: they wait on the stage's barrier, read MMA fragments with 128-bit
// shared loads and run mma.sync m16n8k16 with the unit's <= 8 tokens as M rows, weight rows
// as N, fp32 accumulators.  Tiles are stored unswizzled; the k index inside a 32-wide block
// is permuted identically for both operands so that each thread's fragment is one contiguous
// 16-byte chunk, and rows are padded by 64 bytes (shrink) so those reads are conflict-free.
// The expand updates a staged y tile in shared memory and writes it back with bulk stores.
//
// Every mbarrier wait is bounded: on expiry the thread records an error word in the workspace
// and carries on with the same control flow, so the kernel always terminates.
//
// Semantics: add_lora_bgmv(y, x, wa_T_all, wb_T_all, indicies, layer_idx, scale) of the
// reference (lightllm/models/lora_gpu.py:138,150,162), pools as at :33-40.
#include "lora_common.cuh"

namespace b200lora {

namespace {

constexpr int kStages = 4;
constexpr int kConsWarps = 16;
constexpr int kConsThreads = kConsWarps * 32;
constexpr int kThreads = kConsThreads + 32;       // + one producer warp
constexpr int kRowPad = 64;                       // bytes added to shrink tile rows
constexpr int kShrinkStage = 50688;               // max over rank classes of W + X tiles
constexpr int kYPad = 16;
constexpr int kYBytes = 8 * (1024 * 2 + kYPad);
constexpr int kVPitch = 72;                       // floats per token row of the v tile
constexpr int kVBytes = 8 * kVPitch * 4;
constexpr int kExpandStage = 32768 + kYBytes + kVBytes;
constexpr int kRedBytes = 8 * 8 * 68 * 4;
constexpr unsigned kSpinLimit = 1u << 22;

struct Meta {
    UnitRec u;
    int proj, c0, valid, kc, n_chunks;
    int width_ok;           // columns (shrink) / rows (expand) of the unit inside the projection
    int pad[2];
};
static_assert(sizeof(Meta) == 96, "meta slot");

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait; on expiry records `code` and returns so that control flow stays uniform
__device__ __forceinline__ void mbar_wait(unsigned bar, unsigned parity, unsigned* err, unsigned code) {
    for (unsigned i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return;
        // once any wait anywhere has expired, drain quickly instead of waiting in full again
        if ((i & 0x3fffu) == 0x3fffu && *reinterpret_cast<volatile unsigned*>(err) != 0u) break;
    }
    atomicMax(err, code);
}
__device__ __forceinline__ void bulk_g2s(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, unsigned src, unsigned bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsThreads) : "memory"); }

template <typename T> struct Mma;
template <> struct Mma<__half> {
    static __device__ __forceinline__ void run(float (&c)[4], unsigned a0, unsigned a2, unsigned b0, unsigned b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
    }
};
template <> struct Mma<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float (&c)[4], unsigned a0, unsigned a2, unsigned b0, unsigned b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
    }
};

__device__ __forceinline__ unsigned atom_add_acq_rel(unsigned* p, unsigned v) {
    unsigned old;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}

__device__ __forceinline__ void decode_item(const ApplyParams& p, int it, int n_units, bool expand,
                                            int& unit, int& proj, int& super) {
    unit = it % n_units;
    int sp = it / n_units;
    int pi = 0;
#pragma unroll
    for (int i = 0; i < kMaxProj; ++i) {
        const int ns = expand ? p.proj[i].n_super_out : p.proj[i].n_super_in;
        if (i < p.n_proj - 1 && pi == i && sp >= ns) { sp -= ns; pi = i + 1; }
    }
    proj = pi;
    super = sp;
}

// Producer: fetch the unit record of item `it` (lanes 0..15 one word each), derive the meta
// slot, publish it to shared memory.  Returns with every lane holding the meta in `m`.
__device__ __forceinline__ void producer_meta(const ApplyParams& p, const PlanView& pv, int it, int n_units,
                                              bool expand, int lane, Meta* slot) {
    int unit, proj, super;
    decode_item(p, it, n_units, expand, unit, proj, super);
    if (lane < 16) reinterpret_cast<int*>(&slot->u)[lane] = __ldg(pv.unit_tab + (size_t)unit * 16 + lane);
    __syncwarp();
    if (lane == 0) {
        const int r_pad = pad_rank(slot->u.rank);
        const int width = kSuper / n_sub(r_pad);
        const int c0 = super * kSuper + slot->u.sub * width;
        const int h = expand ? p.proj[proj].h_out : p.proj[proj].h_in;
        slot->proj = proj;
        slot->c0 = c0;
        slot->valid = c0 < h;
        slot->kc = c0 / width;
        slot->n_chunks = (p.proj[proj].h_in + width - 1) / width;
        slot->width_ok = min(width, h - c0);
    }
    __syncwarp();
}

// =============================================================================================
// shrink
// =============================================================================================
template <typename T>
__device__ __forceinline__ void shrink_produce(const ApplyParams& p, const Meta& m, unsigned stage, unsigned bar,
                                               int lane) {
    const ProjArgs& pj = p.proj[m.proj];
    const int r = m.u.rank;
    const int kc_cols = kSuper / n_sub(r);
    const unsigned pitch = kc_cols * 2 + kRowPad;
    const unsigned row_bytes = m.width_ok * 2;
    if (lane == 0) mbar_arrive_expect_tx(bar, row_bytes * (r + m.u.ntok));
    __syncwarp();
    const T* A = reinterpret_cast<const T*>(pj.wa) + block_row0(p, m.u) * (long long)pj.h_in + m.c0;
    for (int row = lane; row < r; row += 32)
        bulk_g2s(stage + row * pitch, A + (long long)row * pj.h_in, row_bytes, bar);
    const unsigned xbase = stage + r * pitch;
    if (lane < m.u.ntok)
        bulk_g2s(xbase + lane * pitch, reinterpret_cast<const T*>(pj.x) + (long long)m.u.tok[lane] * pj.ldx + m.c0,
                 row_bytes, bar);
}

template <typename T>
__device__ __forceinline__ void shrink_consume(const ApplyParams& p, const WorkspaceView& ws, const Meta& m,
                                               const unsigned char* stage, float* red, int tid) {
    const int lane = tid & 31, warp = tid >> 5;
    const int r = m.u.rank;
    const int NB = r / 8;
    const int nsplit = NB >= 2 ? 2 : 1;
    const int ksplit = kConsWarps / nsplit;
    const int NBW = NB / nsplit;                           // 1, 1, 2, 4
    const int kc_cols = kSuper / n_sub(r);
    const int pitch = kc_cols * 2 + kRowPad;
    const int kslot = warp % ksplit, nhalf = warp / ksplit;
    const int nk32 = kc_cols / 32 / ksplit;                // 2, 4, 2, 1
    const int g = lane >> 2, t = lane & 3;
    const unsigned char* xrow = stage + (r + g) * pitch + t * 16;
    const unsigned char* wrow = stage + (nhalf * NBW * 8 + g) * pitch + t * 16;
    const int rp = r + 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int kb = 0; kb < nk32; ++kb) {
        const int col = (kslot * nk32 + kb) * 32;
        if (col < m.width_ok) {
            const uint4 xa = *reinterpret_cast<const uint4*>(xrow + col * 2);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (i < NBW) {
                    const uint4 w = *reinterpret_cast<const uint4*>(wrow + i * 8 * pitch + col * 2);
                    Mma<T>::run(acc[i], xa.x, xa.y, w.x, w.y);
                    Mma<T>::run(acc[i], xa.z, xa.w, w.z, w.w);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (i < NBW) {
            float2* dst = reinterpret_cast<float2*>(red + (kslot * 8 + g) * rp + (nhalf * NBW + i) * 8 + 2 * t);
            *dst = make_float2(acc[i][0], acc[i][1]);
        }
    }
}

template <typename T>
__device__ __forceinline__ void shrink_publish(const ApplyParams& p, const WorkspaceView& ws, const Meta& m,
                                               const float* red, int tid) {
    const int r = m.u.rank, rp = r + 4;
    const int ksplit = kConsWarps / (r >= 16 ? 2 : 1);
    const int outs = m.u.ntok * r;
    const int rshift = 31 - __clz(r);
    for (int idx = tid; idx < outs; idx += kConsThreads) {
        const int tok = idx >> rshift, i = idx & (r - 1);
        float s = 0.f;
        for (int w = 0; w < ksplit; ++w) s += red[(w * 8 + tok) * rp + i];
        ws.partial[(((size_t)m.kc * p.n_proj + m.proj) * p.cap + (m.u.start + tok)) * kMaxRank + i] = s;
    }
}

template <typename T>
__device__ __forceinline__ void shrink_fold(const ApplyParams& p, const WorkspaceView& ws, const Meta& m, int tid) {
    const int r = m.u.rank;
    const bool mid_round = (p.flags & B200_LORA_MID_ROUND) != 0;
    const int outs = m.u.ntok * r;
    const int rshift = 31 - __clz(r);
    const size_t cstride = (size_t)p.n_proj * p.cap * kMaxRank;
    for (int idx = tid; idx < outs; idx += kConsThreads) {
        const int pos = m.u.start + (idx >> rshift), i = idx & (r - 1);
        const float* src = &ws.partial[((size_t)m.proj * p.cap + pos) * kMaxRank + i];
        float s = 0.f;
        int c = 0;
        for (; c + 8 <= m.n_chunks; c += 8) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __ldcg(src + (size_t)(c + j) * cstride);
#pragma unroll
            for (int j = 0; j < 8; ++j) s += v[j];
        }
        for (; c < m.n_chunks; ++c) s += __ldcg(src + (size_t)c * cstride);
        if (mid_round) s = Cvt<T>::round1(s);
        ws.v[((size_t)m.proj * p.cap + pos) * kMaxRank + i] = s;
    }
    if (tid == 0) ws.counters[(size_t)m.proj * p.cap + m.u.wseg] = 0u;
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1) bgmv_shrink_tma_kernel(const __grid_constant__ ApplyParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    float* red = reinterpret_cast<float*>(smem + kStages * kShrinkStage);
    Meta* meta = reinterpret_cast<Meta*>(smem + kStages * kShrinkStage + kRedBytes);
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(meta + 2 * kStages);
    int* s_fold = reinterpret_cast<int*>(bars + 2 * kStages);

    PlanView pv = plan_view(p.plan, p.cap, p.n_adapters);
    WorkspaceView ws = workspace_view(p.workspace, p.cap, p.n_proj);
    const PlanHeader hdr = *pv.hdr;
    if (hdr.error || hdr.cap != p.cap) return;
    const int n_units = (p.flags & B200_LORA_NO_TENSOR) ? hdr.n_units : hdr.n_units_short;
    const int n_items = n_units * p.total_super_in;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int first = blockIdx.x, stride = gridDim.x;
    if (first >= n_items) return;
    const int n_local = (n_items - first + stride - 1) / stride;
    unsigned* err = &ws.ctl->error;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);                 // full: producer's arrive + tx bytes
            mbar_init(smem_u32(&bars[kStages + s]), 1);       // empty: one consumer thread
        }
        *s_fold = -1;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kConsWarps) {
        // ---------------- producer warp ----------------
        for (int n = 0; n < n_local; ++n) {
            const int s = n % kStages;
            const unsigned ph = (n / kStages) & 1;
            mbar_wait(smem_u32(&bars[kStages + s]), ph ^ 1, err, 1);
            Meta* slot = &meta[n % (2 * kStages)];
            producer_meta(p, pv, first + n * stride, n_units, false, lane, slot);
            const unsigned full = smem_u32(&bars[s]);
            if (slot->valid) shrink_produce<T>(p, *slot, smem_u32(smem + s * kShrinkStage), full, lane);
            else if (lane == 0) mbar_arrive(full);
        }
        return;
    }

    // ---------------- consumer warps ----------------
    unsigned ticket = 0;
    for (int n = 0; n < n_local; ++n) {
        const int s = n % kStages;
        const unsigned ph = (n / kStages) & 1;
        const int fold_slot = *s_fold;
        if (fold_slot >= 0) shrink_fold<T>(p, ws, meta[fold_slot], tid);
        const Meta& pm = meta[(n + 2 * kStages - 1) % (2 * kStages)];
        const bool arrive = n > 0 && pm.valid;
        if (tid == 0 && arrive) ticket = atom_add_acq_rel(&ws.counters[(size_t)pm.proj * p.cap + pm.u.wseg], 1u);
        mbar_wait(smem_u32(&bars[s]), ph, err, 2);
        const Meta& m = meta[n % (2 * kStages)];
        if (m.valid) shrink_consume<T>(p, ws, m, smem + s * kShrinkStage, red, tid);
        cons_sync();
        if (tid == 0) mbar_arrive(smem_u32(&bars[kStages + s]));       // stage is free again
        if (m.valid) shrink_publish<T>(p, ws, m, red, tid);
        if (tid == 0) {
            int f = -1;
            if (arrive && ticket == (unsigned)(pm.n_chunks - 1)) f = (n + 2 * kStages - 1) % (2 * kStages);
            *s_fold = f;
        }
        cons_sync();
    }
    const int last_fold = *s_fold;
    if (last_fold >= 0) shrink_fold<T>(p, ws, meta[last_fold], tid);
    cons_sync();
    const Meta& lm = meta[(n_local - 1) % (2 * kStages)];
    if (lm.valid) {
        if (tid == 0) {
            ticket = atom_add_acq_rel(&ws.counters[(size_t)lm.proj * p.cap + lm.u.wseg], 1u);
            *s_fold = (ticket == (unsigned)(lm.n_chunks - 1)) ? 1 : 0;
        }
        cons_sync();
        if (*s_fold == 1) shrink_fold<T>(p, ws, lm, tid);
    }
}

// =============================================================================================
// expand
// =============================================================================================
template <typename T>
__device__ __forceinline__ void expand_produce(const ApplyParams& p, const WorkspaceView& ws, const Meta& m,
                                               unsigned stage, unsigned bar, int lane) {
    const ProjArgs& pj = p.proj[m.proj];
    const int r = m.u.rank;
    const int jc = kSuper / n_sub(r);
    const unsigned w_bytes = m.width_ok * r * 2;
    const unsigned y_bytes = p.y_f32 ? 0u : m.width_ok * 2;
    const unsigned v_bytes = r * 4;
    if (lane == 0) mbar_arrive_expect_tx(bar, w_bytes + m.u.ntok * (y_bytes + v_bytes));
    __syncwarp();
    if (lane == 0) {
        const T* B = reinterpret_cast<const T*>(pj.wb) + (block_row0(p, m.u) * (long long)pj.h_out + (long long)m.c0 * r);
        bulk_g2s(stage, B, w_bytes, bar);
    }
    if (lane < m.u.ntok) {
        if (y_bytes)
            bulk_g2s(stage + 32768 + lane * (jc * 2 + kYPad),
                     reinterpret_cast<const T*>(pj.y) + (long long)m.u.tok[lane] * pj.ldy + m.c0, y_bytes, bar);
        bulk_g2s(stage + 32768 + kYBytes + lane * (kVPitch * 4),
                 ws.v + ((size_t)m.proj * p.cap + m.u.start + lane) * kMaxRank, v_bytes, bar);
    }
}

// hi/lo split of two fp32 values into packed 16-bit pairs
template <typename T>
__device__ __forceinline__ void split2(float v0, float v1, unsigned& hi, unsigned& lo) {
    const float h0 = Cvt<T>::round1(v0), h1 = Cvt<T>::round1(v1);
    hi = Cvt<T>::pack2(h0, h1);
    lo = Cvt<T>::pack2(v0 - h0, v1 - h1);
}

// R = rank class.  Thread (g, t) of a warp owns, for token g and output rows (8*block + 2t, +1):
//   R=64: chunks 2t and 2t+1 of each 128-byte weight row (4 MMA k-steps)
//   R=32: chunk t of each 64-byte row (2 k-steps);  R=16: 8 bytes (1 k-step);  R=8: 4 bytes.
template <typename T, int R>
__device__ __forceinline__ void expand_consume(const ApplyParams& p, const Meta& m, unsigned char* stage, int tid) {
    constexpr int CALLS = R == 64 ? 4 : R == 32 ? 2 : 1;
    constexpr int JC = kSuper / (R <= 16 ? 2 : R / 8);
    constexpr int NBW = JC / 8 / kConsWarps;
    const ProjArgs& pj = p.proj[m.proj];
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int ntok = m.u.ntok;
    const float scale = m.u.scale;
    const float* vt = reinterpret_cast<const float*>(stage + 32768 + kYBytes) + g * kVPitch;

    unsigned ah[CALLS][2], al[CALLS][2];
    if (g < ntok) {
        if (R == 64) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const float4 lo4 = *reinterpret_cast<const float4*>(vt + (2 * t + c) * 8);
                const float4 hi4 = *reinterpret_cast<const float4*>(vt + (2 * t + c) * 8 + 4);
                split2<T>(lo4.x, lo4.y, ah[2 * c][0], al[2 * c][0]);
                split2<T>(lo4.z, lo4.w, ah[2 * c][1], al[2 * c][1]);
                split2<T>(hi4.x, hi4.y, ah[2 * c + 1][0], al[2 * c + 1][0]);
                split2<T>(hi4.z, hi4.w, ah[2 * c + 1][1], al[2 * c + 1][1]);
            }
        } else if (R == 32) {
            const float4 lo4 = *reinterpret_cast<const float4*>(vt + t * 8);
            const float4 hi4 = *reinterpret_cast<const float4*>(vt + t * 8 + 4);
            split2<T>(lo4.x, lo4.y, ah[0][0], al[0][0]);
            split2<T>(lo4.z, lo4.w, ah[0][1], al[0][1]);
            split2<T>(hi4.x, hi4.y, ah[CALLS - 1][0], al[CALLS - 1][0]);
            split2<T>(hi4.z, hi4.w, ah[CALLS - 1][1], al[CALLS - 1][1]);
        } else if (R == 16) {
            const float4 v4 = *reinterpret_cast<const float4*>(vt + t * 4);
            split2<T>(v4.x, v4.y, ah[0][0], al[0][0]);
            split2<T>(v4.z, v4.w, ah[0][1], al[0][1]);
        } else {
            const float2 v2 = *reinterpret_cast<const float2*>(vt + t * 2);
            split2<T>(v2.x, v2.y, ah[0][0], al[0][0]);
            ah[0][1] = 0u; al[0][1] = 0u;
        }
    } else {
#pragma unroll
        for (int c = 0; c < CALLS; ++c) { ah[c][0] = ah[c][1] = al[c][0] = al[c][1] = 0u; }
    }

    unsigned char* ysb = stage + 32768;
    constexpr int ypitch = JC * 2 + kYPad;
    const int jbase = warp * NBW * 8;
#pragma unroll 2
    for (int nb = 0; nb < NBW; ++nb) {
        const int jrow = jbase + nb * 8 + g;                 // this thread's weight row (N index g)
        const unsigned char* wr = stage + jrow * (R * 2);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (R == 64) {
            const uint4 w0 = *reinterpret_cast<const uint4*>(wr + (2 * t) * 16);
            const uint4 w1 = *reinterpret_cast<const uint4*>(wr + (2 * t + 1) * 16);
            Mma<T>::run(acc, ah[0][0], ah[0][1], w0.x, w0.y); Mma<T>::run(acc, al[0][0], al[0][1], w0.x, w0.y);
            Mma<T>::run(acc, ah[1][0], ah[1][1], w0.z, w0.w); Mma<T>::run(acc, al[1][0], al[1][1], w0.z, w0.w);
            Mma<T>::run(acc, ah[2][0], ah[2][1], w1.x, w1.y); Mma<T>::run(acc, al[2][0], al[2][1], w1.x, w1.y);
            Mma<T>::run(acc, ah[3][0], ah[3][1], w1.z, w1.w); Mma<T>::run(acc, al[3][0], al[3][1], w1.z, w1.w);
        } else if (R == 32) {
            const uint4 w0 = *reinterpret_cast<const uint4*>(wr + t * 16);
            Mma<T>::run(acc, ah[0][0], ah[0][1], w0.x, w0.y); Mma<T>::run(acc, al[0][0], al[0][1], w0.x, w0.y);
            Mma<T>::run(acc, ah[CALLS - 1][0], ah[CALLS - 1][1], w0.z, w0.w);
            Mma<T>::run(acc, al[CALLS - 1][0], al[CALLS - 1][1], w0.z, w0.w);
        } else if (R == 16) {
            const uint2 w0 = *reinterpret_cast<const uint2*>(wr + t * 8);
            Mma<T>::run(acc, ah[0][0], ah[0][1], w0.x, w0.y); Mma<T>::run(acc, al[0][0], al[0][1], w0.x, w0.y);
        } else {
            const unsigned w0 = *reinterpret_cast<const unsigned*>(wr + t * 4);
            Mma<T>::run(acc, ah[0][0], 0u, w0, 0u); Mma<T>::run(acc, al[0][0], 0u, w0, 0u);
        }
        // y[token g][j, j+1] += scale * acc
        const int j = jbase + nb * 8 + 2 * t;
        if (g < ntok && j < m.width_ok) {
            const float d0 = scale * acc[0], d1 = scale * acc[1];
            if (p.y_f32) {
                float2* yp = reinterpret_cast<float2*>(reinterpret_cast<float*>(pj.y) + (long long)m.u.tok[g] * pj.ldy + m.c0 + j);
                float2 yv = *yp;
                yv.x += d0; yv.y += d1;
                *yp = yv;
            } else {
                unsigned* yp = reinterpret_cast<unsigned*>(ysb + g * ypitch + j * 2);
                const unsigned w = *yp;
                float lo, hi;
                if (Cvt<T>::is_bf16) {
                    lo = __uint_as_float(w << 16); hi = __uint_as_float(w & 0xffff0000u);
                } else {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
                    lo = f.x; hi = f.y;
                }
                *yp = Cvt<T>::pack2(lo + d0, hi + d1);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1) bgmv_expand_tma_kernel(const __grid_constant__ ApplyParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    Meta* meta = reinterpret_cast<Meta*>(smem + kStages * kExpandStage);
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(meta + 2 * kStages);

    PlanView pv = plan_view(p.plan, p.cap, p.n_adapters);
    WorkspaceView ws = workspace_view(p.workspace, p.cap, p.n_proj);
    const PlanHeader hdr = *pv.hdr;
    if (hdr.error || hdr.cap != p.cap) return;
    const int n_units = (p.flags & B200_LORA_NO_TENSOR) ? hdr.n_units : hdr.n_units_short;
    const int n_items = n_units * p.total_super_out;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int first = blockIdx.x, stride = gridDim.x;
    if (first >= n_items) return;
    const int n_local = (n_items - first + stride - 1) / stride;
    unsigned* err = &ws.ctl->error;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[kStages + s]), kConsWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kConsWarps) {
        for (int n = 0; n < n_local; ++n) {
            const int s = n % kStages;
            const unsigned ph = (n / kStages) & 1;
            mbar_wait(smem_u32(&bars[kStages + s]), ph ^ 1, err, 3);
            Meta* slot = &meta[n % (2 * kStages)];
            producer_meta(p, pv, first + n * stride, n_units, true, lane, slot);
            const unsigned full = smem_u32(&bars[s]);
            if (slot->valid) expand_produce<T>(p, ws, *slot, smem_u32(smem + s * kExpandStage), full, lane);
            else if (lane == 0) mbar_arrive(full);
        }
        return;
    }

    for (int n = 0; n < n_local; ++n) {
        const int s = n % kStages;
        const unsigned ph = (n / kStages) & 1;
        mbar_wait(smem_u32(&bars[s]), ph, err, 4);
        const Meta& m = meta[n % (2 * kStages)];
        unsigned char* stage = smem + s * kExpandStage;
        if (m.valid) {
            switch (m.u.rank) {
                case 8:  expand_consume<T, 8>(p, m, stage, tid); break;
                case 16: expand_consume<T, 16>(p, m, stage, tid); break;
                case 32: expand_consume<T, 32>(p, m, stage, tid); break;
                default: expand_consume<T, 64>(p, m, stage, tid); break;
            }
        }
        cons_sync();
        if (m.valid && !p.y_f32) {
            // coalesced write-back of the updated y tile, 16 bytes per thread
            const ProjArgs& pj = p.proj[m.proj];
            const int jc = kSuper / n_sub(m.u.rank);
            const int cpt = jc / 8, cpt_shift = 31 - __clz(cpt);
            const int c = tid & (cpt - 1), rstep = kConsThreads >> cpt_shift;
            if (c * 8 < m.width_ok) {
                for (int row = tid >> cpt_shift; row < m.u.ntok; row += rstep) {
                    const uint4 val = *reinterpret_cast<const uint4*>(stage + 32768 + row * (jc * 2 + kYPad) + c * 16);
                    *reinterpret_cast<uint4*>(reinterpret_cast<T*>(pj.y) + (long long)m.u.tok[row] * pj.ldy + m.c0 + c * 8) = val;
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars[kStages + s]));     // one arrival per consumer warp
    }
}

constexpr int kShrinkSmem = kStages * kShrinkStage + kRedBytes + 2 * kStages * (int)sizeof(Meta) + 2 * kStages * 8 + 16;
constexpr int kExpandSmem = kStages * kExpandStage + 2 * kStages * (int)sizeof(Meta) + 2 * kStages * 8 + 16;
static_assert(kShrinkSmem <= 232448 && kExpandSmem <= 232448, "exceeds the 227 KB shared memory of one CTA");

template <typename T>
cudaError_t launch_pair(const ApplyParams& p, int n_sm, cudaStream_t s) {
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(bgmv_shrink_tma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kShrinkSmem);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(bgmv_expand_tma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kExpandSmem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    if (!(p.flags & B200_LORA_ONLY_EXPAND)) bgmv_shrink_tma_kernel<T><<<n_sm, kThreads, kShrinkSmem, s>>>(p);
    if (!(p.flags & B200_LORA_ONLY_SHRINK)) bgmv_expand_tma_kernel<T><<<n_sm, kThreads, kExpandSmem, s>>>(p);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_bgmv_tma(const ApplyParams& p, int io_dtype, int n_sm, cudaStream_t s) {
    if (io_dtype == B200_LORA_F16) return launch_pair<__half>(p, n_sm, s);
    return launch_pair<__nv_bfloat16>(p, n_sm, s);
}

}  // namespace b200lora
