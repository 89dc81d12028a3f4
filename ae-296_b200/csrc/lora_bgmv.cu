// Decode BGMV: shrink (v = x . A^T) and expand (y += scale * v . B^T) on adapter-sorted work
// segments of at most 8 tokens.
//
// Both kernels are HBM-bound weight streamers built the same way: one persistent CTA per SM
// walks <= 16 KB weight units through a 6-stage shared-memory ring filled with 128-bit cp.async
// loads (weights, the unit's activation rows, and for the expand the y tile it will update),
// so ~100 KB of loads per SM are in flight while earlier units are being computed.  Tiles are
// XOR-swizzled at 16-byte granularity so ldmatrix reads are conflict-free, and the arithmetic
// is mma.sync m16n8k16 with the unit's <= 8 tokens as (half of) the M dimension, weight rows as
// N, and fp32 accumulators.
// The unit size is constant in bytes: the k-columns (shrink) or output rows (expand) per unit
// shrink as the rank grows.  A segment's weights are read from HBM once for all its tokens.
//
// The split-K partial sums of the shrink are folded in a fixed order by the CTA that arrives
// last at a per-(projection, work segment) counter, so results are bit-reproducible; the
// arrival's round trip is hidden behind the next unit's work.  The expand keeps the fp32
// intermediate exact to ~2^-22 by feeding it to the tensor cores as a hi + lo pair.
//
// Semantics follow the call `add_lora_bgmv(y, x, wa_T_all, wb_T_all, indicies, layer_idx, scale)`
// of the reference (lightllm/models/lora_gpu.py:138,150,162) with pools laid out as at :33-40.
#include "lora_common.cuh"

namespace b200lora {

namespace {

constexpr int kStages = 6;
constexpr int kMetaSlots = 16;
constexpr int kWBytes = 16384;                 // weights of one unit (rank 8 pads to 16 rows)
constexpr int kXBytes = 8192;                  // shrink: 8 tokens x <= 512 columns
constexpr int kYPitchPad = 16;                 // bytes added to a y-tile row against bank conflicts
constexpr int kYBytes = 8 * (512 * 2 + kYPitchPad);
constexpr int kVPitch = 72;                    // floats per token row of the v tile
constexpr int kVBytes = 8 * kVPitch * 4;
constexpr int kShrinkStage = kWBytes + kXBytes;
constexpr int kExpandStage = kWBytes + kYBytes + kVBytes;
constexpr int kWarps = kCtaThreads / 32;       // 16
constexpr int kRedBytes = 8 * 8 * 68 * 4;      // largest cross-warp reduction tile (rank 64: 8 k-slots)

struct Meta {               // per in-flight unit, in shared memory
    UnitRec u;
    int proj, c0;           // projection and first column (shrink) / row (expand) of the unit
    int valid;              // 0: the unit's range lies outside the projection
    int kc;                 // split-K chunk index (shrink)
    int n_chunks;           // split-K chunk count of this (projection, work segment)
    int pad[3];
};
static_assert(sizeof(Meta) == 96, "meta slot");

// ---- small PTX wrappers ---------------------------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(unsigned dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned addr, unsigned& r0, unsigned& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}

template <typename T> struct Mma;
template <> struct Mma<__half> {
    static __device__ __forceinline__ void run(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
};
template <> struct Mma<__nv_bfloat16> {
    static __device__ __forceinline__ void run(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
};

__device__ __forceinline__ unsigned atom_add_acq_rel(unsigned* p, unsigned v) {
    unsigned old;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}

// item -> (unit, projection, super-chunk)
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

// Starts the load of one item's unit record (warp 0; lanes 0..15 carry one word each).
__device__ __forceinline__ void fetch_meta_regs(const ApplyParams& p, const PlanView& pv, int it, int n_units,
                                                bool expand, int lane, int& word, int& proj, int& super) {
    int unit;
    decode_item(p, it, n_units, expand, unit, proj, super);
    word = 0;
    if (lane < 16) word = __ldg(pv.unit_tab + (size_t)unit * 16 + lane);
}

__device__ __forceinline__ void store_meta(const ApplyParams& p, Meta* m, int lane, int word, int proj, int super,
                                           bool expand) {
    if (lane < 16) reinterpret_cast<int*>(&m->u)[lane] = word;
    __syncwarp();
    if (lane == 0) {
        const int r_pad = pad_rank(m->u.rank);
        const int width = kSuper / n_sub(r_pad);
        const int c0 = super * kSuper + m->u.sub * width;
        const int h = expand ? p.proj[proj].h_out : p.proj[proj].h_in;
        m->proj = proj;
        m->c0 = c0;
        m->valid = c0 < h;
        m->kc = c0 / width;
        m->n_chunks = (p.proj[proj].h_in + width - 1) / width;
    }
}

// =============================================================================================
// shrink
// =============================================================================================
// Shared tile of A: r16 = max(r_pad, 16) rows x KC columns, row pitch KC*2 bytes, 16-byte chunk
// c of row i stored at chunk (c ^ (i & 7)).  The x tile uses the same layout with row = token.
template <typename T>
__device__ __forceinline__ void shrink_issue(const ApplyParams& p, const Meta& m, unsigned char* stage, int tid) {
    if (!m.valid) return;
    const ProjArgs& pj = p.proj[m.proj];
    const int r = m.u.rank, r_pad = pad_rank(r);
    const int kc_cols = kSuper / n_sub(r_pad);           // 1024, 1024, 512, 256
    const int cpr = kc_cols / 8;                         // 16-byte chunks per row: 128, 128, 64, 32
    const int cpr_shift = 31 - __clz(cpr);
    const int pitch = kc_cols * 2;
    const T* A = reinterpret_cast<const T*>(pj.wa) + block_row0(p, m.u) * (long long)pj.h_in + m.c0;
    const unsigned wbase = smem_u32(stage);
    // thread -> (row0, c); successive chunks of a thread are rstep rows apart
    const int c = tid & (cpr - 1), row0 = tid >> cpr_shift, rstep = kCtaThreads >> cpr_shift;
    const bool col_ok = (m.c0 + c * 8) < pj.h_in;
    for (int row = row0; row < r_pad; row += rstep) {
        const bool ok = col_ok && row < r;
        const T* src = ok ? A + row * pj.h_in + c * 8 : reinterpret_cast<const T*>(pj.wa);
        cp_async16(wbase + row * pitch + ((c ^ (row & 7)) << 4), src, ok ? 16 : 0);
    }
    const T* X = reinterpret_cast<const T*>(pj.x) + m.c0 + c * 8;
    const unsigned xbase = wbase + kWBytes;
    for (int row = row0; row < m.u.ntok; row += rstep) {
        const T* src = col_ok ? X + (long long)m.u.tok[row] * pj.ldx : reinterpret_cast<const T*>(pj.x);
        cp_async16(xbase + row * pitch + ((c ^ (row & 7)) << 4), src, col_ok ? 16 : 0);
    }
}

// Tokens are the M rows of the MMA (rows 8..15 are zero), weight rows the N columns, so each
// thread ends up with two adjacent ranks of one token.  16 warps = (1 or 2 halves of the rank
// blocks) x (16 or 8 slices of the unit's columns); slices are summed through shared memory.
template <typename T>
__device__ __forceinline__ void shrink_compute(const ApplyParams& p, const WorkspaceView& ws, const Meta& m,
                                               unsigned char* stage, float* red, int tid) {
    if (!m.valid) return;                                  // uniform across the CTA
    const int lane = tid & 31, warp = tid >> 5;
    const int r_pad = pad_rank(m.u.rank);
    const int NB = r_pad / 8;                              // 8-row weight blocks: 1, 2, 4, 8
    const int nsplit = NB >= 2 ? 2 : 1;
    const int ksplit = kWarps / nsplit;                    // 16 or 8
    const int NBW = NB / nsplit;                           // blocks per warp: 1, 1, 2, 4
    const int kc_cols = kSuper / n_sub(r_pad);
    const int pitch = kc_cols * 2;
    const int kslot = warp % ksplit, nhalf = warp / ksplit;
    const int nk16 = kc_cols / 16 / ksplit;                // k16 steps per warp: 4, 8, 4, 2
    const int cw = kslot * nk16 * 2;                       // first 16-byte chunk of this warp
    const unsigned wbase = smem_u32(stage), xbase = wbase + kWBytes;
    const int rp = r_pad + 4;                              // pitch of a reduction row
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const int l7 = lane & 7, mi = lane >> 3;
    for (int ks = 0; ks < nk16; ++ks) {
        const int c = cw + 2 * ks;
        unsigned a0, a2;
        ldmatrix_x2(xbase + l7 * pitch + (((c + (mi & 1)) ^ l7) << 4), a0, a2);
        if (NBW == 1) {
            const int row = nhalf * 8 + l7;
            unsigned b0, b1;
            ldmatrix_x2(wbase + row * pitch + (((c + (mi & 1)) ^ (row & 7)) << 4), b0, b1);
            Mma<T>::run(acc[0], a0, 0u, a2, 0u, b0, b1);
        } else {
#pragma unroll
            for (int pr = 0; pr < 2; ++pr) {
                if (2 * pr < NBW) {
                    const int row = (nhalf * NBW + 2 * pr + (mi >> 1)) * 8 + l7;
                    unsigned b0, b1, b2, b3;
                    ldmatrix_x4(wbase + row * pitch + (((c + (mi & 1)) ^ (row & 7)) << 4), b0, b1, b2, b3);
                    Mma<T>::run(acc[2 * pr], a0, 0u, a2, 0u, b0, b1);
                    Mma<T>::run(acc[2 * pr + 1], a0, 0u, a2, 0u, b2, b3);
                }
            }
        }
    }
    // red[kslot][token][rank]: token g, ranks (block*8 + 2t, +1)
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (i < NBW) {
            float2* dst = reinterpret_cast<float2*>(red + (kslot * 8 + g) * rp + (nhalf * NBW + i) * 8 + 2 * t);
            *dst = make_float2(acc[i][0], acc[i][1]);
        }
    }
    __syncthreads();
    // fold the column slices in slice order and publish this unit's split-K partial
    const int outs = m.u.ntok * r_pad;
    for (int idx = tid; idx < outs; idx += kCtaThreads) {
        const int tok = idx / r_pad, i = idx % r_pad;
        float s = 0.f;
        for (int w = 0; w < ksplit; ++w) s += red[(w * 8 + tok) * rp + i];
        ws.partial[(((size_t)m.kc * p.n_proj + m.proj) * p.cap + (m.u.start + tok)) * kMaxRank + i] = s;
    }
}

// The CTA that arrived last folds all split-K partials of one (projection, work segment) in k order.
template <typename T>
__device__ __forceinline__ void shrink_fold(const ApplyParams& p, const WorkspaceView& ws, const Meta& m, int tid) {
    const int r_pad = pad_rank(m.u.rank);
    const bool mid_round = (p.flags & B200_LORA_MID_ROUND) != 0;
    const int outs = m.u.ntok * r_pad;
    for (int idx = tid; idx < outs; idx += kCtaThreads) {
        const int pos = m.u.start + idx / r_pad, i = idx % r_pad;
        const float* src = &ws.partial[((size_t)m.proj * p.cap + pos) * kMaxRank + i];
        const size_t cstride = (size_t)p.n_proj * p.cap * kMaxRank;
        float s = 0.f;
        int c = 0;
        for (; c + 8 <= m.n_chunks; c += 8) {            // 8 loads in flight, summed in k order
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
__global__ void __launch_bounds__(kCtaThreads, 1) bgmv_shrink_kernel(const __grid_constant__ ApplyParams p) {
    pdl_wait_prior();
    pdl_launch_dependents();            // only after the wait: see lora_common.cuh
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* stages = smem;
    float* red = reinterpret_cast<float*>(smem + kStages * kShrinkStage);   // 8 or 16 slices x 8 tokens x (r_pad + 4)
    Meta* meta = reinterpret_cast<Meta*>(smem + kStages * kShrinkStage + kRedBytes);
    int* s_fold = reinterpret_cast<int*>(meta + kMetaSlots);

    PlanView pv = plan_view(p.plan, p.cap, p.n_adapters);
    WorkspaceView ws = workspace_view(p.workspace, p.cap, p.n_proj);
    const PlanHeader hdr = *pv.hdr;
    if (!plan_usable(hdr, p, &ws.ctl->error)) return;
    const int n_units = (p.flags & B200_LORA_NO_TENSOR) ? hdr.n_units : hdr.n_units_short;
    const int n_items = n_units * p.total_super_in;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int first = blockIdx.x, stride = gridDim.x;
    if (first >= n_items) return;
    const int n_local = (n_items - first + stride - 1) / stride;

    // prologue: metadata of the first kStages items (one warp each), loads of the first kStages - 1
    if (warp < kStages && warp < n_local) {
        int word, proj, super;
        fetch_meta_regs(p, pv, first + warp * stride, n_units, false, lane, word, proj, super);
        store_meta(p, &meta[warp % kMetaSlots], lane, word, proj, super, false);
    }
    if (tid == 0) *s_fold = -1;
    __syncthreads();
    for (int n = 0; n < kStages - 1; ++n) {
        if (n < n_local) shrink_issue<T>(p, meta[n % kMetaSlots], stages + (n % kStages) * kShrinkStage, tid);
        cp_async_commit();
    }

    unsigned ticket = 0;          // thread 0: arrival count returned for the previous item
    for (int n = 0; n < n_local; ++n) {
        // fold a segment whose last arrival was ours (decided before the previous barrier)
        const int fold_slot = *s_fold;
        if (fold_slot >= 0) shrink_fold<T>(p, ws, meta[fold_slot], tid);
        // arrive for item n-1: its partials were written before the barrier that ended iteration n-1
        const bool arrive = n > 0 && meta[(n - 1) % kMetaSlots].valid;
        if (tid == 0 && arrive) {
            const Meta& pm = meta[(n - 1) % kMetaSlots];
            ticket = atom_add_acq_rel(&ws.counters[(size_t)pm.proj * p.cap + pm.u.wseg], 1u);
        }
        const int nn = n + kStages - 1;
        if (nn < n_local) shrink_issue<T>(p, meta[nn % kMetaSlots], stages + (nn % kStages) * kShrinkStage, tid);
        cp_async_commit();
        int word = 0, mproj = 0, msuper = 0;
        const int nm = n + kStages;
        if (warp == 0 && nm < n_local) fetch_meta_regs(p, pv, first + nm * stride, n_units, false, lane, word, mproj, msuper);
        cp_async_wait<kStages - 1>();
        __syncthreads();
        shrink_compute<T>(p, ws, meta[n % kMetaSlots], stages + (n % kStages) * kShrinkStage, red, tid);
        if (warp == 0 && nm < n_local) store_meta(p, &meta[nm % kMetaSlots], lane, word, mproj, msuper, false);
        if (tid == 0) {
            int f = -1;
            if (arrive && ticket == (unsigned)(meta[(n - 1) % kMetaSlots].n_chunks - 1)) f = (n - 1) % kMetaSlots;
            *s_fold = f;
        }
        __syncthreads();
    }
    // drain: a pending fold, then the arrival (and possible fold) of the last item
    const int last_fold = *s_fold;
    if (last_fold >= 0) shrink_fold<T>(p, ws, meta[last_fold], tid);
    __syncthreads();
    const Meta& lm = meta[(n_local - 1) % kMetaSlots];
    if (lm.valid) {
        if (tid == 0) {
            ticket = atom_add_acq_rel(&ws.counters[(size_t)lm.proj * p.cap + lm.u.wseg], 1u);
            *s_fold = (ticket == (unsigned)(lm.n_chunks - 1)) ? 1 : 0;
        }
        __syncthreads();
        if (*s_fold == 1) shrink_fold<T>(p, ws, lm, tid);
    }
    cp_async_wait<0>();
}

// =============================================================================================
// expand
// =============================================================================================
// Shared tile of B: JC rows x r_pad columns (row pitch r_pad*2 bytes = CPR 16-byte chunks).
// With RPL = 8 / CPR rows per 128-byte line, chunk c of row j sits in line j / RPL at slot
// (j % RPL) * CPR + (c ^ ((j / RPL) % CPR)): any 8 consecutive rows hit 8 different slots.
__device__ __forceinline__ int b_tile_off(int row, int c, int cpr, int cpr_shift) {
    const int rpl_shift = 3 - cpr_shift;
    const int line = row >> rpl_shift;
    const int slot = ((row & ((1 << rpl_shift) - 1)) << cpr_shift) + (c ^ (line & (cpr - 1)));
    return line * 128 + slot * 16;
}

template <typename T>
__device__ __forceinline__ void expand_issue(const ApplyParams& p, const WorkspaceView& ws, const Meta& m,
                                             unsigned char* stage, int tid) {
    if (!m.valid) return;
    const ProjArgs& pj = p.proj[m.proj];
    const int r = m.u.rank, r_pad = pad_rank(r);
    const int jc = kSuper / n_sub(r_pad);                 // 1024, 1024, 512, 256 rows
    const int cpr = r_pad / 8, cpr_shift = 31 - __clz(cpr);
    const int pitch = b_pitch(p, r);
    const T* B = reinterpret_cast<const T*>(pj.wb) + block_row0(p, m.u) * (long long)pj.h_out +
                 (long long)m.c0 * pitch;
    const unsigned wbase = smem_u32(stage);
    {
        const int c = tid & (cpr - 1), row0 = tid >> cpr_shift, rstep = kCtaThreads >> cpr_shift;
        int nb = (r - c * 8) * 2;
        nb = nb > 16 ? 16 : (nb < 0 ? 0 : nb);
        const int rows_ok = pj.h_out - m.c0;              // rows of this unit inside the projection
        for (int row = row0; row < jc; row += rstep) {
            const int nbytes = row < rows_ok ? nb : 0;
            const T* src = nbytes ? B + row * pitch + c * 8 : reinterpret_cast<const T*>(pj.wb);
            cp_async16(wbase + b_tile_off(row, c, cpr, cpr_shift), src, nbytes);
        }
    }
    // y tile (16-bit outputs only): ntok rows x jc columns
    if (!p.y_f32) {
        const unsigned ybase = wbase + kWBytes;
        const int ypitch = jc * 2 + kYPitchPad;
        const int cpt = jc / 8, cpt_shift = 31 - __clz(cpt);
        const int c = tid & (cpt - 1), row0 = tid >> cpt_shift, rstep = kCtaThreads >> cpt_shift;
        const bool ok = (m.c0 + c * 8) < pj.h_out;
        const T* Y = reinterpret_cast<const T*>(pj.y) + m.c0 + c * 8;
        for (int row = row0; row < m.u.ntok; row += rstep) {
            const T* src = ok ? Y + (long long)m.u.tok[row] * pj.ldy : reinterpret_cast<const T*>(pj.y);
            cp_async16(ybase + row * ypitch + c * 16, src, ok ? 16 : 0);
        }
    }
    // v tile: ntok rows x r_pad floats
    const unsigned vbase = wbase + kWBytes + kYBytes;
    const int vpt = r_pad / 4, vpt_shift = 31 - __clz(vpt);
    const int vt = m.u.ntok * vpt;
    if (tid < vt) {
        const int row = tid >> vpt_shift, c = tid & (vpt - 1);
        const float* src = ws.v + ((size_t)m.proj * p.cap + m.u.start + row) * kMaxRank + c * 4;
        cp_async16(vbase + row * (kVPitch * 4) + c * 16, src, 16);
    }
}

// Tokens are the M rows of the MMA (rows 8..15 zero), 8 output rows of B the N columns: each
// thread owns two adjacent outputs of one token and updates them in the shared y tile.
template <typename T>
__device__ __forceinline__ void expand_compute(const ApplyParams& p, const Meta& m, unsigned char* stage, int tid) {
    if (!m.valid) return;
    const ProjArgs& pj = p.proj[m.proj];
    const int lane = tid & 31, warp = tid >> 5;
    const int r_pad = pad_rank(m.u.rank);
    const int jc = kSuper / n_sub(r_pad);
    const int cpr = r_pad / 8, cpr_shift = 31 - __clz(cpr);
    const int KS = r_pad <= 16 ? 1 : r_pad / 16;          // k16 steps
    const unsigned wbase = smem_u32(stage);
    const float* vt = reinterpret_cast<const float*>(stage + kWBytes + kYBytes);
    const int g = lane >> 2, t = lane & 3;
    const int ntok = m.u.ntok;
    const float scale = m.u.scale;

    // A fragments: the fp32 intermediate of token g as a hi + lo pair of 16-bit values
    unsigned ah[4][2], al[4][2];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float v0 = 0.f, v1 = 0.f;
            const int k = ks * 16 + h * 8 + 2 * t;
            if (ks < KS && k < r_pad && g < ntok) {
                const float2 vv = *reinterpret_cast<const float2*>(vt + g * kVPitch + k);
                v0 = vv.x; v1 = vv.y;
            }
            const float h0 = Cvt<T>::round1(v0), h1 = Cvt<T>::round1(v1);
            ah[ks][h] = Cvt<T>::pack2(h0, h1);
            al[ks][h] = Cvt<T>::pack2(v0 - h0, v1 - h1);
        }
    }

    const int NBW = jc / 8 / kWarps;                       // 8-row blocks per warp: 8, 8, 4, 2
    const int jbase = warp * NBW * 8;
    const int l7 = lane & 7, mi = lane >> 3;
    unsigned char* ysb = stage + kWBytes;
    const int ypitch = jc * 2 + kYPitchPad;
    const int group = cpr == 1 ? 4 : 2;                    // blocks fetched by one ldmatrix.x4
    for (int nb0 = 0; nb0 < NBW; nb0 += group) {
        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
        if (cpr == 1) {
            const int row = jbase + (nb0 + mi) * 8 + l7;
            unsigned b0, b1, b2, b3;
            ldmatrix_x4(wbase + b_tile_off(row, 0, 1, 0), b0, b1, b2, b3);
            Mma<T>::run(acc[0], ah[0][0], 0u, ah[0][1], 0u, b0, 0u);
            Mma<T>::run(acc[0], al[0][0], 0u, al[0][1], 0u, b0, 0u);
            Mma<T>::run(acc[1], ah[0][0], 0u, ah[0][1], 0u, b1, 0u);
            Mma<T>::run(acc[1], al[0][0], 0u, al[0][1], 0u, b1, 0u);
            Mma<T>::run(acc[2], ah[0][0], 0u, ah[0][1], 0u, b2, 0u);
            Mma<T>::run(acc[2], al[0][0], 0u, al[0][1], 0u, b2, 0u);
            Mma<T>::run(acc[3], ah[0][0], 0u, ah[0][1], 0u, b3, 0u);
            Mma<T>::run(acc[3], al[0][0], 0u, al[0][1], 0u, b3, 0u);
        } else {
            const int row = jbase + (nb0 + (mi >> 1)) * 8 + l7;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                if (ks < KS) {
                    unsigned b0, b1, b2, b3;
                    ldmatrix_x4(wbase + b_tile_off(row, 2 * ks + (mi & 1), cpr, cpr_shift), b0, b1, b2, b3);
                    Mma<T>::run(acc[0], ah[ks][0], 0u, ah[ks][1], 0u, b0, b1);
                    Mma<T>::run(acc[0], al[ks][0], 0u, al[ks][1], 0u, b0, b1);
                    Mma<T>::run(acc[1], ah[ks][0], 0u, ah[ks][1], 0u, b2, b3);
                    Mma<T>::run(acc[1], al[ks][0], 0u, al[ks][1], 0u, b2, b3);
                }
            }
        }
        // y[token g][j, j+1] += scale * acc
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (i < group) {
                const int j = jbase + (nb0 + i) * 8 + 2 * t;
                if (nb0 + i < NBW && g < ntok && m.c0 + j < pj.h_out) {
                    const float d0 = scale * acc[i][0], d1 = scale * acc[i][1];
                    if (p.y_f32) {
                        float2* yp = reinterpret_cast<float2*>(reinterpret_cast<float*>(pj.y) +
                                                               (long long)m.u.tok[g] * pj.ldy + m.c0 + j);
                        float2 yv = *yp;
                        yv.x += d0; yv.y += d1;
                        *yp = yv;
                    } else {
                        unsigned* yp = reinterpret_cast<unsigned*>(ysb + g * ypitch + j * 2);
                        const unsigned w = *yp;
                        float lo, hi;
                        if (sizeof(T) == 2 && Cvt<T>::is_bf16) {
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
    }
    if (p.y_f32) return;
    __syncthreads();
    // coalesced write-back of the updated y tile
    const int cpt = jc / 8, cpt_shift = 31 - __clz(cpt);
    const int c = tid & (cpt - 1), row0 = tid >> cpt_shift, rstep = kCtaThreads >> cpt_shift;
    if (m.c0 + c * 8 < pj.h_out) {
        for (int row = row0; row < ntok; row += rstep) {
            const uint4 val = *reinterpret_cast<const uint4*>(ysb + row * ypitch + c * 16);
            *reinterpret_cast<uint4*>(reinterpret_cast<T*>(pj.y) + (long long)m.u.tok[row] * pj.ldy + m.c0 + c * 8) = val;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kCtaThreads, 1) bgmv_expand_kernel(const __grid_constant__ ApplyParams p) {
    pdl_wait_prior();
    pdl_launch_dependents();            // only after the wait: see lora_common.cuh
    extern __shared__ __align__(1024) unsigned char smem[];
    unsigned char* stages = smem;
    Meta* meta = reinterpret_cast<Meta*>(smem + kStages * kExpandStage);

    PlanView pv = plan_view(p.plan, p.cap, p.n_adapters);
    WorkspaceView ws = workspace_view(p.workspace, p.cap, p.n_proj);
    const PlanHeader hdr = *pv.hdr;
    if (!plan_usable(hdr, p, &ws.ctl->error)) return;
    const int n_units = (p.flags & B200_LORA_NO_TENSOR) ? hdr.n_units : hdr.n_units_short;
    const int n_items = n_units * p.total_super_out;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int first = blockIdx.x, stride = gridDim.x;
    if (first >= n_items) return;
    const int n_local = (n_items - first + stride - 1) / stride;

    if (warp < kStages && warp < n_local) {
        int word, proj, super;
        fetch_meta_regs(p, pv, first + warp * stride, n_units, true, lane, word, proj, super);
        store_meta(p, &meta[warp % kMetaSlots], lane, word, proj, super, true);
    }
    __syncthreads();
    for (int n = 0; n < kStages - 1; ++n) {
        if (n < n_local) expand_issue<T>(p, ws, meta[n % kMetaSlots], stages + (n % kStages) * kExpandStage, tid);
        cp_async_commit();
    }
    for (int n = 0; n < n_local; ++n) {
        const int nn = n + kStages - 1;
        if (nn < n_local) expand_issue<T>(p, ws, meta[nn % kMetaSlots], stages + (nn % kStages) * kExpandStage, tid);
        cp_async_commit();
        int word = 0, mproj = 0, msuper = 0;
        const int nm = n + kStages;
        if (warp == 0 && nm < n_local) fetch_meta_regs(p, pv, first + nm * stride, n_units, true, lane, word, mproj, msuper);
        cp_async_wait<kStages - 1>();
        __syncthreads();
        expand_compute<T>(p, meta[n % kMetaSlots], stages + (n % kStages) * kExpandStage, tid);
        if (warp == 0 && nm < n_local) store_meta(p, &meta[nm % kMetaSlots], lane, word, mproj, msuper, true);
        __syncthreads();
    }
    cp_async_wait<0>();
}

constexpr int kShrinkSmem = kStages * kShrinkStage + kRedBytes + kMetaSlots * (int)sizeof(Meta) + 16;
constexpr int kExpandSmem = kStages * kExpandStage + kMetaSlots * (int)sizeof(Meta) + 16;

template <typename T>
cudaError_t launch_pair(const ApplyParams& p, int n_sm, cudaStream_t s) {
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(bgmv_shrink_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kShrinkSmem);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(bgmv_expand_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kExpandSmem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    if (!(p.flags & B200_LORA_ONLY_EXPAND)) bgmv_shrink_kernel<T><<<n_sm, kCtaThreads, kShrinkSmem, s>>>(p);
    if (!(p.flags & B200_LORA_ONLY_SHRINK)) bgmv_expand_kernel<T><<<n_sm, kCtaThreads, kExpandSmem, s>>>(p);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_bgmv(const ApplyParams& p, int io_dtype, int n_sm, cudaStream_t s) {
    if (io_dtype == B200_LORA_F16) return launch_pair<__half>(p, n_sm, s);
    return launch_pair<__nv_bfloat16>(p, n_sm, s);
}

}  // namespace b200lora
