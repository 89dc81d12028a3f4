// Decode BGMV, fast path: TMA copies + mbarrier pipeline + mma.sync (sm_100a).
//
// Used when every adapter rank is 8, 16, 32 or 64 and every projection width is a multiple of
// 256.  One apply is two launches, a shrink kernel (v = x . A^T per work segment) and an expand
// kernel (y += scale * v . B^T); both are lists of <= 16 KB weight units, ordered projection by
// projection and work segment by work segment, of which every CTA takes a contiguous range.
// A CTA is two producer warps plus eight consumer warps around a 4-stage shared-memory ring;
// two CTAs share an SM, so ~100 KB of loads per SM are in flight.  The producers walk the range
// (alternate units each) and fill a stage with ONE instruction per kind:
//   shrink  A rows [r, KC]   -> one [r x 128] box of a 2-D tensor map over the A pool per 128 columns
//           x rows [ntok, KC]-> one bulk copy per token
//   expand  B rows [JC, r]   -> one contiguous bulk copy; plus one copy per token for the y
//           tile that will be updated
// Each stage's arrival is tracked by an mbarrier transaction count; consumers never compute a
// load address.  They read MMA fragments with wide shared loads (tiles are stored unswizzled;
// the k index is permuted identically for both operands so that a thread's fragment is one
// contiguous chunk) and run mma.sync m16n8k16 with fp32 accumulators.  The legacy MMA path of
// this part has a long dependent-issue latency, so every warp keeps several independent
// accumulators in flight.
//
// Both kernels are launched with programmatic stream serialisation and their producers request
// the first weight tiles before they wait for the predecessor kernel (weights and plan are not
// written by any kernel that can still be running), so a kernel's start-up overlaps its
// predecessor's tail.
//
// shrink: weight rows are the M rows, the unit's <= 8 tokens the N columns.  Consecutive units
// of one (projection, work segment) are accumulated in registers; when the run ends the CTA
// writes ONE split-K partial into the slot numbered by the run's first unit.  Which slots a
// segment has follows from the CTAs' ranges alone, so there are no counters, flags or fences:
// the kernel boundary publishes the partials.
// expand: the first unit a CTA has of a segment brings the intermediate along: its producer
// adds up the segment's slots in ascending k order (bit-reproducible) straight into the stage.
// The weight tile is the MMA's A operand (16 output columns x 16 rank indices), the N columns
// hold the hi and lo 16-bit halves of four tokens' fp32 intermediate, so one MMA is exact for
// four tokens; results are added into the staged y tile, which each warp writes back itself.
//
// Every mbarrier wait is bounded: on expiry the thread records an error word in the workspace
// and carries on with the same control flow, so the kernel always terminates.
//
// Semantics: add_lora_bgmv(y, x, wa_T_all, wb_T_all, indicies, layer_idx, scale) of the
// reference (lightllm/models/lora_gpu.py:138,150,162), pools as at :33-40.
#include "lora_common.cuh"
#include "lora_fold.cuh"

namespace b200lora {

namespace {

constexpr int kStages = 4;
constexpr int kMetaSlots = 2 * kStages;
constexpr int kConsWarps = 8;
constexpr int kConsThreads = kConsWarps * 32;
constexpr int kProdWarps = 2;                     // producer warps take alternate items
constexpr int kThreads = kConsThreads + kProdWarps * 32;
constexpr int kCtasPerSm = 2;
constexpr int kBoxCols = 128;                     // columns of a shrink weight box; its rows are the adapter's rank rows
constexpr int kWTile = 16384;                     // weight tile of one unit
constexpr int kXPad = 64;                         // bytes added to an x-tile row (bank spread)
constexpr int kXBytes = 8 * (512 * 2 + kXPad);
constexpr int kShrinkStage = kWTile + kXBytes;
constexpr int kYPad = 32;                        // y-tile rows 32 bytes apart modulo 128: no bank conflicts
constexpr int kYBytes = 8 * (512 * 2 + kYPad);
constexpr int kVPitch = 72;                       // floats per token row of the v tile
constexpr int kVBytes = 8 * kVPitch * 4;
constexpr int kExpandStage = kWTile + kYBytes + kVBytes;
constexpr int kRedBytes = 8 * 8 * 20 * 4;         // cross-warp reduction tile (largest: rank 16, 8 slices)
constexpr unsigned kSpinLimit = 1u << 22;

struct Meta {
    UnitRec u;
    int proj, c0, valid, kc, n_chunks, width_ok;
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
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
__device__ __forceinline__ void tensor_g2s_2d(unsigned dst, const void* tmap, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsThreads) : "memory"); }

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

// Cursor over a CTA's contiguous range of items.  The items are ordered projection by
// projection, work segment by work segment, and inside a segment super-chunk by super-chunk and
// sub-range by sub-range, so all units of one (projection, work segment) are neighbours: a CTA
// usually sees whole segments, and the expand units it gets belong to the segments it shrank.
// The plan's unit table holds one record per (work segment, sub-range), the records of a
// segment next to each other and equal but for the sub-range, so any of them describes it.
struct Cursor {
    int unit;       // first plan unit of the work segment
    int sp, sub;    // super-chunk and sub-range inside the segment
    int proj, super;
    int ns;         // super-chunks of the projection in this list
    int nsub_log;   // log2(sub-ranges per super-chunk): 2, 2, 3, 4 for rank 8, 16, 32, 64
};
__device__ __forceinline__ int ns_of(const ApplyParams& p, int pi, bool expand) {
    return expand ? p.proj[pi].n_super_out : p.proj[pi].n_super_in;
}
__device__ __forceinline__ int nsub_log_of(int rank) { return rank <= 16 ? 2 : rank <= 32 ? 3 : 4; }
__device__ __forceinline__ int load_record(const int* unit_tab, int unit, int lane) {
    return lane < 16 ? __ldg(unit_tab + (size_t)unit * 16 + lane) : 0;
}
// positions the cursor at item `it` and fetches the record of its work segment
__device__ __forceinline__ Cursor cursor_at(const ApplyParams& p, int it, int n_units, bool expand, const int* unit_tab,
                                            int lane, int& rec) {
    Cursor c;
    int local = it, pi = 0;
#pragma unroll
    for (int i = 0; i < kMaxProj - 1; ++i) {
        const int cnt = n_units * ns_of(p, i, expand);
        if (i < p.n_proj - 1 && pi == i && local >= cnt) { local -= cnt; pi = i + 1; }
    }
    c.proj = pi;
    c.ns = ns_of(p, pi, expand);
    const int up = local / c.ns;                           // a unit of the item's segment
    rec = load_record(unit_tab, up, lane);
    c.nsub_log = nsub_log_of(__shfl_sync(0xffffffffu, rec, 1));
    c.unit = up - (__shfl_sync(0xffffffffu, rec, 2) & 0xffff);
    const int l2 = local - c.unit * c.ns;
    c.sp = c.super = l2 >> c.nsub_log;
    c.sub = l2 & ((1 << c.nsub_log) - 1);
    return c;
}
// advances by `steps` items; fetches the new record whenever the work segment changes
__device__ __forceinline__ void cursor_advance(const ApplyParams& p, int n_units, bool expand, const int* unit_tab, int lane,
                                               int steps, Cursor& c, int& rec) {
    for (int q = 0; q < steps; ++q) {
        if (++c.sub < (1 << c.nsub_log)) continue;
        c.sub = 0;
        if (++c.sp < c.ns) { c.super = c.sp; continue; }
        c.sp = c.super = 0;
        c.unit += 1 << c.nsub_log;
        if (c.unit >= n_units) {
            c.unit = 0;
            c.proj = min(c.proj + 1, p.n_proj - 1);
            c.ns = ns_of(p, c.proj, expand);
        }
        rec = load_record(unit_tab, c.unit, lane);
        c.nsub_log = nsub_log_of(__shfl_sync(0xffffffffu, rec, 1));
    }
}

// A consumer's private copy of a meta slot: six wide loads issued back to back, so that the
// control flow that follows runs on registers instead of a chain of dependent shared loads.
__device__ __forceinline__ Meta load_meta(const Meta* slot) {
    Meta m;
    const uint4* src = reinterpret_cast<const uint4*>(slot);
    uint4* dst = reinterpret_cast<uint4*>(&m);
#pragma unroll
    for (int i = 0; i < (int)(sizeof(Meta) / 16); ++i) dst[i] = src[i];
    return m;
}

// What the producer derives for one item; every lane computes it from the broadcast record.
struct Item {
    int adapter, rank, sub, ntok, start;
    long long cum;
    int proj, c0, valid, kc, n_chunks, width_ok;
};
__device__ __forceinline__ Item make_item(const ApplyParams& p, int rec, const Cursor& c, bool expand) {
    Item it;
    it.adapter = __shfl_sync(0xffffffffu, rec, 0);
    it.rank = __shfl_sync(0xffffffffu, rec, 1);
    const int w2 = __shfl_sync(0xffffffffu, rec, 2);
    it.sub = c.sub;
    it.ntok = (w2 >> 16) & 0xffff;
    it.start = __shfl_sync(0xffffffffu, rec, 5);
    const unsigned lo = (unsigned)__shfl_sync(0xffffffffu, rec, 6);
    const int hi = __shfl_sync(0xffffffffu, rec, 7);
    it.cum = ((long long)hi << 32) | lo;
    const int wshift = it.rank <= 16 ? 9 : it.rank == 32 ? 8 : 7;        // sub-range width 512 / 256 / 128
    const int h = expand ? p.proj[c.proj].h_out : p.proj[c.proj].h_in;
    it.proj = c.proj;
    it.c0 = c.super * kSuper + (it.sub << wshift);
    it.valid = it.c0 < h;
    it.kc = it.c0 >> wshift;
    it.n_chunks = (p.proj[c.proj].h_in + (1 << wshift) - 1) >> wshift;
    it.width_ok = min(1 << wshift, h - it.c0);
    return it;
}
// lanes 0..15 store the record words, lanes 16..21 the derived fields
__device__ __forceinline__ void publish_meta(Meta* slot, int rec, const Item& it, int lane) {
    int* w = reinterpret_cast<int*>(slot);
    if (lane < 16) w[lane] = rec;
    else if (lane == 16) w[16] = it.proj;
    else if (lane == 17) w[17] = it.c0;
    else if (lane == 18) w[18] = it.valid;
    else if (lane == 19) w[19] = it.kc;
    else if (lane == 20) w[20] = it.n_chunks;
    else if (lane == 21) w[21] = it.width_ok;
    __syncwarp();
}
__device__ __forceinline__ long long item_row0(const ApplyParams& p, const Item& it) {
    if (p.packed) return (long long)p.n_layers * it.cum + (long long)p.layer * it.rank;
    return ((long long)it.adapter * p.n_layers + p.layer) * p.r_pool;
}

// =============================================================================================
// shrink
// =============================================================================================
// Stage layout: one weight box per 128-column block of the unit, each [r rows x 128 cols]
// contiguous (row pitch 256 B); then the x tile, one row per token, pitch KC*2 + 64 bytes.
// `parts` bit 0: the barrier's byte count and the weight boxes (never written while kernels of
// this library run, so they may be requested before the predecessor kernel has ended); bit 1:
// the x rows.
template <typename T>
__device__ __forceinline__ void shrink_produce(const ApplyParams& p, const Item& m, int rec, unsigned stage,
                                               unsigned bar, int lane, int parts = 3) {
    const ProjArgs& pj = p.proj[m.proj];
    const int r = m.rank;
    const int kc_cols = kSuper / n_sub(r);                // 512, 512, 256, 128
    const int ncb = kc_cols / kBoxCols;                   // boxes of the unit: 4, 4, 2, 1
    const int box_bytes = r * kBoxCols * 2;
    const int cls = r <= 8 ? 0 : r <= 16 ? 1 : r <= 32 ? 2 : 3;
    const unsigned row_bytes = m.width_ok * 2;
    if (parts & 1) {
        if (lane == 0) mbar_arrive_expect_tx(bar, ncb * box_bytes + m.ntok * row_bytes);
        __syncwarp();
        if (lane < ncb)
            tensor_g2s_2d(stage + lane * box_bytes, &p.amap[m.proj][cls], m.c0 + lane * kBoxCols, (int)item_row0(p, m), bar);
    }
    // lanes 8..15 hold the token rows of the unit record
    if ((parts & 2) && lane >= 8 && lane < 8 + m.ntok)
        bulk_g2s(stage + kWTile + (lane - 8) * (kc_cols * 2 + kXPad),
                 reinterpret_cast<const T*>(pj.x) + (long long)rec * pj.ldx + m.c0, row_bytes, bar);
}

// An item and its record as the meta slot holds them (for the parts of a unit that are
// requested after the rest).
__device__ __forceinline__ Item item_of_meta(const Meta& m) {
    Item it;
    it.adapter = m.u.adapter; it.rank = m.u.rank; it.sub = m.u.sub; it.ntok = m.u.ntok; it.start = m.u.start;
    it.cum = ((long long)m.u.cum_hi << 32) | (unsigned)m.u.cum_lo;
    it.proj = m.proj; it.c0 = m.c0; it.valid = m.valid; it.kc = m.kc; it.n_chunks = m.n_chunks; it.width_ok = m.width_ok;
    return it;
}
__device__ __forceinline__ int record_of_meta(const Meta& m, int lane) {
    return lane < 16 ? reinterpret_cast<const int*>(&m)[lane] : 0;
}

// Weight rows are the M rows of the MMA (16 per block), the unit's tokens its N columns.  The 8
// warps = (1, 2 or 4 row blocks) x (8, 4 or 2 slices of the unit's columns); a warp adds 4 MMAs
// per unit into four independent accumulators that live across the units of one run.
template <typename T, int R>
__device__ __forceinline__ void shrink_consume(const Meta& m, const unsigned char* stage, float (&acc)[4][4], int tid) {
    constexpr int MB = R >= 16 ? R / 16 : 1;               // 16-row blocks: 1, 1, 2, 4
    constexpr int KSPLIT = kConsWarps / MB;                // 8, 8, 4, 2
    constexpr int KC_COLS = R <= 16 ? 512 : R == 32 ? 256 : 128;
    const int lane = tid & 31, warp = tid >> 5;
    const int kslot = warp % KSPLIT, mblk = warp / KSPLIT;
    const int g = lane >> 2, t = lane & 3;
    const unsigned char* xrow = stage + kWTile + g * (KC_COLS * 2 + kXPad) + t * 16;
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {                        // every warp owns two 32-column blocks
        const int col = (kslot * 2 + kb) * 32;
        if (col < m.width_ok) {
            const int cb = col >> 7, cin = col & 127;
            const unsigned char* wbox = stage + cb * (R * kBoxCols * 2) + (mblk * 16 + g) * 256 + cin * 2 + t * 16;
            const uint4 xb = *reinterpret_cast<const uint4*>(xrow + col * 2);
            const uint4 w = *reinterpret_cast<const uint4*>(wbox);
            uint4 u = make_uint4(0u, 0u, 0u, 0u);
            if (R >= 16) u = *reinterpret_cast<const uint4*>(wbox + 8 * 256);           // rank 8 has no rows 8..15
            Mma<T>::run(acc[2 * kb], w.x, u.x, w.y, u.y, xb.x, xb.y);
            Mma<T>::run(acc[2 * kb + 1], w.z, u.z, w.w, u.w, xb.z, xb.w);
        }
    }
}
template <typename T>
__device__ __forceinline__ void shrink_consume_any(const Meta& m, const unsigned char* stage, float (&acc)[4][4], int tid) {
    switch (m.u.rank) {
        case 8:  shrink_consume<T, 8>(m, stage, acc, tid); break;
        case 16: shrink_consume<T, 16>(m, stage, acc, tid); break;
        case 32: shrink_consume<T, 32>(m, stage, acc, tid); break;
        default: shrink_consume<T, 64>(m, stage, acc, tid); break;
    }
}

// One run = consecutive units of one (projection, work segment) in this CTA.
struct Run {
    int proj, wseg, start, ntok, rank, first_kc, count, n_chunks;
};

// Ends a run: cross-warp reduction and one split-K partial in slot `first_kc` of the workspace.
// Nothing else: which slots a (projection, work segment) has follows from the CTAs' item ranges,
// so whoever needs the intermediate adds the slots up after this kernel has ended (the expand
// kernel's producers, or fold_partials_kernel for tensor-parallel callers).  No atomics, no
// fences; the reduction tile alternates between two buffers, so one barrier per run suffices.
template <typename T>
__device__ __forceinline__ void shrink_flush(const ApplyParams& p, const WorkspaceView& ws, const Run& run,
                                             float (&acc)[4][4], float* red2, int& red_sel, int tid) {
    float* red = red2 + red_sel * (kRedBytes / 4);
    red_sel ^= 1;
    const int lane = tid & 31, warp = tid >> 5;
    const int r = run.rank, rp = r + 4;
    const int mb_log = r >= 64 ? 2 : r >= 32 ? 1 : 0;
    const int ksplit = kConsWarps >> mb_log;
    const int kslot = warp & (ksplit - 1), mblk = warp >> (3 - mb_log);
    const int g = lane >> 2, t = lane & 3;
    float c[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        c[j] = (acc[0][j] + acc[1][j]) + (acc[2][j] + acc[3][j]);
        acc[0][j] = acc[1][j] = acc[2][j] = acc[3][j] = 0.f;
    }
    // red[kslot][token][rank]: ranks (mblk*16 + g, +8), tokens (2t, 2t+1)
    float* base = red + kslot * 8 * rp + mblk * 16 + g;
    base[(2 * t) * rp] = c[0];
    base[(2 * t + 1) * rp] = c[1];
    if (r >= 16) {
        base[(2 * t) * rp + 8] = c[2];
        base[(2 * t + 1) * rp + 8] = c[3];
    }
    cons_sync();
    const int outs = run.ntok * r;
    const int rshift = 31 - __clz(r);
    const size_t cstride = (size_t)p.n_proj * p.cap * kMaxRank;
    float* dst = ws.partial + (size_t)run.first_kc * cstride + ((size_t)run.proj * p.cap + run.start) * kMaxRank;
    for (int idx = tid; idx < outs; idx += kConsThreads) {
        const int tok = idx >> rshift, i = idx & (r - 1);
        float s = 0.f;
        for (int w = 0; w < ksplit; ++w) s += red[(w * 8 + tok) * rp + i];
        dst[tok * kMaxRank + i] = s;
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) bgmv_shrink_tma_kernel(const __grid_constant__ ApplyParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    float* red2 = reinterpret_cast<float*>(smem + kStages * kShrinkStage);      // two reduction tiles
    Meta* meta = reinterpret_cast<Meta*>(smem + kStages * kShrinkStage + 2 * kRedBytes);
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(meta + kMetaSlots);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);                 // full: producer's arrive + tx bytes
            mbar_init(smem_u32(&bars[kStages + s]), kConsWarps);   // empty: one arrival per consumer warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // The consumers wait for the predecessor kernel here.  The producers read only the plan and
    // the weight pools at first, which no kernel that may still be running writes, and wait
    // before they touch x: the first weight copies overlap the predecessor's tail.
    if (warp < kConsWarps) {
        pdl_wait_prior();
        if (tid == 0) pdl_launch_dependents();
    }

    PlanView pv = plan_view(p.plan, p.cap, p.n_adapters);
    WorkspaceView ws = workspace_view(p.workspace, p.cap, p.n_proj);
    const PlanHeader hdr = *pv.hdr;
    if (!plan_usable(hdr, p, &ws.ctl->error)) return;
    const int n_units = (p.flags & B200_LORA_NO_TENSOR) ? hdr.n_units : hdr.n_units_short;
    const int n_items = n_units * p.total_super_in;
    // each CTA takes a contiguous range of items
    const int per_cta = (n_items + (int)gridDim.x - 1) / (int)gridDim.x;
    const int first = blockIdx.x * per_cta;
    if (first >= n_items) return;
    const int n_local = min(per_cta, n_items - first);
    unsigned* err = &ws.ctl->error;

    if (warp >= kConsWarps) {
        // ---------------- producer warps ----------------
        const int pw = warp - kConsWarps;
        if (pw >= n_local) return;
        int rec;
        Cursor cur = cursor_at(p, first + pw, n_units, false, pv.unit_tab, lane, rec);
        bool waited = false;
        // after the wait: the x rows of the units whose weights were requested before it
        auto late_parts = [&](int upto) {
            pdl_wait_prior();
            waited = true;
            for (int k = pw; k < upto; k += kProdWarps) {
                const Meta& mk = meta[k % kMetaSlots];
                if (mk.valid)
                    shrink_produce<T>(p, item_of_meta(mk), record_of_meta(mk, lane), smem_u32(smem + (k % kStages) * kShrinkStage),
                                      smem_u32(&bars[k % kStages]), lane, 2);
            }
        };
        for (int n = pw; n < n_local; n += kProdWarps) {
            if (!waited && n >= kStages) late_parts(n);
            const int s = n % kStages;
            const unsigned ph = (n / kStages) & 1;
            const Item it = make_item(p, rec, cur, false);
            // There are twice as many meta slots as stages, so unit n's slot is free once unit
            // n - kStages has been handed over: fill it before waiting for the stage itself, and
            // nothing but the copies stands between that wait and the stage being in flight again.
            publish_meta(&meta[n % kMetaSlots], rec, it, lane);
            mbar_wait(smem_u32(&bars[kStages + s]), ph ^ 1, err, 1);
            const unsigned full = smem_u32(&bars[s]);
            if (it.valid) shrink_produce<T>(p, it, rec, smem_u32(smem + s * kShrinkStage), full, lane, waited ? 3 : 1);
            else if (lane == 0) mbar_arrive(full);
            if (n + kProdWarps < n_local) cursor_advance(p, n_units, false, pv.unit_tab, lane, kProdWarps, cur, rec);
        }
        if (!waited) late_parts(n_local);
        return;
    }

    // ---------------- consumer warps ----------------
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    Run run;
    run.proj = -1; run.wseg = -1; run.count = 0;
    run.start = run.ntok = run.rank = run.first_kc = run.n_chunks = 0;
    int red_sel = 0;
    for (int n = 0; n < n_local; ++n) {
        const int s = n % kStages;
        const unsigned ph = (n / kStages) & 1;
        mbar_wait(smem_u32(&bars[s]), ph, err, 2);
        const Meta m = load_meta(&meta[n % kMetaSlots]);
        if (m.valid) {
            if (m.proj != run.proj || m.u.wseg != run.wseg) {
                if (run.count > 0) shrink_flush<T>(p, ws, run, acc, red2, red_sel, tid);
                run.proj = m.proj; run.wseg = m.u.wseg; run.start = m.u.start; run.ntok = m.u.ntok;
                run.rank = m.u.rank; run.first_kc = m.kc; run.count = 0; run.n_chunks = m.n_chunks;
            }
            shrink_consume_any<T>(m, smem + s * kShrinkStage, acc, tid);
            ++run.count;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars[kStages + s]));      // this warp is done with the stage
    }
    if (run.count > 0) shrink_flush<T>(p, ws, run, acc, red2, red_sel, tid);
}

// =============================================================================================
// expand
// =============================================================================================
// What the expand producers need to add up a segment's split-K slots themselves.
struct FoldCtx {
    int n_units;      // units of the plan (0: the intermediate is final in the workspace already)
    int per_cta;      // length of a CTA's item range in the shrink kernel
};

// `parts` bit 0: the barrier's byte count and the weight tile (never written while kernels of
// this library run, so they may be requested before the predecessor kernel has ended); bit 2:
// the y rows (final once the kernel before the predecessor has completed); bit 1, always last:
// the intermediate v and the producer's arrival.  v is needed
// only by the first unit a CTA has of a (projection, work segment) - the consumers keep its
// fragments for the units that follow - and comes either from the workspace (a tensor-parallel
// caller has summed it over the ranks) or from the shrink kernel's split-K slots, which the
// producer warp adds up in ascending k order straight into the stage.
template <typename T>
__device__ __forceinline__ void expand_produce(const ApplyParams& p, const WorkspaceView& ws, const Item& m, int rec,
                                               unsigned char* stage_ptr, unsigned bar, int lane, int parts, bool need_v,
                                               const FoldCtx& fc, int u0) {
    const unsigned stage = smem_u32(stage_ptr);
    const ProjArgs& pj = p.proj[m.proj];
    const int r = m.rank;
    const int jc = kSuper / n_sub(r);
    const unsigned w_bytes = m.width_ok * r * 2;
    const unsigned y_bytes = (p.y_f32 || (p.flags & B200_LORA_DELTA_THEN_ADD)) ? 0u : m.width_ok * 2;
    const bool v_copy = need_v && fc.n_units == 0;
    const unsigned v_bytes = v_copy ? r * 4 : 0u;
    if (parts & 1) {
        if (lane == 0) mbar_expect_tx(bar, w_bytes + m.ntok * (y_bytes + v_bytes));
        __syncwarp();
    }
    // one instruction: lane 0 the weight tile, lanes 8..15 the y rows, lanes 16..23 the v rows
    const int tok = __shfl_sync(0xffffffffu, rec, 8 + (lane & 7));
    unsigned dst = 0, bytes = 0;
    const void* src = pj.wb;
    if (lane == 0) {
        dst = stage;
        src = reinterpret_cast<const T*>(pj.wb) + (item_row0(p, m) * (long long)pj.h_out + (long long)m.c0 * r);
        bytes = (parts & 1) ? w_bytes : 0u;
    } else if (lane >= 8 && lane < 8 + m.ntok) {
        dst = stage + kWTile + (lane - 8) * (jc * 2 + kYPad);
        src = reinterpret_cast<const T*>(pj.y) + (long long)tok * pj.ldy + m.c0;
        bytes = (parts & 4) ? y_bytes : 0u;
    } else if (lane >= 16 && lane < 16 + m.ntok) {
        dst = stage + kWTile + kYBytes + (lane - 16) * (kVPitch * 4);
        src = ws.v + ((size_t)m.proj * p.cap + m.start + (lane - 16)) * kMaxRank;
        bytes = (parts & 2) ? v_bytes : 0u;
    }
    if (bytes) bulk_g2s(dst, src, bytes, bar);
    if (parts & 2) {
        if (need_v && !v_copy) {
            float* vt = reinterpret_cast<float*>(stage_ptr + kWTile + kYBytes);
            const int seg_first = shrink_seg_first(p, fc.n_units, m.proj, u0);
            const int n_chunks = shrink_chunks(p, m.proj, r);
            const int qshift = 31 - __clz(r >> 2);             // quads of four rank indices per token
            const int nq = (m.ntok * r) >> 2;
            for (int base = 0; base < nq; base += 64) {        // two quads per lane and pass
                size_t off[2];
                bool on[2];
                int dst[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int idx = base + 32 * i + lane;
                    const int t = idx >> qshift, k4 = (idx & ((r >> 2) - 1)) * 4;
                    on[i] = idx < nq;
                    off[i] = ((size_t)m.proj * p.cap + m.start + t) * kMaxRank + k4;
                    dst[i] = t * kVPitch + k4;
                }
                float4 sum[2];
                fold_quads<T, 2>(p, ws, off, on, seg_first, fc.per_cta, n_chunks, sum);
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    if (on[i]) *reinterpret_cast<float4*>(vt + dst[i]) = sum[i];
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar);                       // releases the v tile with it
    }
}

// One packed 16-bit pair of the hi halves (the values rounded to T) or of the lo halves (what
// the rounding dropped) of two fp32 values.
template <typename T>
__device__ __forceinline__ unsigned hl_pack(float v0, float v1, bool lo) {
    const float h0 = Cvt<T>::round1(v0), h1 = Cvt<T>::round1(v1);
    return lo ? Cvt<T>::pack2(v0 - h0, v1 - h1) : Cvt<T>::pack2(h0, h1);
}

// R = rank class.  The weight tile is the MMA's A operand: 16 output columns (M) by 16 rank
// indices (K, in a fixed permutation that lets a thread fetch its fragments with one wide load
// per row).  The N columns are the tokens: column 2q holds the hi half of token q's
// intermediate and column 2q+1 the lo half, so one MMA serves four tokens and a second one,
// issued only for units of more than four tokens, serves tokens 4..7.  Thread (g, t) ends up
// with the hi and lo products of token t for output columns g and g + 8 of the block.
//   R=64: chunks 2t and 2t+1 of each 128-byte weight row (4 MMA k-steps)
//   R=32: chunk t of each 64-byte row (2 k-steps);  R=16: 8 bytes (1 k-step);  R=8: 4 bytes.
// A warp owns NBW consecutive 16-column blocks; the consumer warps never meet at a barrier.
// A warp first moves everything it needs of the stage into registers (intermediate fragments,
// weight fragments, the staged y values), hands the stage back (`empty_bar`) and only then
// computes: the time a stage stays out of flight does not include the arithmetic.
template <typename T, int R>
__device__ __forceinline__ void expand_consume(const ApplyParams& p, const Meta& m, const int* tok_rows, unsigned char* stage,
                                               int tid, unsigned (&bf)[2][4][2], bool reuse, unsigned empty_bar) {
    constexpr int KS = R == 64 ? 4 : R == 32 ? 2 : 1;
    constexpr int JC = kSuper / (R <= 16 ? 4 : R / 4);
    constexpr int NBW = JC / 16 / kConsWarps;              // 16-column blocks per warp: 4, 4, 2, 1
    const ProjArgs& pj = p.proj[m.proj];
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int ntok = m.u.ntok;
    const int ngrp = ntok > 4 ? 2 : 1;
    const float scale = m.u.scale;
    const bool lo_half = (g & 1) != 0;

    // B fragments of token (g >> 1) + 4 * group, hi or lo half by the parity of g; they are the
    // same for every unit of one (projection, work segment), so consecutive units reuse them
    if (!reuse) {
#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
#pragma unroll
        for (int k = 0; k < KS; ++k) bf[grp][k][0] = bf[grp][k][1] = 0u;
        const int q = (g >> 1) + 4 * grp;
        if (q < ntok) {
            const float* vt = reinterpret_cast<const float*>(stage + kWTile + kYBytes) + q * kVPitch;
            if constexpr (R == 64) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const float4 lo4 = *reinterpret_cast<const float4*>(vt + (2 * t + c) * 8);
                    const float4 hi4 = *reinterpret_cast<const float4*>(vt + (2 * t + c) * 8 + 4);
                    bf[grp][2 * c][0] = hl_pack<T>(lo4.x, lo4.y, lo_half);
                    bf[grp][2 * c][1] = hl_pack<T>(lo4.z, lo4.w, lo_half);
                    bf[grp][2 * c + 1][0] = hl_pack<T>(hi4.x, hi4.y, lo_half);
                    bf[grp][2 * c + 1][1] = hl_pack<T>(hi4.z, hi4.w, lo_half);
                }
            } else if constexpr (R == 32) {
                const float4 lo4 = *reinterpret_cast<const float4*>(vt + t * 8);
                const float4 hi4 = *reinterpret_cast<const float4*>(vt + t * 8 + 4);
                bf[grp][0][0] = hl_pack<T>(lo4.x, lo4.y, lo_half);
                bf[grp][0][1] = hl_pack<T>(lo4.z, lo4.w, lo_half);
                bf[grp][1][0] = hl_pack<T>(hi4.x, hi4.y, lo_half);
                bf[grp][1][1] = hl_pack<T>(hi4.z, hi4.w, lo_half);
            } else if constexpr (R == 16) {
                const float4 v4 = *reinterpret_cast<const float4*>(vt + t * 4);
                bf[grp][0][0] = hl_pack<T>(v4.x, v4.y, lo_half);
                bf[grp][0][1] = hl_pack<T>(v4.z, v4.w, lo_half);
            } else {
                const float2 v2 = *reinterpret_cast<const float2*>(vt + t * 2);
                bf[grp][0][0] = hl_pack<T>(v2.x, v2.y, lo_half);
            }
        }
    }
    }

    const int jbase = warp * NBW * 16;
    // the weight fragments of all of the warp's blocks
    unsigned a[NBW][KS][4];
#pragma unroll
    for (int nb = 0; nb < NBW; ++nb) {
        const unsigned char* w0 = stage + (jbase + nb * 16 + g) * (R * 2);   // output column g of the block
        const unsigned char* w1 = w0 + 8 * (R * 2);                          // output column g + 8
        if constexpr (R == 64) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const uint4 r0 = *reinterpret_cast<const uint4*>(w0 + (2 * t + c) * 16);
                const uint4 r1 = *reinterpret_cast<const uint4*>(w1 + (2 * t + c) * 16);
                a[nb][2 * c][0] = r0.x; a[nb][2 * c][1] = r1.x; a[nb][2 * c][2] = r0.y; a[nb][2 * c][3] = r1.y;
                a[nb][2 * c + 1][0] = r0.z; a[nb][2 * c + 1][1] = r1.z; a[nb][2 * c + 1][2] = r0.w; a[nb][2 * c + 1][3] = r1.w;
            }
        } else if constexpr (R == 32) {
            const uint4 r0 = *reinterpret_cast<const uint4*>(w0 + t * 16);
            const uint4 r1 = *reinterpret_cast<const uint4*>(w1 + t * 16);
            a[nb][0][0] = r0.x; a[nb][0][1] = r1.x; a[nb][0][2] = r0.y; a[nb][0][3] = r1.y;
            a[nb][1][0] = r0.z; a[nb][1][1] = r1.z; a[nb][1][2] = r0.w; a[nb][1][3] = r1.w;
        } else if constexpr (R == 16) {
            const uint2 r0 = *reinterpret_cast<const uint2*>(w0 + t * 8);
            const uint2 r1 = *reinterpret_cast<const uint2*>(w1 + t * 8);
            a[nb][0][0] = r0.x; a[nb][0][1] = r1.x; a[nb][0][2] = r0.y; a[nb][0][3] = r1.y;
        } else {
            a[nb][0][0] = *reinterpret_cast<const unsigned*>(w0 + t * 4);
            a[nb][0][1] = *reinterpret_cast<const unsigned*>(w1 + t * 4);
            a[nb][0][2] = a[nb][0][3] = 0u;
        }
    }
    // Token t (+4): hi + lo products for columns g and g + 8.  Lanes g and g ^ 1 swap one value
    // so that each ends up with two adjacent columns: (g, g+1) for even g, (g+7, g+8) for odd g.
    const unsigned char* ysb = stage + kWTile;
    constexpr int ypitch = JC * 2 + kYPad;
    const bool staged = !(p.y_f32 || (p.flags & B200_LORA_DELTA_THEN_ADD));
    const int jl = jbase + (lo_half ? g + 7 : g);
    const bool col_ok = jbase < m.width_ok;                // the warp's columns lie inside the matrix
    // the staged y values this lane will update, and the rows they go back to
    unsigned yw[2][NBW];
    int row[2];
#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
        const int q = t + 4 * grp;
        row[grp] = (grp < ngrp && q < ntok && col_ok) ? tok_rows[q] : -1;
#pragma unroll
        for (int nb = 0; nb < NBW; ++nb) yw[grp][nb] = 0u;
        if (staged && row[grp] >= 0) {
            const unsigned* ys = reinterpret_cast<const unsigned*>(ysb + q * ypitch + jl * 2);
#pragma unroll
            for (int nb = 0; nb < NBW; ++nb) yw[grp][nb] = ys[nb * 8];
        }
    }
    // the stage is no longer needed
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar);

#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
        if (grp >= ngrp) break;                            // uniform across the warp
        float d0[NBW], d1[NBW];
#pragma unroll
        for (int nb = 0; nb < NBW; ++nb) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 0; k < KS; ++k) Mma<T>::run(acc, a[nb][k][0], a[nb][k][1], a[nb][k][2], a[nb][k][3], bf[grp][k][0], bf[grp][k][1]);
            const float c_lo = scale * (acc[0] + acc[1]);
            const float c_hi = scale * (acc[2] + acc[3]);
            const float got = __shfl_xor_sync(0xffffffffu, lo_half ? c_lo : c_hi, 4);
            d0[nb] = lo_half ? got : c_lo;
            d1[nb] = lo_half ? c_hi : got;
        }
        if (row[grp] < 0) continue;
        const long long yoff = (long long)row[grp] * pj.ldy + m.c0 + jl;
        if (staged) {
            // every lane adds its pairs and stores them straight to global memory, eight lanes
            // filling one 32-byte sector of a token's row
            unsigned* yg = reinterpret_cast<unsigned*>(reinterpret_cast<T*>(pj.y) + yoff);
#pragma unroll
            for (int nb = 0; nb < NBW; ++nb) {
                float lo, hi;
                if (Cvt<T>::is_bf16) {
                    lo = __uint_as_float(yw[grp][nb] << 16); hi = __uint_as_float(yw[grp][nb] & 0xffff0000u);
                } else {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&yw[grp][nb]));
                    lo = f.x; hi = f.y;
                }
                yg[nb * 8] = Cvt<T>::pack2(lo + d0[nb], hi + d1[nb]);
            }
        } else if (p.y_f32) {
            float2* yp = reinterpret_cast<float2*>(reinterpret_cast<float*>(pj.y) + yoff);
            float2 yv[NBW];
#pragma unroll
            for (int nb = 0; nb < NBW; ++nb) yv[nb] = yp[nb * 8];
#pragma unroll
            for (int nb = 0; nb < NBW; ++nb) {
                yv[nb].x += d0[nb]; yv[nb].y += d1[nb];
                yp[nb * 8] = yv[nb];
            }
        } else {
            // the delta is rounded to the I/O type and added to y in that type, two outputs
            // per reduction, straight in global memory: no y tile, no write-back
            T* yp = reinterpret_cast<T*>(pj.y) + yoff;
#pragma unroll
            for (int nb = 0; nb < NBW; ++nb) {
                const unsigned d = Cvt<T>::pack2(d0[nb], d1[nb]);
                if (Cvt<T>::is_bf16) asm volatile("red.global.add.noftz.bf16x2 [%0], %1;" ::"l"(yp + nb * 16), "r"(d) : "memory");
                else asm volatile("red.global.add.noftz.f16x2 [%0], %1;" ::"l"(yp + nb * 16), "r"(d) : "memory");
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) bgmv_expand_tma_kernel(const __grid_constant__ ApplyParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    Meta* meta = reinterpret_cast<Meta*>(smem + kStages * kExpandStage);
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(meta + kMetaSlots);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[kStages + s]), kConsWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp < kConsWarps) {                               // the producers wait before they touch v
        pdl_wait_prior();
        if (tid == 0) pdl_launch_dependents();
    }

    PlanView pv = plan_view(p.plan, p.cap, p.n_adapters);
    WorkspaceView ws = workspace_view(p.workspace, p.cap, p.n_proj);
    const PlanHeader hdr = *pv.hdr;
    if (!plan_usable(hdr, p, &ws.ctl->error)) return;
    const int n_units = (p.flags & B200_LORA_NO_TENSOR) ? hdr.n_units : hdr.n_units_short;
    const int n_items = n_units * p.total_super_out;
    const int per_cta = (n_items + (int)gridDim.x - 1) / (int)gridDim.x;
    const int first = blockIdx.x * per_cta;
    if (first >= n_items) return;
    const int n_local = min(per_cta, n_items - first);
    unsigned* err = &ws.ctl->error;

    if (warp >= kConsWarps) {
        const int pw = warp - kConsWarps;
        if (pw >= n_local) return;
        int rec;
        Cursor cur = cursor_at(p, first + pw, n_units, true, pv.unit_tab, lane, rec);
        FoldCtx fc;
        fc.n_units = (p.flags & B200_LORA_ONLY_EXPAND) ? 0 : n_units;
        fc.per_cta = (n_units * p.total_super_in + (int)gridDim.x - 1) / (int)gridDim.x;
        bool waited = false;
        // Before the wait: weights and y rows (when this CTA runs, every kernel before the
        // predecessor has completed - see the note on programmatic launches in lora_common.cuh -
        // and the predecessor, this apply's shrink or reduction step, does not write y).  After
        // the wait: the intermediates of those units; the meta slot's spare words hold what that
        // takes (first unit of the segment, does it need v)
        auto late_parts = [&](int upto) {
            pdl_wait_prior();
            waited = true;
            for (int k = pw; k < upto; k += kProdWarps) {
                const Meta& mk = meta[k % kMetaSlots];
                if (mk.valid)
                    expand_produce<T>(p, ws, item_of_meta(mk), record_of_meta(mk, lane), smem + (k % kStages) * kExpandStage,
                                      smem_u32(&bars[k % kStages]), lane, 2, mk.pad[0] != 0, fc, mk.pad[1]);
            }
        };
        for (int n = pw; n < n_local; n += kProdWarps) {
            if (!waited && n >= kStages) late_parts(n);
            const int s = n % kStages;
            const unsigned ph = (n / kStages) & 1;
            const Item it = make_item(p, rec, cur, true);
            // the CTA's first unit of a (projection, work segment) brings the intermediate along
            const bool need_v = n == 0 || (cur.sp == 0 && cur.sub == 0);
            // ... except the CTA's very first unit, whose intermediate the (still idle) consumer
            // warps add up with all their threads: it is on the kernel's critical path
            const bool by_consumers = n == 0 && fc.n_units != 0;
            Meta* slot = &meta[n % kMetaSlots];          // free already (see the shrink kernel)
            publish_meta(slot, rec, it, lane);
            if (lane == 0) { slot->pad[0] = (need_v && !by_consumers) ? 1 : 0; slot->pad[1] = cur.unit; }
            __syncwarp();
            if (n == 0) asm volatile("bar.arrive 2, %0;" ::"n"(kConsThreads + 32) : "memory");   // meta slot 0 is published
            mbar_wait(smem_u32(&bars[kStages + s]), ph ^ 1, err, 3);
            const unsigned full = smem_u32(&bars[s]);
            if (it.valid) expand_produce<T>(p, ws, it, rec, smem + s * kExpandStage, full, lane, waited ? 7 : 1 | 4, need_v && !by_consumers, fc, cur.unit);
            else if (lane == 0) mbar_arrive(full);
            if (n + kProdWarps < n_local) cursor_advance(p, n_units, true, pv.unit_tab, lane, kProdWarps, cur, rec);
        }
        if (!waited) late_parts(n_local);
        return;
    }

    // The intermediate of the CTA's first unit: one quad per thread, up to eight slots in flight.
    asm volatile("bar.sync 2, %0;" ::"n"(kConsThreads + 32) : "memory");       // producer 0 has published meta slot 0
    if (!(p.flags & B200_LORA_ONLY_EXPAND)) {
        const Meta m0 = load_meta(&meta[0]);
        if (m0.valid) {
            const int r = m0.u.rank;
            const int per_a = (n_units * p.total_super_in + (int)gridDim.x - 1) / (int)gridDim.x;
            const int seg_first = shrink_seg_first(p, n_units, m0.proj, m0.pad[1]);
            const int n_chunks = shrink_chunks(p, m0.proj, r);
            const int qshift = 31 - __clz(r >> 2);
            float* vt = reinterpret_cast<float*>(smem + kWTile + kYBytes);
            for (int idx = tid; idx < ((m0.u.ntok * r) >> 2); idx += kConsThreads) {
                const int t = idx >> qshift, k4 = (idx & ((r >> 2) - 1)) * 4;
                const size_t off[1] = {((size_t)m0.proj * p.cap + m0.u.start + t) * kMaxRank + k4};
                const bool on[1] = {true};
                float4 sum[1];
                fold_quads<T, 1, 8>(p, ws, off, on, seg_first, per_a, n_chunks, sum);
                *reinterpret_cast<float4*>(vt + t * kVPitch + k4) = sum[0];
            }
        }
        cons_sync();
    }
    unsigned bf[2][4][2];                                  // v fragments of the last (projection, work segment)
    int bf_key = -1;
    for (int n = 0; n < n_local; ++n) {
        const int s = n % kStages;
        const unsigned ph = (n / kStages) & 1;
        mbar_wait(smem_u32(&bars[s]), ph, err, 4);
        const Meta m = load_meta(&meta[n % kMetaSlots]);
        unsigned char* stage = smem + s * kExpandStage;
        if (m.valid) {
            const int key = m.proj * p.cap + m.u.wseg;
            const bool reuse = key == bf_key;
            bf_key = key;
            const unsigned empty_bar = smem_u32(&bars[kStages + s]);      // one arrival per consumer warp, made inside
            switch (m.u.rank) {
                case 8:  expand_consume<T, 8>(p, m, meta[n % kMetaSlots].u.tok, stage, tid, bf, reuse, empty_bar); break;
                case 16: expand_consume<T, 16>(p, m, meta[n % kMetaSlots].u.tok, stage, tid, bf, reuse, empty_bar); break;
                case 32: expand_consume<T, 32>(p, m, meta[n % kMetaSlots].u.tok, stage, tid, bf, reuse, empty_bar); break;
                default: expand_consume<T, 64>(p, m, meta[n % kMetaSlots].u.tok, stage, tid, bf, reuse, empty_bar); break;
            }
        } else {
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars[kStages + s]));
        }
    }
}

// For tensor-parallel callers, who sum the intermediate over the ranks between the two halves:
// adds up the split-K slots of every (projection, work segment) into v in the workspace.
template <typename T>
__global__ void __launch_bounds__(128) fold_partials_kernel(const __grid_constant__ ApplyParams p, int shrink_grid) {
    pdl_wait_prior();
    pdl_launch_dependents();
    PlanView pv = plan_view(p.plan, p.cap, p.n_adapters);
    WorkspaceView ws = workspace_view(p.workspace, p.cap, p.n_proj);
    const PlanHeader hdr = *pv.hdr;
    if (!plan_usable(hdr, p, &ws.ctl->error)) return;
    const int n_units = (p.flags & B200_LORA_NO_TENSOR) ? hdr.n_units : hdr.n_units_short;
    const int per_cta = (n_units * p.total_super_in + shrink_grid - 1) / shrink_grid;
    const int proj = blockIdx.y;
    // The units with sub-range 0 are the first units of the work segments.  A warp looks at 32 records at
    // once (one load round) and then works through the heads among them.
    const int lane = threadIdx.x & 31, warp_g = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int n_warps = gridDim.x * (blockDim.x >> 5);
    for (int base = warp_g * 32; base < n_units; base += n_warps * 32) {
        const int u = base + lane;
        int r = 0, ntok = 0, start = 0;
        if (u < n_units) {
            const UnitRec* rec = reinterpret_cast<const UnitRec*>(pv.unit_tab) + u;
            if (rec->sub == 0) { r = rec->rank; ntok = rec->ntok; start = rec->start; }
        }
        unsigned heads = __ballot_sync(0xffffffffu, ntok > 0);
        while (heads) {
            const int src = __ffs(heads) - 1;
            heads &= heads - 1;
            const int hr = __shfl_sync(0xffffffffu, r, src), hn = __shfl_sync(0xffffffffu, ntok, src);
            const int hs = __shfl_sync(0xffffffffu, start, src);
            const int seg_first = shrink_seg_first(p, n_units, proj, base + src);
            const int n_chunks = shrink_chunks(p, proj, hr);
            const int qshift = 31 - __clz(hr >> 2);
            for (int idx = lane; idx < ((hn * hr) >> 2); idx += 32) {
                const int t = idx >> qshift, k4 = (idx & ((hr >> 2) - 1)) * 4;
                const size_t off = ((size_t)proj * p.cap + hs + t) * kMaxRank + k4;
                const size_t offs[1] = {off};
                const bool on[1] = {true};
                float4 sum[1];
                fold_quads<T, 1>(p, ws, offs, on, seg_first, per_cta, n_chunks, sum);
                *reinterpret_cast<float4*>(ws.v + off) = sum[0];
            }
        }
    }
}

constexpr int kShrinkSmem = kStages * kShrinkStage + 2 * kRedBytes + kMetaSlots * (int)sizeof(Meta) + 2 * kStages * 8 + 16;
constexpr int kExpandSmem = kStages * kExpandStage + kMetaSlots * (int)sizeof(Meta) + 2 * kStages * 8 + 16;
static_assert(kCtasPerSm * (kShrinkSmem + 1024) <= 233472 && kCtasPerSm * (kExpandSmem + 1024) <= 233472,
              "two CTAs must fit the 228 KB of shared memory of one SM");

// shrink kernel, then expand kernel (whose producers add up the split-K slots), each launched so
// that its prologue and first weight copies overlap its predecessor's tail; callers that want
// only one half get that half, and after a lone shrink half the intermediate is written out.
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
    const int grid = n_sm * kCtasPerSm;
    cudaError_t e = cudaSuccess;
    if (!(p.flags & B200_LORA_ONLY_EXPAND)) {
        e = launch_pdl(bgmv_shrink_tma_kernel<T>, grid, kThreads, kShrinkSmem, s, p);
        if (e == cudaSuccess && (p.flags & B200_LORA_ONLY_SHRINK) && !(p.flags & B200_LORA_KEEP_PARTIALS))
            e = launch_pdl(fold_partials_kernel<T>, dim3(n_sm, p.n_proj), 128, 0, s, p, grid);
    }
    if (e == cudaSuccess && !(p.flags & B200_LORA_ONLY_SHRINK))
        e = launch_pdl(bgmv_expand_tma_kernel<T>, grid, kThreads, kExpandSmem, s, p);
    return e;
}

}  // namespace

int bgmv_tma_shrink_grid(int n_sm) { return n_sm * kCtasPerSm; }

cudaError_t launch_bgmv_tma(const ApplyParams& p, int io_dtype, int n_sm, cudaStream_t s) {
    if (io_dtype == B200_LORA_F16) return launch_pair<__half>(p, n_sm, s);
    return launch_pair<__nv_bfloat16>(p, n_sm, s);
}

}  // namespace b200lora
