// Prefill SGMV for tall segments: TMA-fed tcgen05 tiles with TMEM accumulators.
//
// A "tall" run is >= 32 consecutive token rows that share one adapter of rank 16, 32 or 64
// (the plan finds them inside the adapter segments); everything else stays on the BGMV kernels.  One work item is
// (128-row tile of a tall segment, projection).  For it a CTA computes, entirely on chip,
//
//   phase 1   D1[128, r]    = X[128, h_in] . A^T          tcgen05.mma, M=128 N=r, K in blocks of 64
//   convert   V = D1 as 16-bit (hi, and lo unless the intermediate is to be rounded)   -> smem
//   phase 2   D2[128, 128]  = V . B[n0:n0+128, :]^T        per 128-column slice of the output
//   epilogue  y[rows, n0:n0+128] += scale * D2
//
// Warp roles: warps 0 and 3 issue TMA tensor copies (x and A boxes for phase 1, B boxes for
// phase 2) into mbarrier-tracked rings; warp 1 allocates TMEM and has one thread issue the tcgen05.mma of
// phase 1 into one of two D1 buffers, one item ahead; warp 2 has one thread issue those of phase
// 2 and moves y through shared memory (a [128, 128] block per slice comes in by tensor copy ahead of
// its accumulator; blocks of whole tiles leave by tensor store, rows of a run's last, partial tile are
// stored by their threads); both MMA warps release ring slots and publish accumulators with tcgen05.commit; warps 4..11 read
// accumulators with tcgen05.ld (each warp its own 32-lane quadrant of TMEM, two warps per
// quadrant sharing a slice's columns) and do the conversion and the y update.  Operand tiles use the 128/64/32-byte swizzled K-major layouts
// that TMA writes and the MMA descriptors name.  Two D2 buffers let the MMA of slice n+1 overlap
// the epilogue of slice n.  Single-CTA launch; every copy reads this GPU's own memory.
//
// Every mbarrier wait is bounded: on expiry the thread records an error word in the workspace
// and carries on with unchanged control flow, so the kernel terminates and TMEM is released.
//
// Semantics: the reference's prefill op bmm(bmm(x, A^T), B^T) (lightllm/models/lora_gpu.py:127-128)
// generalised to adapter-sorted segments; with B200_LORA_MID_ROUND the [T, r] intermediate is
// rounded to the I/O type exactly as that op's fp16 tensors do.
#include "lora_common.cuh"

namespace b200lora {

namespace {

constexpr int kBM = 128;            // token rows per tile
constexpr int kBK = 64;             // k columns per phase-1 block (one 128-byte swizzle atom)
constexpr int kBN = 128;            // output columns per phase-2 slice
constexpr int kS1 = 4;              // phase-1 ring slots (deeper rings measured no faster: one SM's copy
                                    // engine sustains about 50 GB/s whatever is in flight)
constexpr int kS2 = 2;              // phase-2 ring slots
constexpr int kXTile = kBM * kBK * 2;            // 16 KB
constexpr int kATile = 64 * kBK * 2;             // 8 KB (rank 64)
constexpr int kStage1 = kXTile + kATile;
constexpr int kBTile = kBN * 64 * 2;             // 16 KB (rank 64)
constexpr int kVTile = kBM * 64 * 2;             // 16 KB
constexpr int kYS = 2;               // y staging slots (16-bit y) when both phases run in one launch
constexpr int kYSMax = 4;            // ... when a launch runs phase 2 only (they take the phase-1 ring's room)
constexpr int kYTile = kBM * kBN * 2;            // 32 KB: two boxes of 64 columns, 128-byte swizzled rows
constexpr int kSmemTiles = kS1 * kStage1 + kS2 * kBTile + 2 * kVTile + kYS * kYTile;
constexpr int kNumBars = 2 * kS1 + 2 * kS2 + 6 + 4 + 2 * kYSMax;
static_assert(kS1 * kStage1 + kYS * kYTile >= kYSMax * kYTile, "the y slots of a phase-2 launch fit the ring's room");
static_assert((kYS & (kYS - 1)) == 0 && (kYSMax & (kYSMax - 1)) == 0, "slot counts are powers of two");
constexpr int kSgmvSmem = kSmemTiles + kNumBars * 8 + 128 + 1024;    // + TMEM address and y slot state + alignment slack
constexpr int kEpiWarps = 8;         // two per TMEM lane quadrant: each takes half the columns of a slice
constexpr int kSgmvThreads = 128 + kEpiWarps * 32;   // phase-1 TMA, phase-1 MMA, phase-2 MMA, phase-2 TMA, epilogue
constexpr int kTmemCols = 512;
constexpr int kD1Col = 0, kD2Col = 128;     // two D1 buffers of 64 columns, two D2 buffers of 128
constexpr unsigned kSpinLimit = 1u << 22;
// Launcher-internal flag (above the public bits): the two launches of a batch with few tiles.  The
// phase-1 launch cuts every (tile, projection) pair along k, one CTA per part; the parts' fp32 sums
// go to the split-K partial buffers and nothing else happens there: a small kernel between the two
// launches adds a pair's parts, in part order, into v (all SMs, coalesced, every part's load in
// flight at once; having the CTA that finishes a pair last add them kept a few SMs busy for longer
// than the whole of phase 1, and having every phase-2 CTA add them itself reads them once per
// column part).
constexpr int kFlagKSplit = 1 << 16;
constexpr int kMaxKSplit = 8;
// Launcher-internal: the phase-2 launch that follows it.  It is launched with programmatic stream
// serialization and waits for the phase-1 launch only where it reads v; its set-up and its first
// B and y copies (nothing the phase-1 launch writes) overlap that launch's tail.
constexpr int kFlagLateWait = 1 << 17;

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
__device__ __forceinline__ void mbar_wait(unsigned bar, unsigned parity, unsigned* err, unsigned code) {
    for (unsigned i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return;
        if ((i & 0x3fffu) == 0x3fffu && *reinterpret_cast<volatile unsigned*>(err) != 0u) break;
    }
    atomicMax(err, code);
}
__device__ __forceinline__ void tensor_g2s_2d(unsigned dst, const void* tmap, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tensor_s2g_2d(const void* tmap, int x, int y, unsigned src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(tmap), "r"(x), "r"(y), "r"(src) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the committed stores have read their shared-memory source / have completed
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---- tcgen05 wrappers -----------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(unsigned smem_dst, unsigned ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(unsigned d_tmem, unsigned long long adesc, unsigned long long bdesc,
                                           unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld16(unsigned taddr, float (&v)[16]) {
    unsigned r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// K-major shared-memory operand descriptor.  layout: 2 = 128-byte, 4 = 64-byte, 6 = 32-byte swizzle;
// sbo = bytes between 8-row groups.
__device__ __forceinline__ unsigned long long make_desc(unsigned saddr, unsigned layout, unsigned sbo) {
    unsigned long long d = (unsigned long long)((saddr >> 4) & 0x3fffu);
    d |= 1ull << 16;                                         // leading byte offset: unused with swizzle
    d |= (unsigned long long)((sbo >> 4) & 0x3fffu) << 32;
    d |= 1ull << 46;                                         // descriptor version of this architecture
    d |= (unsigned long long)layout << 61;
    return d;
}
// kind::f16 instruction descriptor: fp32 accumulate, both operands K-major
__device__ __forceinline__ unsigned make_idesc(bool bf16, int M, int N) {
    const unsigned fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((unsigned)(N >> 3) << 17) | ((unsigned)(M >> 4) << 24);
}

struct TileInfo {
    int adapter, rank, row0, valid, cls;     // cls: 0 -> 16, 1 -> 32, 2 -> 64
    int pos0;                                // sorted position of the tile's first row (index into v)
    float scale;
    long long a_row0;                        // first row of the A block in the [rows, h_in] view
    long long b_row0;                        // first row of the B block in the [rows, rank] view
};

__device__ __forceinline__ TileInfo tile_info(const SgmvParams& sp, const ApplyParams& p, const PlanView& pv,
                                              int tile, int proj) {
    TileInfo t;
    const int pos0 = pv.tile_tab[2 * tile], e1 = pv.tile_tab[2 * tile + 1];
    const int seg = e1 >> 8;
    t.adapter = pv.seg_adapter[seg];
    t.rank = pv.seg_rank[seg];
    t.pos0 = pos0;
    t.row0 = pv.perm[pos0];                   // rows of a run are consecutive
    t.valid = (e1 & 255) + 1;
    t.cls = t.rank == 16 ? 0 : t.rank == 32 ? 1 : 2;
    t.scale = p.scalings ? p.scalings[t.adapter] : p.scale;
    t.a_row0 = block_row0(p, t.adapter, t.rank);
    // B block [h_out, rank] starts at element a_row0 * h_out; in the [rows, rank] view that is row
    // a_row0 * (h_out / rank) (h_out is a multiple of 64).  Dense pools have rank == R.
    t.b_row0 = p.packed ? t.a_row0 * (long long)(p.proj[proj].h_out / t.rank)
                        : ((long long)t.adapter * p.n_layers + p.layer) * p.proj[proj].h_out;
    (void)sp;
    return t;
}

// k parts per (tile, projection) pair of a phase-1 launch with few pairs: as many as there are CTAs
// per pair, bounded by the k blocks of the narrowest input and by the partial buffers of the workspace
__device__ __forceinline__ int ksplit_of(const ApplyParams& p, int n_cta, int base_items) {
    if (base_items <= 0) return 1;
    int ksplit = max(1, min(kMaxKSplit, n_cta / base_items));
    int h_min = p.proj[0].h_in, h_max = p.proj[0].h_in;
    for (int i = 1; i < p.n_proj; ++i) { h_min = min(h_min, p.proj[i].h_in); h_max = max(h_max, p.proj[i].h_in); }
    return max(1, min(ksplit, min(h_min / kBK, max_kchunks(h_max))));
}

// Adds the k parts of every (tile, projection) pair into v after a k-split phase-1 launch of
// `n_cta` CTAs.  One unit = 16 rows of a pair = 256 threads, a thread per four rank columns.
__global__ void __launch_bounds__(256) sgmv_ksum_kernel(const __grid_constant__ ApplyParams p, int n_cta) {
    pdl_wait_prior();
    if (threadIdx.x == 0) pdl_launch_dependents();
    PlanView pv = plan_view(p.plan, p.cap, p.n_adapters);
    WorkspaceView ws = workspace_view(p.workspace, p.cap, p.n_proj);
    const PlanHeader hdr = *pv.hdr;
    if (!plan_usable(hdr, p, &ws.ctl->error)) return;
    const int base_items = hdr.n_tiles * p.n_proj;
    const int ksplit = ksplit_of(p, n_cta, base_items);
    if (ksplit <= 1) return;                               // phase 1 wrote v itself
    const size_t kstride = (size_t)p.n_proj * p.cap * kMaxRank;
    const int r16 = threadIdx.x >> 4, f = threadIdx.x & 15;
    for (int u = blockIdx.x; u < base_items * (kBM / 16); u += gridDim.x) {
        const int pair = u >> 3, tile = pair / p.n_proj, proj = pair - tile * p.n_proj;
        const int pos0 = pv.tile_tab[2 * tile], e1 = pv.tile_tab[2 * tile + 1];
        const int rank = pv.seg_rank[e1 >> 8], valid = (e1 & 255) + 1;
        const int row = (u & 7) * 16 + r16;
        if (row >= valid || f * 4 >= rank) continue;
        const size_t vidx = ((size_t)proj * p.cap + pos0 + row) * kMaxRank + f * 4;
        float4 g[kMaxKSplit];
#pragma unroll
        for (int kp = 0; kp < kMaxKSplit; ++kp) {
            g[kp] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (kp < ksplit) g[kp] = __ldcg(reinterpret_cast<const float4*>(ws.partial + kp * kstride + vidx));
        }
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int kp = 0; kp < kMaxKSplit; ++kp)
            if (kp < ksplit) { a.x += g[kp].x; a.y += g[kp].y; a.z += g[kp].z; a.w += g[kp].w; }
        *reinterpret_cast<float4*>(ws.v + vidx) = a;
    }
}

template <typename T>
__global__ void __launch_bounds__(kSgmvThreads, 1)
sgmv_tile_kernel(const __grid_constant__ ApplyParams p, const __grid_constant__ SgmvParams sp) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // tensor-parallel callers, and the launcher when tiles are few, run the two halves separately
    const bool do1 = !(p.flags & B200_LORA_ONLY_EXPAND), do2 = !(p.flags & B200_LORA_ONLY_SHRINK);
    // Shared memory: B ring, V (hi, lo), then the phase-1 ring followed by the y slots.  A launch
    // of phase 2 only has more y slots, in the ring's room.
    constexpr int ns1 = kS1;
    const int nys = !do1 ? kYSMax : kYS, nys_log = !do1 ? 2 : 1;
    unsigned char* stage2 = smem;
    unsigned char* vhi = stage2 + kS2 * kBTile;
    unsigned char* vlo = vhi + kVTile;
    unsigned char* flex = vlo + kVTile;
    unsigned char* stage1 = flex;
    unsigned char* ystage = !do1 ? flex : flex + kS1 * kStage1;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + kSmemTiles);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + kNumBars);
    int* ystate = reinterpret_cast<int*>(tmem_slot + 1);        // per y slot: projection (< 0: no store), column, row
    // barrier indices
    const int FULL1 = 0, EMPTY1 = kS1, FULL2 = 2 * kS1, EMPTY2 = 2 * kS1 + kS2;
    const int D1_FULL = 2 * kS1 + 2 * kS2, D1_EMPTY = D1_FULL + 2, V_READY = D1_FULL + 4, V_FREE = D1_FULL + 5;
    const int D2_FULL = D1_FULL + 6, D2_EMPTY = D1_FULL + 8, Y_FULL = D1_FULL + 10, Y_DONE = Y_FULL + kYSMax;
    auto bar = [&](int i) { return smem_u32(&bars[i]); };

    if (!(p.flags & kFlagLateWait)) {
        pdl_wait_prior();
        if (threadIdx.x == 0) pdl_launch_dependents();
    }
    PlanView pv = plan_view(p.plan, p.cap, p.n_adapters);
    WorkspaceView ws = workspace_view(p.workspace, p.cap, p.n_proj);
    const PlanHeader hdr = *pv.hdr;
    unsigned* err = &ws.ctl->error;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_tiles = plan_usable(hdr, p, err) ? hdr.n_tiles : 0;
    // Work items: (tile, projection) pairs, dealt to the CTAs round by round.  The pairs of the
    // last, incomplete round are cut by output columns into `nsplit` parts each (every part redoes
    // the cheap phase 1, mostly from L2), so that the round keeps all SMs busy for a fraction of a
    // pair's time instead of a few SMs for all of it.
    const int base_items = n_tiles * p.n_proj;
    const int n_cta = (int)gridDim.x;
    const int n_full = (base_items / n_cta) * n_cta, n_rem = base_items - n_full;
    const int ksplit = (p.flags & kFlagKSplit) ? ksplit_of(p, n_cta, base_items) : 1;
    const bool k_items = ksplit > 1 && (p.flags & B200_LORA_ONLY_SHRINK);
    // a launch of phase 2 only: both column halves of the epilogue build V (each its half of the rank columns)
    const bool both = !do1;
    // Column parts of the pairs of the last round.  A launch of both phases cuts them in about 2 * n_cta parts
    // (every part redoes phase 1, and measured against fewer parts the finer cut still wins).  A launch of
    // phase 2 only has nothing to redo: the CTAs work through ceil(n_rem * parts / n_cta) parts each and a part
    // costs a fixed start (reading v, building V) plus 1/parts of the pair's copies.
    int nsplit = 1;
    if (n_rem > 0 && !(p.flags & B200_LORA_ONLY_SHRINK)) {
        int max_parts = 8;
        float c2 = 0.f;                                    // KB of B and y boxes per pair, at the largest rank
        for (int i = 0; i < p.n_proj; ++i) {              // every part must own at least one column slice
            max_parts = min(max_parts, (p.proj[i].h_out + kBN - 1) / kBN);
            c2 += (float)(2 * kBM + 64) * p.proj[i].h_out * 2.f / 1024.f;
        }
        c2 /= p.n_proj;
        if (do1) nsplit = min(max_parts, max(1, (2 * n_cta) / n_rem));
        else {
            float best = 3.0e38f;
            for (int ns = 1; ns <= max_parts; ++ns) {
                const int rounds = (n_rem * ns + n_cta - 1) / n_cta;
                const float cost = rounds * (96.f + c2 / ns);
                if (cost < best * 0.98f) { best = cost; nsplit = ns; }   // more parts only where they clearly pay
            }
        }
    }
    const int n_items = k_items ? base_items * ksplit : n_full + n_rem * nsplit;
    // item -> pair, part, parts of the pair (parts of k in a k-split phase-1 launch, else of the output columns)
    auto decode = [&](int item, int& rest, int& part, int& parts) {
        if (k_items) { rest = item / ksplit; part = item - rest * ksplit; parts = ksplit; }
        else if (item < n_full) { rest = item; part = 0; parts = 1; }
        else { const int j = item - n_full; rest = n_full + j / nsplit; part = j % nsplit; parts = nsplit; }
    };
    const bool mid_round = (p.flags & B200_LORA_MID_ROUND) != 0;
    // 16-bit y goes through shared memory: tensor copies bring a slice's [128, 128] block in ahead
    // of its accumulator and, for tiles whose 128 rows all belong to the run, carry the sum back
    const bool y_staged = !p.y_f32;

    if (tid == 0) {
        for (int s = 0; s < kS1; ++s) { mbar_init(bar(FULL1 + s), 1); mbar_init(bar(EMPTY1 + s), 1); }
        for (int s = 0; s < kS2; ++s) { mbar_init(bar(FULL2 + s), 1); mbar_init(bar(EMPTY2 + s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar(D1_FULL + b), 1); mbar_init(bar(D1_EMPTY + b), 128); }
        mbar_init(bar(V_READY), do1 ? 128 : 256);
        mbar_init(bar(V_FREE), 1);
        for (int b = 0; b < 2; ++b) { mbar_init(bar(D2_FULL + b), 1); mbar_init(bar(D2_EMPTY + b), kEpiWarps * 32); }
        for (int b = 0; b < kYSMax; ++b) { mbar_init(bar(Y_FULL + b), 1); mbar_init(bar(Y_DONE + b), kEpiWarps * 32); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                    // one warp owns the TMEM allocation
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = *reinterpret_cast<volatile unsigned*>(tmem_slot);

    if (warp == 0) {
        // ================= TMA producer, phase 1: x and A boxes =================
        unsigned n1 = 0;                // ring uses so far
        for (int item = blockIdx.x; do1 && item < n_items; item += gridDim.x) {
            int rest, part, parts;
            decode(item, rest, part, parts);
            const int tile = rest / p.n_proj, proj = rest - tile * p.n_proj;   // a tile's projections are neighbours: x is read from DRAM once
            const TileInfo t = tile_info(sp, p, pv, tile, proj);
            const int nkb_all = p.proj[proj].h_in / kBK;
            const int kb0 = k_items ? part * nkb_all / parts : 0, kb1 = k_items ? (part + 1) * nkb_all / parts : nkb_all;
            for (int kb = kb0; kb < kb1; ++kb, ++n1) {
                const int s = n1 % ns1;
                mbar_wait(bar(EMPTY1 + s), ((n1 / ns1) & 1) ^ 1, err, 11);
                const unsigned dst = smem_u32(stage1 + s * kStage1);
                if (lane == 0) mbar_arrive_expect_tx(bar(FULL1 + s), kXTile + t.rank * kBK * 2);
                __syncwarp();
                // two copies per block (the copy count, not the byte count, is what this kernel is short
                // of): lane 1 the x box [64 x 128], lane 0 the A box [64 x rank]
                if (lane == 1)
                    tensor_g2s_2d(dst, &sp.xmap[proj], kb * kBK, t.row0, bar(FULL1 + s));
                else if (lane == 0)
                    tensor_g2s_2d(dst + kXTile, &sp.amap[proj][t.cls], kb * kBK, (int)t.a_row0, bar(FULL1 + s));
            }
        }
    } else if (warp == 3) {
        // ================= TMA producer, phase 2: B boxes =================
        // (a warp of its own: phase 1 runs an item ahead and must not queue behind these copies)
        // It also moves y: the load of slice n goes out as soon as the epilogue has finished with
        // the slice that used the slot before, and after that slice's store has read the slot.
        unsigned n2 = 0, ny = 0;
        auto retire = [&](unsigned k) {                       // slice k of this CTA
            const int ys = k & (nys - 1);
            mbar_wait(bar(Y_DONE + ys), (k >> nys_log) & 1, err, 21);
            if (lane == 0 && ystate[3 * ys] >= 0) {
                const int sp_ = ystate[3 * ys], sc = ystate[3 * ys + 1], sr = ystate[3 * ys + 2];
                const unsigned src = smem_u32(ystage + ys * kYTile);
                tensor_s2g_2d(&sp.ymap[sp_], sc, sr, src);
                if (sc + 64 < p.proj[sp_].h_out) tensor_s2g_2d(&sp.ymap[sp_], sc + 64, sr, src + kYTile / 2);
                bulk_commit();
                bulk_wait_read();
            }
            __syncwarp();
        };
        for (int item = blockIdx.x; do2 && item < n_items; item += gridDim.x) {
            int rest, part, parts;
            decode(item, rest, part, parts);
            const int tile = rest / p.n_proj, proj = rest - tile * p.n_proj;   // a tile's projections are neighbours: x is read from DRAM once
            const TileInfo t = tile_info(sp, p, pv, tile, proj);
            const ProjArgs& pj = p.proj[proj];
            const int nnt_all = (pj.h_out + kBN - 1) / kBN;
            const int nt0 = part * nnt_all / parts, nnt = (part + 1) * nnt_all / parts;
            for (int nt = nt0; nt < nnt; ++nt, ++n2) {
                const int s = n2 % kS2;
                mbar_wait(bar(EMPTY2 + s), ((n2 / kS2) & 1) ^ 1, err, 12);
                if (lane == 0) {
                    mbar_arrive_expect_tx(bar(FULL2 + s), kBN * t.rank * 2);
                    tensor_g2s_2d(smem_u32(stage2 + s * kBTile), &sp.bmap[proj][t.cls], 0, (int)t.b_row0 + nt * kBN,
                                  bar(FULL2 + s));
                }
                __syncwarp();
                if (y_staged) {
                    const int ys = ny & (nys - 1);
                    if (ny >= (unsigned)nys) retire(ny - nys);
                    if (lane == 0) {
                        const unsigned dst = smem_u32(ystage + ys * kYTile);
                        mbar_arrive_expect_tx(bar(Y_FULL + ys), kYTile);
                        tensor_g2s_2d(dst, &sp.ymap[proj], nt * kBN, t.row0, bar(Y_FULL + ys));
                        tensor_g2s_2d(dst + kYTile / 2, &sp.ymap[proj], nt * kBN + 64, t.row0, bar(Y_FULL + ys));
                        ystate[3 * ys] = t.valid == kBM ? proj : -1;      // other tiles are stored row by row by the epilogue
                        ystate[3 * ys + 1] = nt * kBN;
                        ystate[3 * ys + 2] = t.row0;
                    }
                    __syncwarp();
                    ++ny;
                }
            }
        }
        for (unsigned k = ny > (unsigned)nys ? ny - nys : 0u; k < ny; ++k) retire(k);
        if (lane == 0) bulk_wait_all();
    } else if (warp == 1) {
        // ================= MMA issuer, phase 1: D1[item & 1] = X . A^T =================
        // runs one item ahead of phase 2, so the x stream of the next item overlaps the y update
        // of this one
        unsigned n1 = 0, n_item = 0;
        const bool bf16 = Cvt<T>::is_bf16;
        for (int item = blockIdx.x; do1 && item < n_items; item += gridDim.x, ++n_item) {
            int rest, part, parts;
            decode(item, rest, part, parts);
            const int tile = rest / p.n_proj, proj = rest - tile * p.n_proj;   // a tile's projections are neighbours: x is read from DRAM once
            const TileInfo t = tile_info(sp, p, pv, tile, proj);
            const int nkb_all = p.proj[proj].h_in / kBK;
            const int kb0 = k_items ? part * nkb_all / parts : 0, kb1 = k_items ? (part + 1) * nkb_all / parts : nkb_all;
            const int b1 = n_item & 1;
            // the buffer must have been drained by the epilogue of the item two before
            mbar_wait(bar(D1_EMPTY + b1), ((n_item >> 1) & 1) ^ 1, err, 13);
            tc_fence_after();
            const unsigned idesc1 = make_idesc(bf16, kBM, t.rank);
            for (int kb = kb0; kb < kb1; ++kb, ++n1) {
                const int s = n1 % ns1;
                mbar_wait(bar(FULL1 + s), (n1 / ns1) & 1, err, 14);
                tc_fence_after();
                if (lane == 0) {
                    const unsigned xa = smem_u32(stage1 + s * kStage1), aa = xa + kXTile;
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)
                        tc_mma_f16(tmem + kD1Col + b1 * 64, make_desc(xa + k * 32, 2, 1024), make_desc(aa + k * 32, 2, 1024),
                                   idesc1, ((kb - kb0) | k) != 0);
                    tc_commit(bar(EMPTY1 + s));                       // slot reusable once these MMAs finish
                    if (kb == kb1 - 1) tc_commit(bar(D1_FULL + b1));
                }
                __syncwarp();
            }
        }
    } else if (warp == 2) {
        // ================= MMA issuer, phase 2: D2[buf] = V . B_slice^T =================
        unsigned n2 = 0, nd = 0, n_item = 0;
        const bool bf16 = Cvt<T>::is_bf16;
        for (int item = blockIdx.x; do2 && item < n_items; item += gridDim.x, ++n_item) {
            int rest, part, parts;
            decode(item, rest, part, parts);
            const int tile = rest / p.n_proj, proj = rest - tile * p.n_proj;   // a tile's projections are neighbours: x is read from DRAM once
            const TileInfo t = tile_info(sp, p, pv, tile, proj);
            const ProjArgs& pj = p.proj[proj];
            mbar_wait(bar(V_READY), n_item & 1, err, 15);
            tc_fence_after();
            const unsigned layout = t.cls == 2 ? 2u : t.cls == 1 ? 4u : 6u;
            const unsigned sbo = 8u * t.rank * 2u;
            const unsigned idesc2 = make_idesc(bf16, kBM, kBN);
            const int nnt_all = (pj.h_out + kBN - 1) / kBN;
            const int nt0 = part * nnt_all / parts, nnt = (part + 1) * nnt_all / parts;
            for (int nt = nt0; nt < nnt; ++nt, ++n2, ++nd) {
                const int s = n2 % kS2, buf = nd & 1;
                mbar_wait(bar(FULL2 + s), (n2 / kS2) & 1, err, 16);
                mbar_wait(bar(D2_EMPTY + buf), ((nd >> 1) & 1) ^ 1, err, 17);
                tc_fence_after();
                if (lane == 0) {
                    const unsigned ba = smem_u32(stage2 + s * kBTile);
                    const unsigned d2 = tmem + kD2Col + buf * kBN;
                    const int ksteps = t.rank / 16;
                    for (int k = 0; k < ksteps; ++k)
                        tc_mma_f16(d2, make_desc(smem_u32(vhi) + k * 32, layout, sbo), make_desc(ba + k * 32, layout, sbo),
                                   idesc2, k != 0);
                    if (!mid_round)
                        for (int k = 0; k < ksteps; ++k)
                            tc_mma_f16(d2, make_desc(smem_u32(vlo) + k * 32, layout, sbo),
                                       make_desc(ba + k * 32, layout, sbo), idesc2, 1u);
                    tc_commit(bar(EMPTY2 + s));
                    tc_commit(bar(D2_FULL + buf));
                    if (nt == nnt - 1) tc_commit(bar(V_FREE));        // V may be overwritten after this
                }
                __syncwarp();
            }
        }
    } else {
        // ================= epilogue warps =================
        const int quad = warp & 3;                          // TMEM lanes 32*quad .. +31
        const int half = (warp - 4) >> 2;                   // which 64 columns of every 128-column slice
        const int row = quad * 32 + lane;
        const unsigned lane_base = (unsigned)(quad * 32) << 16;
        unsigned nd = 0, n_item = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++n_item) {
            int rest, part, parts;
            decode(item, rest, part, parts);
            const int tile = rest / p.n_proj, proj = rest - tile * p.n_proj;   // a tile's projections are neighbours: x is read from DRAM once
            const TileInfo t = tile_info(sp, p, pv, tile, proj);
            const ProjArgs& pj = p.proj[proj];
            if (half != 0 && !do2) continue;
            // ---- D1 -> V (16-bit hi / lo), swizzled K-major rows of rank*2 bytes: first warp of the quadrant
            if (half == 0 || both) {
            float d1[64];
            // fp32 row of the intermediate: the reduced v, or this k part's slot when phase 1 is cut along k
            const size_t vidx = ((size_t)proj * p.cap + t.pos0 + row) * kMaxRank;
            const size_t kstride = (size_t)p.n_proj * p.cap * kMaxRank;
            float* vrow = k_items ? ws.partial + part * kstride + vidx : ws.v + vidx;
            if (do1) {
                const int b1 = n_item & 1;
                mbar_wait(bar(D1_FULL + b1), (n_item >> 1) & 1, err, 18);
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (c * 16 < t.rank) {
                        float v[16];
                        tc_ld16(tmem + lane_base + kD1Col + b1 * 64 + c * 16, v);
#pragma unroll
                        for (int i = 0; i < 16; ++i) d1[c * 16 + i] = v[i];
                    }
                }
                tc_fence_before();
                mbar_arrive(bar(D1_EMPTY + b1));
                if (!do2) {                                  // shrink half only: publish the fp32 rows
                    if (row < t.valid) {
#pragma unroll
                        for (int c = 0; c < 16; ++c)
                            if (c * 4 < t.rank)
                                reinterpret_cast<float4*>(vrow)[c] = make_float4(d1[4 * c], d1[4 * c + 1], d1[4 * c + 2], d1[4 * c + 3]);
                    }
                    continue;
                }
            } else {
                // expand half only: v was summed by the caller (or by the kernel that adds the k parts)
                if (p.flags & kFlagLateWait) { pdl_wait_prior(); pdl_launch_dependents(); }
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
                    if ((c >> 3) == half && c * 4 < t.rank && row < t.valid) f = __ldcg(reinterpret_cast<const float4*>(vrow) + c);
                    d1[4 * c] = f.x; d1[4 * c + 1] = f.y; d1[4 * c + 2] = f.z; d1[4 * c + 3] = f.w;
                }
            }
            mbar_wait(bar(V_FREE), (n_item & 1) ^ 1, err, 19);       // previous item's phase 2 finished with V
            {
                const int rb = t.rank * 2;                            // row bytes: 32, 64, 128
                const int sw = t.cls == 2 ? (row & 7) : t.cls == 1 ? ((row >> 1) & 3) : ((row >> 2) & 1);
                unsigned char* rh = vhi + (row >> 3) * (8 * rb) + (row & 7) * rb;
                unsigned char* rl = vlo + (row >> 3) * (8 * rb) + (row & 7) * rb;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    if (c * 8 < t.rank && (!both || (c >> 2) == half)) {
                        uint4 h, l;
                        unsigned* hp = reinterpret_cast<unsigned*>(&h);
                        unsigned* lp = reinterpret_cast<unsigned*>(&l);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float a = d1[c * 8 + 2 * i], b = d1[c * 8 + 2 * i + 1];
                            const float ha = Cvt<T>::round1(a), hb = Cvt<T>::round1(b);
                            hp[i] = Cvt<T>::pack2(ha, hb);
                            lp[i] = Cvt<T>::pack2(a - ha, b - hb);
                        }
                        *reinterpret_cast<uint4*>(rh + ((c ^ sw) << 4)) = h;
                        if (!mid_round) *reinterpret_cast<uint4*>(rl + ((c ^ sw) << 4)) = l;
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic writes -> tensor-core reads
            mbar_arrive(bar(V_READY));
            }
            // ---- D2 slices -> y
            const int nnt_all = (pj.h_out + kBN - 1) / kBN;
            const int nt0 = part * nnt_all / parts, nnt = (part + 1) * nnt_all / parts;
            const bool live = row < t.valid, whole = t.valid == kBM;
            for (int nt = nt0; nt < nnt; ++nt, ++nd) {
                const int buf = nd & 1, ys = nd & (nys - 1);
                // this thread's 128 bytes of the staged y block: row `row` of the box of its column half;
                // the 16-byte chunk c of a row sits at chunk c ^ (row & 7)
                unsigned char* ysm = ystage + ys * kYTile + half * (kYTile / 2) + row * 128;
                uint4* yrow = reinterpret_cast<uint4*>(reinterpret_cast<T*>(pj.y) + (long long)(t.row0 + row) * pj.ldy + nt * kBN) + half * (kBN / 16);
                if (y_staged) mbar_wait(bar(Y_FULL + ys), (nd >> nys_log) & 1, err, 22);
                mbar_wait(bar(D2_FULL + buf), (nd >> 1) & 1, err, 20);
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < kBN / 32; ++c) {
                    float v[16];
                    tc_ld16(tmem + lane_base + kD2Col + buf * kBN + half * (kBN / 2) + c * 16, v);
                    const int col = nt * kBN + half * (kBN / 2) + c * 16;
                    if (p.y_f32) {
                        if (live && col < pj.h_out) {
                            float4* yp = reinterpret_cast<float4*>(reinterpret_cast<float*>(pj.y) +
                                                                   (long long)(t.row0 + row) * pj.ldy + col);
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                float4 y4 = yp[q];
                                y4.x += t.scale * v[4 * q]; y4.y += t.scale * v[4 * q + 1];
                                y4.z += t.scale * v[4 * q + 2]; y4.w += t.scale * v[4 * q + 3];
                                yp[q] = y4;
                            }
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            uint4* ys4 = reinterpret_cast<uint4*>(ysm + (((2 * c + q) ^ (row & 7)) << 4));
                            uint4 y4 = *ys4;
                            float f[8];
                            Cvt<T>::unpack8(y4, f);
                            y4.x = Cvt<T>::pack2(f[0] + t.scale * v[8 * q], f[1] + t.scale * v[8 * q + 1]);
                            y4.y = Cvt<T>::pack2(f[2] + t.scale * v[8 * q + 2], f[3] + t.scale * v[8 * q + 3]);
                            y4.z = Cvt<T>::pack2(f[4] + t.scale * v[8 * q + 4], f[5] + t.scale * v[8 * q + 5]);
                            y4.w = Cvt<T>::pack2(f[6] + t.scale * v[8 * q + 6], f[7] + t.scale * v[8 * q + 7]);
                            if (whole) *ys4 = y4;                                   // leaves with the slot's tensor store
                            else if (live && col < pj.h_out) yrow[2 * c + q] = y4;
                        }
                    }
                }
                if (y_staged) {
                    if (whole) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tensor store
                    mbar_arrive(bar(Y_DONE + ys));
                }
                tc_fence_before();
                mbar_arrive(bar(D2_EMPTY + buf));
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, kTmemCols);
    // a CTA that waited nowhere above (no item that reads v) still waits before it leaves
    if ((p.flags & kFlagLateWait) && threadIdx.x == 0) { pdl_wait_prior(); pdl_launch_dependents(); }
}

}  // namespace

bool sgmv_tiles_supported(const ApplyParams& p) {
    for (int i = 0; i < p.n_proj; ++i)
        if ((p.proj[i].h_in % kBK) || (p.proj[i].h_out % 64)) return false;
    return true;
}

cudaError_t launch_sgmv_tiles(const ApplyParams& p, const SgmvParams& sp, int io_dtype, int n_sm, cudaStream_t s) {
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(sgmv_tile_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSgmvSmem);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(sgmv_tile_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSgmvSmem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    auto launch = [&](const ApplyParams& q) {
        if (io_dtype == B200_LORA_F16) sgmv_tile_kernel<__half><<<n_sm, kSgmvThreads, kSgmvSmem, s>>>(q, sp);
        else sgmv_tile_kernel<__nv_bfloat16><<<n_sm, kSgmvThreads, kSgmvSmem, s>>>(q, sp);
        return cudaGetLastError();
    };
    // With fewer (tile, projection) pairs than SMs a single launch has to cut every pair by output
    // columns, and each part streams the pair's x rows again for phase 1 at the rate one SM's
    // copy engine sustains.  Two launches avoid that: the first does phase 1 once per pair, cut
    // along k over the idle SMs, and leaves fp32 sums in the workspace; the second cuts only
    // phase 2.  The tile count is known on the device only; the token count bounds it.
    const bool halves_given = (p.flags & (B200_LORA_ONLY_SHRINK | B200_LORA_ONLY_EXPAND)) != 0;
    const long long max_pairs = ((long long)p.n_tokens / kBM + 1) * p.n_proj;
    if (max_pairs >= n_sm) return launch(p);
    ApplyParams q = p;
    if (halves_given) return launch(q);
    q.flags = p.flags | B200_LORA_ONLY_SHRINK | kFlagKSplit;
    cudaError_t e = launch(q);
    if (e != cudaSuccess) return e;
    e = launch_pdl(sgmv_ksum_kernel, dim3(n_sm), dim3(256), 0, s, q, n_sm);
    if (e != cudaSuccess) return e;
    q.flags = p.flags | B200_LORA_ONLY_EXPAND | kFlagLateWait;
    if (io_dtype == B200_LORA_F16)
        return launch_pdl(sgmv_tile_kernel<__half>, dim3(n_sm), dim3(kSgmvThreads), kSgmvSmem, s, q, sp);
    return launch_pdl(sgmv_tile_kernel<__nv_bfloat16>, dim3(n_sm), dim3(kSgmvThreads), kSgmvSmem, s, q, sp);
}

}  // namespace b200lora
