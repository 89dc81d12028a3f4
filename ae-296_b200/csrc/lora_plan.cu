// Plan build: adapter-index gather and segment bookkeeping on the device.
//
// One CTA turns the per-token adapter ids into
//   perm         stable counting sort (token order kept inside one adapter)
//   seg_*        one segment per adapter that has tokens, ascending adapter id
//   unit_tab     the <= 16 KB weight units the BGMV kernels walk: short segments first
//   tile_tab     128-row tiles of tall runs (>= 32 consecutive rows of one adapter) for the tensor-core kernel
// It replaces the reference's precomputed index tensor (lightllm/models/lora_gpu.py:120,124)
// and is integer work only: the tests require it bit-exact against a stable argsort.
#include "lora_common.cuh"

namespace b200lora {

constexpr int kPlanThreads = 1024;

// exclusive scan of one int per thread over the CTA; returns the prefix, `total` the CTA sum
__device__ int block_scan_excl(int val, int& total, int* warp_sums) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int inc = val;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();                       // warp_sums may still be read from a previous call
    if (lane == 31) warp_sums[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        int w = warp_sums[lane];
        int winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        warp_sums[lane] = winc - w;        // exclusive prefix of warp totals
        if (lane == 31) warp_sums[32] = winc;
    }
    __syncthreads();
    total = warp_sums[32];
    return warp_sums[wid] + inc - val;
}

template <typename IdT>
__device__ __forceinline__ int load_id(const void* ids, int t) {
    return (int)reinterpret_cast<const IdT*>(ids)[t];
}

// Phase A (ids known): histogram, segment table, stable placement.
template <typename IdT>
__device__ void build_from_ids(PlanView pv, const void* ids, int T, int N, int* smem, int* s_cur, int* s_perm) {
    const int tid = threadIdx.x;
    int* warp_sums = smem;              // 33 words
    int* s_bad = smem + 40;
    if (tid == 0) *s_bad = 0;
    // histogram, in shared memory when the adapter table fits (hot adapters would serialise
    // hundreds of global atomics on one address)
    int* hist = s_cur ? s_cur : pv.hist;
    for (int a = tid; a <= N; a += kPlanThreads) hist[a] = 0;
    __syncthreads();
    for (int t = tid; t < T; t += kPlanThreads) {
        int a = load_id<IdT>(ids, t);
        if (a < 0 || a >= N) *s_bad = 1;
        else atomicAdd(&hist[a], 1);
    }
    __syncthreads();
    if (*s_bad) {                        // leave an empty plan that applies nothing
        if (tid == 0) { pv.hdr->error = 1; pv.hdr->n_segs = 0; pv.hdr->n_tokens = 0; }
        return;
    }
    // exclusive scan over adapters: token offset and segment index
    int tok_carry = 0, seg_carry = 0;
    for (int base = 0; base < N; base += kPlanThreads) {
        int a = base + tid;
        int c = a < N ? hist[a] : 0;
        int tot_c, tot_s;
        int off = block_scan_excl(c, tot_c, warp_sums);
        int sidx = block_scan_excl(c > 0 ? 1 : 0, tot_s, warp_sums);
        if (a < N) {
            if (c > 0) {
                pv.seg_start[seg_carry + sidx] = tok_carry + off;
                pv.seg_adapter[seg_carry + sidx] = a;
            }
            pv.hist[a] = tok_carry + off;   // becomes the placement cursor
            if (s_cur) s_cur[a] = tok_carry + off;
        }
        tok_carry += tot_c;
        seg_carry += tot_s;
    }
    if (tid == 0) { pv.seg_start[seg_carry] = T; pv.hdr->n_segs = seg_carry; pv.hdr->n_tokens = T; }
    __syncthreads();
    // stable placement, one CTA-wide tile of tokens at a time, warps in order; the cursors live in
    // shared memory when the adapter table fits (a global read-modify-write per warp and step
    // would cost a memory round trip each)
    int* cur = s_cur ? s_cur : pv.hist;
    const int lane = tid & 31, wid = tid >> 5;
    for (int base = 0; base < T; base += kPlanThreads) {
        int t = base + tid;
        bool valid = t < T;
        int a = valid ? load_id<IdT>(ids, t) : -1 - lane;      // distinct dummies never match
        unsigned peers = __match_any_sync(0xffffffffu, a);
        int rank_in_warp = __popc(peers & ((1u << lane) - 1));
        int leader = __ffs(peers) - 1;
        int cnt = __popc(peers);
        int n_warps = min(kPlanThreads / 32, (T - base + 31) / 32);
        int slot = 0;
        for (int w = 0; w < n_warps; ++w) {
            if (wid == w && valid && lane == leader) {
                slot = cur[a];
                cur[a] = slot + cnt;
            }
            __syncthreads();
        }
        slot = __shfl_sync(0xffffffffu, slot, leader);
        if (valid) {
            pv.perm[slot + rank_in_warp] = t;
            if (s_perm) s_perm[slot + rank_in_warp] = t;
            if (slot + rank_in_warp != t) *s_bad = 2;          // some token moved: rows are not pre-grouped
        }
    }
    __syncthreads();
    if (tid == 0 && *s_bad == 0) pv.hdr->identity = 1;     // sorted already: tall runs are whole segments
    __syncthreads();
}

// Walks one adapter segment (sorted positions [b, e)) as a sequence of pieces: maximal runs of
// consecutive token rows that are long enough for the tensor-core tiles ("tall", kind 1), and the
// stretches of positions in between (kind 0).  f(kind, begin, end).
template <class F>
__device__ __forceinline__ void walk_segment(const int* perm, int b, int e, bool identity, bool tile_rank, F f) {
    int i = b, short_begin = b;
    while (i < e) {
        int j = i + 1;
        if (identity) j = e;
        else while (j < e && perm[j] == perm[j - 1] + 1) ++j;
        if (tile_rank && j - i >= kTallMin) {
            if (i > short_begin) f(0, short_begin, i);
            f(1, i, j);
            short_begin = j;
        }
        i = j;
    }
    if (e > short_begin) f(0, short_begin, e);
}

// Phase B: split segments into tall runs and short stretches, cut both into work segments of at
// most kChunkTok tokens, lay out unit records (short ones first) and the tile list.
__device__ void build_units(PlanView pv, const PlanAdapters ad, int* smem, const int* perm) {
    const int* ranks = ad.ranks;
    const long long* cum_ranks = ad.cum_ranks;
    const int r_pool = ad.r_pool;
    const int tid = threadIdx.x;
    int* warp_sums = smem;
    const int S = pv.hdr->n_segs;
    const bool identity = pv.hdr->identity != 0;
    // pass 0 totals the units of short stretches (they are listed first); pass 1 writes
    int tot_short = 0, tot_tall = 0, tot_tiles = 0, tot_ws = 0;
    for (int pass = 0; pass < 2; ++pass) {
        int c_short = 0, c_tall = 0, c_tiles = 0, c_ws = 0;
        for (int base = 0; base < S; base += kPlanThreads) {
            int s = base + tid;
            int us = 0, ut = 0, nt = 0, r = 0, nchunk = 0, b = 0, e = 0, a = 0, nsub = 0;
            bool tile_rank = false;
            if (s < S) {
                a = pv.seg_adapter[s];
                r = ranks ? ranks[a] : r_pool;
                if (ad.ranks_pow2 && !((r == 8 || r == 16 || r == 32 || r == 64) && (cum_ranks || r == r_pool)))
                    pv.hdr->error = 3;                  // the fast kernels were promised these ranks
                if (r < 1) r = 1;
                if (r > kMaxRank) r = kMaxRank;
                b = pv.seg_start[s];
                e = pv.seg_start[s + 1];
                nsub = n_sub(pad_rank(r));
                // tensor-core tiles take ranks 16/32/64 in a layout whose B rows are contiguous
                tile_rank = (r == 16 || r == 32 || r == 64) && (cum_ranks || r == r_pool);
                walk_segment(perm, b, e, identity, tile_rank, [&](int kind, int pb, int pe) {
                    const int ch = (pe - pb + kChunkTok - 1) / kChunkTok;
                    nchunk += ch;
                    if (kind) { ut += ch * nsub; nt += (pe - pb + kTileM - 1) / kTileM; }
                    else us += ch * nsub;
                });
            }
            int t0, t1, t2, t3;
            int o_s = block_scan_excl(us, t0, warp_sums);
            int o_t = block_scan_excl(ut, t1, warp_sums);
            int o_m = block_scan_excl(nt, t2, warp_sums);
            int o_w = block_scan_excl(nchunk, t3, warp_sums);
            if (pass == 1 && s < S) {
                pv.seg_rank[s] = r;
                pv.seg_flags[s] = nt > 0 ? 1 : 0;
                int u_short = c_short + o_s, u_tall = tot_short + c_tall + o_t;
                int w = c_ws + o_w, tile = c_tiles + o_m;
                // this thread lists the segment's work segments; their unit records are written
                // afterwards by all threads, one work segment each
                walk_segment(perm, b, e, identity, tile_rank, [&](int kind, int pb, int pe) {
                    const int len = pe - pb;
                    const int ch = (len + kChunkTok - 1) / kChunkTok;
                    const int per = (len + ch - 1) / ch;             // balanced chunk length
                    int& u = kind ? u_tall : u_short;
                    for (int c = 0; c < ch; ++c) {
                        pv.ws_start[w] = pb + min(c * per, len);
                        pv.ws_adapter[w] = a;
                        pv.ws_rank[w] = r | (kind << 16);
                        pv.ws_unit0[w] = u;
                        u += nsub;
                        ++w;
                    }
                    if (kind) {
                        for (int m = 0; m * kTileM < len; ++m) {
                            pv.tile_tab[2 * tile] = pb + m * kTileM;
                            pv.tile_tab[2 * tile + 1] = (s << 8) | (min(kTileM, len - m * kTileM) - 1);
                            ++tile;
                        }
                    }
                });
            }
            c_short += t0; c_tall += t1; c_tiles += t2; c_ws += t3;
        }
        tot_short = c_short; tot_tall = c_tall; tot_tiles = c_tiles; tot_ws = c_ws;
    }
    if (tid == 0) {
        pv.ws_start[tot_ws] = pv.hdr->n_tokens;
        pv.hdr->n_wsegs = tot_ws;
        pv.hdr->n_units = tot_short + tot_tall;
        pv.hdr->n_units_short = tot_short;
        pv.hdr->n_tiles = tot_tiles;
    }
    __syncthreads();
    // Where a work segment's units sit in the unit list is free (every record names its own segment).
    // Segments come out of the walk above adapter by adapter, so a popular adapter's many full
    // 8-token segments - the expensive units - would be neighbours and land in the ranges of a few
    // CTAs.  Deal the list positions out with a stride near the golden section of the segment count
    // instead (coprime with it, so every segment gets one position): any window of the list then
    // holds a fair sample of cheap and expensive units.  Short stretches keep coming first.
    if (tot_ws > 2) {
        if (tid == 0) {
            int stride = (int)(tot_ws * 0.6180339887f) | 1;
            auto gcd = [](int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; };
            while (gcd(stride, tot_ws) != 1) stride += 2;
            smem[41] = stride;
        }
        __syncthreads();
        const int stride = smem[41];
        for (int kind = 0; kind < 2; ++kind) {
            int carry = kind ? tot_short : 0;
            for (int base = 0; base < tot_ws; base += kPlanThreads) {
                const int i = base + tid;
                int w = -1, val = 0;
                if (i < tot_ws) {
                    w = (int)(((long long)i * stride) % tot_ws);
                    const int rk = pv.ws_rank[w];
                    if ((rk >> 16) == kind) val = n_sub(pad_rank(rk & 0xffff));
                    else w = -1;
                }
                int tot;
                const int off = block_scan_excl(val, tot, warp_sums);
                if (w >= 0) pv.ws_unit0[w] = carry + off;
                carry += tot;
            }
        }
        __syncthreads();
    }
    // unit records: one work segment per thread, n_sub records of four 16-byte stores each
    for (int w = tid; w < tot_ws; w += kPlanThreads) {
        const int cb = pv.ws_start[w], ce = pv.ws_start[w + 1];
        const int a = pv.ws_adapter[w], r = pv.ws_rank[w] & 0xffff;
        const int nsub = n_sub(pad_rank(r));
        const long long cum = cum_ranks ? cum_ranks[a] : 0;
        UnitRec rec;
        rec.adapter = a; rec.rank = r; rec.sub = 0; rec.ntok = (short)(ce - cb); rec.wseg = w; rec.start = cb;
        rec.scale = ad.scalings ? ad.scalings[a] : ad.scale;
        rec.cum_lo = (int)(cum & 0xffffffffll); rec.cum_hi = (int)(cum >> 32);
        for (int i = 0; i < 8; ++i) rec.tok[i] = perm[cb + min(i, ce - cb - 1)];
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<UnitRec*>(pv.unit_tab) + pv.ws_unit0[w]);
        for (int j = 0; j < nsub; ++j) {
            rec.sub = (short)j;
            const uint4* src = reinterpret_cast<const uint4*>(&rec);
#pragma unroll
            for (int q = 0; q < 4; ++q) dst[4 * j + q] = src[q];
        }
    }
}

template <typename IdT>
__global__ void __launch_bounds__(kPlanThreads, 1)
plan_build_kernel(void* plan, int cap, const void* ids, int T, const PlanAdapters ad, int n_cur, int n_perm) {
    extern __shared__ int dyn_smem[];                      // placement cursors [n_cur], then perm [n_perm]
    int* s_cur = n_cur ? dyn_smem : nullptr;
    int* s_perm = n_perm ? dyn_smem + n_cur : nullptr;
    const int N = ad.n_adapters;
    // no early launch of the successor here: the apply kernels read the plan before they wait
    // for their predecessor, which is safe only because a plan kernel has ended by then
    pdl_wait_prior();
    __shared__ int smem[64];
    PlanView pv = plan_view(plan, cap, N);
    if (threadIdx.x == 0) {
        pv.hdr->error = 0; pv.hdr->cap = cap; pv.hdr->n_adapters = N; pv.hdr->identity = 0;
        pv.hdr->n_units = 0; pv.hdr->n_tiles = 0; pv.hdr->n_units_short = 0; pv.hdr->n_segs = 0; pv.hdr->n_tokens = 0;
    }
    __syncthreads();
    build_from_ids<IdT>(pv, ids, T, N, smem, s_cur, s_perm);
    __syncthreads();
    if (pv.hdr->error) return;
    build_units(pv, ad, smem, s_perm ? s_perm : pv.perm);
}

__global__ void __launch_bounds__(kPlanThreads, 1)
plan_segments_kernel(void* plan, int cap, const int* seg_starts, const int* seg_adapter, int S, int T,
                     const PlanAdapters ad) {
    const int N = ad.n_adapters;
    // no early launch of the successor here: the apply kernels read the plan before they wait
    // for their predecessor, which is safe only because a plan kernel has ended by then
    pdl_wait_prior();
    __shared__ int smem[64];
    PlanView pv = plan_view(plan, cap, N);
    const int tid = threadIdx.x;
    if (tid == 0) {
        pv.hdr->error = 0; pv.hdr->cap = cap; pv.hdr->n_adapters = N; pv.hdr->identity = 1;
        pv.hdr->n_units = 0; pv.hdr->n_tiles = 0; pv.hdr->n_units_short = 0; pv.hdr->n_segs = 0; pv.hdr->n_tokens = 0;
        smem[40] = 0;
    }
    __syncthreads();
    // validate: offsets start at 0, end at T, strictly increase; adapters in range
    for (int s = tid; s < S; s += kPlanThreads) {
        int b = seg_starts[s], e = seg_starts[s + 1], a = seg_adapter[s];
        if (b < 0 || e <= b || e > T) smem[40] = 2;
        if (a < 0 || a >= N) smem[40] = 1;
        if (s == 0 && b != 0) smem[40] = 2;
        if (s == S - 1 && e != T) smem[40] = 2;
    }
    __syncthreads();
    if (smem[40]) { if (tid == 0) pv.hdr->error = smem[40]; return; }
    for (int s = tid; s < S; s += kPlanThreads) { pv.seg_start[s] = seg_starts[s]; pv.seg_adapter[s] = seg_adapter[s]; }
    for (int t = tid; t < T; t += kPlanThreads) pv.perm[t] = t;
    if (tid == 0) { pv.seg_start[S] = T; pv.hdr->n_segs = S; pv.hdr->n_tokens = T; }
    __syncthreads();
    build_units(pv, ad, smem, pv.perm);
}

cudaError_t launch_plan_build(void* plan, int cap, const void* ids, int ids_i64, int n_tokens,
                              const PlanAdapters& ad, cudaStream_t s) {
    // shared-memory copies of the placement cursors and of perm, when they fit
    const int n_cur = (size_t)(ad.n_adapters + 1) * 4 <= 48 * 1024 ? ad.n_adapters + 1 : 0;
    const int n_perm = (size_t)n_tokens * 4 <= 144 * 1024 ? n_tokens : 0;
    const size_t smem = (size_t)(n_cur + n_perm) * 4;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(plan_build_kernel<long long>, cudaFuncAttributeMaxDynamicSharedMemorySize, 192 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(plan_build_kernel<int>, cudaFuncAttributeMaxDynamicSharedMemorySize, 192 * 1024);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    if (ids_i64)
        plan_build_kernel<long long><<<1, kPlanThreads, smem, s>>>(plan, cap, ids, n_tokens, ad, n_cur, n_perm);
    else
        plan_build_kernel<int><<<1, kPlanThreads, smem, s>>>(plan, cap, ids, n_tokens, ad, n_cur, n_perm);
    return cudaGetLastError();
}

cudaError_t launch_plan_from_segments(void* plan, int cap, const int* seg_starts, const int* seg_adapter,
                                      int n_segs, int n_tokens, const PlanAdapters& ad, cudaStream_t s) {
    plan_segments_kernel<<<1, kPlanThreads, 0, s>>>(plan, cap, seg_starts, seg_adapter, n_segs, n_tokens, ad);
    return cudaGetLastError();
}

}  // namespace b200lora
