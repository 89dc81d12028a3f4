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

// Working copies of the tables the build reads back (segments, work segments): shared memory when
// the batch is small enough, the plan's own global arrays otherwise.  A decode batch's plan is a
// chain of dependent steps on one CTA; with the tables on chip each step costs a barrier instead
// of a round trip to L2.
struct Scratch {
    int* seg_start;     // [S + 1]
    int* seg_adapter;   // [S]
    int* seg_rank;      // [S]
    int* ws_start;      // [W + 1]
    int* ws_adapter;    // [W]
    int* ws_rank;       // [W]   rank | kind << 16
    int* ws_unit0;      // [W]
    bool on_chip;
};

template <typename IdT>
__device__ __forceinline__ int load_id(const void* ids, int t) {
    return (int)reinterpret_cast<const IdT*>(ids)[t];
}

// Phase A (ids known): histogram, segment table, stable placement.
template <typename IdT>
__device__ void build_from_ids(PlanView pv, const Scratch& sc, const void* ids, int T, int N, int* smem, int* s_cur, int* s_perm) {
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
                if (sc.on_chip) { sc.seg_start[seg_carry + sidx] = tok_carry + off; sc.seg_adapter[seg_carry + sidx] = a; }
            }
            pv.hist[a] = tok_carry + off;   // becomes the placement cursor
            if (s_cur) s_cur[a] = tok_carry + off;
        }
        tok_carry += tot_c;
        seg_carry += tot_s;
    }
    if (tid == 0) {
        pv.seg_start[seg_carry] = T; pv.hdr->n_segs = seg_carry; pv.hdr->n_tokens = T;
        if (sc.on_chip) sc.seg_start[seg_carry] = T;
        smem[42] = seg_carry;
    }
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
    if (tid == 0) {
        const int ident = *s_bad == 0 ? 1 : 0;             // sorted already: tall runs are whole segments
        if (ident) pv.hdr->identity = 1;
        smem[43] = ident;
    }
    __syncthreads();
}

// ---- block-wide scans over an array of n ints (shared or global), in place ----------------------
// inclusive maximum, front to back
__device__ void scan_max_forward(int* arr, int n, int* warp_sums) {
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    int carry = -1;
    for (int base = 0; base < n; base += kPlanThreads) {
        const int i = base + tid;
        int v = i < n ? arr[i] : -1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v = max(v, t); }
        __syncthreads();
        if (lane == 31) warp_sums[wid] = v;
        __syncthreads();
        if (wid == 0) {
            int w = warp_sums[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, w, o); if (lane >= o) w = max(w, t); }
            warp_sums[lane] = w;                            // inclusive maximum over the warps so far
        }
        __syncthreads();
        v = max(v, carry);
        if (wid > 0) v = max(v, warp_sums[wid - 1]);
        if (i < n) arr[i] = v;
        carry = max(carry, warp_sums[31]);
    }
    __syncthreads();
}
// inclusive minimum, back to front
__device__ void scan_min_backward(int* arr, int n, int* warp_sums) {
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int kInf = 0x7fffffff;
    int carry = kInf;
    const int rounds = (n + kPlanThreads - 1) / kPlanThreads;
    for (int rd = rounds - 1; rd >= 0; --rd) {
        const int i = rd * kPlanThreads + (kPlanThreads - 1 - tid);     // thread 0 takes the round's last element
        int v = i < n ? arr[i] : kInf;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v = min(v, t); }
        __syncthreads();
        if (lane == 31) warp_sums[wid] = v;
        __syncthreads();
        if (wid == 0) {
            int w = warp_sums[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, w, o); if (lane >= o) w = min(w, t); }
            warp_sums[lane] = w;
        }
        __syncthreads();
        v = min(v, carry);
        if (wid > 0) v = min(v, warp_sums[wid - 1]);
        if (i < n) arr[i] = v;
        carry = min(carry, warp_sums[31]);
    }
    __syncthreads();
}

// Phase B: cut every segment into pieces - maximal runs of consecutive token rows that are long
// enough for the tensor-core tiles ("tall", kind 1) and the stretches in between (kind 0) - and the
// pieces into work segments of at most kChunkTok tokens; list the 128-row tiles of the tall pieces;
// place the work segments' units in the unit list; write the unit records.
//
// Everything is computed per sorted position with block-wide scans (a thread per position), so the
// time does not depend on how long a segment or a run is:
//   seg(i)    segment of position i                     max-scan of the segment starts
//   R(i)      start of the run that holds i             max-scan of the run heads (row not the previous row + 1)
//   N(i)      start of the next run (or segment)        min-scan, back to front
//   tall(i)   N - R >= kTallMin and the rank has tiles
//   piece heads: segment heads, heads of tall runs, heads of runs that follow a tall run
//   PS(i), PE(i) piece bounds, by the same two scans; the piece's work segments and tiles start at
//   fixed offsets from PS.
// t0..t3: four int arrays of T entries (shared memory, or the unit table's room, which is written last).
__device__ void build_units(PlanView pv, const Scratch& sc, const PlanAdapters ad, int* smem, const int* perm, int S,
                            int T, int* t0, int* t1, int* t2, int* t3) {
    const int* ranks = ad.ranks;
    const long long* cum_ranks = ad.cum_ranks;
    const int r_pool = ad.r_pool;
    const int tid = threadIdx.x;
    int* warp_sums = smem;
    const int kInf = 0x7fffffff;
    // segments: rank (checked against the promise made to the fast kernels), start marks
    for (int i = tid; i < T; i += kPlanThreads) t0[i] = -1;
    __syncthreads();
    for (int s = tid; s < S; s += kPlanThreads) {
        const int a = sc.seg_adapter[s];
        int r = ranks ? ranks[a] : r_pool;
        if (ad.ranks_pow2 && !((r == 8 || r == 16 || r == 32 || r == 64) && (cum_ranks || r == r_pool)))
            pv.hdr->error = 3;                          // the fast kernels were promised these ranks
        r = min(max(r, 1), kMaxRank);
        pv.seg_rank[s] = r;
        pv.seg_flags[s] = 0;
        sc.seg_rank[s] = r;
        t0[sc.seg_start[s]] = s;
    }
    __syncthreads();
    scan_max_forward(t0, T, warp_sums);                 // t0 = seg(i)
    // run heads
    for (int i = tid; i < T; i += kPlanThreads) {
        const bool head = i == sc.seg_start[t0[i]] || perm[i] != perm[i - 1] + 1;
        t1[i] = head ? i : -1;
        t2[i] = head ? i : kInf;
    }
    __syncthreads();
    scan_max_forward(t1, T, warp_sums);                 // t1 = R(i)
    scan_min_backward(t2, T, warp_sums);                // t2 = first run head >= i
    // tall runs and piece heads; t3 = head flag | tall << 1
    auto tall_at = [&](int i) {
        const int r = sc.seg_rank[t0[i]];
        // tensor-core tiles take ranks 16/32/64 in a layout whose B rows are contiguous
        const bool tile_rank = (r == 16 || r == 32 || r == 64) && (cum_ranks || r == r_pool);
        const int next = i + 1 < T ? min(t2[i + 1], T) : T;         // no further head: the run ends with the batch
        return tile_rank && next - t1[i] >= kTallMin;
    };
    for (int i = tid; i < T; i += kPlanThreads) {
        const bool seg_head = i == sc.seg_start[t0[i]];
        const bool tall = tall_at(i);
        const bool head = seg_head || (t1[i] == i && (tall || tall_at(i - 1)));
        t3[i] = (head ? 1 : 0) | (tall ? 2 : 0);
    }
    __syncthreads();
    for (int i = tid; i < T; i += kPlanThreads) {
        const bool head = (t3[i] & 1) != 0;
        t1[i] = head ? i : -1;
        t2[i] = head ? i : kInf;
    }
    __syncthreads();
    scan_max_forward(t1, T, warp_sums);                 // t1 = PS(i)
    scan_min_backward(t2, T, warp_sums);                // t2 = first piece head >= i
    // work segments and tiles: heads at fixed offsets inside a piece, numbered in position order
    int ws_carry = 0, tile_carry = 0;
    for (int base = 0; base < T; base += kPlanThreads) {
        const int i = base + tid;
        int wh = 0, th = 0, s = 0, kind = 0, pe = 0;
        if (i < T) {
            const int pb = t1[i];
            pe = i + 1 < T ? min(t2[i + 1], T) : T;
            const int len = pe - pb, k = i - pb;
            const int ch = (len + kChunkTok - 1) / kChunkTok;
            const int per = (len + ch - 1) / ch;            // balanced chunk length
            s = t0[i];
            kind = (t3[i] >> 1) & 1;
            wh = (k % per) == 0 ? 1 : 0;
            th = (kind && (k % kTileM) == 0) ? 1 : 0;
        }
        int tot_w, tot_t;
        const int w = ws_carry + block_scan_excl(wh, tot_w, warp_sums);
        const int tile = tile_carry + block_scan_excl(th, tot_t, warp_sums);
        if (wh) {
            sc.ws_start[w] = i;
            sc.ws_adapter[w] = sc.seg_adapter[s];
            sc.ws_rank[w] = sc.seg_rank[s] | (kind << 16);
        }
        if (th) {
            pv.tile_tab[2 * tile] = i;
            pv.tile_tab[2 * tile + 1] = (s << 8) | (min(kTileM, pe - i) - 1);
            pv.seg_flags[s] = 1;
        }
        ws_carry += tot_w;
        tile_carry += tot_t;
    }
    const int tot_ws = ws_carry, tot_tiles = tile_carry;
    if (tid == 0) sc.ws_start[tot_ws] = T;
    __syncthreads();
    // Where a work segment's units sit in the unit list is free (every record names its own segment),
    // except that short stretches come first.  Segments come adapter by adapter, so a popular
    // adapter's many full 8-token segments - the expensive units - would be neighbours and land in
    // the ranges of a few CTAs.  Deal the list positions out with a stride near the golden section of
    // the segment count instead (coprime with it, so every segment gets one position): any window of
    // the list then holds a fair sample of cheap and expensive units.
    if (tid == 0) {
        int stride = 1;
        if (tot_ws > 2) {
            stride = (int)(tot_ws * 0.6180339887f) | 1;
            auto gcd = [](int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; };
            while (gcd(stride, tot_ws) != 1) stride += 2;
        }
        smem[41] = stride;
    }
    __syncthreads();
    const int stride = smem[41];
    int tot_short = 0, tot_tall = 0;
    for (int kind = 0; kind < (tot_tiles > 0 ? 2 : 1); ++kind) {
        int carry = kind ? tot_short : 0;
        for (int base = 0; base < tot_ws; base += kPlanThreads) {
            const int i = base + tid;
            int w = -1, val = 0;
            if (i < tot_ws) {
                w = (int)(((long long)i * stride) % tot_ws);
                const int rk = sc.ws_rank[w];
                if ((rk >> 16) == kind) val = n_sub(pad_rank(rk & 0xffff));
                else w = -1;
            }
            int tot;
            const int off = block_scan_excl(val, tot, warp_sums);
            if (w >= 0) sc.ws_unit0[w] = carry + off;
            carry += tot;
        }
        if (kind) tot_tall = carry - tot_short;
        else tot_short = carry;
    }
    if (tid == 0) {
        pv.hdr->n_wsegs = tot_ws;
        pv.hdr->n_units = tot_short + tot_tall;
        pv.hdr->n_units_short = tot_short;
        pv.hdr->n_tiles = tot_tiles;
    }
    __syncthreads();
    // unit records: one work segment per thread, n_sub records of four 16-byte stores each
    for (int w = tid; w < tot_ws; w += kPlanThreads) {
        const int cb = sc.ws_start[w], ce = sc.ws_start[w + 1];
        const int a = sc.ws_adapter[w], r = sc.ws_rank[w] & 0xffff;
        const int nsub = n_sub(pad_rank(r));
        const long long cum = cum_ranks ? cum_ranks[a] : 0;
        UnitRec rec;
        rec.adapter = a; rec.rank = r; rec.sub = 0; rec.ntok = (short)(ce - cb); rec.wseg = w; rec.start = cb;
        rec.scale = ad.scalings ? ad.scalings[a] : ad.scale;
        rec.cum_lo = (int)(cum & 0xffffffffll); rec.cum_hi = (int)(cum >> 32);
        for (int i = 0; i < 8; ++i) rec.tok[i] = perm[cb + min(i, ce - cb - 1)];
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<UnitRec*>(pv.unit_tab) + sc.ws_unit0[w]);
        for (int j = 0; j < nsub; ++j) {
            rec.sub = (short)j;
            const uint4* src = reinterpret_cast<const uint4*>(&rec);
#pragma unroll
            for (int q = 0; q < 4; ++q) dst[4 * j + q] = src[q];
        }
    }
}

// Working tables in dynamic shared memory after `used` ints, when they fit; else the plan's own arrays.
__device__ __forceinline__ Scratch make_scratch(PlanView pv, int* dyn, int used, int n_ws_cap, int n_seg_cap, bool fits) {
    Scratch sc;
    sc.on_chip = fits;
    if (fits) {
        int* w = dyn + used;
        sc.seg_start = w;   w += n_seg_cap + 1;
        sc.seg_adapter = w; w += n_seg_cap;
        sc.seg_rank = w;    w += n_seg_cap;
        sc.ws_start = w;    w += n_ws_cap + 1;
        sc.ws_adapter = w;  w += n_ws_cap;
        sc.ws_rank = w;     w += n_ws_cap;
        sc.ws_unit0 = w;
    } else {
        sc.seg_start = pv.seg_start; sc.seg_adapter = pv.seg_adapter; sc.seg_rank = pv.seg_rank;
        sc.ws_start = pv.ws_start; sc.ws_adapter = pv.ws_adapter; sc.ws_rank = pv.ws_rank; sc.ws_unit0 = pv.ws_unit0;
    }
    return sc;
}
// ints of the working tables plus the four per-position temporaries of build_units
__host__ __device__ inline size_t scratch_ints(int n_ws_cap, int n_seg_cap) { return 3 * (size_t)n_seg_cap + 1 + 8 * (size_t)n_ws_cap + 1; }
// the four temporaries: behind the working tables on chip, else in the room of the unit table (written last)
// (mode 1: everything on chip; 2: only the temporaries, at `dyn`; 0: nothing)
__device__ __forceinline__ void temporaries(PlanView pv, const Scratch& sc, int* dyn, int mode, int T, int*& t0, int*& t1, int*& t2, int*& t3) {
    int* base = mode == 1 ? sc.ws_unit0 + T : mode == 2 ? dyn : pv.unit_tab;
    t0 = base; t1 = base + T; t2 = base + 2 * (size_t)T; t3 = base + 3 * (size_t)T;
}

template <typename IdT>
__global__ void __launch_bounds__(kPlanThreads, 1)
plan_build_kernel(void* plan, int cap, const void* ids, int T, const PlanAdapters ad, int n_cur, int n_perm, int n_scr) {
    extern __shared__ int dyn_smem[];                      // placement cursors [n_cur], perm [n_perm], working tables
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
    const Scratch sc = make_scratch(pv, dyn_smem, n_cur + n_perm, T, min(T, N), n_scr == 1);
    __syncthreads();
    build_from_ids<IdT>(pv, sc, ids, T, N, smem, s_cur, s_perm);
    __syncthreads();
    if (pv.hdr->error) return;
    int *t0, *t1, *t2, *t3;
    temporaries(pv, sc, dyn_smem + n_cur + n_perm, n_scr, T, t0, t1, t2, t3);
    build_units(pv, sc, ad, smem, s_perm ? s_perm : pv.perm, smem[42], T, t0, t1, t2, t3);
}

__global__ void __launch_bounds__(kPlanThreads, 1)
plan_segments_kernel(void* plan, int cap, const int* seg_starts, const int* seg_adapter, int S, int T,
                     const PlanAdapters ad, int n_scr) {
    extern __shared__ int dyn_smem[];                      // working tables, when they fit
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
    const Scratch sc = make_scratch(pv, dyn_smem, 0, T, S, n_scr == 1);
    for (int s = tid; s < S; s += kPlanThreads) {
        const int b = seg_starts[s], a = seg_adapter[s];
        pv.seg_start[s] = b; pv.seg_adapter[s] = a;
        if (sc.on_chip) { sc.seg_start[s] = b; sc.seg_adapter[s] = a; }
    }
    for (int t = tid; t < T; t += kPlanThreads) pv.perm[t] = t;
    if (tid == 0) {
        pv.seg_start[S] = T; pv.hdr->n_segs = S; pv.hdr->n_tokens = T;
        if (sc.on_chip) sc.seg_start[S] = T;
    }
    __syncthreads();
    int *t0, *t1, *t2, *t3;
    temporaries(pv, sc, dyn_smem, n_scr, T, t0, t1, t2, t3);
    build_units(pv, sc, ad, smem, pv.perm, S, T, t0, t1, t2, t3);
}

cudaError_t launch_plan_build(void* plan, int cap, const void* ids, int ids_i64, int n_tokens,
                              const PlanAdapters& ad, cudaStream_t s) {
    // shared-memory copies of the placement cursors and of perm, when they fit
    const int n_cur = (size_t)(ad.n_adapters + 1) * 4 <= 48 * 1024 ? ad.n_adapters + 1 : 0;
    const int n_perm = (size_t)n_tokens * 4 <= 144 * 1024 ? n_tokens : 0;
    // the working tables and the per-position temporaries too when everything fits, else the temporaries alone
    size_t scr = scratch_ints(n_tokens, n_tokens < ad.n_adapters ? n_tokens : ad.n_adapters);
    int n_scr = 1;
    if (!n_perm || (size_t)(n_cur + n_perm + scr) * 4 > 200 * 1024) {
        scr = 4 * (size_t)n_tokens;
        n_scr = (size_t)(n_cur + n_perm + scr) * 4 <= 200 * 1024 ? 2 : 0;
    }
    const size_t smem = (size_t)(n_cur + n_perm + (n_scr ? scr : 0)) * 4;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(plan_build_kernel<long long>, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(plan_build_kernel<int>, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    if (ids_i64)
        plan_build_kernel<long long><<<1, kPlanThreads, smem, s>>>(plan, cap, ids, n_tokens, ad, n_cur, n_perm, n_scr);
    else
        plan_build_kernel<int><<<1, kPlanThreads, smem, s>>>(plan, cap, ids, n_tokens, ad, n_cur, n_perm, n_scr);
    return cudaGetLastError();
}

cudaError_t launch_plan_from_segments(void* plan, int cap, const int* seg_starts, const int* seg_adapter,
                                      int n_segs, int n_tokens, const PlanAdapters& ad, cudaStream_t s) {
    size_t scr = scratch_ints(n_tokens, n_segs);
    int n_scr = 1;
    if (scr * 4 > 200 * 1024) {
        scr = 4 * (size_t)n_tokens;
        n_scr = scr * 4 <= 200 * 1024 ? 2 : 0;
    }
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(plan_segments_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    plan_segments_kernel<<<1, kPlanThreads, n_scr ? scr * 4 : 0, s>>>(plan, cap, seg_starts, seg_adapter, n_segs, n_tokens, ad, n_scr);
    return cudaGetLastError();
}

}  // namespace b200lora
