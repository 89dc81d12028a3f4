// Tensor-parallel exchange of the shrink result without a collective library.
//
// Every rank holds A sharded along h_in, so after its shrink half the fp32 intermediate
// v [n_proj][T][64] in its workspace is a partial sum that has to be added over the ranks before
// the expand half.  One kernel per rank does that over NVLink with plain peer stores and loads of
// LOCAL memory only, and with no flag, fence or barrier between the data and its consumer:
//   push    every rank writes its partial into slot `rank` of a landing buffer in every OTHER
//           rank's memory as 8-byte packets (value, number of this exchange): an 8-byte store
//           arrives whole, so a packet that shows the exchange's number carries its value;
//   gather  every thread then reads, from its own rank's landing buffer, the packets of the
//           elements it owns until they show this exchange's number (bounded), and adds the
//           ranks' values in rank order 0..tp-1, so that all ranks end up with bit-identical
//           sums; the result replaces v in the workspace.
// So that tens of thousands of threads do not poll while the kernels everybody waits for need the
// memory system, a CTA first sleeps on one word per peer: the peer's CTA of the same index, which
// moves the same elements, writes it after its packets.  That word is only a hint (nothing orders
// it behind the packets); the packets' own numbers decide.
// The latency of an exchange is one trip over NVLink plus the polling; nothing waits for a whole
// buffer.  The number of the exchange lives in device memory and is advanced by the kernel itself
// (its last CTA to finish), so a CUDA graph that contains the kernel stays correct when replayed.
// Two landing buffers alternate: a rank can run at most one exchange ahead of its slowest peer
// (it needs that peer's push to finish its own gather), so a buffer is never overwritten while
// its reader is still in the gather that uses it.  Numbers start at 1 and buffers at zero, and a
// number returns to a buffer only after 2^32 exchanges.  No bulk/TMA copy touches peer memory and
// nothing here uses multicast.
//
// Large exchanges over many ranks go through an owner instead (`via_owner`): every group of rows has
// one owning rank (group number modulo tp); the others send their partial to the owner alone, the
// owner adds them up in rank order and sends the sum to everybody (a landing slot of its own).  A
// rank then sends 2 (tp-1)/tp of the data instead of tp-1 times the data, for one more trip over
// NVLink; the rows of tall runs take this route from four ranks on, everything else stays direct.
//
// A tensor-parallel apply runs two such exchanges side by side, one for the rows of tall runs
// (between the two tile launches, on the side stream) and one for all other rows (between the
// BGMV halves): each takes its rows and their rank columns from the plan, and each has its own
// landing buffers and counters ("set"), because a peer may be one exchange ahead in either.
// After the TMA shrink kernel the exchange of the BGMV rows starts from that kernel's split-K
// slots: it adds them up itself (in slot order, as the expand kernel's producers do), so no
// kernel stands between the shrink half and the exchange.
#include <stdlib.h>
#include <string.h>

#include "lora_common.cuh"
#include "lora_fold.cuh"

namespace b200lora {

namespace {

constexpr int kTpMaxRanks = B200_LORA_TP_MAX_RANKS;
constexpr unsigned kTpSpinLimit = 1u << 20;          // polls of one packet pair before giving up (a second or two)
constexpr int kTpHintCtas = 160;                     // CTAs of an exchange kernel at most (one per SM)
constexpr int kTpHintBase = 64;                      // word offset of the hints inside a set's counter block
// per set: exchange counter, CTA counter, then the hint words [2 buffers][8 ranks][kTpHintCtas]
constexpr int kTpSetWords = kTpHintBase + 2 * kTpMaxRanks * kTpHintCtas;
static_assert(2 * kTpSetWords * 4 <= B200_LORA_TP_COUNTER_BYTES, "both sets' counter blocks fit the space the allocation leaves");

struct TpArgs {
    uint4* peer_landing[kTpMaxRanks][2];     // [rank][buffer]: that rank's landing buffers as mapped here (own: local)
    unsigned* peer_hints[kTpMaxRanks];       // [rank]: that rank's hint words [2][kTpMaxRanks][kTpHintCtas] of this set
    unsigned* epoch;                         // this rank's exchange counter (device)
    unsigned* done;                          // this rank's count of finished CTAs (zero at rest)
    int tp, rank;
};

TpArgs tp_args(const b200_lora_tp* tp, int set) {
    TpArgs a;
    memset(&a, 0, sizeof(a));
    for (int r = 0; r < tp->tp; ++r)
        for (int b = 0; b < 2; ++b)
            a.peer_landing[r][b] = reinterpret_cast<uint4*>(static_cast<char*>(tp->landing[r][b]) + (size_t)set * tp->set_stride);
    for (int r = 0; r < tp->tp; ++r) a.peer_hints[r] = static_cast<unsigned*>(tp->flags[r]) + set * kTpSetWords + kTpHintBase;
    a.epoch = static_cast<unsigned*>(tp->flags[tp->rank]) + set * kTpSetWords;
    a.done = a.epoch + 1;
    a.tp = tp->tp;
    a.rank = tp->rank;
    return a;
}

// two packets at once; the halves are checked separately, so it does not matter whether the 16 bytes arrive together
__device__ __forceinline__ uint4 ld_packets(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_packet(uint4* p16, int half, float value, unsigned epoch) {
    asm volatile("st.global.v2.u32 [%0], {%1, %2};" ::"l"(reinterpret_cast<char*>(p16) + 8 * half), "r"(__float_as_uint(value)), "r"(epoch)
                 : "memory");
}

// Which float4s of v an exchange moves: kind 0 every row below n_tokens, all 64 columns; kind 1
// the rows of the plan's BGMV work segments (the first `n_units` unit records) and kind 2 the
// rows of its 128-row tiles, of every row the float4s that hold its adapter's rank columns.  A
// warp takes a group of <= 8 rows at a time and calls f(index of the float4 in v) for each of its
// float4s in every projection; both passes of the kernel visit the same float4s in the same threads.
struct RowSel {
    int kind, n_groups, n_tokens, n_proj, cap;
};
template <typename F>
__device__ __forceinline__ void tp_for_rows(const PlanView& pv, const RowSel& rs, F&& f) {
    const int lane = threadIdx.x & 31;
    // The work of a thread is a chain of dependent memory round trips, so the exchange is as quick as that
    // chain is short: the warps are dealt over the projections and over the quarters of a group first (a
    // group of 8 rows of rank 64 is 128 float4s: one per lane of four warps).
    const int warp_all = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), warps_all = gridDim.x * (blockDim.x >> 5);
    const int ways = rs.n_proj * 4, sub = warp_all % ways;
    const int pj = sub >> 2, quarter = sub & 3, warp_g = warp_all / ways, n_warps = warps_all / ways;
    if (warp_g >= n_warps) return;
    // Unit records: a warp looks at 32 at once (one load round for all of them) and works through the few
    // that head a work segment.  Rows and tiles: every candidate is a group, one per warp and round.
    const int batch = rs.kind == 1 ? 32 : 1;
    for (int base = warp_g * batch; base < rs.n_groups; base += n_warps * batch) {
        const int gi = base + (batch == 1 ? 0 : lane);
        int pos = 0, rows = 0, rank = 0;
        if (gi < rs.n_groups && (batch == 32 || lane == 0)) {
            if (rs.kind == 0) {
                pos = gi * 8;
                rows = min(8, rs.n_tokens - pos);
                rank = kMaxRank;
            } else if (rs.kind == 2) {
                const int tile = gi >> 4, e1 = pv.tile_tab[2 * tile + 1];
                pos = pv.tile_tab[2 * tile] + (gi & 15) * 8;
                rows = min(8, (e1 & 255) + 1 - (gi & 15) * 8);
                rank = pv.seg_rank[e1 >> 8];
            } else {
                const int* rec = pv.unit_tab + (size_t)gi * 16;
                const int w2 = rec[2];
                if ((w2 & 0xffff) == 0) {                     // the records of a work segment differ in the sub-range only
                    pos = rec[5];
                    rows = (w2 >> 16) & 0xffff;
                    rank = rec[1];
                }
            }
        }
        unsigned live = __ballot_sync(0xffffffffu, rows > 0);
        while (live) {
            const int src = __ffs(live) - 1;
            live &= live - 1;
            const int g_pos = __shfl_sync(0xffffffffu, pos, src), g_rows = __shfl_sync(0xffffffffu, rows, src);
            const int q = (__shfl_sync(0xffffffffu, rank, src) + 3) >> 2, n = g_rows * q;
            const int g_unit = base + src, g_rank = __shfl_sync(0xffffffffu, rank, src);
            for (int idx = quarter * 32 + lane; idx < n; idx += 128) {
                const int r = idx / q;
                f(((size_t)pj * rs.cap + g_pos + r) * (kMaxRank / 4) + (idx - r * q), pj, g_unit, g_rank);
            }
        }
    }
}

// `p`: of an apply, what the exchange needs (plan, workspace, sizes; for the fold also the projections'
// widths and the flags).  `fold_grid` > 0: v of the BGMV rows is still the split-K slots of a TMA shrink
// kernel of that many CTAs.
template <typename T>
__global__ void __launch_bounds__(256) tp_exchange_kernel(const TpArgs a, const __grid_constant__ ApplyParams p, int kind,
                                                          int all_units, int fold_grid, int skip_push, int via_owner) {
    pdl_wait_prior();                        // the shrink half's result is complete
    if (threadIdx.x == 0) pdl_launch_dependents();
    const int cap = p.cap, n_tokens = p.n_tokens, n_proj = p.n_proj;
    WorkspaceView ws = workspace_view(p.workspace, p.cap, p.n_proj);
    float* v = ws.v;
    unsigned* err = &ws.ctl->error;
    const unsigned epoch = *reinterpret_cast<volatile unsigned*>(a.epoch) + 1u;     // advanced after every CTA has read it
    const int buf = (int)(epoch & 1u);
    RowSel rs;
    rs.kind = kind; rs.n_tokens = n_tokens; rs.n_proj = n_proj; rs.cap = cap;
    rs.n_groups = (n_tokens + 7) / 8;
    PlanView pv;
    memset(&pv, 0, sizeof(pv));
    if (kind != 0) {
        pv = plan_view(p.plan, cap, p.n_adapters);
        const PlanHeader hdr = *pv.hdr;
        // an unusable plan moves nothing; the exchange counters stay in step all the same
        const bool usable = hdr.error == 0 && hdr.cap == cap && hdr.n_tokens == n_tokens;
        rs.n_groups = !usable ? 0 : kind == 2 ? hdr.n_tiles * (kTileM / 8) : all_units ? hdr.n_units : hdr.n_units_short;
    }
    const size_t slot_f4 = (size_t)n_proj * cap * (kMaxRank / 4);       // float4s of v = packet quads of one landing slot
    float4* v4 = reinterpret_cast<float4*>(v);

    // ---- push: four packets per float4 into slot `rank` of every peer ----
    const int fold_per_cta = fold_grid > 0 ? (rs.n_groups * p.total_super_in + fold_grid - 1) / fold_grid : 0;
    if (!skip_push || fold_grid > 0)
        tp_for_rows(pv, rs, [&](size_t idx, int pj, int unit, int rank) {
            float4 val;
            if (fold_grid > 0) {                                          // this rank's own sum first
                const size_t offs[1] = {idx * 4};
                const bool on[1] = {true};
                float4 sum[1];
                fold_quads<T, 1>(p, ws, offs, on, shrink_seg_first(p, rs.n_groups, pj, unit), fold_per_cta,
                                 shrink_chunks(p, pj, rank), sum);
                val = sum[0];
                v4[idx] = val;
            } else val = v4[idx];
            if (skip_push) return;
            const int owner = via_owner ? unit % a.tp : -1;
            for (int s = 0; s < a.tp; ++s) {
                if (s == a.rank || (via_owner && s != owner)) continue;
                uint4* dst = a.peer_landing[s][buf] + ((size_t)a.rank * slot_f4 + idx) * 2;
                st_packet(dst, 0, val.x, epoch);
                st_packet(dst, 1, val.y, epoch);
                st_packet(dst + 1, 0, val.z, epoch);
                st_packet(dst + 1, 1, val.w, epoch);
            }
        });
    // ---- the hint: this CTA's packets are on their way / the peers' CTAs of this index have sent theirs ----
    __syncthreads();
    if (!skip_push && threadIdx.x < a.tp && (int)threadIdx.x != a.rank)
        *reinterpret_cast<volatile unsigned*>(a.peer_hints[threadIdx.x] + (buf * kTpMaxRanks + a.rank) * kTpHintCtas + blockIdx.x) = epoch;
    if (threadIdx.x < a.tp && (int)threadIdx.x != a.rank) {
        const volatile unsigned* hint = a.peer_hints[a.rank] + (buf * kTpMaxRanks + threadIdx.x) * kTpHintCtas + blockIdx.x;
        for (unsigned i = 0; i < kTpSpinLimit && (int)(*hint - epoch) < 0; ++i) {
            if ((i & 0xffu) == 0xffu && *reinterpret_cast<volatile unsigned*>(err) != 0u) break;
            __nanosleep(i < 8 ? 100 : 400);
        }
    }
    __syncthreads();
    // ---- gather: read the own landing buffer until the packets are this exchange's, add in rank order ----
    bool gave_up = false;
    // one float4 = two packet pairs at `src`; polls until all four packets are this exchange's
    auto wait4 = [&](const uint4* src, uint4 p0, uint4 p1, unsigned nap) {
        for (unsigned i = 0; !gave_up && (p0.y != epoch || p0.w != epoch || p1.y != epoch || p1.w != epoch); ++i) {
            if (i >= kTpSpinLimit || ((i & 0xffu) == 0xffu && *reinterpret_cast<volatile unsigned*>(err) != 0u)) {
                gave_up = true;                                           // this thread stops waiting for anything
                break;
            }
            if (i > 16 || nap > 64) __nanosleep(nap);
            p0 = ld_packets(src);
            p1 = ld_packets(src + 1);
        }
        return make_float4(__uint_as_float(p0.x), __uint_as_float(p0.z), __uint_as_float(p1.x), __uint_as_float(p1.z));
    };
    tp_for_rows(pv, rs, [&](size_t idx, int, int unit, int) {
        if (via_owner && unit % a.tp != a.rank) return;                   // somebody else adds this group up
        const float4 own = v4[idx];
        const uint4* mine = a.peer_landing[a.rank][buf] + idx * 2;
        uint4 pk[kTpMaxRanks][2];                                         // every peer's packets requested before any is looked at
#pragma unroll
        for (int s = 0; s < kTpMaxRanks; ++s)
            if (s < a.tp && s != a.rank) {
                pk[s][0] = ld_packets(mine + (size_t)s * slot_f4 * 2);
                pk[s][1] = ld_packets(mine + (size_t)s * slot_f4 * 2 + 1);
            }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < kTpMaxRanks; ++s) {                           // rank order: the same sum on every rank
            if (s >= a.tp) continue;
            float4 x = own;
            if (s != a.rank) x = wait4(mine + (size_t)s * slot_f4 * 2, pk[s][0], pk[s][1], 64);
            acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
        }
        v4[idx] = acc;
        if (via_owner && !skip_push)                                      // the sum goes out to everybody's slot number tp
            for (int s = 0; s < a.tp; ++s) {
                if (s == a.rank) continue;
                uint4* dst = a.peer_landing[s][buf] + ((size_t)a.tp * slot_f4 + idx) * 2;
                st_packet(dst, 0, acc.x, epoch);
                st_packet(dst, 1, acc.y, epoch);
                st_packet(dst + 1, 0, acc.z, epoch);
                st_packet(dst + 1, 1, acc.w, epoch);
            }
    });
    if (via_owner)                                                        // the groups other ranks own: their sums
        tp_for_rows(pv, rs, [&](size_t idx, int, int unit, int) {
            if (unit % a.tp == a.rank) return;
            const uint4* src = a.peer_landing[a.rank][buf] + ((size_t)a.tp * slot_f4 + idx) * 2;
            v4[idx] = wait4(src, ld_packets(src), ld_packets(src + 1), 200);
        });
    if (gave_up) atomicMax(err, 8u);
    // ---- the last CTA to get here advances the exchange counter ----
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned before = atomicAdd(a.done, 1u);
        if (before == gridDim.x - 1) {
            *reinterpret_cast<volatile unsigned*>(a.done) = 0u;
            *reinterpret_cast<volatile unsigned*>(a.epoch) = epoch;
        }
    }
}

int exchange_grid(int n_tokens, int n_proj, int n_sm) {
    // a warp per (group of <= 8 rows, projection) where the batch allows it: the work of a thread is a
    // chain of dependent memory round trips, so the exchange is as quick as that chain is short
    long long grid = ((long long)(n_tokens + 7) / 8 * n_proj * 4 + 7) / 8;
    if (grid > n_sm) grid = n_sm;
    if (grid > kTpHintCtas) grid = kTpHintCtas;
    return grid < 8 ? 8 : (int)grid;
}

}  // namespace

template <typename... Args>
cudaError_t launch_exchange(int io_dtype, int grid, cudaStream_t s, Args&&... args) {
    if (io_dtype == B200_LORA_F16) return launch_pdl(tp_exchange_kernel<__half>, dim3(grid), dim3(256), 0, s, std::forward<Args>(args)...);
    return launch_pdl(tp_exchange_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, std::forward<Args>(args)...);
}

cudaError_t launch_tp_exchange_rows(const b200_lora_tp* tp, int set, bool tall, bool all_units, const ApplyParams& p, int fold_grid,
                                    int io_dtype, int skip_push, int n_sm, cudaStream_t s) {
    const TpArgs a = tp_args(tp, set);
    // B200_LORA_TP_VIA_OWNER=0/1 in the environment overrides the route (for tests on two GPUs)
    static const int forced = [] { const char* v = getenv("B200_LORA_TP_VIA_OWNER"); return v ? (v[0] == '1' ? 1 : 0) : -1; }();
    const int via_owner = forced >= 0 ? forced : (tall && tp->tp >= 4) ? 1 : 0;
    return launch_exchange(io_dtype, exchange_grid(p.n_tokens, p.n_proj, n_sm), s, a, p, tall ? 2 : 1, all_units ? 1 : 0,
                           tall ? 0 : fold_grid, skip_push, via_owner);
}

cudaError_t launch_tp_exchange(const b200_lora_tp* tp, void* workspace, int n_proj, int cap, int n_tokens, int skip_push,
                               int n_sm, cudaStream_t s) {
    const TpArgs a = tp_args(tp, 0);
    ApplyParams p;
    memset(&p, 0, sizeof(p));
    p.n_proj = n_proj;
    p.cap = cap;
    p.n_tokens = n_tokens;
    p.workspace = workspace;
    return launch_exchange(B200_LORA_BF16, exchange_grid(n_tokens, n_proj, n_sm), s, a, p, 0, 0, 0, skip_push, 0);
}

}  // namespace b200lora
