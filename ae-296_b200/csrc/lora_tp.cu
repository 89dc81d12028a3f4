// Tensor-parallel exchange of the shrink result without a collective library.
//
// Every rank holds A sharded along h_in, so after its shrink half the fp32 intermediate
// v [n_proj][T][64] in its workspace is a partial sum that has to be added over the ranks before
// the expand half.  One kernel per rank does that over NVLink with plain peer stores and loads of
// LOCAL memory only:
//   push    every rank writes its partial into slot `rank` of a landing buffer in every OTHER
//           rank's memory (st.global to the peer mapping), fences at system scope, and its last
//           CTA raises this rank's arrival word in every peer's memory;
//   gather  every CTA then waits (bounded) until the arrival words of all peers show this
//           exchange, and adds the landing slots to its own partial in rank order 0..tp-1, so that
//           all ranks end up with bit-identical sums; the result replaces v in the workspace.
// The number of the exchange lives in device memory and is advanced by the kernel itself, so a CUDA
// graph that contains the kernel stays correct when replayed.  Two landing buffers alternate: a
// rank can run at most one exchange ahead of its slowest peer (it needs that peer's push to finish
// its own gather), so a buffer is never overwritten while its reader is still in the gather that
// uses it.  No bulk/TMA copy touches peer memory and nothing here uses multicast.
#include <string.h>

#include "lora_common.cuh"

namespace b200lora {

namespace {

constexpr int kTpMaxRanks = B200_LORA_TP_MAX_RANKS;
constexpr unsigned kTpSpinLimit = 1u << 20;          // polls of an arrival word before giving up (a second or two)

struct TpArgs {
    float* peer_landing[kTpMaxRanks][2];     // [rank][buffer]: that rank's landing buffers as mapped here (own: local)
    unsigned* peer_flags[kTpMaxRanks];       // that rank's arrival words [2][kTpMaxRanks]
    unsigned* epoch;                         // this rank's exchange counter (device)
    unsigned* done;                          // this rank's CTA counter of the push phase (zero at rest)
    int tp, rank;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(256) tp_exchange_kernel(const TpArgs a, float* v, int n_proj, int cap, int n_tokens,
                                                          unsigned* err, int skip_push) {
    pdl_wait_prior();                        // the shrink half's result is complete
    pdl_launch_dependents();
    __shared__ unsigned s_epoch;
    if (threadIdx.x == 0) s_epoch = *reinterpret_cast<volatile unsigned*>(a.epoch) + 1u;
    __syncthreads();
    const unsigned epoch = s_epoch;
    const int buf = (int)(epoch & 1u);
    // items: float4 number c4 of row t of projection p, rows below n_tokens only
    const size_t per_proj = (size_t)n_tokens * 16;
    const size_t n_items = per_proj * n_proj;
    const size_t slot_f4 = (size_t)n_proj * cap * 16;                    // float4s of one landing slot
    const size_t chunk = (n_items + gridDim.x - 1) / gridDim.x;
    const size_t lo = blockIdx.x * chunk, hi = lo + chunk < n_items ? lo + chunk : n_items;
    float4* v4 = reinterpret_cast<float4*>(v);
    auto index_of = [&](size_t it) { const size_t p = it / per_proj, r = it - p * per_proj; return p * (size_t)cap * 16 + r; };

    // ---- push ----
    for (size_t it = lo + threadIdx.x; it < hi; it += blockDim.x) {
        const size_t idx = index_of(it);
        const float4 val = v4[idx];
        for (int s = 0; s < a.tp; ++s)
            if (s != a.rank) reinterpret_cast<float4*>(a.peer_landing[s][buf])[(size_t)a.rank * slot_f4 + idx] = val;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned before = atomicAdd(a.done, 1u);
        if (before == gridDim.x - 1) {                                    // every CTA's stores are out
            __threadfence_system();
            if (!skip_push)
                for (int s = 0; s < a.tp; ++s)
                    if (s != a.rank) st_release_sys(a.peer_flags[s] + buf * kTpMaxRanks + a.rank, epoch);
            *reinterpret_cast<volatile unsigned*>(a.done) = 0u;
            *reinterpret_cast<volatile unsigned*>(a.epoch) = epoch;
        }
    }
    // ---- gather ----
    if (threadIdx.x < a.tp && (int)threadIdx.x != a.rank) {
        const unsigned* flag = a.peer_flags[a.rank] + buf * kTpMaxRanks + threadIdx.x;
        bool ok = false;
        for (unsigned i = 0; i < kTpSpinLimit; ++i) {
            if ((int)(ld_acquire_sys(flag) - epoch) >= 0) { ok = true; break; }
            if ((i & 0xffu) == 0xffu && *reinterpret_cast<volatile unsigned*>(err) != 0u) break;
            __nanosleep(100);
        }
        if (!ok) atomicMax(err, 8u);
    }
    __syncthreads();
    for (size_t it = lo + threadIdx.x; it < hi; it += blockDim.x) {
        const size_t idx = index_of(it);
        const float4 own = v4[idx];
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < a.tp; ++s) {                                  // rank order: the same sum on every rank
            const float4 x = s == a.rank ? own
                                         : __ldcg(reinterpret_cast<const float4*>(a.peer_landing[a.rank][buf]) + (size_t)s * slot_f4 + idx);
            acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
        }
        v4[idx] = acc;
    }
}

}  // namespace

cudaError_t launch_tp_exchange(const b200_lora_tp* tp, float* v, int n_proj, int cap, int n_tokens, unsigned* err,
                               int skip_push, int n_sm, cudaStream_t s) {
    TpArgs a;
    memset(&a, 0, sizeof(a));
    for (int r = 0; r < tp->tp; ++r) {
        a.peer_landing[r][0] = static_cast<float*>(tp->landing[r][0]);
        a.peer_landing[r][1] = static_cast<float*>(tp->landing[r][1]);
        a.peer_flags[r] = static_cast<unsigned*>(tp->flags[r]);
    }
    a.epoch = static_cast<unsigned*>(tp->flags[tp->rank]) + 2 * kTpMaxRanks;
    a.done = a.epoch + 1;
    a.tp = tp->tp;
    a.rank = tp->rank;
    const size_t n_items = (size_t)n_proj * n_tokens * 16;
    int grid = (int)((n_items + 1023) / 1024);
    if (grid > n_sm) grid = n_sm;
    if (grid < 1) grid = 1;
    return launch_pdl(tp_exchange_kernel, dim3(grid), dim3(256), 0, s, a, v, n_proj, cap, n_tokens, err, skip_push);
}

}  // namespace b200lora
