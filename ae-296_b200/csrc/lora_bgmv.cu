// Decode BGMV: shrink (v = x . A^T) and expand (y += scale * v . B^T) on adapter-sorted segments.
//
// Both kernels are HBM-bound weight streamers.  Work is cut into units of 32 KB of weights
// (8 independent 128-bit loads per thread, 256 threads): the number of k-columns (shrink) or
// output rows (expand) per unit shrinks as the rank grows, so every unit costs the same bytes.
// A segment's weights are read from HBM once and applied to all of its tokens, four tokens per
// register pass.  fp32 accumulation throughout; cross-lane sums use a halving butterfly of warp
// shuffles.  The split-K partial sums of the shrink are combined in a fixed order by the last
// CTA to arrive at a per-(projection, segment) counter, so results are bit-reproducible.
//
// Semantics follow the call `add_lora_bgmv(y, x, wa_T_all, wb_T_all, indicies, layer_idx, scale)`
// of the reference (lightllm/models/lora_gpu.py:138,150,162) with pools laid out as at :33-40.
#include "lora_common.cuh"

namespace b200lora {

namespace {

__device__ __forceinline__ uint4 zero4() { return make_uint4(0u, 0u, 0u, 0u); }

// keep the first `nvalid` 16-bit lanes of a 128-bit word, clear the rest
__device__ __forceinline__ uint4 mask_lanes(uint4 u, int nvalid) {
    if (nvalid >= 8) return u;
    if (nvalid <= 0) return zero4();
    unsigned* w = reinterpret_cast<unsigned*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int lo = 2 * i, hi = 2 * i + 1;
        unsigned m = (lo < nvalid ? 0x0000ffffu : 0u) | (hi < nvalid ? 0xffff0000u : 0u);
        w[i] &= m;
    }
    return u;
}

// Sum NV per-lane values over groups of G consecutive lanes.  Afterwards lane g (within its
// group) holds the NV/G totals with original indices [g*NV/G, (g+1)*NV/G) in v[0 .. NV/G).
// If NV < G the remaining steps are plain all-reduces and every lane of a sub-group holds
// the same single total.
template <int NV, int G>
__device__ __forceinline__ void halving_reduce(float (&v)[NV], int lane) {
    int n = NV;
#pragma unroll
    for (int o = G / 2; o >= 1; o >>= 1) {
        if (n > 1) {
            n >>= 1;
            const bool hi = (lane & o) != 0;
#pragma unroll
            for (int i = 0; i < NV / 2; ++i) {
                if (i < n) {
                    float send = hi ? v[i] : v[i + n];
                    float keep = hi ? v[i + n] : v[i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                }
            }
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
        }
    }
}

struct Item {
    int seg, sub, proj, super;
};

// item -> (unit, projection, super-chunk); n_super[] per projection
__device__ __forceinline__ Item decode_item(const ApplyParams& p, const PlanView& pv, int it, int n_units,
                                            bool expand) {
    Item r;
    int u = it % n_units;
    int sp = it / n_units;
    int pi = 0;
#pragma unroll
    for (int i = 0; i < kMaxProj; ++i) {
        int ns = expand ? p.proj[i].n_super_out : p.proj[i].n_super_in;
        if (i < p.n_proj && sp >= ns && pi == i) { sp -= ns; pi = i + 1; }
    }
    int e = pv.unit_tab[u];
    r.seg = e >> 3;
    r.sub = e & 7;
    r.proj = pi;
    r.super = sp;
    return r;
}

// ---------------------------------------------------------------------------------------------
// shrink: one unit = rows [0, r) x KC columns of A_a, KC = 16384 / r_pad
// ---------------------------------------------------------------------------------------------
template <typename T, int RPW>
__device__ void shrink_item(const ApplyParams& p, const PlanView& pv, const WorkspaceView& ws, const Item it,
                            int* s_flag) {
    constexpr int KS = kSlots / RPW;            // k-steps of 256 columns per unit
    constexpr int KC = KS * 256;
    constexpr int RPAD = RPW * 8;
    constexpr int NV = RPW * kTokTile;
    const ProjArgs& pj = p.proj[it.proj];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int k0 = it.super * kSuper + it.sub * KC;
    if (k0 >= pj.h_in) return;
    const int a = pv.seg_adapter[it.seg];
    const int r = pv.seg_rank[it.seg];
    const int b = pv.seg_start[it.seg], e = pv.seg_start[it.seg + 1];
    const T* A = reinterpret_cast<const T*>(pj.wa) + block_row0(p, a, r) * (long long)pj.h_in;

    uint4 w[kSlots];
#pragma unroll
    for (int q = 0; q < kSlots; ++q) {
        const int rl = q % RPW, ks = q / RPW;
        const int i = warp * RPW + rl;
        const int k = k0 + ks * 256 + lane * 8;
        w[q] = (i < r && k < pj.h_in) ? ldg_nc16(A + (long long)i * pj.h_in + k) : zero4();
    }

    const int kc = k0 / KC;
    const T* X = reinterpret_cast<const T*>(pj.x);
    for (int pos0 = b; pos0 < e; pos0 += kTokTile) {
        const int nt = min(kTokTile, e - pos0);
        float acc[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) acc[i] = 0.f;
        int tok[kTokTile];
#pragma unroll
        for (int tt = 0; tt < kTokTile; ++tt) tok[tt] = pv.perm[pos0 + (tt < nt ? tt : 0)];
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int k = k0 + ks * 256 + lane * 8;
            float xf[kTokTile][8];
#pragma unroll
            for (int tt = 0; tt < kTokTile; ++tt) {
                uint4 xv = (tt < nt && k < pj.h_in) ? ldg16(X + (long long)tok[tt] * pj.ldx + k) : zero4();
                Cvt<T>::unpack8(xv, xf[tt]);
            }
#pragma unroll
            for (int rl = 0; rl < RPW; ++rl) {
                float wf[8];
                Cvt<T>::unpack8(w[ks * RPW + rl], wf);
#pragma unroll
                for (int tt = 0; tt < kTokTile; ++tt) {
                    if (tt < nt) {
                        float s = acc[rl * kTokTile + tt];
#pragma unroll
                        for (int j = 0; j < 8; ++j) s = fmaf(wf[j], xf[tt][j], s);
                        acc[rl * kTokTile + tt] = s;
                    }
                }
            }
        }
        halving_reduce<NV, 32>(acc, lane);
        // writer lanes: low (5 - log2 NV) bits clear; value index = lane >> (5 - log2 NV)
        constexpr int SH = (NV == 32) ? 0 : (NV == 16) ? 1 : (NV == 8) ? 2 : 3;
        if ((lane & ((1 << SH) - 1)) == 0) {
            const int vi = lane >> SH;
            const int rl = vi / kTokTile, tt = vi % kTokTile;
            if (tt < nt) {
                const int i = warp * RPW + rl;
                ws.partial[(((size_t)kc * p.n_proj + it.proj) * p.cap + (pos0 + tt)) * kMaxRank + i] = acc[0];
            }
        }
    }

    // arrive; the last CTA of this (projection, segment) folds the partials in k order
    const int n_chunks = (pj.h_in + KC - 1) / KC;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned old = atomicAdd(&ws.counters[(size_t)it.proj * p.cap + it.seg], 1u);
        *s_flag = (old == (unsigned)(n_chunks - 1));
    }
    __syncthreads();
    if (*s_flag) {
        __threadfence();
        const int len = e - b;
        const bool mid_round = (p.flags & B200_LORA_MID_ROUND) != 0;
        for (int idx = tid; idx < len * RPAD; idx += kCtaThreads) {
            const int pos = b + idx / RPAD, i = idx % RPAD;
            float s = 0.f;
            for (int c = 0; c < n_chunks; ++c)
                s += __ldcg(&ws.partial[(((size_t)c * p.n_proj + it.proj) * p.cap + pos) * kMaxRank + i]);
            if (mid_round) s = Cvt<T>::round1(s);
            ws.v[((size_t)it.proj * p.cap + pos) * kMaxRank + i] = s;
        }
        if (tid == 0) ws.counters[(size_t)it.proj * p.cap + it.seg] = 0u;
    }
    __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(kCtaThreads, 2) bgmv_shrink_kernel(const __grid_constant__ ApplyParams p) {
    __shared__ int s_item;
    __shared__ int s_flag;
    PlanView pv = plan_view(p.plan, p.cap, p.n_adapters);
    WorkspaceView ws = workspace_view(p.workspace, p.cap, p.n_proj);
    const PlanHeader hdr = *pv.hdr;
    if (hdr.error || hdr.cap != p.cap) return;
    const int n_units = (p.flags & B200_LORA_NO_TENSOR) ? hdr.n_units : hdr.n_units_short;
    const int n_items = n_units * p.total_super_in;
    while (true) {
        if (threadIdx.x == 0) s_item = (int)atomicAdd(&ws.ctl->ticket[0], 1u);
        __syncthreads();
        const int it = s_item;
        __syncthreads();
        if (it >= n_items) break;
        Item item = decode_item(p, pv, it, n_units, false);
        const int rpad = pad_rank(pv.seg_rank[item.seg]);
        switch (rpad) {
            case 8:  shrink_item<T, 1>(p, pv, ws, item, &s_flag); break;
            case 16: shrink_item<T, 2>(p, pv, ws, item, &s_flag); break;
            case 32: shrink_item<T, 4>(p, pv, ws, item, &s_flag); break;
            default: shrink_item<T, 8>(p, pv, ws, item, &s_flag); break;
        }
    }
    if (threadIdx.x == 0) {
        unsigned d = atomicAdd(&ws.ctl->done[0], 1u);
        if (d == gridDim.x - 1) { ws.ctl->ticket[0] = 0u; ws.ctl->done[0] = 0u; }
    }
}

// ---------------------------------------------------------------------------------------------
// expand: one unit = JC rows x r columns of B_a, JC = 16384 / r_pad
// ---------------------------------------------------------------------------------------------
template <typename T, int G>
__device__ void expand_item(const ApplyParams& p, const PlanView& pv, const WorkspaceView& ws, const Item it,
                            float* stage) {
    constexpr int RL = kCtaThreads / G;          // rows covered by one CTA-wide load
    constexpr int RLP = RL + 4;                  // padded pitch of one load's rows in the staging tile
    constexpr int JC = kSlots * RL;
    constexpr int JCP = kSlots * RLP;
    constexpr int NV = kSlots * kTokTile;        // 32
    constexpr int NKEEP = NV / G;                // values a lane keeps after the reduce
    const ProjArgs& pj = p.proj[it.proj];
    const int tid = threadIdx.x, lane = tid & 31;
    const int j0 = it.super * kSuper + it.sub * JC;
    if (j0 >= pj.h_out) return;
    const int a = pv.seg_adapter[it.seg];
    const int r = pv.seg_rank[it.seg];
    const int b = pv.seg_start[it.seg], e = pv.seg_start[it.seg + 1];
    const int pitch = b_pitch(p, r);
    const T* B = reinterpret_cast<const T*>(pj.wb) + block_row0(p, a, r) * (long long)pj.h_out;
    const int g = tid % G, k0 = g * 8, row_in_load = tid / G;
    const float scale = p.scalings ? p.scalings[a] : p.scale;

    uint4 w[kSlots];
#pragma unroll
    for (int q = 0; q < kSlots; ++q) {
        const int row = j0 + q * RL + row_in_load;
        w[q] = (row < pj.h_out && k0 < r) ? mask_lanes(ldg_nc16(B + (long long)row * pitch + k0), r - k0) : zero4();
    }

    for (int pos0 = b; pos0 < e; pos0 += kTokTile) {
        const int nt = min(kTokTile, e - pos0);
        float vf[kTokTile][8];
#pragma unroll
        for (int tt = 0; tt < kTokTile; ++tt) {
            if (tt < nt) {
                const float4* vp = reinterpret_cast<const float4*>(
                    &ws.v[((size_t)it.proj * p.cap + pos0 + tt) * kMaxRank + k0]);
                float4 v0 = vp[0], v1 = vp[1];
                vf[tt][0] = v0.x; vf[tt][1] = v0.y; vf[tt][2] = v0.z; vf[tt][3] = v0.w;
                vf[tt][4] = v1.x; vf[tt][5] = v1.y; vf[tt][6] = v1.z; vf[tt][7] = v1.w;
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) vf[tt][j] = 0.f;
            }
        }
        float acc[NV];
#pragma unroll
        for (int q = 0; q < kSlots; ++q) {
            float wf[8];
            Cvt<T>::unpack8(w[q], wf);
#pragma unroll
            for (int tt = 0; tt < kTokTile; ++tt) {
                float s = 0.f;
                if (tt < nt) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) s = fmaf(wf[j], vf[tt][j], s);
                }
                acc[q * kTokTile + tt] = s;
            }
        }
        halving_reduce<NV, G>(acc, lane);
        // lane g keeps value indices [g*NKEEP, (g+1)*NKEEP): vi = q * kTokTile + tt
#pragma unroll
        for (int i = 0; i < NKEEP; ++i) {
            const int vi = g * NKEEP + i;
            const int q = vi / kTokTile, tt = vi % kTokTile;
            stage[tt * JCP + q * RLP + row_in_load] = scale * acc[i];
        }
        __syncthreads();
        // coalesced read-modify-write of y, 8 outputs per thread
        const int chunks = JC / 8;
        for (int idx = tid; idx < nt * chunks; idx += kCtaThreads) {
            const int tt = idx / chunks, j8 = (idx % chunks) * 8;
            const int col = j0 + j8;
            if (col < pj.h_out) {
                const int tok = pv.perm[pos0 + tt];
                const float4* sp = reinterpret_cast<const float4*>(&stage[tt * JCP + (j8 / RL) * RLP + (j8 % RL)]);
                const float4 s0 = sp[0], s1 = sp[1];
                const float st[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                if (p.y_f32) {
                    float4* yp = reinterpret_cast<float4*>(reinterpret_cast<float*>(pj.y) + (long long)tok * pj.ldy + col);
                    float4 y0 = yp[0], y1 = yp[1];
                    y0.x += st[0]; y0.y += st[1]; y0.z += st[2]; y0.w += st[3];
                    y1.x += st[4]; y1.y += st[5]; y1.z += st[6]; y1.w += st[7];
                    yp[0] = y0; yp[1] = y1;
                } else {
                    uint4* yp = reinterpret_cast<uint4*>(reinterpret_cast<T*>(pj.y) + (long long)tok * pj.ldy + col);
                    uint4 yv = *yp;
                    float yf[8];
                    Cvt<T>::unpack8(yv, yf);
                    yv.x = Cvt<T>::pack2(yf[0] + st[0], yf[1] + st[1]);
                    yv.y = Cvt<T>::pack2(yf[2] + st[2], yf[3] + st[3]);
                    yv.z = Cvt<T>::pack2(yf[4] + st[4], yf[5] + st[5]);
                    yv.w = Cvt<T>::pack2(yf[6] + st[6], yf[7] + st[7]);
                    *yp = yv;
                }
            }
        }
        __syncthreads();
    }
}

template <typename T>
__global__ void __launch_bounds__(kCtaThreads, 2) bgmv_expand_kernel(const __grid_constant__ ApplyParams p) {
    __shared__ int s_item;
    __shared__ __align__(16) float stage[kTokTile * (kSuper + 4 * kSlots)];   // 32.5 KB
    PlanView pv = plan_view(p.plan, p.cap, p.n_adapters);
    WorkspaceView ws = workspace_view(p.workspace, p.cap, p.n_proj);
    const PlanHeader hdr = *pv.hdr;
    if (hdr.error || hdr.cap != p.cap) return;
    const int n_units = (p.flags & B200_LORA_NO_TENSOR) ? hdr.n_units : hdr.n_units_short;
    const int n_items = n_units * p.total_super_out;
    while (true) {
        if (threadIdx.x == 0) s_item = (int)atomicAdd(&ws.ctl->ticket[1], 1u);
        __syncthreads();
        const int it = s_item;
        __syncthreads();
        if (it >= n_items) break;
        Item item = decode_item(p, pv, it, n_units, true);
        const int rpad = pad_rank(pv.seg_rank[item.seg]);
        switch (rpad) {
            case 8:  expand_item<T, 1>(p, pv, ws, item, stage); break;
            case 16: expand_item<T, 2>(p, pv, ws, item, stage); break;
            case 32: expand_item<T, 4>(p, pv, ws, item, stage); break;
            default: expand_item<T, 8>(p, pv, ws, item, stage); break;
        }
    }
    if (threadIdx.x == 0) {
        unsigned d = atomicAdd(&ws.ctl->done[1], 1u);
        if (d == gridDim.x - 1) { ws.ctl->ticket[1] = 0u; ws.ctl->done[1] = 0u; }
    }
}

}  // namespace

cudaError_t launch_bgmv(const ApplyParams& p, int io_dtype, int n_sm, cudaStream_t s) {
    const int grid = n_sm * 2;
    const bool do_shrink = !(p.flags & B200_LORA_ONLY_EXPAND);
    const bool do_expand = !(p.flags & B200_LORA_ONLY_SHRINK);
    if (io_dtype == B200_LORA_F16) {
        if (do_shrink) bgmv_shrink_kernel<__half><<<grid, kCtaThreads, 0, s>>>(p);
        if (do_expand) bgmv_expand_kernel<__half><<<grid, kCtaThreads, 0, s>>>(p);
    } else {
        if (do_shrink) bgmv_shrink_kernel<__nv_bfloat16><<<grid, kCtaThreads, 0, s>>>(p);
        if (do_expand) bgmv_expand_kernel<__nv_bfloat16><<<grid, kCtaThreads, 0, s>>>(p);
    }
    return cudaGetLastError();
}

}  // namespace b200lora
