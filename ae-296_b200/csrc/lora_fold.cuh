// Adding up the split-K slots the TMA shrink kernel leaves (shared by the expand kernel's producers,
// the fold kernel and the tensor-parallel exchange).
#pragma once

#include "lora_common.cuh"

namespace b200lora {

namespace {

// The split-K slots of one (projection, work segment): the runs of the shrink kernel start at
// the segment's first unit and wherever a CTA's item range starts inside the segment, and a
// run's slot is the index, inside the segment, of its first unit.  `seg_first` is the list
// index of the segment's first unit, `per_cta` the length of a CTA's range, `n_chunks` the
// units of the segment that lie inside the matrix (they come first).
struct SlotWalk {
    int j, step, n_chunks;
    __device__ __forceinline__ SlotWalk(int seg_first, int per_cta, int n_chunks_) : j(0), n_chunks(n_chunks_) {
        step = per_cta - seg_first % per_cta;              // distance to the next range start
    }
    __device__ __forceinline__ bool valid() const { return j < n_chunks; }
    __device__ __forceinline__ void next(int per_cta) { j += step; step = per_cta; }
};
// list index of the first shrink unit of the segment that starts at plan unit `u0`
__device__ __forceinline__ int shrink_seg_first(const ApplyParams& p, int n_units, int proj, int u0) {
    int base = 0;
#pragma unroll
    for (int i = 0; i < kMaxProj - 1; ++i)
        if (i < proj) base += n_units * p.proj[i].n_super_in;
    return base + u0 * p.proj[proj].n_super_in;
}
__device__ __forceinline__ int shrink_chunks(const ApplyParams& p, int proj, int rank) {
    const int wshift = rank <= 16 ? 9 : rank == 32 ? 8 : 7;
    return (p.proj[proj].h_in + (1 << wshift) - 1) >> wshift;
}

// Adds up the slots of one segment, ascending, for NQ quads (four consecutive rank indices of
// one token each) at once: the loads of all quads and of up to NS slots are in flight together.
template <typename T, int NQ, int NS = 4>
__device__ __forceinline__ void fold_quads(const ApplyParams& p, const WorkspaceView& ws, const size_t (&off)[NQ],
                                           const bool (&on)[NQ], int seg_first, int per_cta, int n_chunks, float4 (&s)[NQ]) {
    const size_t cstride = (size_t)p.n_proj * p.cap * kMaxRank;
#pragma unroll
    for (int i = 0; i < NQ; ++i) s[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    SlotWalk sw(seg_first, per_cta, n_chunks);
    while (sw.valid()) {
        float4 v[NS][NQ];
#pragma unroll
        for (int q = 0; q < NS; ++q) {
            const bool live = sw.valid();
#pragma unroll
            for (int i = 0; i < NQ; ++i) {
                v[q][i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live && on[i]) v[q][i] = __ldcg(reinterpret_cast<const float4*>(ws.partial + (size_t)sw.j * cstride + off[i]));
            }
            if (live) sw.next(per_cta);
        }
#pragma unroll
        for (int q = 0; q < NS; ++q)
#pragma unroll
            for (int i = 0; i < NQ; ++i) { s[i].x += v[q][i].x; s[i].y += v[q][i].y; s[i].z += v[q][i].z; s[i].w += v[q][i].w; }
    }
    if (p.flags & B200_LORA_MID_ROUND) {
#pragma unroll
        for (int i = 0; i < NQ; ++i) {
            s[i].x = Cvt<T>::round1(s[i].x); s[i].y = Cvt<T>::round1(s[i].y);
            s[i].z = Cvt<T>::round1(s[i].z); s[i].w = Cvt<T>::round1(s[i].w);
        }
    }
}

}  // namespace

}  // namespace b200lora
