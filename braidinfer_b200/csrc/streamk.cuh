// Reading the partial products that the stream-k form of the tensor-core GEMM leaves in
// its workspace (see gemm_tc.cu: mode 3).
//
// The k blocks of all [128 x BLOCK_N] output tiles form one line of w = tiles * total_kb
// blocks; CTA c of `grid` owns blocks [floor(c w / grid), floor((c + 1) w / grid)) and
// writes the partial product of its j-th run inside one tile to slot c * max_segs + j,
// a [n_rows][128] float32 block.  The slots of a tile are added in ascending CTA order,
// so a sum does not depend on which CTA finished first.
#pragma once
#include "common.cuh"

#define STREAMK_TILE_M 128

struct StreamK {
    const float* partial;
    int grid, max_segs, total_kb, n_tiles, n_rows, block_n;
    long long w;               // m_tiles * n_tiles * total_kb
};

// The CTAs whose ranges meet one tile, and the slot of the first of them.
struct StreamKSpan { int c_first, c_last; long long slot_first; };

__device__ __forceinline__ int streamk_owner(const StreamK& k, long long x) {
    // the largest c with floor(c w / grid) <= x
    const long long c = ((x + 1) * k.grid - 1) / k.w;
    return (int)(c < k.grid - 1 ? c : k.grid - 1);
}

__device__ __forceinline__ StreamKSpan streamk_span(const StreamK& k, int n, int col) {
    const int tile = (col / STREAMK_TILE_M) * k.n_tiles + n / k.block_n;
    const long long x0 = (long long)tile * k.total_kb;
    StreamKSpan s;
    s.c_first = streamk_owner(k, x0);
    s.c_last = streamk_owner(k, x0 + k.total_kb - 1);
    const long long lo = (long long)s.c_first * k.w / k.grid;
    s.slot_first = (long long)s.c_first * k.max_segs + (tile - (int)(lo / k.total_kb));
    return s;
}

// The sums below ask for the slots of a tile STREAMK_BATCH at a time before they add any of
// them: the loads do not depend on one another, so their trips to L2 overlap, and the adds
// still go in ascending CTA order.  (One load and one add in turn would cost a trip each.)
#define STREAMK_BATCH 8

// Sum over the slots of element (n, col).
__device__ __forceinline__ float streamk_sum(const StreamK& k, const StreamKSpan& s, int n, int col) {
    const size_t slot_elems = (size_t)k.n_rows * STREAMK_TILE_M;
    const float* base = k.partial + (size_t)n * STREAMK_TILE_M + (col % STREAMK_TILE_M);
    const size_t stride = (size_t)k.max_segs * slot_elems;
    float acc = base[(size_t)s.slot_first * slot_elems];
    for (int c0 = s.c_first + 1; c0 <= s.c_last; c0 += STREAMK_BATCH) {
        float v[STREAMK_BATCH];
#pragma unroll
        for (int i = 0; i < STREAMK_BATCH; ++i) v[i] = (c0 + i <= s.c_last) ? base[(size_t)(c0 + i) * stride] : 0.f;
#pragma unroll
        for (int i = 0; i < STREAMK_BATCH; ++i)
            if (c0 + i <= s.c_last) acc += v[i];
    }
    return acc;
}

// Two elements of row n at once (the two halves of a rotary pair): the slots of both are asked
// for together.  Each sum adds its own slots in ascending CTA order, as streamk_sum does.
__device__ __forceinline__ void streamk_sum_pair(const StreamK& k, const StreamKSpan& s0, const StreamKSpan& s1, int n,
                                                 int col0, int col1, float& out0, float& out1) {
    const size_t slot_elems = (size_t)k.n_rows * STREAMK_TILE_M;
    const float* b0 = k.partial + (size_t)n * STREAMK_TILE_M + (col0 % STREAMK_TILE_M);
    const float* b1 = k.partial + (size_t)n * STREAMK_TILE_M + (col1 % STREAMK_TILE_M);
    const size_t stride = (size_t)k.max_segs * slot_elems;
    float a0 = b0[(size_t)s0.slot_first * slot_elems];
    float a1 = b1[(size_t)s1.slot_first * slot_elems];
    const int n0 = s0.c_last - s0.c_first, n1 = s1.c_last - s1.c_first;
    for (int j0 = 1; j0 <= max(n0, n1); j0 += STREAMK_BATCH) {
        float v0[STREAMK_BATCH], v1[STREAMK_BATCH];
#pragma unroll
        for (int i = 0; i < STREAMK_BATCH; ++i) {
            v0[i] = (j0 + i <= n0) ? b0[(size_t)(s0.c_first + j0 + i) * stride] : 0.f;
            v1[i] = (j0 + i <= n1) ? b1[(size_t)(s1.c_first + j0 + i) * stride] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < STREAMK_BATCH; ++i) {
            if (j0 + i <= n0) a0 += v0[i];
            if (j0 + i <= n1) a1 += v1[i];
        }
    }
    out0 = a0;
    out1 = a1;
}

// Four consecutive columns (col a multiple of 4, so they lie in one tile).
__device__ __forceinline__ float4 streamk_sum4(const StreamK& k, const StreamKSpan& s, int n, int col) {
    const size_t slot_elems = (size_t)k.n_rows * STREAMK_TILE_M;
    const float* base = k.partial + (size_t)n * STREAMK_TILE_M + (col % STREAMK_TILE_M);
    const size_t stride = (size_t)k.max_segs * slot_elems;
    float4 acc = *reinterpret_cast<const float4*>(base + (size_t)s.slot_first * slot_elems);
    for (int c0 = s.c_first + 1; c0 <= s.c_last; c0 += STREAMK_BATCH) {
        float4 v[STREAMK_BATCH];
#pragma unroll
        for (int i = 0; i < STREAMK_BATCH; ++i)
            v[i] = (c0 + i <= s.c_last) ? *reinterpret_cast<const float4*>(base + (size_t)(c0 + i) * stride)
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < STREAMK_BATCH; ++i)
            if (c0 + i <= s.c_last) { acc.x += v[i].x; acc.y += v[i].y; acc.z += v[i].z; acc.w += v[i].w; }
    }
    return acc;
}
