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

// Sum over the slots of element (n, col).
__device__ __forceinline__ float streamk_sum(const StreamK& k, const StreamKSpan& s, int n, int col) {
    const size_t in_slot = (size_t)n * STREAMK_TILE_M + (col % STREAMK_TILE_M);
    const size_t slot_elems = (size_t)k.n_rows * STREAMK_TILE_M;
    float acc = k.partial[(size_t)s.slot_first * slot_elems + in_slot];
    for (int c = s.c_first + 1; c <= s.c_last; ++c)
        acc += k.partial[(size_t)c * k.max_segs * slot_elems + in_slot];
    return acc;
}

// Four consecutive columns (col a multiple of 4, so they lie in one tile).
__device__ __forceinline__ float4 streamk_sum4(const StreamK& k, const StreamKSpan& s, int n, int col) {
    const size_t in_slot = (size_t)n * STREAMK_TILE_M + (col % STREAMK_TILE_M);
    const size_t slot_elems = (size_t)k.n_rows * STREAMK_TILE_M;
    float4 acc = *reinterpret_cast<const float4*>(k.partial + (size_t)s.slot_first * slot_elems + in_slot);
    for (int c = s.c_first + 1; c <= s.c_last; ++c) {
        const float4 v = *reinterpret_cast<const float4*>(k.partial + (size_t)c * k.max_segs * slot_elems + in_slot);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    return acc;
}
