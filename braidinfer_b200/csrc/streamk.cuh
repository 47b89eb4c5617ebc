// Reading the partial products that the stream-k form of the tensor-core GEMM leaves in
// its workspace (see gemm_tc.cu: mode 3).
//
// Output tiles ([128 weight rows x block_n tokens]) are numbered in the order the product
// walks them (tc_tile_index).  The k blocks of tiles tile_begin, tile_begin + 1, ... form one
// line of w = tiles * total_kb blocks; CTA c of `grid` owns blocks [floor(c w / grid),
// floor((c + 1) w / grid)) and writes the partial product of its j-th run inside one tile to
// slot c * max_segs + j, a [block_n][128] float32 block.  The slots of a tile are added in
// ascending CTA order, so a sum does not depend on which CTA finished first.
#pragma once
#include "common.cuh"

#define STREAMK_TILE_M 128
#define STREAMK_GROUP_N 8            // token tiles that share their stay in L2 (see tc_tile_coords)

// The order in which the product walks its output tiles.  Token tiles vary fastest, so that CTAs
// running side by side share weight tiles in L2; with more than STREAMK_GROUP_N token tiles they go
// in groups of that many, each group against all weight tiles before the next, or a group's tokens
// would not stay in L2 while the weights stream past.
__host__ __device__ __forceinline__ void tc_tile_coords(int tile, int m_tiles, int n_tiles, int& mt, int& nt) {
    if (n_tiles <= STREAMK_GROUP_N) {
        nt = tile % n_tiles;
        mt = tile / n_tiles;
        return;
    }
    const int per_group = STREAMK_GROUP_N * m_tiles;
    const int grp = tile / per_group, r = tile - grp * per_group;
    const int width = (n_tiles - grp * STREAMK_GROUP_N) < STREAMK_GROUP_N ? (n_tiles - grp * STREAMK_GROUP_N) : STREAMK_GROUP_N;
    mt = r / width;
    nt = grp * STREAMK_GROUP_N + (r - mt * width);
}
__host__ __device__ __forceinline__ int tc_tile_index(int mt, int nt, int m_tiles, int n_tiles) {
    if (n_tiles <= STREAMK_GROUP_N) return mt * n_tiles + nt;
    const int grp = nt / STREAMK_GROUP_N;
    const int width = (n_tiles - grp * STREAMK_GROUP_N) < STREAMK_GROUP_N ? (n_tiles - grp * STREAMK_GROUP_N) : STREAMK_GROUP_N;
    return grp * STREAMK_GROUP_N * m_tiles + mt * width + (nt - grp * STREAMK_GROUP_N);
}

struct StreamK {
    const float* partial;
    int grid, max_segs, total_kb, n_tiles, n_rows, block_n;
    long long w;               // (tiles in the line) * total_kb
    int m_tiles, tile_begin;   // the line starts at tile `tile_begin` of the walk
};

// A plan as the host hands it from the product to the kernel that adds up:
// {grid, max_segs, total_kb, n_tiles, block_n, w, m_tiles, tile_begin}.
#define STREAMK_PLAN_INTS 8
static inline StreamK streamk_from_plan(const float* partial, const int* plan, int n_rows) {
    return StreamK{partial, plan[0], plan[1], plan[2], plan[3], n_rows, plan[4], (long long)plan[5], plan[6], plan[7]};
}

// The CTAs whose ranges meet one tile, and the slot of the first of them.
struct StreamKSpan { int c_first, c_last; long long slot_first; };

__device__ __forceinline__ int streamk_owner(const StreamK& k, long long x) {
    // the largest c with floor(c w / grid) <= x
    const long long c = ((x + 1) * k.grid - 1) / k.w;
    return (int)(c < k.grid - 1 ? c : k.grid - 1);
}

// `tile`: index in the line (walk index minus tile_begin).
__device__ __forceinline__ StreamKSpan streamk_span_of_tile(const StreamK& k, int tile) {
    const long long x0 = (long long)tile * k.total_kb;
    StreamKSpan s;
    s.c_first = streamk_owner(k, x0);
    s.c_last = streamk_owner(k, x0 + k.total_kb - 1);
    const long long lo = (long long)s.c_first * k.w / k.grid;
    s.slot_first = (long long)s.c_first * k.max_segs + (tile - (int)(lo / k.total_kb));
    return s;
}

// The span of the tile that holds element (token n, weight row col).
__device__ __forceinline__ StreamKSpan streamk_span(const StreamK& k, int n, int col) {
    return streamk_span_of_tile(k, tc_tile_index(col / STREAMK_TILE_M, n / k.block_n, k.m_tiles, k.n_tiles) - k.tile_begin);
}

__device__ __forceinline__ size_t streamk_slot_elems(const StreamK& k) { return (size_t)k.block_n * STREAMK_TILE_M; }
__device__ __forceinline__ size_t streamk_in_slot(const StreamK& k, int n, int col) {
    return (size_t)(n % k.block_n) * STREAMK_TILE_M + (col % STREAMK_TILE_M);
}

// The sums below ask for the slots of a tile STREAMK_BATCH at a time before they add any of
// them: the loads do not depend on one another, so their trips to L2 overlap, and the adds
// still go in ascending CTA order.  (One load and one add in turn would cost a trip each.)
#define STREAMK_BATCH 8

// Sum over the slots of element (n, col).
__device__ __forceinline__ float streamk_sum(const StreamK& k, const StreamKSpan& s, int n, int col) {
    const size_t slot_elems = streamk_slot_elems(k);
    const float* base = k.partial + streamk_in_slot(k, n, col);
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
    const size_t slot_elems = streamk_slot_elems(k);
    const float* b0 = k.partial + streamk_in_slot(k, n, col0);
    const float* b1 = k.partial + streamk_in_slot(k, n, col1);
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
    const size_t slot_elems = streamk_slot_elems(k);
    const float* base = k.partial + streamk_in_slot(k, n, col);
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

// Two groups of four consecutive columns of one tile at once (a SwiGLU output's gate and up sums): the
// slots of both are asked for together, so the two sums cost one trip, not two.  Each sum adds its own
// slots in ascending CTA order, as streamk_sum4 does.
__device__ __forceinline__ void streamk_sum4_pair(const StreamK& k, const StreamKSpan& s, int n, int col0, int col1,
                                                  float4& out0, float4& out1) {
    const size_t slot_elems = streamk_slot_elems(k);
    const float* b0 = k.partial + streamk_in_slot(k, n, col0);
    const float* b1 = k.partial + streamk_in_slot(k, n, col1);
    const size_t stride = (size_t)k.max_segs * slot_elems;
    float4 a0 = *reinterpret_cast<const float4*>(b0 + (size_t)s.slot_first * slot_elems);
    float4 a1 = *reinterpret_cast<const float4*>(b1 + (size_t)s.slot_first * slot_elems);
    constexpr int B = STREAMK_BATCH / 2;
    for (int c0 = s.c_first + 1; c0 <= s.c_last; c0 += B) {
        float4 v0[B], v1[B];
#pragma unroll
        for (int i = 0; i < B; ++i) {
            const bool in = c0 + i <= s.c_last;
            v0[i] = in ? *reinterpret_cast<const float4*>(b0 + (size_t)(c0 + i) * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
            v1[i] = in ? *reinterpret_cast<const float4*>(b1 + (size_t)(c0 + i) * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < B; ++i)
            if (c0 + i <= s.c_last) {
                a0.x += v0[i].x; a0.y += v0[i].y; a0.z += v0[i].z; a0.w += v0[i].w;
                a1.x += v1[i].x; a1.y += v1[i].y; a1.z += v1[i].z; a1.w += v1[i].w;
            }
    }
    out0 = a0;
    out1 = a1;
}
