// Row scales: an RMSNorm whose scale is applied after the product that follows it.
//
// y = RMSNorm(h) W^T = rs(h) * ((h * g) W^T), with rs(h) = rsqrt(mean(h^2) + eps) one number a row and g
// the norm's weights.  In a step of a few tokens the kernel that completes h (the adding-up of a product's
// partial sums, see fused_reduce.cu) can therefore work on a few columns of many rows per CTA instead of
// on whole rows: it writes h, bfloat16(h * g), and its columns' share of each row's sum of squares, and
// whoever multiplies bfloat16(h * g) by a matrix multiplies its results by rs, which it gets from the
// shares: a product of whole tiles in its epilogue; a stream-k product has its first CTA turn the shares
// into one float a row (rs_rows) for the kernel that adds its partial sums up.  The sum of squares and rs
// are float32, the shares are added in ascending order.
#pragma once
#include "common.cuh"

struct RowScaleArgs {
    const float* shares;       // [n_shares][stride >= rows], or null: no scale (1)
    int n_shares;
    long long stride;
    float width, eps;          // rs = rsqrt(sum of the shares / width + eps)
};

#define ROWSCALE_BATCH 16      // shares asked for at once (a width of 8192 has 16)

// The shares are read with ordinary loads, through L1: every thread of a kernel that applies a scale reads
// the same few floats, and loads that go to L2 each time (ld.global.cg) queue up on those few lines
// (measured: a step of 8 rows 1.7 % slower instead of 1.7 % faster).

__device__ __forceinline__ float row_scale_of(const RowScaleArgs& r, int row) {
    if (!r.shares) return 1.f;
    float ss = 0.f;
    for (int t0 = 0; t0 < r.n_shares; t0 += ROWSCALE_BATCH) {
        float p[ROWSCALE_BATCH];
#pragma unroll
        for (int i = 0; i < ROWSCALE_BATCH; ++i)
            p[i] = (t0 + i < r.n_shares) ? r.shares[(size_t)(t0 + i) * r.stride + row] : 0.f;
#pragma unroll
        for (int i = 0; i < ROWSCALE_BATCH; ++i) ss += p[i];
    }
    return rsqrtf(ss / r.width + r.eps);
}

// What the host checks before it hands a scale to a kernel.
static inline const char* row_scale_problem(const RowScaleArgs& r, int rows) {
    if (!r.shares) return nullptr;
    if (r.n_shares <= 0) return "no shares";
    if (r.stride < rows) return "stride below the number of rows";
    if (!(r.width > 0.f)) return "width must be positive";
    return nullptr;
}
