// Token choice on the device: argmax, and the sampling chain of the reference
// (crates/braidinfer-runtime/src/sampling.rs:49-171) in its order: logit bias,
// repetition penalty, temperature (0 means argmax), top-k, min-p, top-p, softmax,
// inverse CDF with a uniform number that the caller supplies per row.
//
// One block per row of logits; all arithmetic float32.  Where the reference sorts,
// this finds the cut value on the bit pattern of the floats (top-k: the k-th largest key
// digit by digit, eight bits a pass, from counts in shared memory; top-p: the same walk
// over a histogram of probability mass in fixed point, four passes over a whole row, or a
// bisection bit by bit when top-k has left a block's worth of candidates), and keeps the
// lowest indices of a tie at the cut (the
// reference's unstable sort leaves that order open).  When top-k leaves at most a
// block's worth of candidates, they are gathered into shared memory in index order and
// the rest of the chain runs on them alone.  Argmax returns the lowest index of the maximum.
#include "common.cuh"

#define SAMP_THREADS 1024

__device__ __forceinline__ unsigned int float_key(float x) {
    // Monotone map float -> uint: larger float, larger key (-inf lowest, NaN above +inf).
    const unsigned int b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float block_reduce_sum(float v, float* sh) {
    return block_sum(v, sh);
}
__device__ __forceinline__ float block_reduce_max(float v, float* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float t = (lane < nw) ? sh[lane] : -INFINITY;
    return warp_max(t);
}
__device__ __forceinline__ int block_reduce_isum(int v, int* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    int t = (lane < nw) ? sh[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}
__device__ __forceinline__ int block_reduce_imin(int v, int* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    int t = (lane < nw) ? sh[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = min(t, __shfl_xor_sync(0xffffffffu, t, o));
    return t;
}
// Exclusive prefix over the threads of the block (thread order), float and int.
__device__ __forceinline__ float block_exclusive_scan(float v, float* sh /* [32] */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();
    if (lane == 31) sh[warp] = inc;
    __syncthreads();
    float base = 0.f;
    for (int i = 0; i < warp; ++i) base += sh[i];
    return base + inc - v;
}
__device__ __forceinline__ int block_exclusive_iscan(int v, int* sh /* [32] */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();
    if (lane == 31) sh[warp] = inc;
    __syncthreads();
    int base = 0;
    for (int i = 0; i < warp; ++i) base += sh[i];
    return base + inc - v;
}

// A row of logits.  In shared memory it is laid out with one float of padding after every 32: the chain
// reads it both with consecutive threads on consecutive elements and with every thread on a run of
// elements of its own (the sums along the index), and without the padding the runs of a warp's threads
// start 32 floats apart, on one bank.
struct Row {
    float* p;
    int padded;
    __device__ __forceinline__ float& operator[](int i) const { return p[padded ? i + (i >> 5) : i]; }
};

// Every element of the row once, the block's threads in stride: f(value, index).  A row in global memory (one
// too long for shared memory) that starts on 16 bytes is read 16 bytes at a time, four loads in flight a thread:
// with one 4-byte load at a time a thread, a row of 512 KB is 128 round trips to L2 a pass, and the chain
// makes a dozen passes.  (A thread then meets its elements in another order than in the plain loop; rows in
// shared memory keep the plain loop, and their sums the order they had.)
template <typename F>
__device__ __forceinline__ void row_each(const Row& x, int n, F f) {
    if (!x.padded && (((uintptr_t)x.p & 15) == 0)) {
        const int n4 = n >> 2;
        const float4* x4 = reinterpret_cast<const float4*>(x.p);
        constexpr int U = 4;
        for (int base = threadIdx.x; base < n4; base += blockDim.x * U) {
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int g = base + u * (int)blockDim.x;
                v[u] = g < n4 ? x4[g] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int g = base + u * (int)blockDim.x;
                if (g < n4) { f(v[u].x, 4 * g); f(v[u].y, 4 * g + 1); f(v[u].z, 4 * g + 2); f(v[u].w, 4 * g + 3); }
            }
        }
        for (int i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) f(x.p[i], i);
        return;
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x) f(x[i], i);
}
// The same with a new value for every element: x[i] = f(x[i], i).
template <typename F>
__device__ __forceinline__ void row_update(const Row& x, int n, F f) {
    if (!x.padded && (((uintptr_t)x.p & 15) == 0)) {
        const int n4 = n >> 2;
        float4* x4 = reinterpret_cast<float4*>(x.p);
        constexpr int U = 4;
        for (int base = threadIdx.x; base < n4; base += blockDim.x * U) {
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int g = base + u * (int)blockDim.x;
                v[u] = g < n4 ? x4[g] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int g = base + u * (int)blockDim.x;
                if (g < n4) x4[g] = make_float4(f(v[u].x, 4 * g), f(v[u].y, 4 * g + 1), f(v[u].z, 4 * g + 2), f(v[u].w, 4 * g + 3));
            }
        }
        for (int i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) x.p[i] = f(x.p[i], i);
        return;
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x) x[i] = f(x[i], i);
}

// One thread's candidate after looking at (v, i): the largest value, the lowest index among equals.
__device__ __forceinline__ void argmax_take(float v, int i, float& best, int& best_i, bool& saw_nan) {
    if (v != v) saw_nan = true;
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
}

// The block's winner from every thread's candidate.
__device__ __forceinline__ int argmax_finish(float best, int best_i, bool saw_nan, float* shf, int* shi, int* nan_flag) {
    if (saw_nan && nan_flag) atomicExch(nan_flag, 1);
    const float m = block_reduce_max(best, shf);
    const int cand = (best == m) ? best_i : 0x7fffffff;
    int r = block_reduce_imin(cand, shi);
    if (r == 0x7fffffff) r = 0;     // all values were -inf or NaN
    return r;
}

// Lowest index of the largest value of x[0..n); a NaN anywhere raises *nan_flag.
__device__ int block_argmax(Row x, int n, float* shf, int* shi, int* nan_flag) {
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    bool saw_nan = false;
    row_each(x, n, [&](float v, int i) { argmax_take(v, i, best, best_i, saw_nan); });
    return argmax_finish(best, best_i, saw_nan, shf, shi, nan_flag);
}

// The same over a row in global memory that starts on 16 bytes: 16-byte loads, four of them in flight a thread.
__device__ int block_argmax_vec(const float* __restrict__ x, int n, float* shf, int* shi, int* nan_flag) {
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    bool saw_nan = false;
    const int n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    constexpr int U = 4;
    for (int base = threadIdx.x; base < n4; base += blockDim.x * U) {
        float4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int g = base + u * (int)blockDim.x;
            v[u] = g < n4 ? x4[g] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = (base + u * (int)blockDim.x) * 4;
            if (i < n4 * 4) {
                argmax_take(v[u].x, i, best, best_i, saw_nan);
                argmax_take(v[u].y, i + 1, best, best_i, saw_nan);
                argmax_take(v[u].z, i + 2, best, best_i, saw_nan);
                argmax_take(v[u].w, i + 3, best, best_i, saw_nan);
            }
        }
    }
    for (int i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) argmax_take(x[i], i, best, best_i, saw_nan);
    return argmax_finish(best, best_i, saw_nan, shf, shi, nan_flag);
}

__global__ void __launch_bounds__(SAMP_THREADS)
argmax_kernel(const float* __restrict__ logits, long long ld, int* __restrict__ out, int vocab, int* nan_flag) {
    pdl_trigger();
    pdl_wait();
    __shared__ float shf[32];
    __shared__ int shi[32];
    const float* row = logits + (size_t)blockIdx.x * ld;
    const int r = (((uintptr_t)row & 15) == 0) ? block_argmax_vec(row, vocab, shf, shi, nan_flag)
                                                : block_argmax(Row{const_cast<float*>(row), 0}, vocab, shf, shi, nan_flag);
    if (threadIdx.x == 0) out[blockIdx.x] = r;
}

extern "C" int braid_argmax(const float* logits, long long ld, int* out, int rows, int vocab,
                            int* nan_flag, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (vocab <= 0) BRAID_REFUSE("argmax: vocab=%d must be positive", vocab);
    braid_launch(argmax_kernel, dim3(rows), dim3(SAMP_THREADS), 0, (cudaStream_t)stream, logits, ld, out, vocab, nan_flag);
    BRAID_LAUNCH_CHECK();
}

// Per-row options, one entry per row of logits.
struct SampleArgs {
    const float* logits;     // [rows, ld]
    float* work;             // [rows, vocab] scratch that the kernel may overwrite (may be logits)
    long long ld;
    int* out;                // [rows]
    int vocab;
    const float* temperature;
    const int* top_k;
    const float* top_p;
    const float* min_p;
    const float* rep_penalty;
    const float* uniform;    // u in [0, 1) per row
    // repetition history as (token, count) pairs: row r owns [hist_off[r], hist_off[r+1])
    const int* hist_off;
    const int* hist_tok;
    const int* hist_cnt;
    // logit bias as (token, delta) pairs: row r owns [bias_off[r], bias_off[r+1])
    const int* bias_off;
    const int* bias_tok;
    const float* bias_val;
    int* nan_flag;
    int row_in_smem;         // the launch has vocab floats of dynamic shared memory for the row
};

// The passes that go along the index (ranks among equal keys, the gathering of candidates, the cumulative
// sum) give every thread a run of elements of its own where the row lies in shared memory.  In global memory
// such runs put the 32 loads of a warp on 32 lines, so there a warp owns a span of the row instead
// ([warp * span, (warp + 1) * span), span a multiple of 32), reads it 32 consecutive elements at a time, and
// ranks and running sums go across the lanes by ballot and shuffle.
struct Span { int b, e, lane, warp; };
__device__ __forceinline__ Span span_of(int n) {
    const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5;
    const int len = ((n + nw - 1) / nw + 31) / 32 * 32;
    Span s;
    s.b = min(n, warp * len);
    s.e = min(n, s.b + len);
    s.lane = threadIdx.x & 31;
    s.warp = warp;
    return s;
}
__device__ __forceinline__ int warp_isum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// The sum of the warps' values before this warp's (sh: one int a warp).
__device__ __forceinline__ int warps_before(int v, int* sh, const Span& sp) {
    __syncthreads();
    if (sp.lane == 0) sh[sp.warp] = v;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < sp.warp; ++w) before += sh[w];
    return before;
}

__device__ void apply_cut_span(float* x, int n, unsigned int cut, int keep_equal, int* shi) {
    const Span sp = span_of(n);
    int eq = 0;
    for (int i = sp.b + sp.lane; i < sp.e; i += 32) eq += (float_key(x[i]) == cut);
    int before = warps_before(warp_isum(eq), shi, sp);
    for (int i0 = sp.b; i0 < sp.e; i0 += 32) {
        const int i = i0 + sp.lane;
        const bool in = i < sp.e;
        const unsigned int key = float_key(in ? x[i] : 0.f);
        const bool is_eq = in && key == cut;
        const unsigned int bal = __ballot_sync(0xffffffffu, is_eq);
        const int rank = before + __popc(bal & ((1u << sp.lane) - 1u));
        if (in && (key < cut || (is_eq && rank >= keep_equal))) x[i] = -INFINITY;
        before += __popc(bal);
    }
    __syncthreads();
}

// Keep the `keep` lowest-index elements whose key equals `cut` and everything above
// it; set the rest to -inf.
__device__ void apply_cut(Row x, int n, unsigned int cut, int keep_equal, int* shi) {
    if (!x.padded) { apply_cut_span(x.p, n, cut, keep_equal, shi); return; }
    const int chunk = (n + blockDim.x - 1) / blockDim.x;
    const int b = min(n, (int)threadIdx.x * chunk), e = min(n, b + chunk);
    int eq = 0;
    for (int i = b; i < e; ++i) eq += (float_key(x[i]) == cut);
    int before = block_exclusive_iscan(eq, shi);
    for (int i = b; i < e; ++i) {
        const unsigned int k = float_key(x[i]);
        if (k < cut) x[i] = -INFINITY;
        else if (k == cut) {
            if (before >= keep_equal) x[i] = -INFINITY;
            ++before;
        }
    }
    __syncthreads();
}

// The k-th largest key of x[0..n): most significant digit first, eight bits a pass.  After a
// pass `prefix` holds the digits found so far and `want` the rank still looked for among
// the keys that share them.  Counts are integers, so the result does not depend on timing.
__device__ unsigned int kth_largest_key(Row x, int n, int k, int* hist /* [256] */, int* shi) {
    unsigned int prefix = 0;
    int want = k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        const unsigned int mask = (shift == 24) ? 0u : (0xffffffffu << (shift + 8));
        row_each(x, n, [&](float v, int) {
            const unsigned int key = float_key(v);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
        });
        __syncthreads();
        // the highest digit d with count(digits >= d) >= want: one warp walks the 256 counts from the top
        if (threadIdx.x < 32) {
            int carried = 0, digit = 0, left = want;
            bool done = false;
            for (int base = 224; base >= 0 && !done; base -= 32) {
                const int c = hist[base + 31 - threadIdx.x];                 // lane 0 holds the highest digit of the group
                int inc = c;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, inc, o);
                    if ((int)threadIdx.x >= o) inc += t;
                }
                const unsigned int hit = __ballot_sync(0xffffffffu, carried + inc >= want);
                if (hit) {
                    const int lane = __ffs(hit) - 1;
                    digit = base + 31 - lane;
                    const int before = carried + __shfl_sync(0xffffffffu, inc, lane) - __shfl_sync(0xffffffffu, c, lane);
                    left = want - before;
                    done = true;
                } else {
                    carried += __shfl_sync(0xffffffffu, inc, 31);
                }
            }
            if (threadIdx.x == 0) { shi[0] = digit; shi[1] = left; }
        }
        __syncthreads();
        prefix |= ((unsigned int)shi[0]) << shift;
        want = shi[1];
        __syncthreads();
    }
    return prefix;
}

// Probability mass in fixed point (48 fractional bits): sums of integers do not depend on the order in which the
// threads add, so a histogram of mass may be built with atomics and still give the same cut every time.
#define MASS_ONE 281474976710656.f            // 2^48
__device__ __forceinline__ unsigned long long mass_of(float p) { return __float2ull_rd(p * MASS_ONE); }
// A 64-bit sum kept as two 32-bit words, so that the adds are the shared-memory atomics the hardware has
// (a 64-bit add would be a compare-and-swap loop, which queues when many threads meet on a few counters).
__device__ __forceinline__ void mass_add(unsigned int* lo, unsigned int* hi, unsigned long long q) {
    const unsigned int ql = (unsigned int)q, qh = (unsigned int)(q >> 32);
    const unsigned int old = atomicAdd(lo, ql);
    const unsigned int carry = (old + ql < old) ? 1u : 0u;
    if (qh + carry) atomicAdd(hi, qh + carry);
}

// The cut of top-p: the largest key c such that the mass of the elements with key >= c reaches `target`
// (0 if even the whole row does not).  `*above` receives the mass of the keys strictly greater than the cut.
// Most significant digit first, eight bits a pass, as kth_largest_key, with mass in the place of counts:
// four passes over the row instead of the thirty-two of a bisection bit by bit.
// p(x) = expf(x - m) / total, as the rest of the chain computes it.
__device__ unsigned int top_p_cut(Row x, int n, float m, float total, unsigned long long target,
                                  unsigned int* mhist /* [512]: low words, then high words */,
                                  unsigned long long* shl /* [1] */, int* shi, unsigned long long* above) {
    unsigned int prefix = 0;
    unsigned long long carried = 0;          // mass of the keys above every key that shares the prefix
    bool any = true;
    for (int shift = 24; shift >= 0 && any; shift -= 8) {
        for (int i = threadIdx.x; i < 512; i += blockDim.x) mhist[i] = 0;
        __syncthreads();
        const unsigned int mask = (shift == 24) ? 0u : (0xffffffffu << (shift + 8));
        // a thread adds up runs of equal digits by itself before it goes to the histogram: the top digits of a
        // row are nearly all the same, and a thousand threads on one counter would queue
        int run_digit = -1;
        unsigned long long run = 0;
        row_each(x, n, [&](float v, int) {
            const unsigned int key = float_key(v);
            if ((key & mask) != prefix) return;
            const int d = (int)((key >> shift) & 255u);
            const unsigned long long q = mass_of(expf(v - m) / total);
            if (d == run_digit) { run += q; return; }
            if (run) mass_add(&mhist[run_digit], &mhist[256 + run_digit], run);
            run_digit = d;
            run = q;
        });
        if (run) mass_add(&mhist[run_digit], &mhist[256 + run_digit], run);
        __syncthreads();
        // the highest digit d with carried + mass(digits >= d) >= target: one warp walks the 256 sums from the top
        if (threadIdx.x < 32) {
            unsigned long long acc = carried, before = carried;
            int digit = -1;
            for (int base = 224; base >= 0 && digit < 0; base -= 32) {
                const int d = base + 31 - (int)threadIdx.x;                           // lane 0 holds the highest digit of the group
                const unsigned long long c = ((unsigned long long)mhist[256 + d] << 32) + mhist[d];
                unsigned long long inc = c;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const unsigned long long t = __shfl_up_sync(0xffffffffu, inc, o);
                    if ((int)threadIdx.x >= o) inc += t;
                }
                const unsigned int hit = __ballot_sync(0xffffffffu, acc + inc >= target);
                if (hit) {
                    const int lane = __ffs(hit) - 1;
                    digit = base + 31 - lane;
                    before = acc + __shfl_sync(0xffffffffu, inc, lane) - __shfl_sync(0xffffffffu, c, lane);
                } else {
                    acc += __shfl_sync(0xffffffffu, inc, 31);
                }
            }
            if (threadIdx.x == 0) { shi[0] = digit; shl[0] = before; }
        }
        __syncthreads();
        const int digit = shi[0];
        if (digit < 0) any = false;           // the whole row does not reach the target: keep everything
        else {
            prefix |= ((unsigned int)digit) << shift;
            carried = shl[0];
        }
        __syncthreads();
    }
    *above = carried;
    return any ? prefix : 0u;
}

// The rest of the chain after top-k, on at most blockDim.x candidates held in shared memory in
// index order (cv: values, ci: indices; thread t owns candidate t).  Same steps, same order of
// sums along the index as the full-row form below.
__device__ int sample_few(float* cv, const int* ci, int m, float mp, float tp, float u, float* shf, int* shi,
                          int* found, int* nan_flag) {
    const int t = threadIdx.x;
    float v = (t < m) ? cv[t] : -INFINITY;
    if (mp > 0.f) {                                                  // min-p
        const float mx = block_reduce_max(v, shf);
        if (v > -INFINITY && expf(v - mx) < mp) v = -INFINITY;
        __syncthreads();
    }
    if (tp < 1.f) {                                                  // top-p
        const float mx = block_reduce_max(v, shf);
        const float total = block_reduce_sum(expf(v - mx), shf);
        const float p = expf(v - mx) / total;
        const unsigned int key = float_key(v);
        unsigned int cut = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned int cand = cut | (1u << bit);
            if (block_reduce_sum(key >= cand ? p : 0.f, shf) >= tp) cut = cand;
        }
        const float above = block_reduce_sum(key > cut ? p : 0.f, shf);
        const float pv = block_reduce_max(key == cut ? p : 0.f, shf);
        int keep = 1;
        if (pv > 0.f) {
            float c = above;
            keep = 0;
            do { c += pv; ++keep; } while (c < tp && keep < m);
        }
        if (cut != 0) {
            const int before = block_exclusive_iscan(key == cut ? 1 : 0, shi);
            if (key < cut || (key == cut && before >= keep)) v = -INFINITY;
            __syncthreads();
        }
    }
    if (v != v && nan_flag) atomicExch(nan_flag, 1);
    const float mx = block_reduce_max(v, shf);
    const float total = block_reduce_sum(expf(v - mx), shf);
    const float p = expf(v - mx) / total;
    const float c = block_exclusive_scan(p, shf) + p;
    if (t == 0) *found = 0x7fffffff;
    __syncthreads();
    if (t < m && u <= c) atomicMin(found, t);
    __syncthreads();
    int r = *found;
    if (r == 0x7fffffff) {                                           // falls back to the largest (lowest index of a tie)
        const int cand = (t < m && v == mx) ? t : 0x7fffffff;
        r = block_reduce_imin(cand, shi);
        if (r == 0x7fffffff) r = 0;
    }
    return ci[r];
}

#define SAMP_ROW_SMEM_BYTES (216 * 1024)
// bytes of a padded row of n floats (see Row)
static inline size_t samp_row_bytes(int n) { return ((size_t)n + (size_t)(n >> 5) + 1) * sizeof(float); }

__global__ void __launch_bounds__(SAMP_THREADS)
sample_kernel(SampleArgs a) {
    pdl_trigger();
    pdl_wait();
    __shared__ float shf[32];
    __shared__ int shi[32];
    __shared__ int found;
    __shared__ int hist[256];
    __shared__ __align__(8) float cand_v[SAMP_THREADS];
    __shared__ int cand_i[SAMP_THREADS];
    extern __shared__ float row_s[];                     // the row itself, when it fits (a.row_in_smem)
    const int row = blockIdx.x, n = a.vocab;
    const float* in = a.logits + (size_t)row * a.ld;
    // The chain passes over the row a dozen times; a row that fits in shared memory is copied there
    // once and never touches global memory again.  Longer rows live in the caller's scratch.
    const Row x{a.row_in_smem ? row_s : a.work + (size_t)row * n, a.row_in_smem};
    const Row src{const_cast<float*>(in), 0};            // read 16 bytes at a time where it starts on 16 (row_each)
    const float temp = a.temperature[row];
    const float rp = a.rep_penalty ? a.rep_penalty[row] : 1.f;
    const bool biased = a.bias_off && a.bias_off[row + 1] > a.bias_off[row];
    const bool penalised = rp != 1.f && a.hist_off && a.hist_off[row + 1] > a.hist_off[row];
    if (!biased && !penalised) {
        // nothing touches single logits before the temperature: no copy of the row for an argmax, and the copy and
        // the division in one pass otherwise
        if (temp == 0.f) {                               // sampling.rs:82-84
            const int r = block_argmax(src, n, shf, shi, a.nan_flag);
            if (threadIdx.x == 0) a.out[row] = r;
            return;
        }
        row_each(src, n, [&](float v, int i) { x[i] = v / temp; });
    } else {
    if (x.p != in) row_each(src, n, [&](float v, int i) { x[i] = v; });
    __syncthreads();
    // logit bias: additive, one entry after another (sampling.rs:57-65)
    if (a.bias_off && threadIdx.x == 0)
        for (int i = a.bias_off[row]; i < a.bias_off[row + 1]; ++i) {
            const int t = a.bias_tok[i];
            if (t >= 0 && t < n) x[t] += a.bias_val[i];
        }
    __syncthreads();
    // repetition penalty, once per occurrence in the history (sampling.rs:68-79)
    if (rp != 1.f && a.hist_off) {
        for (int i = a.hist_off[row] + threadIdx.x; i < a.hist_off[row + 1]; i += blockDim.x) {
            const int t = a.hist_tok[i];
            if (t < 0 || t >= n) continue;
            float v = x[t];
            for (int c = 0; c < a.hist_cnt[i]; ++c) v = (v > 0.f) ? v / rp : v * rp;
            x[t] = v;
        }
    }
    __syncthreads();
    if (temp == 0.f) {                                   // sampling.rs:82-84
        const int r = block_argmax(x, n, shf, shi, a.nan_flag);
        if (threadIdx.x == 0) a.out[row] = r;
        return;
    }
    row_update(x, n, [&](float v, int) { return v / temp; });
    }
    __syncthreads();

    // top-k (sampling.rs:90-104): the k-th largest key, digit by digit
    const int k = a.top_k ? a.top_k[row] : 0;
    if (k > 0 && k < n) {
        const unsigned int cut = kth_largest_key(x, n, k, hist, shi);
        int c = 0;
        row_each(x, n, [&](float v, int) { c += (float_key(v) > cut); });
        const int above = block_reduce_isum(c, shi);
        if (k <= (int)blockDim.x) {
            // few candidates: gather them in index order (those above the cut, and the lowest
            // indices of the tie at it), and finish the chain on them alone
            const int keep_equal = k - above;
            if (!x.padded) {
                const Span sp = span_of(n);
                int eq = 0, gt = 0;
                for (int i = sp.b + sp.lane; i < sp.e; i += 32) {
                    const unsigned int key = float_key(x.p[i]);
                    eq += (key == cut);
                    gt += (key > cut);
                }
                eq = warp_isum(eq);
                gt = warp_isum(gt);
                int eq_before = warps_before(eq, shi, sp);
                const int kept_eq = max(0, min(eq, keep_equal - eq_before));
                int at = warps_before(gt + kept_eq, shi, sp);
                for (int i0 = sp.b; i0 < sp.e; i0 += 32) {
                    const int i = i0 + sp.lane;
                    const bool in = i < sp.e;
                    const float v = in ? x.p[i] : 0.f;
                    const unsigned int key = float_key(v);
                    const bool is_eq = in && key == cut;
                    const unsigned int bal_eq = __ballot_sync(0xffffffffu, is_eq);
                    const int rank = eq_before + __popc(bal_eq & ((1u << sp.lane) - 1u));
                    const bool keep = in && (key > cut || (is_eq && rank < keep_equal));
                    const unsigned int bal = __ballot_sync(0xffffffffu, keep);
                    if (keep) {
                        const int pos = at + __popc(bal & ((1u << sp.lane) - 1u));
                        cand_v[pos] = v;
                        cand_i[pos] = i;
                    }
                    eq_before += __popc(bal_eq);
                    at += __popc(bal);
                }
            } else {
            const int chunk = (n + blockDim.x - 1) / blockDim.x;
            const int b = min(n, (int)threadIdx.x * chunk), e = min(n, b + chunk);
            int eq = 0, gt = 0;
            for (int i = b; i < e; ++i) {
                const unsigned int key = float_key(x[i]);
                eq += (key == cut);
                gt += (key > cut);
            }
            int eq_before = block_exclusive_iscan(eq, shi);
            __syncthreads();
            const int kept_eq = max(0, min(eq, keep_equal - eq_before));
            int at = block_exclusive_iscan(gt + kept_eq, shi);
            for (int i = b; i < e; ++i) {
                const float v = x[i];
                const unsigned int key = float_key(v);
                bool keep = key > cut;
                if (key == cut) { keep = eq_before < keep_equal; ++eq_before; }
                if (keep) { cand_v[at] = v; cand_i[at] = i; ++at; }
            }
            }
            __syncthreads();
            const int r = sample_few(cand_v, cand_i, k, a.min_p ? a.min_p[row] : 0.f, a.top_p ? a.top_p[row] : 1.f,
                                     a.uniform[row], shf, shi, &found, a.nan_flag);
            if (threadIdx.x == 0) a.out[row] = r;
            return;
        }
        apply_cut(x, n, cut, k - above, shi);
    }

    // min-p (sampling.rs:107-118)
    const float mp = a.min_p ? a.min_p[row] : 0.f;
    if (mp > 0.f) {
        float m = -INFINITY;
        row_each(x, n, [&](float v, int) { m = fmaxf(m, v); });
        m = block_reduce_max(m, shf);
        row_update(x, n, [&](float v, int) { return (v > -INFINITY && expf(v - m) < mp) ? -INFINITY : v; });
        __syncthreads();
    }

    // top-p (sampling.rs:121-151): smallest set of largest probabilities whose sum reaches top_p
    const float tp = a.top_p ? a.top_p[row] : 1.f;
    if (tp < 1.f) {
        float m = -INFINITY;
        row_each(x, n, [&](float v, int) { m = fmaxf(m, v); });
        m = block_reduce_max(m, shf);
        float s = 0.f;
        row_each(x, n, [&](float v, int) { s += expf(v - m); });
        const float total = block_reduce_sum(s, shf);
        // the histogram of mass lives where the candidates of the few-candidates form would: that form has returned
        unsigned int* mhist = reinterpret_cast<unsigned int*>(cand_v);
        unsigned long long* shl = reinterpret_cast<unsigned long long*>(mhist + 512);
        static_assert(sizeof(float) * SAMP_THREADS >= 4 * 512 + 8, "the mass histogram outgrows the candidates' array");
        unsigned long long above_q = 0;
        const unsigned int cut = top_p_cut(x, n, m, total, (unsigned long long)((double)tp * (double)MASS_ONE), mhist, shl,
                                           shi, &above_q);
        // mass strictly above the cut, and the size of one member of the tie at the cut
        const float above = (float)((double)above_q / (double)MASS_ONE);
        float pv = 0.f;
        if (cut != 0) {
            const unsigned int b = (cut & 0x80000000u) ? (cut & 0x7fffffffu) : ~cut;      // float_key backwards
            pv = expf(__uint_as_float(b) - m) / total;
        }
        int keep = 1;
        if (pv > 0.f) {
            float c = above;
            keep = 0;
            do { c += pv; ++keep; } while (c < tp && keep < n);
        }
        if (cut != 0) apply_cut(x, n, cut, keep, shi);
    }

    // softmax and inverse CDF in index order (sampling.rs:154-170)
    float m = -INFINITY;
    row_each(x, n, [&](float v, int) {
        if (v != v && a.nan_flag) atomicExch(a.nan_flag, 1);
        m = fmaxf(m, v);
    });
    m = block_reduce_max(m, shf);
    float s = 0.f;
    row_each(x, n, [&](float v, int) { s += expf(v - m); });
    const float total = block_reduce_sum(s, shf);
    const float u = a.uniform[row];
    if (!x.padded) {
        // a warp's share of the sum, the shares before it, then along its span with a running sum across the lanes
        const Span sp = span_of(n);
        float mine = 0.f;
        for (int i = sp.b + sp.lane; i < sp.e; i += 32) mine += expf(x.p[i] - m) / total;
        mine = warp_sum(mine);
        __syncthreads();
        if (sp.lane == 0) shf[sp.warp] = mine;
        if (threadIdx.x == 0) found = 0x7fffffff;
        __syncthreads();
        float c = 0.f;
        for (int w = 0; w < sp.warp; ++w) c += shf[w];
        if (u <= c + mine * 1.001f + 1e-6f) {              // the draw may fall in this span (the walk adds in another order)
            for (int i0 = sp.b; i0 < sp.e; i0 += 32) {
                const int i = i0 + sp.lane;
                float inc = i < sp.e ? expf(x.p[i] - m) / total : 0.f;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float t = __shfl_up_sync(0xffffffffu, inc, o);
                    if (sp.lane >= o) inc += t;
                }
                const unsigned int hit = __ballot_sync(0xffffffffu, i < sp.e && u <= c + inc);
                if (hit) {
                    if (sp.lane == 0) atomicMin(&found, i0 + __ffs(hit) - 1);
                    break;
                }
                c += __shfl_sync(0xffffffffu, inc, 31);
            }
        }
        __syncthreads();
    } else {
    const int chunk = (n + blockDim.x - 1) / blockDim.x;
    const int b = min(n, (int)threadIdx.x * chunk), e = min(n, b + chunk);
    float mine = 0.f;
    for (int i = b; i < e; ++i) mine += expf(x[i] - m) / total;
    float c = block_exclusive_scan(mine, shf);
    if (threadIdx.x == 0) found = 0x7fffffff;
    __syncthreads();
    for (int i = b; i < e; ++i) {
        c += expf(x[i] - m) / total;
        if (u <= c) { atomicMin(&found, i); break; }
    }
    __syncthreads();
    }
    int r = found;
    if (r == 0x7fffffff) {
        __syncthreads();
        r = block_argmax(x, n, shf, shi, nullptr);   // sampling.rs:170 falls back to the largest
    }
    if (threadIdx.x == 0) a.out[row] = r;
}

extern "C" int braid_sample(const float* logits, float* work, long long ld, int* out, int rows, int vocab,
                            const float* temperature, const int* top_k, const float* top_p,
                            const float* min_p, const float* rep_penalty, const float* uniform,
                            const int* hist_off, const int* hist_tok, const int* hist_cnt,
                            const int* bias_off, const int* bias_tok, const float* bias_val,
                            int* nan_flag, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (vocab <= 0) BRAID_REFUSE("sample: vocab=%d must be positive", vocab);
    if (!temperature || !uniform) BRAID_REFUSE("sample: temperature and uniform arrays are required");
    // a row of up to SAMP_ROW_SMEM_BYTES stays in shared memory for the whole chain
    const size_t row_bytes = samp_row_bytes(vocab);
    const int in_smem = row_bytes <= SAMP_ROW_SMEM_BYTES;
    if (in_smem) {
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SAMP_ROW_SMEM_BYTES);
            if (e != cudaSuccess) { braid_set_error("sample: cannot reserve %d bytes of shared memory: %s", SAMP_ROW_SMEM_BYTES, cudaGetErrorString(e)); return (int)e; }
            configured = true;
        }
    } else if (!work) {
        BRAID_REFUSE("sample: a row of %d logits does not fit in shared memory and needs the work buffer", vocab);
    }
    SampleArgs a{logits, work, ld, out, vocab, temperature, top_k, top_p, min_p, rep_penalty, uniform,
                 hist_off, hist_tok, hist_cnt, bias_off, bias_tok, bias_val, nan_flag, in_smem};
    braid_launch(sample_kernel, dim3(rows), dim3(SAMP_THREADS), in_smem ? row_bytes : 0, (cudaStream_t)stream, a);
    BRAID_LAUNCH_CHECK();
}
