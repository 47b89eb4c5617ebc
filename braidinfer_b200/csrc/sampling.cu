// Token choice on the device: argmax, and the sampling chain of the reference
// (crates/braidinfer-runtime/src/sampling.rs:49-171) in its order: logit bias,
// repetition penalty, temperature (0 means argmax), top-k, min-p, top-p, softmax,
// inverse CDF with a uniform number that the caller supplies per row.
//
// One block per row of logits; all arithmetic float32.  Where the reference sorts,
// this finds the cut value by bisection on the bit pattern of the floats, and keeps
// the lowest indices of a tie at the cut (the reference's unstable sort leaves that
// order open).  Argmax returns the lowest index of the maximum.
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

// Lowest index of the largest value of x[0..n); a NaN anywhere raises *nan_flag.
__device__ int block_argmax(const float* x, int n, float* shf, int* shi, int* nan_flag) {
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    bool saw_nan = false;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = x[i];
        if (v != v) saw_nan = true;
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
    if (saw_nan && nan_flag) atomicExch(nan_flag, 1);
    const float m = block_reduce_max(best, shf);
    const int cand = (best == m) ? best_i : 0x7fffffff;
    int r = block_reduce_imin(cand, shi);
    if (r == 0x7fffffff) r = 0;     // all values were -inf or NaN
    return r;
}

__global__ void __launch_bounds__(SAMP_THREADS)
argmax_kernel(const float* __restrict__ logits, long long ld, int* __restrict__ out, int vocab, int* nan_flag) {
    pdl_trigger();
    pdl_wait();
    __shared__ float shf[32];
    __shared__ int shi[32];
    const int r = block_argmax(logits + (size_t)blockIdx.x * ld, vocab, shf, shi, nan_flag);
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
};

// Keep the `keep` lowest-index elements whose key equals `cut` and everything above
// it; set the rest to -inf.
__device__ void apply_cut(float* x, int n, unsigned int cut, int keep_equal, int* shi) {
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

__global__ void __launch_bounds__(SAMP_THREADS)
sample_kernel(SampleArgs a) {
    pdl_trigger();
    pdl_wait();
    __shared__ float shf[32];
    __shared__ int shi[32];
    __shared__ int found;
    const int row = blockIdx.x, n = a.vocab;
    const float* in = a.logits + (size_t)row * a.ld;
    float* x = a.work + (size_t)row * n;
    if (x != in)
        for (int i = threadIdx.x; i < n; i += blockDim.x) x[i] = in[i];
    __syncthreads();
    // logit bias: additive, one entry after another (sampling.rs:57-65)
    if (a.bias_off && threadIdx.x == 0)
        for (int i = a.bias_off[row]; i < a.bias_off[row + 1]; ++i) {
            const int t = a.bias_tok[i];
            if (t >= 0 && t < n) x[t] += a.bias_val[i];
        }
    __syncthreads();
    // repetition penalty, once per occurrence in the history (sampling.rs:68-79)
    const float rp = a.rep_penalty ? a.rep_penalty[row] : 1.f;
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
    const float temp = a.temperature[row];
    if (temp == 0.f) {                                   // sampling.rs:82-84
        const int r = block_argmax(x, n, shf, shi, a.nan_flag);
        if (threadIdx.x == 0) a.out[row] = r;
        return;
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x) x[i] = x[i] / temp;
    __syncthreads();

    // top-k (sampling.rs:90-104): the k-th largest key by bisection
    const int k = a.top_k ? a.top_k[row] : 0;
    if (k > 0 && k < n) {
        unsigned int cut = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned int cand = cut | (1u << bit);
            int c = 0;
            for (int i = threadIdx.x; i < n; i += blockDim.x) c += (float_key(x[i]) >= cand);
            if (block_reduce_isum(c, shi) >= k) cut = cand;
        }
        int c = 0;
        for (int i = threadIdx.x; i < n; i += blockDim.x) c += (float_key(x[i]) > cut);
        const int above = block_reduce_isum(c, shi);
        apply_cut(x, n, cut, k - above, shi);
    }

    // min-p (sampling.rs:107-118)
    const float mp = a.min_p ? a.min_p[row] : 0.f;
    if (mp > 0.f) {
        float m = -INFINITY;
        for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, x[i]);
        m = block_reduce_max(m, shf);
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float v = x[i];
            if (v > -INFINITY && expf(v - m) < mp) x[i] = -INFINITY;
        }
        __syncthreads();
    }

    // top-p (sampling.rs:121-151): smallest set of largest probabilities whose sum reaches top_p
    const float tp = a.top_p ? a.top_p[row] : 1.f;
    if (tp < 1.f) {
        float m = -INFINITY;
        for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, x[i]);
        m = block_reduce_max(m, shf);
        float s = 0.f;
        for (int i = threadIdx.x; i < n; i += blockDim.x) s += expf(x[i] - m);
        const float total = block_reduce_sum(s, shf);
        unsigned int cut = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned int cand = cut | (1u << bit);
            float ms = 0.f;
            for (int i = threadIdx.x; i < n; i += blockDim.x)
                if (float_key(x[i]) >= cand) ms += expf(x[i] - m) / total;
            if (block_reduce_sum(ms, shf) >= tp) cut = cand;
        }
        // mass strictly above the cut, and the size of one member of the tie at the cut
        float ms = 0.f, pv = 0.f;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const unsigned int key = float_key(x[i]);
            if (key > cut) ms += expf(x[i] - m) / total;
            else if (key == cut) pv = expf(x[i] - m) / total;
        }
        const float above = block_reduce_sum(ms, shf);
        pv = block_reduce_max(pv, shf);
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
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = x[i];
        if (v != v && a.nan_flag) atomicExch(a.nan_flag, 1);
        m = fmaxf(m, v);
    }
    m = block_reduce_max(m, shf);
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += expf(x[i] - m);
    const float total = block_reduce_sum(s, shf);
    const int chunk = (n + blockDim.x - 1) / blockDim.x;
    const int b = min(n, (int)threadIdx.x * chunk), e = min(n, b + chunk);
    float mine = 0.f;
    for (int i = b; i < e; ++i) mine += expf(x[i] - m) / total;
    float c = block_exclusive_scan(mine, shf);
    if (threadIdx.x == 0) found = 0x7fffffff;
    __syncthreads();
    const float u = a.uniform[row];
    for (int i = b; i < e; ++i) {
        c += expf(x[i] - m) / total;
        if (u <= c) { atomicMin(&found, i); break; }
    }
    __syncthreads();
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
    SampleArgs a{logits, work, ld, out, vocab, temperature, top_k, top_p, min_p, rep_penalty, uniform,
                 hist_off, hist_tok, hist_cnt, bias_off, bias_tok, bias_val, nan_flag};
    braid_launch(sample_kernel, dim3(rows), dim3(SAMP_THREADS), 0, (cudaStream_t)stream, a);
    BRAID_LAUNCH_CHECK();
}
