// Kernels that add up the partial products of a stream-k GEMM and go straight on with
// what follows the product, for steps of few tokens (up to a few hundred) where every launch counts:
//
//   braid_streamk_reduce_norm     h = h + sum (the residual sum, float32, written back),
//                                 then RMSNorm of the new h: out = h * rsqrt(mean(h^2) + eps) * w.
//                                 One CTA of up to 1024 threads a row, so that the row's sum of
//                                 squares needs one block-wide sum and nothing between CTAs.
//   braid_streamk_reduce_rope_kv  qkv = sum, rotary encoding of the query and key heads,
//                                 keys and values into the paged cache (what elementwise.cu's
//                                 rope_kv_kernel does after a plain product).
//   braid_streamk_reduce_prep     h = h + sum, and what an RMSNorm whose scale is left to the next
//                                 product needs (rowscale.cuh): bfloat16(h * w) and each CTA's share
//                                 of the rows' sums of squares.  A CTA owns 512 columns of one row, so
//                                 a step of 8 rows of 4096 is finished by 64 CTAs, not by 8.
//
// Formulas are those of the unfused kernels (elementwise.cu cites the reference lines).
#include "common.cuh"
#include "rowscale.cuh"
#include "streamk.cuh"
#include "trace.cuh"

// Slots of a traced reduce + norm launch: 0 entry, 1 before the dependency wait, 2 after it,
// 3 partial sums and row loaded and added, 4 block-wide sum done, 5 stored.
BRAID_TRACE_BUFFER(reduce_norm, 64)

#define RN_MAX_THREADS 1024

// One CTA per output row, one thread per group of four columns (a thread takes further groups
// in turn when the row is wider than four times the block).  The first group of a thread
// stays in registers between the two passes, so a row of up to 4096 columns is read once.
template <typename TW, typename TO>
__global__ void __launch_bounds__(RN_MAX_THREADS)
streamk_reduce_norm_kernel(StreamK k, float* h, const TW* __restrict__ w, TO* __restrict__ out,
                           const int* __restrict__ row_index, int width, float eps) {
#ifdef BRAID_TRACE
    unsigned long long* trace_row = nullptr;
    if (threadIdx.x == 0) {
        trace_row = braid_trace_open(reduce_norm, 64);
        BRAID_STAMP(trace_row, 0);
    }
#endif
    pdl_trigger();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const int src = row_index ? row_index[r] : r;       // the step's tables are on the device before its first kernel
    const bool write_back = (row_index == nullptr);      // gathered rows may repeat: leave h alone
    const int groups = (width + 3) / 4;                  // groups of four columns
    const bool vec = (width & 3) == 0;                   // rows of h start on 16 bytes
    TO* o = out + (size_t)r * width;
    float ss = 0.f;
    // where this thread's first group of partial sums lies, and the norm's weights of that group
    // (no kernel writes them), are worked out before the wait
    const int g_first = threadIdx.x;
    StreamKSpan sp_first = {};
    float w_first[4] = {0.f, 0.f, 0.f, 0.f};
    if (src >= 0 && g_first < groups) {
        sp_first = streamk_span(k, src, g_first * 4);
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (g_first * 4 + e < width) w_first[e] = to_f32(w[g_first * 4 + e]);
    }
    BRAID_STAMP(trace_row, 1);
    pdl_wait();
    BRAID_STAMP(trace_row, 2);
    float v_first[4] = {0.f, 0.f, 0.f, 0.f};              // the new h of this thread's first group
    if (src >= 0) {
        float* hr = h + (size_t)src * width;
        for (int g = g_first; g < groups; g += blockDim.x) {
            const int c = g * 4;
            // the row's old values are asked for before the partial sums are added up: one trip for all
            float old[4] = {0.f, 0.f, 0.f, 0.f};
            if (vec) {
                const float4 o4 = *reinterpret_cast<const float4*>(hr + c);
                old[0] = o4.x; old[1] = o4.y; old[2] = o4.z; old[3] = o4.w;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (c + e < width) old[e] = hr[c + e];
            }
            const float4 s4 = streamk_sum4(k, g == g_first ? sp_first : streamk_span(k, src, c), src, c);
            const float s[4] = {s4.x, s4.y, s4.z, s4.w};
            float v[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                v[e] = (c + e < width) ? old[e] + s[e] : 0.f;
                ss = fmaf(v[e], v[e], ss);
            }
            if (write_back) {
                if (vec) *reinterpret_cast<float4*>(hr + c) = make_float4(v[0], v[1], v[2], v[3]);
                else {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (c + e < width) hr[c + e] = v[e];
                }
            }
            if (g == g_first) { v_first[0] = v[0]; v_first[1] = v[1]; v_first[2] = v[2]; v_first[3] = v[3]; }
        }
    }
    BRAID_STAMP(trace_row, 3);
    const float total = block_sum(ss, red);
    BRAID_STAMP(trace_row, 4);
    if (src < 0) {
        for (int g = g_first; g < groups; g += blockDim.x)
            for (int e = 0; e < 4 && g * 4 + e < width; ++e) o[g * 4 + e] = from_f32<TO>(0.f);
        return;
    }
    const float scale = rsqrtf(total / (float)width + eps);
    const float* hr = h + (size_t)src * width;
    for (int g = g_first; g < groups; g += blockDim.x) {
        const int c = g * 4;
        if (g == g_first) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (c + e < width) o[c + e] = from_f32<TO>(v_first[e] * scale * w_first[e]);
            continue;
        }
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        if (!write_back) {
            const float4 s4 = streamk_sum4(k, streamk_span(k, src, c), src, c);
            s[0] = s4.x; s[1] = s4.y; s[2] = s4.z; s[3] = s4.w;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (c + e >= width) break;
            const float v = hr[c + e] + s[e];             // written back above by this very thread, or recomputed
            o[c + e] = from_f32<TO>(v * scale * to_f32(w[c + e]));
        }
    }
    BRAID_STAMP(trace_row, 5);
}

extern "C" int braid_streamk_reduce_norm(const float* partial, const int* plan, int n_rows, float* h, const void* w,
                                         int w_dtype, void* out, int out_dtype, const int* row_index, int rows_out,
                                         int width, float eps, void* stream) {
    if (rows_out <= 0) return BRAID_OK;
    if (width <= 0) BRAID_REFUSE("reduce_norm: width=%d must be positive", width);
    const StreamK k = streamk_from_plan(partial, plan, n_rows);
    const int groups = (width + 3) / 4;
    int threads = ((groups + 31) / 32) * 32;
    if (threads > RN_MAX_THREADS) threads = RN_MAX_THREADS;
    cudaStream_t s = (cudaStream_t)stream;
#define RN_LAUNCH(TW, TO) braid_launch(streamk_reduce_norm_kernel<TW, TO>, dim3(rows_out), dim3(threads), 0, s, k, h, (const TW*)w, (TO*)out, row_index, width, eps)
    if (w_dtype == BRAID_F32 && out_dtype == BRAID_F32) RN_LAUNCH(float, float);
    else if (w_dtype == BRAID_F32 && out_dtype == BRAID_BF16) RN_LAUNCH(float, __nv_bfloat16);
    else if (w_dtype == BRAID_BF16 && out_dtype == BRAID_F32) RN_LAUNCH(__nv_bfloat16, float);
    else if (w_dtype == BRAID_BF16 && out_dtype == BRAID_BF16) RN_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else BRAID_REFUSE("reduce_norm: unknown dtype codes w=%d out=%d", w_dtype, out_dtype);
#undef RN_LAUNCH
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ reduce + what a scaled norm needs
#define PREP_THREADS 128
#define PREP_COLS (PREP_THREADS * 4)           // columns of a row that one CTA owns

// h[row, c..] += sum of the partial products (k.partial null: h is complete already), hb = bfloat16(h * w),
// shares[blockIdx.x][row] = sum over the CTA's columns of h^2.  Width a multiple of 4, rows of h and hb
// start on 16 and 8 bytes.
template <typename TW>
__global__ void __launch_bounds__(PREP_THREADS)
streamk_reduce_prep_kernel(StreamK k, float* __restrict__ h, const TW* __restrict__ w, __nv_bfloat16* __restrict__ hb,
                           float* __restrict__ shares, long long share_stride, int width) {
    pdl_trigger();
    __shared__ float red[PREP_THREADS / 32];
    const int row = blockIdx.y;
    const int c = blockIdx.x * PREP_COLS + threadIdx.x * 4;
    const bool live = c < width;
    // where the partial sums lie and the norm's weights (no kernel writes them): before the wait
    StreamKSpan sp = {};
    float g[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
        if (k.partial) sp = streamk_span(k, row, c);
#pragma unroll
        for (int e = 0; e < 4; ++e) g[e] = to_f32(w[c + e]);
    }
    pdl_wait();
    float ss = 0.f;
    if (live) {
        float* hr = h + (size_t)row * width + c;
        const float4 old = *reinterpret_cast<const float4*>(hr);
        float4 v = old;
        if (k.partial) {
            const float4 s4 = streamk_sum4(k, sp, row, c);
            v = make_float4(old.x + s4.x, old.y + s4.y, old.z + s4.z, old.w + s4.w);
            *reinterpret_cast<float4*>(hr) = v;
        }
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * g[0], v.y * g[1]), hi = __floats2bfloat162_rn(v.z * g[2], v.w * g[3]);
        uint2 pk;
        pk.x = *reinterpret_cast<unsigned int*>(&lo);
        pk.y = *reinterpret_cast<unsigned int*>(&hi);
        *reinterpret_cast<uint2*>(hb + (size_t)row * width + c) = pk;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = red[0];
#pragma unroll
        for (int i = 1; i < PREP_THREADS / 32; ++i) total += red[i];
        shares[(size_t)blockIdx.x * share_stride + row] = total;
    }
}

// `partial` and `plan` null: h is complete and only hb and the shares are made.  shares: [ceil(width / 512)][share_stride].
extern "C" int braid_streamk_reduce_prep(const float* partial, const int* plan, int n_rows, float* h, const void* w,
                                         int w_dtype, void* hb, float* shares, long long share_stride, int width,
                                         void* stream) {
    if (n_rows <= 0) return BRAID_OK;
    if (width <= 0 || (width & 3)) BRAID_REFUSE("reduce_prep: width=%d must be a positive multiple of 4", width);
    if (((uintptr_t)h & 15) || ((uintptr_t)hb & 7)) BRAID_REFUSE("reduce_prep: h and hb must be aligned to 16 and 8 bytes");
    if (!shares || share_stride < n_rows) BRAID_REFUSE("reduce_prep: shares with a stride of at least %d are required", n_rows);
    if ((partial == nullptr) != (plan == nullptr)) BRAID_REFUSE("reduce_prep: partial sums come with their plan");
    if (n_rows > 65535) BRAID_REFUSE("reduce_prep: %d rows exceed the grid limit", n_rows);
    StreamK k = {};
    if (partial) k = streamk_from_plan(partial, plan, n_rows);
    const dim3 grid((width + PREP_COLS - 1) / PREP_COLS, n_rows);
    cudaStream_t s = (cudaStream_t)stream;
    if (w_dtype == BRAID_F32)
        braid_launch(streamk_reduce_prep_kernel<float>, grid, dim3(PREP_THREADS), 0, s, k, h, (const float*)w, (__nv_bfloat16*)hb, shares, share_stride, width);
    else if (w_dtype == BRAID_BF16)
        braid_launch(streamk_reduce_prep_kernel<__nv_bfloat16>, grid, dim3(PREP_THREADS), 0, s, k, h, (const __nv_bfloat16*)w, (__nv_bfloat16*)hb, shares, share_stride, width);
    else BRAID_REFUSE("reduce_prep: unknown dtype code w=%d", w_dtype);
    BRAID_LAUNCH_CHECK();
}
extern "C" int braid_streamk_reduce_prep_cols(void) { return PREP_COLS; }

// ------------------------------------------------------------------ reduce + rotary + cache write
struct ReduceRopeArgs {
    StreamK k;
    __nv_bfloat16* qkv;          // [rows, (nqh + 2 nkh) * hd], written here
    const float* inv_freq;
    const int* positions;
    const int* token_seq;
    const int* page_table;
    __nv_bfloat16* cache;        // one layer, or null (no write)
    int rows, nqh, nkh, hd, rope_dim, adjacent;
    int page_size, table_cols, num_pages;
    int* error_flag;
    const float* rs_rows;        // the scale of every row that the product's input still wants (rowscale.cuh), or null
};

__global__ void streamk_reduce_rope_kv_kernel(ReduceRopeArgs a) {
    pdl_trigger();
    // Up to pdl_wait(): the step's tables (on the device before the step's first kernel), the
    // rotation angle and the places of the partial sums; the partial sums themselves after it.
    const int row = blockIdx.x;
    const int seq = a.token_seq[row];
    if (seq < 0) return;
    const int head = blockIdx.y;
    const int pos = a.positions[row];
    const int width = (a.nqh + 2 * a.nkh) * a.hd;
    const int col0 = head * a.hd;
    __nv_bfloat16* dst_row = a.qkv + (size_t)row * width + col0;
    const bool is_q = head < a.nqh;
    const bool is_k = !is_q && head < a.nqh + a.nkh;
    __nv_bfloat16* dst = nullptr;
    if (!is_q && a.cache) {
        const int kvh = is_k ? head - a.nqh : head - a.nqh - a.nkh;
        const int block = pos / a.page_size, off = pos - block * a.page_size;
        int page = (block < a.table_cols) ? a.page_table[(size_t)seq * a.table_cols + block] : -1;
        if (page < 0 || page >= a.num_pages) {
            if (threadIdx.x == 0) atomicExch(a.error_flag, 1);
            page = -1;
        }
        if (page >= 0)
            dst = a.cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * a.nkh + kvh) * a.page_size + off) * a.hd;
    }
    const int half = a.rope_dim / 2;
    if (is_q || is_k) {
        // the first pair of this thread (the only one when head_dim / 2 <= blockDim.x)
        const int p_first = threadIdx.x;
        float sn0 = 0.f, cs0 = 1.f;
        StreamKSpan sp0 = {}, sp1 = {};
        if (p_first < half) {
            sincosf((float)pos * a.inv_freq[p_first], &sn0, &cs0);
            sp0 = streamk_span(a.k, row, col0 + (a.adjacent ? 2 * p_first : p_first));
            sp1 = streamk_span(a.k, row, col0 + (a.adjacent ? 2 * p_first + 1 : p_first + half));
        }
        pdl_wait();
        const float rs = a.rs_rows ? a.rs_rows[row] : 1.f;     // asked for with the first partial sums: one trip
        for (int p = threadIdx.x; p < half; p += blockDim.x) {
            const int i0 = a.adjacent ? 2 * p : p;
            const int i1 = a.adjacent ? 2 * p + 1 : p + half;
            float sn = sn0, cs = cs0;
            StreamKSpan s0 = sp0, s1 = sp1;
            if (p != p_first) {
                sincosf((float)pos * a.inv_freq[p], &sn, &cs);
                s0 = streamk_span(a.k, row, col0 + i0);
                s1 = streamk_span(a.k, row, col0 + i1);
            }
            // the product is rounded to bfloat16 before it is rotated, as after a plain product
            float f0, f1;
            streamk_sum_pair(a.k, s0, s1, row, col0 + i0, col0 + i1, f0, f1);
            const float x0 = __bfloat162float(__float2bfloat16_rn(f0 * rs));
            const float x1 = __bfloat162float(__float2bfloat16_rn(f1 * rs));
            const __nv_bfloat16 y0 = __float2bfloat16_rn(x0 * cs - x1 * sn);
            const __nv_bfloat16 y1 = __float2bfloat16_rn(x0 * sn + x1 * cs);
            dst_row[i0] = y0;
            dst_row[i1] = y1;
            if (dst) { dst[i0] = y0; dst[i1] = y1; }
        }
        for (int i = a.rope_dim + threadIdx.x; i < a.hd; i += blockDim.x) {
            const __nv_bfloat16 y = __float2bfloat16_rn(streamk_sum(a.k, streamk_span(a.k, row, col0 + i), row, col0 + i) * rs);
            dst_row[i] = y;
            if (dst) dst[i] = y;
        }
    } else {
        const int i_first = threadIdx.x;
        StreamKSpan sp0 = {};
        if (i_first < a.hd) sp0 = streamk_span(a.k, row, col0 + i_first);
        pdl_wait();
        const float rs = a.rs_rows ? a.rs_rows[row] : 1.f;
        for (int i = threadIdx.x; i < a.hd; i += 2 * blockDim.x) {
            const StreamKSpan s0 = (i == i_first) ? sp0 : streamk_span(a.k, row, col0 + i);
            const int i2 = i + blockDim.x;                  // a thread's elements go two at a time
            if (i2 < a.hd) {
                float f0, f1;
                streamk_sum_pair(a.k, s0, streamk_span(a.k, row, col0 + i2), row, col0 + i, col0 + i2, f0, f1);
                const __nv_bfloat16 y0 = __float2bfloat16_rn(f0 * rs), y1 = __float2bfloat16_rn(f1 * rs);
                dst_row[i] = y0; dst_row[i2] = y1;
                if (dst) { dst[i] = y0; dst[i2] = y1; }
            } else {
                const __nv_bfloat16 y = __float2bfloat16_rn(streamk_sum(a.k, s0, row, col0 + i) * rs);
                dst_row[i] = y;
                if (dst) dst[i] = y;
            }
        }
    }
}

extern "C" int braid_streamk_reduce_rope_kv(const float* partial, const int* plan, void* qkv, const float* inv_freq,
                                            const int* positions, const int* token_seq, const int* page_table,
                                            void* cache, int rows, int nqh, int nkh, int hd, int rope_dim, int adjacent,
                                            int page_size, int table_cols, int num_pages, const float* rs_rows,
                                            int* error_flag, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (nqh <= 0 || nkh <= 0 || hd <= 0) BRAID_REFUSE("reduce_rope_kv: heads/head_dim must be positive");
    if (rope_dim < 0 || rope_dim > hd || (rope_dim & 1)) BRAID_REFUSE("reduce_rope_kv: rope_dim=%d must be even and <= head_dim=%d", rope_dim, hd);
    if (nqh + 2 * nkh > 65535) BRAID_REFUSE("reduce_rope_kv: %d heads exceed the grid limit", nqh + 2 * nkh);
    ReduceRopeArgs a{streamk_from_plan(partial, plan, rows),
                     (__nv_bfloat16*)qkv, inv_freq, positions, token_seq, page_table, (__nv_bfloat16*)cache,
                     rows, nqh, nkh, hd, rope_dim, adjacent, page_size, table_cols, num_pages, error_flag, rs_rows};
    braid_launch(streamk_reduce_rope_kv_kernel, dim3(rows, nqh + 2 * nkh), dim3(hd >= 128 ? 64 : 32), 0, (cudaStream_t)stream, a);
    BRAID_LAUNCH_CHECK();
}
