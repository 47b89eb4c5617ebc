// Row-wise kernels: embedding gather, RMSNorm, SiLU*up, residual add, rotary encoding
// with the write of keys and values into the paged cache.
//
// Formulas follow the reference ops they replace (by that project's paths):
//   embedding      kernels/megakernel_ops.hip:1757-1768
//   rmsnorm        kernels/megakernel_ops.hip:862-904
//   silu * up      kernels/megakernel_ops.hip:374-407
//   residual add   kernels/megakernel_ops.hip:1185-1212
//   rotation       kernels/megakernel_ops.hip:2019-2030 (adjacent pairs)
//   cache write    kernels/op_kv_write_paged_batch.hip:38-78
// The residual stream is float32 in both run modes; sums of squares, rsqrt, angles,
// sin/cos and the residual sum are float32.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int n_tokens, int hidden, int vocab) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    int id = ids[t];
    const bool valid = (id >= 0 && id < vocab);
    const T* row = table + (size_t)(valid ? id : 0) * hidden;
    float* o = out + (size_t)t * hidden;
    // rows that start on 16 bytes and hold a whole number of 16-byte groups go group by group
    constexpr int VEC = 16 / sizeof(T);
    if (valid && hidden % VEC == 0 && (((uintptr_t)row | (uintptr_t)o) & 15) == 0) {
        for (int g = threadIdx.x; g < hidden / VEC; g += blockDim.x) {
            T v[VEC];
            *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(row + g * VEC);
#pragma unroll
            for (int e = 0; e < VEC; e += 4)
                *reinterpret_cast<float4*>(o + g * VEC + e) = make_float4(to_f32(v[e]), to_f32(v[e + 1]), to_f32(v[e + 2]), to_f32(v[e + 3]));
        }
        return;
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = valid ? to_f32(row[i]) : 0.f;
}

extern "C" int braid_embed(const void* table, int table_dtype, const int* ids, float* out,
                           int n_tokens, int hidden, int vocab, void* stream) {
    if (n_tokens <= 0) return BRAID_OK;
    if (hidden <= 0 || vocab <= 0) BRAID_REFUSE("embed: hidden=%d vocab=%d must be positive", hidden, vocab);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == BRAID_F32)
        braid_launch(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const float*)table, ids, out, n_tokens, hidden, vocab);
    else if (table_dtype == BRAID_BF16)
        braid_launch(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, (const __nv_bfloat16*)table, ids, out, n_tokens, hidden, vocab);
    else
        BRAID_REFUSE("embed: unknown table dtype code %d", table_dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ rmsnorm
// One block per output row.  `row_index` (may be null) picks the input row of each
// output row, which gathers the rows whose logits are wanted before the final norm.
template <typename TW, typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ row_index, int rows, int width, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const int r = blockIdx.x;
    if (r >= rows) return;
    const int src = row_index ? row_index[r] : r;
    TO* o = out + (size_t)r * width;
    if (src < 0) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<TO>(0.f);
        return;
    }
    const float* xr = x + (size_t)src * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = from_f32<TO>(xr[i] * scale * to_f32(w[i]));
}

// Rows whose width is a multiple of 4 (and at most 4 * 8 * 512): one pass over x with
// 16-byte loads, the row kept in registers between the sum of squares and the scaling.
template <typename TW, typename TO, int PER>
__global__ void __launch_bounds__(512)
rmsnorm_vec_kernel(const float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                   const int* __restrict__ row_index, int rows, int width, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const int src = row_index ? row_index[r] : r;
    TO* o = out + (size_t)r * width;
    const int groups = width >> 2;
    if (src < 0) {
        for (int g = threadIdx.x; g < groups; g += blockDim.x)
            for (int e = 0; e < 4; ++e) o[g * 4 + e] = from_f32<TO>(0.f);
        return;
    }
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * width);
    float4 v[PER];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int g = threadIdx.x + i * blockDim.x;
        if (g < groups) {
            v[i] = xr[g];
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / (float)width + eps);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int g = threadIdx.x + i * blockDim.x;
        if (g < groups) {
            const int c = g * 4;
            const float y0 = v[i].x * scale * to_f32(w[c]), y1 = v[i].y * scale * to_f32(w[c + 1]);
            const float y2 = v[i].z * scale * to_f32(w[c + 2]), y3 = v[i].w * scale * to_f32(w[c + 3]);
            if (sizeof(TO) == 2) {
                __nv_bfloat162 a = __floats2bfloat162_rn(y0, y1), b = __floats2bfloat162_rn(y2, y3);
                uint2 pk;
                pk.x = *reinterpret_cast<unsigned int*>(&a);
                pk.y = *reinterpret_cast<unsigned int*>(&b);
                *reinterpret_cast<uint2*>(o + c) = pk;
            } else {
                *reinterpret_cast<float4*>(o + c) = make_float4(y0, y1, y2, y3);
            }
        }
    }
}

extern "C" int braid_rmsnorm(const float* x, const void* w, int w_dtype, void* out, int out_dtype,
                             const int* row_index, int rows, int width, float eps, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (width <= 0) BRAID_REFUSE("rmsnorm: width=%d must be positive", width);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    const bool aligned = (width % 4 == 0) && (((uintptr_t)x & 15) == 0) && (((uintptr_t)out & 15) == 0);
    if (aligned && width <= 4 * 8 * threads) {
        const int per = (width / 4 + threads - 1) / threads;          // float4 groups a thread
#define BRAID_RMSV(TW, TO)                                                                                           \
        do {                                                                                                         \
            if (per <= 1) braid_launch(rmsnorm_vec_kernel<TW, TO, 1>, dim3(rows), dim3(threads), 0, s, x, (const TW*)w, (TO*)out, row_index, rows, width, eps); \
            else if (per <= 2) braid_launch(rmsnorm_vec_kernel<TW, TO, 2>, dim3(rows), dim3(threads), 0, s, x, (const TW*)w, (TO*)out, row_index, rows, width, eps); \
            else if (per <= 4) braid_launch(rmsnorm_vec_kernel<TW, TO, 4>, dim3(rows), dim3(threads), 0, s, x, (const TW*)w, (TO*)out, row_index, rows, width, eps); \
            else braid_launch(rmsnorm_vec_kernel<TW, TO, 8>, dim3(rows), dim3(threads), 0, s, x, (const TW*)w, (TO*)out, row_index, rows, width, eps); \
        } while (0)
        if (w_dtype == BRAID_F32 && out_dtype == BRAID_F32) BRAID_RMSV(float, float);
        else if (w_dtype == BRAID_F32 && out_dtype == BRAID_BF16) BRAID_RMSV(float, __nv_bfloat16);
        else if (w_dtype == BRAID_BF16 && out_dtype == BRAID_F32) BRAID_RMSV(__nv_bfloat16, float);
        else if (w_dtype == BRAID_BF16 && out_dtype == BRAID_BF16) BRAID_RMSV(__nv_bfloat16, __nv_bfloat16);
        else BRAID_REFUSE("rmsnorm: unknown dtype codes w=%d out=%d", w_dtype, out_dtype);
#undef BRAID_RMSV
        BRAID_LAUNCH_CHECK();
    }
#define BRAID_RMS(TW, TO) braid_launch(rmsnorm_kernel<TW, TO>, dim3(rows), dim3(threads), 0, s, x, (const TW*)w, (TO*)out, row_index, rows, width, eps)
    if (w_dtype == BRAID_F32 && out_dtype == BRAID_F32) BRAID_RMS(float, float);
    else if (w_dtype == BRAID_F32 && out_dtype == BRAID_BF16) BRAID_RMS(float, __nv_bfloat16);
    else if (w_dtype == BRAID_BF16 && out_dtype == BRAID_F32) BRAID_RMS(__nv_bfloat16, float);
    else if (w_dtype == BRAID_BF16 && out_dtype == BRAID_BF16) BRAID_RMS(__nv_bfloat16, __nv_bfloat16);
    else BRAID_REFUSE("rmsnorm: unknown dtype codes w=%d out=%d", w_dtype, out_dtype);
#undef BRAID_RMS
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ silu(gate) * up
// gu is [rows, 2*inter]: gate in columns [0, inter), up in [inter, 2*inter).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long long total, int inter) {
    pdl_trigger();
    pdl_wait();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long r = i / inter;
    const int c = (int)(i - r * inter);
    const float g = to_f32(gu[r * 2 * inter + c]);
    const float u = to_f32(gu[r * 2 * inter + inter + c]);
    out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
}

extern "C" int braid_silu_mul(const void* gu, void* out, int dtype, int rows, int inter, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (inter <= 0) BRAID_REFUSE("silu_mul: inter=%d must be positive", inter);
    const long long total = (long long)rows * inter;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("silu_mul: %lld elements exceed one launch", total);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BRAID_F32) braid_launch(silu_mul_kernel<float>, dim3((int)blocks), dim3(threads), 0, s, (const float*)gu, (float*)out, total, inter);
    else if (dtype == BRAID_BF16) braid_launch(silu_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, total, inter);
    else BRAID_REFUSE("silu_mul: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ residual add
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ h, const T* __restrict__ delta, long long total) {
    pdl_trigger();
    pdl_wait();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) h[i] = h[i] + to_f32(delta[i]);
}

extern "C" int braid_residual_add(float* h, const void* delta, int delta_dtype, long long total, void* stream) {
    if (total <= 0) return BRAID_OK;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("residual_add: %lld elements exceed one launch", total);
    cudaStream_t s = (cudaStream_t)stream;
    if (delta_dtype == BRAID_F32) braid_launch(residual_add_kernel<float>, dim3((int)blocks), dim3(threads), 0, s, h, (const float*)delta, total);
    else if (delta_dtype == BRAID_BF16) braid_launch(residual_add_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, s, h, (const __nv_bfloat16*)delta, total);
    else BRAID_REFUSE("residual_add: unknown dtype code %d", delta_dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ rotary + cache write
// qkv: [rows, (nqh + 2*nkh) * hd], heads in the order q..., k..., v....
// Queries are rotated in place.  Keys are rotated and written to the cache (and in
// place); values are copied to the cache.  A row whose token_seq is negative is
// padding and is left alone.  Cache of one layer: [page][2][nkh][page_size][hd].
struct RopeKvArgs {
    void* qkv;
    const float* inv_freq;       // [rope_dim / 2]
    const int* positions;        // [rows]
    const int* token_seq;        // [rows], index into the step's sequences, or -1
    const int* page_table;       // [n_seqs, table_cols], page of each logical block
    void* cache;                 // base of the layer's pool, or null (no write)
    int rows, nqh, nkh, hd, rope_dim, adjacent;
    int page_size, table_cols, num_pages;
    int* error_flag;
};

template <typename T>
__global__ void rope_kv_kernel(RopeKvArgs a) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int seq = a.token_seq[row];
    if (seq < 0) return;
    const int head = blockIdx.y;                     // [0, nqh + 2 nkh)
    const int pos = a.positions[row];
    const int width = (a.nqh + 2 * a.nkh) * a.hd;
    T* src = (T*)a.qkv + (size_t)row * width + (size_t)head * a.hd;
    const bool is_q = head < a.nqh;
    const bool is_k = !is_q && head < a.nqh + a.nkh;
    T* dst = nullptr;
    if (!is_q && a.cache) {
        const int kvh = is_k ? head - a.nqh : head - a.nqh - a.nkh;
        const int block = pos / a.page_size, off = pos - block * a.page_size;
        int page = (block < a.table_cols) ? a.page_table[(size_t)seq * a.table_cols + block] : -1;
        if (page < 0 || page >= a.num_pages) {
            if (threadIdx.x == 0) atomicExch(a.error_flag, 1);
            page = -1;
        }
        if (page >= 0)
            dst = (T*)a.cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * a.nkh + kvh) * a.page_size + off) * a.hd;
    }
    const int half = a.rope_dim / 2;
    if (is_q || is_k) {
        for (int p = threadIdx.x; p < half; p += blockDim.x) {
            const int i0 = a.adjacent ? 2 * p : p;
            const int i1 = a.adjacent ? 2 * p + 1 : p + half;
            const float ang = (float)pos * a.inv_freq[p];
            float sn, cs;
            sincosf(ang, &sn, &cs);
            const float x0 = to_f32(src[i0]), x1 = to_f32(src[i1]);
            const T y0 = from_f32<T>(x0 * cs - x1 * sn);
            const T y1 = from_f32<T>(x0 * sn + x1 * cs);
            src[i0] = y0;
            src[i1] = y1;
            if (dst) { dst[i0] = y0; dst[i1] = y1; }
        }
        if (dst)
            for (int i = a.rope_dim + threadIdx.x; i < a.hd; i += blockDim.x) dst[i] = src[i];
    } else if (dst) {
        for (int i = threadIdx.x; i < a.hd; i += blockDim.x) dst[i] = src[i];
    }
}

// One block per token; angles computed once per (token, pair) and shared by all heads;
// 16-byte loads and stores.  Needs head_dim and rope_dim to be multiples of 2 * VEC
// (VEC = 8 for bfloat16, 4 for float32) and 16-byte aligned rows.
template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_vec_kernel(RopeKvArgs a) {
    pdl_trigger();
    pdl_wait();
    constexpr int VEC = 16 / sizeof(T);
    extern __shared__ float cs_sn[];                   // [rope_dim / 2] cosines, then sines
    const int row = blockIdx.x;
    const int seq = a.token_seq[row];
    if (seq < 0) return;
    const int pos = a.positions[row];
    const int half = a.rope_dim / 2;
    for (int p = threadIdx.x; p < half; p += blockDim.x) sincosf((float)pos * a.inv_freq[p], &cs_sn[half + p], &cs_sn[p]);
    const int width = (a.nqh + 2 * a.nkh) * a.hd;
    T* base = (T*)a.qkv + (size_t)row * width;
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (a.cache) {
        const int block = pos / a.page_size, off = pos - block * a.page_size;
        int page = (block < a.table_cols) ? a.page_table[(size_t)seq * a.table_cols + block] : -1;
        if (page < 0 || page >= a.num_pages) {
            if (threadIdx.x == 0) atomicExch(a.error_flag, 1);
        } else {
            kdst = (T*)a.cache + (((size_t)page * 2) * a.nkh * a.page_size + off) * a.hd;       // + kvh * page_size * hd
            vdst = kdst + (size_t)a.nkh * a.page_size * a.hd;
        }
    }
    __syncthreads();
    const int rot_vecs = a.adjacent ? a.rope_dim / VEC : half / VEC;      // vectors a head's rotation takes
    const int pass_vecs = (a.hd - a.rope_dim) / VEC;                      // unrotated tail of a q/k head
    const int qk_heads = a.nqh + a.nkh;
    const int per_head = rot_vecs + pass_vecs;
    for (int item = threadIdx.x; item < qk_heads * per_head; item += blockDim.x) {
        const int head = item / per_head, j = item - head * per_head;
        T* h = base + (size_t)head * a.hd;
        T* dst = (head >= a.nqh && kdst) ? kdst + (size_t)(head - a.nqh) * a.page_size * a.hd : nullptr;
        if (j >= rot_vecs) {                            // tail beyond rope_dim: keys copy through to the cache
            const int i0 = a.rope_dim + (j - rot_vecs) * VEC;
            if (dst) *reinterpret_cast<uint4*>(dst + i0) = *reinterpret_cast<const uint4*>(h + i0);
            continue;
        }
        T x0[VEC], x1[VEC];
        if (a.adjacent) {
            const int i0 = j * VEC;                     // VEC / 2 pairs (2p, 2p + 1)
            *reinterpret_cast<uint4*>(x0) = *reinterpret_cast<const uint4*>(h + i0);
#pragma unroll
            for (int e = 0; e < VEC; e += 2) {
                const int p = (i0 + e) >> 1;
                const float c = cs_sn[p], sn = cs_sn[half + p];
                const float u = to_f32(x0[e]), v = to_f32(x0[e + 1]);
                x0[e] = from_f32<T>(u * c - v * sn);
                x0[e + 1] = from_f32<T>(u * sn + v * c);
            }
            *reinterpret_cast<uint4*>(h + i0) = *reinterpret_cast<const uint4*>(x0);
            if (dst) *reinterpret_cast<uint4*>(dst + i0) = *reinterpret_cast<const uint4*>(x0);
        } else {
            const int i0 = j * VEC;                     // VEC pairs (p, p + half)
            *reinterpret_cast<uint4*>(x0) = *reinterpret_cast<const uint4*>(h + i0);
            *reinterpret_cast<uint4*>(x1) = *reinterpret_cast<const uint4*>(h + i0 + half);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float c = cs_sn[i0 + e], sn = cs_sn[half + i0 + e];
                const float u = to_f32(x0[e]), v = to_f32(x1[e]);
                x0[e] = from_f32<T>(u * c - v * sn);
                x1[e] = from_f32<T>(u * sn + v * c);
            }
            *reinterpret_cast<uint4*>(h + i0) = *reinterpret_cast<const uint4*>(x0);
            *reinterpret_cast<uint4*>(h + i0 + half) = *reinterpret_cast<const uint4*>(x1);
            if (dst) {
                *reinterpret_cast<uint4*>(dst + i0) = *reinterpret_cast<const uint4*>(x0);
                *reinterpret_cast<uint4*>(dst + i0 + half) = *reinterpret_cast<const uint4*>(x1);
            }
        }
    }
    if (vdst) {
        const int hv = a.hd / VEC;
        const T* vsrc = base + (size_t)qk_heads * a.hd;
        for (int item = threadIdx.x; item < a.nkh * hv; item += blockDim.x) {
            const int kvh = item / hv, j = item - kvh * hv;
            *reinterpret_cast<uint4*>(vdst + (size_t)kvh * a.page_size * a.hd + j * VEC) =
                *reinterpret_cast<const uint4*>(vsrc + (size_t)kvh * a.hd + j * VEC);
        }
    }
}

extern "C" int braid_rope_kv_write(void* qkv, int dtype, const float* inv_freq, const int* positions,
                                   const int* token_seq, const int* page_table, void* cache,
                                   int rows, int nqh, int nkh, int hd, int rope_dim, int adjacent,
                                   int page_size, int table_cols, int num_pages, int* error_flag,
                                   void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (nqh <= 0 || nkh <= 0 || hd <= 0) BRAID_REFUSE("rope_kv_write: heads/head_dim must be positive");
    if (rope_dim < 0 || rope_dim > hd || (rope_dim & 1)) BRAID_REFUSE("rope_kv_write: rope_dim=%d must be even and <= head_dim=%d", rope_dim, hd);
    if (nqh + 2 * nkh > 65535) BRAID_REFUSE("rope_kv_write: %d heads exceed the grid limit", nqh + 2 * nkh);
    RopeKvArgs a{qkv, inv_freq, positions, token_seq, page_table, cache, rows, nqh, nkh, hd, rope_dim, adjacent,
                 page_size, table_cols, num_pages, error_flag};
    cudaStream_t s = (cudaStream_t)stream;
    const int vec = dtype == BRAID_F32 ? 4 : 8;
    if ((dtype == BRAID_F32 || dtype == BRAID_BF16) && hd % (2 * vec) == 0 && rope_dim % (2 * vec) == 0 &&
        (((uintptr_t)qkv | (uintptr_t)cache) & 15) == 0) {
        const size_t smem = (size_t)rope_dim * sizeof(float);
        if (dtype == BRAID_F32) braid_launch(rope_kv_vec_kernel<float>, dim3(rows), dim3(128), smem, s, a);
        else braid_launch(rope_kv_vec_kernel<__nv_bfloat16>, dim3(rows), dim3(128), smem, s, a);
        BRAID_LAUNCH_CHECK();
    }
    dim3 grid(rows, nqh + 2 * nkh);
    const int threads = hd >= 128 ? 64 : 32;
    if (dtype == BRAID_F32) braid_launch(rope_kv_kernel<float>, dim3(grid), dim3(threads), 0, s, a);
    else if (dtype == BRAID_BF16) braid_launch(rope_kv_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, s, a);
    else BRAID_REFUSE("rope_kv_write: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ casts
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long total) {
    pdl_trigger();
    pdl_wait();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = from_f32<TO>(to_f32(in[i]));
}

extern "C" int braid_cast(const void* in, int in_dtype, void* out, int out_dtype, long long total, void* stream) {
    if (total <= 0) return BRAID_OK;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("cast: %lld elements exceed one launch", total);
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == BRAID_F32 && out_dtype == BRAID_BF16) braid_launch(cast_kernel<float, __nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, s, (const float*)in, (__nv_bfloat16*)out, total);
    else if (in_dtype == BRAID_BF16 && out_dtype == BRAID_F32) braid_launch(cast_kernel<__nv_bfloat16, float>, dim3((int)blocks), dim3(threads), 0, s, (const __nv_bfloat16*)in, (float*)out, total);
    else BRAID_REFUSE("cast: unsupported dtype codes %d -> %d", in_dtype, out_dtype);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ int32 gather
// dst[i] = src[index[i]]: feeds the tokens a sampler left on the device into the next step.
__global__ void gather_i32_kernel(const int* __restrict__ src, const int* __restrict__ index, int* __restrict__ dst, int n) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[index[i]];
}

extern "C" int braid_gather_i32(const int* src, const int* index, int* dst, int n, void* stream) {
    if (n <= 0) return BRAID_OK;
    braid_launch(gather_i32_kernel, dim3((n + 127) / 128), dim3(128), 0, (cudaStream_t)stream, src, index, dst, n);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ logit hash
// One 64-bit hash a row of float32 logits, for finding the first step at which two runs part: for every
// element in order, h ^= its 32 bits; h *= 0x100000001b3, from h = 0xcbf29ce484222325 (the hash that the
// reference writes under BRAIDINFER_LOGIT_TRACE, crates/braidinfer-runtime/src/generate.rs:383-396).
// The chain is sequential, so one thread a row walks it; the block stages the row through shared memory.
#define HASH_CHUNK 4096
__global__ void logit_hash_kernel(const float* __restrict__ logits, long long ld, int vocab, unsigned long long* __restrict__ out) {
    __shared__ float chunk[HASH_CHUNK];
    pdl_trigger();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * ld;
    unsigned long long h = 0xcbf29ce484222325ull;
    for (int c0 = 0; c0 < vocab; c0 += HASH_CHUNK) {
        const int n = min(HASH_CHUNK, vocab - c0);
        for (int i = threadIdx.x; i < n; i += blockDim.x) chunk[i] = row[c0 + i];
        __syncthreads();
        if (threadIdx.x == 0)
            for (int i = 0; i < n; ++i) {
                h ^= (unsigned long long)__float_as_uint(chunk[i]);
                h *= 0x100000001b3ull;
            }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[blockIdx.x] = h;
}

extern "C" int braid_logit_hash(const float* logits, long long ld, int rows, int vocab, unsigned long long* out, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (vocab <= 0 || ld < vocab) BRAID_REFUSE("logit_hash: vocab=%d, row stride=%lld", vocab, ld);
    braid_launch(logit_hash_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, logits, ld, vocab, out);
    BRAID_LAUNCH_CHECK();
}
