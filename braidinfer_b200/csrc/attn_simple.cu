// Plain attention over the paged cache: one warp per (token, query head).
//
// It is the float32 path's attention and the reference kernel that the faster
// bfloat16 kernels are checked against.  It serves prompts, chunks of prompts and
// single decoded tokens alike: every query reads its keys and values from the cache,
// which already holds the step's own tokens.
//
// Formula (kernels/megakernel_ops.hip:2192-2194, 2310-2342 of the reference): head h
// reads kv head h / g; s_j = (q . k_j) * scale; online softmax with running maximum m,
// denominator d and accumulator acc; out = acc / d.  Key j is visible to the query at
// position p iff j <= p and, with a window w > 0, p - j < w (the window is this
// library's own; the reference has none).  Scores, softmax and accumulation are float32.
#include "common.cuh"

struct AttnSimpleArgs {
    const void* q;            // [rows, q_row_stride], head h at column h * hd
    void* out;                // [rows, out_row_stride]
    const void* cache;        // one layer: [page][2][nkh][page_size][hd]
    const int* page_table;    // [n_seqs, table_cols]
    const int* positions;     // [rows]
    const int* token_seq;     // [rows] or -1 for padding
    int q_row_stride, out_row_stride;
    int rows, nqh, nkh, hd, page_size, table_cols, num_pages, window;
    float scale;
    int* error_flag;          // raised when a visible position has no page, or one outside the cache
};

#define ATTN_SIMPLE_WARPS 4
#define ATTN_SIMPLE_MAX_HD 256

template <typename T>
__global__ void __launch_bounds__(ATTN_SIMPLE_WARPS * 32)
attn_simple_kernel(AttnSimpleArgs a) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];                  // [warps][hd] queries, [warps][32] probabilities
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* qs = smem + warp * a.hd;
    float* ps = smem + ATTN_SIMPLE_WARPS * a.hd + warp * 32;
    const long long item = (long long)blockIdx.x * ATTN_SIMPLE_WARPS + warp;
    if (item >= (long long)a.rows * a.nqh) return;
    const int row = (int)(item / a.nqh), head = (int)(item - (long long)row * a.nqh);
    T* o = (T*)a.out + (size_t)row * a.out_row_stride + (size_t)head * a.hd;
    const int seq = a.token_seq[row];
    if (seq < 0) {
        for (int d = lane; d < a.hd; d += 32) o[d] = from_f32<T>(0.f);
        return;
    }
    const int pos = a.positions[row];
    const int kvh = head / (a.nqh / a.nkh);
    const T* q = (const T*)a.q + (size_t)row * a.q_row_stride + (size_t)head * a.hd;
    for (int d = lane; d < a.hd; d += 32) qs[d] = to_f32(q[d]);
    __syncwarp();

    const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    float m = -INFINITY, l = 0.f;
    float acc[ATTN_SIMPLE_MAX_HD / 32];
#pragma unroll
    for (int i = 0; i < ATTN_SIMPLE_MAX_HD / 32; ++i) acc[i] = 0.f;
    const int* table = a.page_table + (size_t)seq * a.table_cols;
    const size_t head_stride = (size_t)a.page_size * a.hd;

    for (int j0 = lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        const T* vrow = nullptr;
        if (j <= pos) {
            const int block = j / a.page_size, off = j - block * a.page_size;
            int page = (block < a.table_cols) ? table[block] : -1;
            if (page < 0 || page >= a.num_pages) {      // never followed: flag it and read page 0 instead
                atomicExch(a.error_flag, 1);
                page = 0;
            }
            const T* kbase = (const T*)a.cache + ((size_t)page * 2 * a.nkh + kvh) * head_stride + (size_t)off * a.hd;
            vrow = kbase + (size_t)a.nkh * head_stride;
            float dot = 0.f;
            for (int d = 0; d < a.hd; ++d) dot = fmaf(qs[d], to_f32(kbase[d]), dot);
            s = dot * a.scale;
        }
        const float cmax = warp_max(s);
        const float m_new = fmaxf(m, cmax);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float p = (j <= pos) ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
        m = m_new;
        ps[lane] = p;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < ATTN_SIMPLE_MAX_HD / 32; ++i) acc[i] *= corr;
        const int n_valid = min(32, pos - j0 + 1);
        for (int jj = 0; jj < n_valid; ++jj) {
            const T* vr = (const T*)__shfl_sync(0xffffffffu, (unsigned long long)vrow, jj);
            const float pj = ps[jj];
#pragma unroll
            for (int i = 0; i < ATTN_SIMPLE_MAX_HD / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < a.hd) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
        __syncwarp();
    }
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < ATTN_SIMPLE_MAX_HD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < a.hd) o[d] = from_f32<T>(acc[i] * inv);
    }
}

extern "C" int braid_attn_simple(const void* q, void* out, int dtype, const void* cache,
                                 const int* page_table, const int* positions, const int* token_seq,
                                 int q_row_stride, int out_row_stride, int rows, int nqh, int nkh, int hd,
                                 int page_size, int table_cols, int num_pages, int window, float scale,
                                 int* error_flag, void* stream) {
    if (rows <= 0) return BRAID_OK;
    if (!error_flag) BRAID_REFUSE("attn_simple: error_flag is required");
    if (num_pages <= 0 || table_cols <= 0 || page_size <= 0) BRAID_REFUSE("attn_simple: the cache has no pages (pages=%d, table columns=%d, page size=%d)", num_pages, table_cols, page_size);
    if (nqh <= 0 || nkh <= 0 || nqh % nkh != 0) BRAID_REFUSE("attn_simple: %d query heads do not divide into %d kv heads", nqh, nkh);
    if (hd <= 0 || hd > ATTN_SIMPLE_MAX_HD) BRAID_REFUSE("attn_simple: head_dim=%d outside (0, %d]", hd, ATTN_SIMPLE_MAX_HD);
    AttnSimpleArgs a{q, out, cache, page_table, positions, token_seq, q_row_stride, out_row_stride,
                     rows, nqh, nkh, hd, page_size, table_cols, num_pages, window, scale, error_flag};
    const long long items = (long long)rows * nqh;
    const long long blocks = (items + ATTN_SIMPLE_WARPS - 1) / ATTN_SIMPLE_WARPS;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("attn_simple: %lld (token, head) pairs exceed one launch", items);
    const size_t smem = (size_t)ATTN_SIMPLE_WARPS * (hd + 32) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == BRAID_F32) braid_launch(attn_simple_kernel<float>, dim3((int)blocks), dim3(ATTN_SIMPLE_WARPS * 32), smem, s, a);
    else if (dtype == BRAID_BF16) braid_launch(attn_simple_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(ATTN_SIMPLE_WARPS * 32), smem, s, a);
    else BRAID_REFUSE("attn_simple: unknown dtype code %d", dtype);
    BRAID_LAUNCH_CHECK();
}
