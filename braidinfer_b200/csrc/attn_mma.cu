// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16,
// float32 accumulation), compiled for one head size: -DBRAID_HD=<head_dim>.
//
// One kernel serves prompts, chunks of prompts and decoded tokens.  A CTA owns BM = 16 x
// NW "rows": the query heads of one kv head (up to BM of them) for BM / heads
// consecutive tokens of one sequence, so the heads of a group share every key and value
// tile they read.  Keys and values come from the cache in tiles of BN positions (a tile
// never straddles a 64-position page) through a cp.async ring; scores, the online
// softmax (running maximum m, denominator l) and the output accumulator are float32;
// probabilities are rounded to bfloat16 for the P.V product.  With n_splits > 1 the key
// range of a CTA is one slice of the context and it writes (m, l, unnormalised out) for
// braid_attn_combine to merge: that is how a single decoded token fills the machine.
//
// Visibility is the one rule of the whole library: key j is visible to the query at
// position p iff j <= p and (window == 0 or p - j < window).
//
// Replaces the reference's op_attn_paged, one 256-thread block per query head walking
// the context token by token (kernels/megakernel_ops.hip:2150-2343).
#include "common.cuh"

#ifndef BRAID_HD
#error "compile with -DBRAID_HD=<head_dim>"
#endif
static_assert(BRAID_HD % 16 == 0 && BRAID_HD >= 16 && BRAID_HD <= 256, "head_dim must be a multiple of 16 in [16, 256]");

#include "page.h"
#define PAGE BRAID_PAGE_SIZE

struct AttnMmaArgs {
    const __nv_bfloat16* q;      // [rows, q_row_stride]; head h at column h * HD
    __nv_bfloat16* out;          // [rows, out_row_stride]
    float* partial;              // [rows * nqh][n_splits][HD + 2] when n_splits > 1
    const __nv_bfloat16* cache;  // one layer: [page][2][nkh][PAGE][HD]
    const int* page_table;       // [n_seqs, table_cols]
    const int* q_start;          // [n_seqs] first row of the sequence
    const int* q_len;            // [n_seqs] rows of the sequence
    const int* kv_before;        // [n_seqs] cache length before this step
    int q_row_stride, out_row_stride;
    int nqh, nkh, table_cols, window, n_splits;
    float scale_log2;            // softmax scale * log2(e)
    int num_pages;               // pages of the cache: a table entry outside [0, num_pages) is never followed
    int* error_flag;             // raised when a tile of visible keys has no page or one outside the cache
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD, int NW, int BN, int ST>
struct AttnCfg {
    static_assert(PAGE % BN == 0, "a key tile must not straddle a page");
    static constexpr int BM = 16 * NW;
    static constexpr int ROW = HD * 2 + 16;               // bytes per padded shared-memory row
    static constexpr int Q_BYTES = BM * ROW;
    static constexpr int TILE_BYTES = BN * ROW;           // one K or V tile
    static constexpr int SMEM = Q_BYTES + ST * 2 * TILE_BYTES;
};

template <int HD, int NW, int BN, int ST>
__global__ void __launch_bounds__(NW * 32)
attn_mma_kernel(AttnMmaArgs a) {
    using C = AttnCfg<HD, NW, BN, ST>;
    pdl_trigger();
    // What follows up to pdl_wait() reads only the step's tables (copied to the device before
    // the step's first kernel) and keys and values of positions cached by earlier steps,
    // which no kernel of this step writes; the queries and the step's own keys come after it.
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sKV = smem + C::Q_BYTES;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = a.nqh / a.nkh;
    const int hpc = g < C::BM ? g : C::BM;                 // heads per CTA
    const int tpc = C::BM / hpc;                           // tokens per CTA
    const int hchunks = (g + hpc - 1) / hpc;
    // CTAs start in the order x, y, z: every kv head and sequence of the last token tile first, then of
    // the tile before: late tokens see the most keys, so the longest CTAs start first
    const int seq = blockIdx.y;
    const int kvh = blockIdx.x / hchunks, hchunk = blockIdx.x - kvh * hchunks;
    const int unit = gridDim.z - 1 - blockIdx.z;
    const int tile = unit / a.n_splits, split = unit - tile * a.n_splits;
    const int q_len = a.q_len[seq];
    const int tok0 = tile * tpc;
    if (tok0 >= q_len) return;
    const int q_start = a.q_start[seq], kv_before = a.kv_before[seq];
    const int n_tok = min(tpc, q_len - tok0);
    const int pos_min = kv_before + tok0, pos_max = pos_min + n_tok - 1;
    const int k_lo = (a.window > 0 && pos_min - a.window + 1 > 0) ? pos_min - a.window + 1 : 0;
    int t_lo = k_lo / BN, t_hi = pos_max / BN + 1;
    if (a.n_splits > 1) {
        const int per = (t_hi - t_lo + a.n_splits - 1) / a.n_splits;
        t_lo = t_lo + split * per;
        t_hi = min(t_hi, t_lo + per);
    }
    const int n_tiles = max(0, t_hi - t_lo);
    const int* table = a.page_table + (size_t)seq * a.table_cols;
    const int head0 = kvh * g + hchunk * hpc;              // first query head of this CTA
    const int n_heads = min(hpc, g - hchunk * hpc);

    constexpr int CH = HD / 8;                             // 16-byte chunks per row
    auto load_tile = [&](int t, int stage) {
        const int key0 = t * BN;
        const int block = key0 / PAGE;
        int page = (block < a.table_cols) ? table[block] : -1;
        if (page < 0 || page >= a.num_pages) {             // flag it and read page 0 instead: no address is made from it
            if (tid == 0) atomicExch(a.error_flag, 1);
            page = 0;
        }
        const int off = key0 - block * PAGE;
        const __nv_bfloat16* kbase = a.cache + (((size_t)page * 2) * a.nkh + kvh) * PAGE * HD + (size_t)off * HD;
        const __nv_bfloat16* vbase = kbase + (size_t)a.nkh * PAGE * HD;
        uint8_t* dk = sKV + stage * 2 * C::TILE_BYTES;
        uint8_t* dv = dk + C::TILE_BYTES;
        for (int i = tid; i < BN * CH; i += NW * 32) {
            const int r = i / CH, c = i - r * CH;
            cp_async16(dk + r * C::ROW + c * 16, kbase + (size_t)r * HD + c * 8);
            cp_async16(dv + r * C::ROW + c * 16, vbase + (size_t)r * HD + c * 8);
        }
    };
    // the first tiles of the ring; those that hold only positions cached before this step
    // are asked for at once, the others after the wait
    bool early[ST];                                      // every stage of the ring is free at the start
#pragma unroll
    for (int s = 0; s < ST; ++s) {
        early[s] = s < n_tiles && (t_lo + s + 1) * BN <= kv_before;
        if (early[s]) load_tile(t_lo + s, s);
    }
    pdl_wait();

    // the tiles of the ring that had to wait (they hold this step's own keys) are asked for first: the trip
    // for the queries, next, then runs beside theirs
#pragma unroll
    for (int s = 0; s < ST; ++s) {
        if (s < n_tiles && !early[s]) load_tile(t_lo + s, s);
        cp_async_commit();                               // one group a stage, as the loop below counts them
    }

    // ---- queries into shared memory (rows of absent tokens or heads are zero)
    for (int i = tid; i < C::BM * CH; i += NW * 32) {
        const int r = i / CH, c = i - r * CH;
        const int tl = r / hpc, hl = r - tl * hpc;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tl < n_tok && hl < n_heads)
            v = *reinterpret_cast<const uint4*>(a.q + (size_t)(q_start + tok0 + tl) * a.q_row_stride + (size_t)(head0 + hl) * HD + c * 8);
        *reinterpret_cast<uint4*>(sQ + r * C::ROW + c * 16) = v;
    }


    // per-thread rows: r0 = lane / 4 and r0 + 8 of this warp's 16
    const int row_a = warp * 16 + (lane >> 2), row_b = row_a + 8;
    int pos_a = -1, pos_b = -1;                            // -1: the row sees nothing
    {
        const int ta = row_a / hpc, ha = row_a - ta * hpc;
        const int tb = row_b / hpc, hb = row_b - tb * hpc;
        if (ta < n_tok && ha < n_heads) pos_a = pos_min + ta;
        if (tb < n_tok && hb < n_heads) pos_b = pos_min + tb;
    }
    const int lo_a = (a.window > 0) ? pos_a - a.window + 1 : 0;
    const int lo_b = (a.window > 0) ? pos_b - a.window + 1 : 0;

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    for (int it = 0; it < n_tiles; ++it) {
        if (it > 0) {                                    // the stage that tile it - 1 has left takes tile it + ST - 1
            const int pre = it + ST - 1;
            if (pre < n_tiles) load_tile(t_lo + pre, pre % ST);
            cp_async_commit();
        }
        cp_async_wait<ST - 1>();
        __syncthreads();
        const uint8_t* sK = sKV + (it % ST) * 2 * C::TILE_BYTES;
        const uint8_t* sV = sK + C::TILE_BYTES;

        // ---- S = Q K^T
        float s[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            uint32_t a0, a1, a2, a3;
            ldsm_x4(a0, a1, a2, a3, sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * C::ROW + (kk * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
            for (int nb = 0; nb < BN / 16; ++nb) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(b0, b1, b2, b3, sK + (nb * 16 + (lane >> 4) * 8 + (lane & 7)) * C::ROW + (kk * 16 + ((lane >> 3) & 1) * 8) * 2);
                mma_bf16(s[nb * 2], a0, a1, a2, a3, b0, b1);
                mma_bf16(s[nb * 2 + 1], a0, a1, a2, a3, b2, b3);
            }
        }

        // ---- mask, online softmax
        const int key0 = (t_lo + it) * BN + (lane & 3) * 2;
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = key0 + nb * 8 + e;
                const bool va = (j <= pos_a) && (j >= lo_a);
                const bool vb = (j <= pos_b) && (j >= lo_b);
                s[nb][e] = va ? s[nb][e] * a.scale_log2 : -INFINITY;
                s[nb][2 + e] = vb ? s[nb][2 + e] * a.scale_log2 : -INFINITY;
                mx_a = fmaxf(mx_a, s[nb][e]);
                mx_b = fmaxf(mx_b, s[nb][2 + e]);
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float ms_a = (mn_a == -INFINITY) ? 0.f : mn_a, ms_b = (mn_b == -INFINITY) ? 0.f : mn_b;
        const float corr_a = exp2f(m_a - ms_a), corr_b = exp2f(m_b - ms_b);      // exp2(-inf) = 0
        m_a = mn_a; m_b = mn_b;
        float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
        for (int nb = 0; nb < BN / 8; ++nb) {
            s[nb][0] = exp2f(s[nb][0] - ms_a); s[nb][1] = exp2f(s[nb][1] - ms_a);
            s[nb][2] = exp2f(s[nb][2] - ms_b); s[nb][3] = exp2f(s[nb][3] - ms_b);
            sum_a += s[nb][0] + s[nb][1];
            sum_b += s[nb][2] + s[nb][3];
        }
        l_a = l_a * corr_a + sum_a;
        l_b = l_b * corr_b + sum_b;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) { o[i][0] *= corr_a; o[i][1] *= corr_a; o[i][2] *= corr_b; o[i][3] *= corr_b; }

        // ---- O += P V
#pragma unroll
        for (int j = 0; j < BN / 16; ++j) {
            const uint32_t p0 = pack_bf16(s[2 * j][0], s[2 * j][1]);
            const uint32_t p1 = pack_bf16(s[2 * j][2], s[2 * j][3]);
            const uint32_t p2 = pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]);
            const uint32_t p3 = pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
            for (int db = 0; db < HD / 16; ++db) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(b0, b1, b2, b3, sV + (j * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * C::ROW + (db * 16 + (lane >> 4) * 8) * 2);
                mma_bf16(o[db * 2], p0, p1, p2, p3, b0, b1);
                mma_bf16(o[db * 2 + 1], p0, p1, p2, p3, b2, b3);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

    // ---- write
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = half ? row_b : row_a;
        const int pos = half ? pos_b : pos_a;
        if (pos < 0) continue;
        const int tl = row / hpc, hl = row - tl * hpc;
        const size_t grow = (size_t)(q_start + tok0 + tl);
        const int head = head0 + hl;
        const float l = half ? l_b : l_a, m = half ? m_b : m_a;
        if (a.n_splits == 1) {
            const float inv = 1.f / l;
            __nv_bfloat16* dst = a.out + grow * a.out_row_stride + (size_t)head * HD + (lane & 3) * 2;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i)
                *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][half * 2] * inv, o[i][half * 2 + 1] * inv);
        } else {
            float* dst = a.partial + ((grow * a.nqh + head) * a.n_splits + split) * (HD + 2);
            if ((lane & 3) == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
            for (int i = 0; i < HD / 8; ++i)
                *reinterpret_cast<float2*>(dst + 2 + i * 8 + (lane & 3) * 2) = make_float2(o[i][half * 2], o[i][half * 2 + 1]);
        }
    }
}

// Merge the slices of one (row, head): out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M).
// A thread owns output dimensions; it loads every slice's (m, l, O_d) at once (the loads do
// not depend on one another) and repeats the few scalar sums of the row itself.
#define COMBINE_MAX_SPLITS 64
template <int HD>
__global__ void attn_combine_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                    const int* __restrict__ token_seq, int out_row_stride, int nqh, int n_splits) {
    pdl_trigger();
    // the step's tables are on the device before the step's first kernel: read before the wait
    const int row = blockIdx.x, head = blockIdx.y;
    const bool padding = token_seq[row] < 0;
    pdl_wait();
    if (padding) return;
    const float* p = partial + ((size_t)row * nqh + head) * n_splits * (HD + 2);
    constexpr int B = 16;                                  // slices asked for at once: one trip for up to 16
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float M = -INFINITY, L = 0.f, acc = 0.f;
        for (int s0 = 0; s0 < n_splits; s0 += B) {
            float m[B], l[B], o[B];
#pragma unroll
            for (int i = 0; i < B; ++i) {
                const bool in = s0 + i < n_splits;
                const float* ps = p + (size_t)(in ? s0 + i : 0) * (HD + 2);
                m[i] = in ? ps[0] : -INFINITY;
                l[i] = in ? ps[1] : 0.f;
                o[i] = in ? ps[2 + d] : 0.f;
            }
            float Mn = M;
#pragma unroll
            for (int i = 0; i < B; ++i) Mn = fmaxf(Mn, m[i]);
            if (Mn == -INFINITY) continue;
            const float c = exp2f(M - Mn);                 // exp2(-inf) = 0 the first time
            L *= c;
            acc *= c;
#pragma unroll
            for (int i = 0; i < B; ++i) {
                const float wgt = (m[i] == -INFINITY) ? 0.f : exp2f(m[i] - Mn);
                L = fmaf(l[i], wgt, L);
                acc = fmaf(o[i], wgt, acc);
            }
            M = Mn;
        }
        out[(size_t)row * out_row_stride + (size_t)head * HD + d] = __float2bfloat16_rn(acc / L);
    }
}

template <int NW, int BN, int ST>
static int launch_attn(const AttnMmaArgs& a, int n_seqs, int max_q_len, cudaStream_t s) {
    using C = AttnCfg<BRAID_HD, NW, BN, ST>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_mma_kernel<BRAID_HD, NW, BN, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) { braid_set_error("attn_mma: cannot reserve %d bytes of shared memory: %s", C::SMEM, cudaGetErrorString(e)); return (int)e; }
        configured = true;
    }
    const int g = a.nqh / a.nkh;
    const int hpc = g < C::BM ? g : C::BM;
    const int tpc = C::BM / hpc;
    const int hchunks = (g + hpc - 1) / hpc;
    const long long gx = (long long)((max_q_len + tpc - 1) / tpc) * a.n_splits;
    if (gx > 65535 || (long long)a.nkh * hchunks > 0x7fffffffLL || n_seqs > 65535)
        BRAID_REFUSE("attn_mma: the step exceeds the grid limits (%lld tiles, %d heads, %d sequences)", gx, a.nkh * hchunks, n_seqs);
    dim3 grid(a.nkh * hchunks, n_seqs, (unsigned)gx);
    braid_launch(attn_mma_kernel<BRAID_HD, NW, BN, ST>, dim3(grid), dim3(NW * 32), C::SMEM, s, a);
    BRAID_LAUNCH_CHECK();
}

extern "C" int braid_attn_mma_head_dim(void) { return BRAID_HD; }

// Floats of scratch that n_splits > 1 needs.
extern "C" long long braid_attn_mma_partial_floats(int rows, int nqh, int n_splits) {
    return n_splits > 1 ? (long long)rows * nqh * n_splits * (BRAID_HD + 2) : 0;
}

// CTAs of the few-token kernel (kind 1) that the device holds at once: the context is
// best sliced so that one wave of CTAs covers the step.
extern "C" int braid_attn_mma_decode_slots(int kind) {
    (void)kind;
    int dev = 0, sms = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    using C = AttnCfg<BRAID_HD, 1, 32, 3>;
    cudaFuncSetAttribute(attn_mma_kernel<BRAID_HD, 1, 32, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_mma_kernel<BRAID_HD, 1, 32, 3>, 32, C::SMEM);
    if (e != cudaSuccess || per_sm <= 0 || sms <= 0) return 148 * 4;
    return per_sm * sms;
}

// kind 0: many tokens per sequence (4 warps, tiles of 64 keys); kind 1: few (1 warp, tiles of 32 keys).
extern "C" int braid_attn_mma(const void* q, void* out, void* partial, const void* cache, const int* page_table,
                              const int* q_start, const int* q_len, const int* kv_before, const int* token_seq,
                              int q_row_stride, int out_row_stride, int rows, int n_seqs, int max_q_len,
                              int nqh, int nkh, int hd, int table_cols, int num_pages, int window, int n_splits, int kind,
                              float scale, int* error_flag, void* stream) {
    if (rows <= 0 || n_seqs <= 0) return BRAID_OK;
    if (!error_flag) BRAID_REFUSE("attn_mma: error_flag is required");
    if (num_pages <= 0 || table_cols <= 0) BRAID_REFUSE("attn_mma: the cache has no pages (pages=%d, table columns=%d)", num_pages, table_cols);
    if (hd != BRAID_HD) BRAID_REFUSE("attn_mma: this library was compiled for head_dim=%d, not %d", BRAID_HD, hd);
    if (nqh <= 0 || nkh <= 0 || nqh % nkh) BRAID_REFUSE("attn_mma: %d query heads do not divide into %d kv heads", nqh, nkh);
    if ((q_row_stride % 8) || ((uintptr_t)q & 15)) BRAID_REFUSE("attn_mma: queries must be 16-byte aligned rows");
    if ((out_row_stride % 2) || ((uintptr_t)out & 3)) BRAID_REFUSE("attn_mma: out rows must be 4-byte aligned");
    if (n_splits < 1) n_splits = 1;
    if (n_splits > 1 && !partial) BRAID_REFUSE("attn_mma: n_splits > 1 needs the partial buffer");
    AttnMmaArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (float*)partial, (const __nv_bfloat16*)cache, page_table,
                  q_start, q_len, kv_before, q_row_stride, out_row_stride, nqh, nkh, table_cols, window, n_splits,
                  scale * 1.4426950408889634f, num_pages, error_flag};
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    if (kind == 0) rc = launch_attn<4, 64, 2>(a, n_seqs, max_q_len, s);
    else rc = launch_attn<1, 32, 3>(a, n_seqs, max_q_len, s);
    if (rc) return rc;
    if (n_splits > 1) {
        dim3 grid(rows, nqh);
        braid_launch(attn_combine_kernel<BRAID_HD>, grid, dim3(BRAID_HD >= 128 ? 128 : 32), 0, s, (const float*)partial, (__nv_bfloat16*)out, token_seq, out_row_stride, nqh, n_splits);
        BRAID_LAUNCH_CHECK();
    }
    return BRAID_OK;
}

// ------------------------------------------------------------------ no-allocation entry point
// See attn_noalloc.h for who needs this and what it costs.
#include "attn_noalloc.h"

// The scratch itself.  In host code this name is only a handle for the runtime: its
// device address has to be asked for (below) before a kernel can be given it.
static __device__ __align__(256) float g_noalloc_scratch[BRAID_ATTN_NOALLOC_MAX_FLOATS];

#define BRAID_NOALLOC_MAX_DEVICES 64
static float* g_noalloc_ptr[BRAID_NOALLOC_MAX_DEVICES];      // device address of the array, per device

extern "C" long long braid_attn_noalloc_capacity_floats(void) { return BRAID_ATTN_NOALLOC_MAX_FLOATS; }

extern "C" int braid_attn_mma_noalloc(const void* q, void* out, const void* cache, const int* page_table,
                                      const int* q_start, const int* q_len, const int* kv_before, const int* token_seq,
                                      int q_row_stride, int out_row_stride, int rows, int n_seqs, int max_q_len,
                                      int nqh, int nkh, int hd, int table_cols, int num_pages, int window, int n_splits,
                                      int kind, float scale, int* error_flag, void* stream) {
    if (rows <= 0 || n_seqs <= 0) return BRAID_OK;
    if (n_splits < 1) n_splits = 1;
    const long long need = braid_attn_mma_partial_floats(rows, nqh, n_splits);
    if (need > BRAID_ATTN_NOALLOC_MAX_FLOATS)
        BRAID_REFUSE("attn_mma_noalloc: the step needs %lld floats of scratch (rows=%d heads=%d slices=%d head_dim=%d), "
                     "the built-in array holds %d; use fewer slices or braid_attn_mma with a buffer of your own",
                     need, rows, nqh, n_splits, BRAID_HD, BRAID_ATTN_NOALLOC_MAX_FLOATS);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { braid_set_error("attn_mma_noalloc: cudaGetDevice: %s", cudaGetErrorString(e)); return (int)e; }
    if (dev < 0 || dev >= BRAID_NOALLOC_MAX_DEVICES) BRAID_REFUSE("attn_mma_noalloc: device index %d is beyond %d", dev, BRAID_NOALLOC_MAX_DEVICES);
    if (!g_noalloc_ptr[dev]) {
        // set-up, once per device, with that device current: the array's address on it
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            braid_set_error("attn_mma_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : BRAID_REFUSED;
        }
        g_noalloc_ptr[dev] = p;
    }
    return braid_attn_mma(q, out, n_splits > 1 ? g_noalloc_ptr[dev] : nullptr, cache, page_table, q_start, q_len,
                          kv_before, token_seq, q_row_stride, out_row_stride, rows, n_seqs, max_q_len, nqh, nkh, hd,
                          table_cols, num_pages, window, n_splits, kind, scale, error_flag, stream);
}
