// bfloat16 attention of prompts over the paged cache on the 5th-generation tensor cores
// (tcgen05), compiled for one head size: -DBRAID_HD=64 or 128.
//
// A CTA owns 128 rows: the query heads of one kv head (up to 128 of them) for 128 / heads
// consecutive tokens of one sequence, and walks the visible keys in tiles of 128 (two
// 64-position pages).
//
//   warp 0      TMA: the query tile once, then key and value tiles into a two-stage ring
//               (cp.async.bulk.tensor, 128-byte swizzle, no multicast);
//   warp 1      one lane issues S = Q K^T (accumulator in tensor memory, two buffers) and,
//               once the softmax warps have written P, O_tile = P V;
//   warps 2..9  two threads per row, 64 keys and 64 output dimensions each: read S from
//               tensor memory, mask, running maximum (the two halves of a row meet in shared
//               memory) and denominator in float32, P = exp2(s - m) rounded to bfloat16 into
//               shared memory (the A operand of the second product), then add O_tile into the
//               row's float32 output held in registers, rescaled when the maximum moved.
//
// Keys are K-major for the first product; values are read MN-major by the second one,
// straight from the [position][head_dim] layout of the cache, so nothing is transposed.
// Every wait on an mbarrier is bounded (see tcgen05.cuh); a wait that runs out raises
// *error_flag and the kernel frees its tensor memory and returns.
//
// Visibility is the rule of the whole library: key j is visible to the query at position
// p iff j <= p and (window == 0 or p - j < window).  Replaces, for prompts, the
// reference's op_attn_paged (kernels/megakernel_ops.hip:2150-2343), as attn_mma.cu does;
// attn_mma.cu stays the kernel for other head sizes and the twin this one is tested against.
#include "common.cuh"
#include "tcgen05.cuh"

#ifndef BRAID_HD
#error "compile with -DBRAID_HD=<head_dim>"
#endif

#if BRAID_HD == 64 || BRAID_HD == 128
#define BRAID_ATTN_TC 1

#define FA_BM 128
#define FA_BN 128
#define FA_PAGE 64
#define FA_THREADS 320                          // TMA warp, MMA warp, 8 softmax warps
#define FA_HB (BRAID_HD / 64)                    // 64-element blocks of the head dimension
#define FA_BLOCK_BYTES (128 * 128)               // [128 rows][64 elements] bf16, 128-byte rows
#define FA_Q_BYTES (FA_HB * FA_BLOCK_BYTES)
#define FA_KV_BYTES (FA_HB * FA_BLOCK_BYTES)     // one K or one V tile
#define FA_STAGE_BYTES (2 * FA_KV_BYTES)
#define FA_P_BYTES (2 * FA_BLOCK_BYTES)
#define FA_SMEM (FA_Q_BYTES + 2 * FA_STAGE_BYTES + FA_P_BYTES + 1024 + 128 + 2 * 2 * 128 * 4)
#define FA_TMEM_COLS 512                          // S0 [0,128) S1 [128,256) O_tile [256, 256 + HD)

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));       // exp2(-inf) = 0, exp2(0) = 1 exactly
    return y;
}
// 64 consecutive columns of this thread's lane: two loads in flight, one wait.
__device__ __forceinline__ void tmem_ld32x2(uint32_t taddr, float* v) {
    uint32_t r[64];
#pragma unroll
    for (int h = 0; h < 2; ++h)
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
            "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(r[h * 32 + 0]), "=r"(r[h * 32 + 1]), "=r"(r[h * 32 + 2]), "=r"(r[h * 32 + 3]), "=r"(r[h * 32 + 4]),
              "=r"(r[h * 32 + 5]), "=r"(r[h * 32 + 6]), "=r"(r[h * 32 + 7]), "=r"(r[h * 32 + 8]), "=r"(r[h * 32 + 9]),
              "=r"(r[h * 32 + 10]), "=r"(r[h * 32 + 11]), "=r"(r[h * 32 + 12]), "=r"(r[h * 32 + 13]), "=r"(r[h * 32 + 14]),
              "=r"(r[h * 32 + 15]), "=r"(r[h * 32 + 16]), "=r"(r[h * 32 + 17]), "=r"(r[h * 32 + 18]), "=r"(r[h * 32 + 19]),
              "=r"(r[h * 32 + 20]), "=r"(r[h * 32 + 21]), "=r"(r[h * 32 + 22]), "=r"(r[h * 32 + 23]), "=r"(r[h * 32 + 24]),
              "=r"(r[h * 32 + 25]), "=r"(r[h * 32 + 26]), "=r"(r[h * 32 + 27]), "=r"(r[h * 32 + 28]), "=r"(r[h * 32 + 29]),
              "=r"(r[h * 32 + 30]), "=r"(r[h * 32 + 31])
            : "r"(taddr + h * 32) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
// BRAID_HD / 2 consecutive columns (32 or 64).
__device__ __forceinline__ void tmem_ld_od(uint32_t taddr, float* v) {
#if BRAID_HD == 128
    tmem_ld32x2(taddr, v);
#else
    tmem_ld32(taddr, v);
#endif
}

struct AttnTcArgs {
    __nv_bfloat16* out;
    const int* page_table;
    const int* q_start;
    const int* q_len;
    const int* kv_before;
    int out_row_stride, nqh, nkh, table_cols, window;
    float scale_log2;
    int* error_flag;
};

__global__ void __launch_bounds__(FA_THREADS, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, AttnTcArgs a) {
    constexpr int HD = BRAID_HD;
    pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;
    uint8_t* sKV = sQ + FA_Q_BYTES;
    uint8_t* sP = sKV + 2 * FA_STAGE_BYTES;
    uint64_t* bars = (uint64_t*)(sP + FA_P_BYTES);
    uint64_t* q_full = bars;            // [1]
    uint64_t* kv_full = bars + 1;       // [2]
    uint64_t* kv_empty = bars + 3;      // [2]
    uint64_t* s_full = bars + 5;        // [2]
    uint64_t* s_empty = bars + 7;       // [2]
    uint64_t* p_ready = bars + 9;       // [1]
    uint64_t* o_full = bars + 10;       // [1]
    uint64_t* o_empty = bars + 11;      // [1]
    uint32_t* tmem_slot = (uint32_t*)(bars + 12);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* xchg = (float*)(bars + 16);                    // [2 parities][2 halves][128 rows]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = a.nqh / a.nkh;
    const int hpc = g < FA_BM ? g : FA_BM;
    const int tpc = FA_BM / hpc;
    const int hchunks = (g + hpc - 1) / hpc;
    const int seq = blockIdx.z;
    const int kvh = blockIdx.y / hchunks, hchunk = blockIdx.y - kvh * hchunks;
    const int tile = gridDim.x - 1 - blockIdx.x;       // late tokens see the most keys: start them first

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1);
            mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 256);
        }
        mbar_init(p_ready, 256); mbar_init(o_full, 1); mbar_init(o_empty, 256);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, FA_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();

    const int q_len = a.q_len[seq];
    const int tok0 = tile * tpc;
    const bool active = tok0 < q_len;             // uniform over the CTA
    const int q_start = a.q_start[seq], kv_before = a.kv_before[seq];
    const int n_tok = active ? min(tpc, q_len - tok0) : 0;
    const int pos_min = kv_before + tok0, pos_max = pos_min + n_tok - 1;
    const int k_lo = (a.window > 0 && pos_min - a.window + 1 > 0) ? pos_min - a.window + 1 : 0;
    const int t_lo = k_lo / FA_BN, t_hi = active ? pos_max / FA_BN + 1 : 0;
    const int n_tiles = active ? t_hi - t_lo : 0;
    const int head0 = kvh * g + hchunk * hpc;
    const int n_heads = min(hpc, g - hchunk * hpc);

    if (warp == 0) {
        if (lane == 0 && active) {
            mbar_expect_tx(q_full, (uint32_t)(hpc * tpc * 128 * FA_HB));      // the box is hpc x tpc rows of 128 bytes
#pragma unroll
            for (int hb = 0; hb < FA_HB; ++hb)
                tma_load_3d(&map_q, q_full, sQ + hb * FA_BLOCK_BYTES, hb * 64, head0, q_start + tok0);
            const int* table = a.page_table + (size_t)seq * a.table_cols;
            bool ok = true;
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int st = j & 1;
                ok = mbar_wait(&kv_empty[st], (uint32_t)((j >> 1) & 1) ^ 1u, abort_flag);
                if (!ok) break;
                uint8_t* sK = sKV + st * FA_STAGE_BYTES;
                uint8_t* sV = sK + FA_KV_BYTES;
                mbar_expect_tx(&kv_full[st], FA_STAGE_BYTES);
                const int block0 = (t_lo + j) * (FA_BN / FA_PAGE);
                const int page0 = table[block0];
#pragma unroll
                for (int pg = 0; pg < FA_BN / FA_PAGE; ++pg) {
                    // a page the sequence does not have (yet) is stood in for by the tile's first
                    // page: its keys are masked, and its values are finite
                    int page = (block0 + pg < a.table_cols) ? table[block0 + pg] : -1;
                    if (page < 0) page = page0;
                    const int krow = ((page * 2 + 0) * a.nkh + kvh) * FA_PAGE;
                    const int vrow = ((page * 2 + 1) * a.nkh + kvh) * FA_PAGE;
#pragma unroll
                    for (int hb = 0; hb < FA_HB; ++hb) {
                        tma_load_2d(&map_kv, &kv_full[st], sK + hb * FA_BLOCK_BYTES + pg * FA_PAGE * 128, hb * 64, krow);
                        tma_load_2d(&map_kv, &kv_full[st], sV + hb * FA_BLOCK_BYTES + pg * FA_PAGE * 128, hb * 64, vrow);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && active) {
            constexpr uint32_t idesc_qk = umma_idesc_bf16(FA_BM, FA_BN);
            constexpr uint32_t idesc_pv = umma_idesc_bf16_b_mn(FA_BM, HD);
            bool ok = mbar_wait(q_full, 0, abort_flag);
            auto issue_pv = [&](int i) -> bool {
                if (!mbar_wait(p_ready, (uint32_t)(i & 1), abort_flag)) return false;
                if (!mbar_wait(o_empty, (uint32_t)(i & 1) ^ 1u, abort_flag)) return false;
                tc_fence_after();
                const uint32_t sV = smem_u32(sKV + (i & 1) * FA_STAGE_BYTES + FA_KV_BYTES);
                const uint32_t sPa = smem_u32(sP);
#pragma unroll
                for (int ks = 0; ks < FA_BN / 16; ++ks)
                    umma_bf16(tmem_base + 256,
                              umma_desc_sw128(sPa + (ks >> 2) * FA_BLOCK_BYTES + (ks & 3) * 32),
                              umma_desc_sw128_mn(sV + ks * 16 * 128, FA_BLOCK_BYTES), idesc_pv, ks > 0 ? 1u : 0u);
                umma_commit(o_full);
                umma_commit(&kv_empty[i & 1]);
                return true;
            };
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int st = j & 1;
                const uint32_t ph = (uint32_t)((j >> 1) & 1);
                ok = mbar_wait(&kv_full[st], ph, abort_flag) && mbar_wait(&s_empty[st], ph ^ 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t sQa = smem_u32(sQ), sK = smem_u32(sKV + st * FA_STAGE_BYTES);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint32_t off = (ks >> 2) * FA_BLOCK_BYTES + (ks & 3) * 32;
                    umma_bf16(tmem_base + st * 128, umma_desc_sw128(sQa + off), umma_desc_sw128(sK + off), idesc_qk,
                              ks > 0 ? 1u : 0u);
                }
                umma_commit(&s_full[st]);
                if (j > 0) ok = issue_pv(j - 1);
            }
            if (ok && n_tiles > 0) issue_pv(n_tiles - 1);
        }
    } else if (active) {
        const int quarter = warp & 3;                          // tensor-memory lanes 32 * quarter ...
        const int half = (warp - 2) >> 2;                      // keys / output dims [64 * half, 64 * half + 64)
        const int r = quarter * 32 + lane;                     // this thread's row
        const int tl = r / hpc, hl = r - tl * hpc;
        const bool valid = tl < n_tok && hl < n_heads;
        const int pos = valid ? pos_min + tl : -1;
        const int lo = (a.window > 0) ? pos - a.window + 1 : 0;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        constexpr int OD = HD / 2;                             // output dimensions a thread keeps
        float o[OD];
#pragma unroll
        for (int i = 0; i < OD; ++i) o[i] = 0.f;
        float m = -INFINITY, l = 0.f, corr_prev = 1.f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int st = j & 1;
            ok = mbar_wait(&s_full[st], (uint32_t)((j >> 1) & 1), abort_flag);
            if (!ok) break;
            tc_fence_after();
            const int key0 = (t_lo + j) * FA_BN + half * 64;
            const bool all_visible = ((t_lo + j) * FA_BN + FA_BN - 1 <= pos_min) &&
                                     (a.window == 0 || (t_lo + j) * FA_BN >= pos_max - a.window + 1);
            float sv[64];
            tmem_ld32x2(tmem_base + st * 128 + half * 64 + lane_addr, sv);
            float mx = -INFINITY;
            if (all_visible) {
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 64; ++i) mx = fmaxf(mx, sv[i]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int key = key0 + i;
                    if (!(key <= pos && key >= lo)) sv[i] = -INFINITY;
                    mx = fmaxf(mx, sv[i]);
                }
            }
            // the two halves of the row agree on the maximum
            float* xm = xchg + (j & 1) * 256;
            xm[half * 128 + r] = mx;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            mx = fmaxf(mx, xm[(half ^ 1) * 128 + r]) * a.scale_log2;   // scale > 0 commutes with the maximum
            const float m_new = fmaxf(m, mx);
            const float ms = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = fast_exp2(m - ms);
            m = m_new;
            // probabilities, rounded to bfloat16 (kept in registers until the P buffer is free)
            float sum = 0.f;
            const bool dead = !valid && all_visible;
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float p0 = dead ? 0.f : fast_exp2(fmaf(sv[2 * i], a.scale_log2, -ms));
                const float p1 = dead ? 0.f : fast_exp2(fmaf(sv[2 * i + 1], a.scale_log2, -ms));
                sum += p0 + p1;
                __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
                pk[i] = *reinterpret_cast<uint32_t*>(&b);
            }
            l = l * corr + sum;
            // the second product of the tile before reads the P buffer until o_full completes
            if (j > 0) {
                ok = mbar_wait(o_full, (uint32_t)((j - 1) & 1), abort_flag);
                if (!ok) break;
            }
            uint8_t* prow = sP + half * FA_BLOCK_BYTES + r * 128;      // this thread's 128-byte row of block `half`
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8)
                *reinterpret_cast<uint4*>(prow + ((c8 ^ (r & 7)) << 4)) =
                    make_uint4(pk[c8 * 4], pk[c8 * 4 + 1], pk[c8 * 4 + 2], pk[c8 * 4 + 3]);
            tc_fence_before();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(p_ready);
            mbar_arrive(&s_empty[st]);
            // the output of the tile before, rescaled by how far the maximum moved since
            if (j > 0) {
                tc_fence_after();
                float ov[OD];
                tmem_ld_od(tmem_base + 256 + half * OD + lane_addr, ov);
#pragma unroll
                for (int i = 0; i < OD; ++i) o[i] = fmaf(o[i], corr_prev, ov[i]);
                tc_fence_before();
                mbar_arrive(o_empty);
            }
            corr_prev = corr;
        }
        if (ok && n_tiles > 0) {
            ok = mbar_wait(o_full, (uint32_t)((n_tiles - 1) & 1), abort_flag);
            if (ok) {
                tc_fence_after();
                float ov[OD];
                tmem_ld_od(tmem_base + 256 + half * OD + lane_addr, ov);
#pragma unroll
                for (int i = 0; i < OD; ++i) o[i] = fmaf(o[i], corr_prev, ov[i]);
                // the two halves of the row add their denominators
                float* xl = xchg + (n_tiles & 1) * 256;
                xl[half * 128 + r] = l;
                asm volatile("bar.sync 1, 256;" ::: "memory");
                l += xl[(half ^ 1) * 128 + r];
                if (valid) {
                    const float inv = 1.f / l;
                    __nv_bfloat16* dst = a.out + (size_t)(q_start + tok0 + tl) * a.out_row_stride +
                                         (size_t)(head0 + hl) * HD + half * OD;
#pragma unroll
                    for (int c = 0; c < OD; c += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            __nv_bfloat162 b = __floats2bfloat162_rn(o[c + 2 * i] * inv, o[c + 2 * i + 1] * inv);
                            w[i] = *reinterpret_cast<uint32_t*>(&b);
                        }
                        *reinterpret_cast<uint4*>(dst + c) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(a.error_flag, 1);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, FA_TMEM_COLS);
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*FaEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static FaEncodeTiledFn fa_encode_fn() {
    static FaEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (FaEncodeTiledFn)p;
    }
    return fn;
}

extern "C" int braid_attn_tc_supported(void) { return 1; }

// Prompt attention on tcgen05.  Arguments as braid_attn_mma (attn_mma.cu); no slicing of
// the context.  `cache_rows` = pages * 2 * nkh * 64 rows of head_dim elements.
extern "C" int braid_attn_tc(const void* q, void* out, const void* cache, long long cache_rows, const int* page_table,
                             const int* q_start, const int* q_len, const int* kv_before,
                             int q_row_stride, int out_row_stride, int rows, int n_seqs, int max_q_len,
                             int nqh, int nkh, int hd, int table_cols, int window, float scale,
                             int* error_flag, void* stream) {
    if (rows <= 0 || n_seqs <= 0) return BRAID_OK;
    if (hd != BRAID_HD) BRAID_REFUSE("attn_tc: this library was compiled for head_dim=%d, not %d", BRAID_HD, hd);
    if (nqh <= 0 || nkh <= 0 || nqh % nkh) BRAID_REFUSE("attn_tc: %d query heads do not divide into %d kv heads", nqh, nkh);
    if ((q_row_stride % 8) || ((uintptr_t)q & 15) || ((uintptr_t)cache & 15)) BRAID_REFUSE("attn_tc: queries and cache must be 16-byte aligned");
    if ((out_row_stride % 8) || ((uintptr_t)out & 15)) BRAID_REFUSE("attn_tc: out rows must be 16-byte aligned");
    if (!error_flag) BRAID_REFUSE("attn_tc: error_flag is required");
    FaEncodeTiledFn fn = fa_encode_fn();
    if (!fn) BRAID_REFUSE("attn_tc: the driver does not export cuTensorMapEncodeTiled");
    const int g = nqh / nkh;
    const int hpc = g < FA_BM ? g : FA_BM, tpc = FA_BM / hpc, hchunks = (g + hpc - 1) / hpc;
    CUtensorMap mq, mkv;
    {
        cuuint64_t dims[3] = {(cuuint64_t)BRAID_HD, (cuuint64_t)nqh, (cuuint64_t)rows};
        cuuint64_t strides[2] = {(cuuint64_t)BRAID_HD * 2, (cuuint64_t)q_row_stride * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)hpc, (cuuint32_t)tpc};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = fn(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) BRAID_REFUSE("attn_tc: cuTensorMapEncodeTiled(q) failed with %d", (int)r);
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)BRAID_HD, (cuuint64_t)cache_rows};
        cuuint64_t strides[1] = {(cuuint64_t)BRAID_HD * 2};
        cuuint32_t box[2] = {64, FA_PAGE};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = fn(&mkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) BRAID_REFUSE("attn_tc: cuTensorMapEncodeTiled(cache) failed with %d", (int)r);
    }
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM);
        if (e != cudaSuccess) { braid_set_error("attn_tc: cannot reserve %d bytes of shared memory: %s", FA_SMEM, cudaGetErrorString(e)); return (int)e; }
        configured = true;
    }
    const long long gx = (max_q_len + tpc - 1) / tpc;
    if (gx > 0x7fffffffLL || (long long)nkh * hchunks > 65535 || n_seqs > 65535)
        BRAID_REFUSE("attn_tc: the step exceeds the grid limits");
    AttnTcArgs a{(__nv_bfloat16*)out, page_table, q_start, q_len, kv_before, out_row_stride, nqh, nkh, table_cols, window,
                 scale * 1.4426950408889634f, error_flag};
    braid_launch(attn_tc_kernel, dim3((unsigned)gx, nkh * hchunks, n_seqs), dim3(FA_THREADS), FA_SMEM,
                 (cudaStream_t)stream, mq, mkv, a);
    BRAID_LAUNCH_CHECK();
}

#else
extern "C" int braid_attn_tc_supported(void) { return 0; }
#endif
