// bfloat16 attention of prompts over the paged cache on the 5th-generation tensor cores
// (tcgen05), compiled for one head size: -DBRAID_HD=64 or 128.
//
// A CTA owns 128 rows: the query heads of one kv head (up to 128 of them) for 128 / heads
// consecutive tokens of one sequence, and walks the visible keys one 64-position page at
// a time.  Two CTAs share an SM (half its shared memory, tensor memory and registers
// each), so that one's chain of dependent steps runs under the other's.
//
//   warp 0      TMA: the query tile once, then key tiles into a ring of two stages and
//               value tiles into a ring of three, each as soon as its stage is free
//               (cp.async.bulk.tensor, 128-byte swizzle, no multicast);
//   warp 1      one lane issues S = Q K^T (accumulator in tensor memory, two buffers) and,
//               once the softmax warps have written P, O += P V, accumulated in tensor memory;
//   warps 2..5  one thread per row: read the 64 scores of S from tensor memory, mask,
//               running maximum and denominator in float32, and write P = exp2(s - m),
//               rounded to bfloat16, back into tensor memory over the first half of the
//               row's scores: the second product takes P from there as its A operand.
//
// S of tile j + 2 overwrites the buffer of tile j; the MMA warp issues it only when the second
// product of tile j, which reads P from there, has completed (issued a tile earlier, so it has).
// The softmax warps look at the completion of every second product, one tile late, which costs
// nothing and keeps their view of that barrier within one phase (see the loop).
//
// The running maximum m is only raised when a tile's maximum exceeds it by more than 8
// (in the exponent of two), and then the thread scales its row of O in tensor memory by
// exp2(m_old - m_new) before the next product adds to it.  In between, probabilities are
// at most 2^8; the denominator is taken against the same m, so the quotient is exact.
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
#define FA_BN 64                                 // keys per tile: one page
#include "page.h"
#define FA_PAGE BRAID_PAGE_SIZE
static_assert(FA_PAGE == 64, "a key tile of this kernel is one page of 64 positions");
#define FA_THREADS 192                           // TMA warp, MMA warp, 4 softmax warps
#define FA_HB (BRAID_HD / 64)                    // 64-element blocks of the head dimension
#define FA_QBLOCK_BYTES (128 * 128)              // [128 rows][64 elements] bf16, 128-byte rows
#define FA_KBLOCK_BYTES (64 * 128)               // [64 positions][64 elements]
#define FA_Q_BYTES (FA_HB * FA_QBLOCK_BYTES)
#define FA_KV_BYTES (FA_HB * FA_KBLOCK_BYTES)    // one K or one V tile
#define FA_KST 2                                 // stages of the key ring
#define FA_VST 3                                 // stages of the value ring
#define FA_BAR_BYTES 192
#define FA_SMEM (FA_Q_BYTES + (FA_KST + FA_VST) * FA_KV_BYTES + FA_BAR_BYTES)
#define FA_TMEM_COLS 256                         // S0 [0,64) S1 [64,128) (P over their first 32 columns), O [128, 128 + HD)
#define FA_RAISE 8.f                             // how far a tile's maximum may exceed m before m is raised

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
// tcgen05.mma with both operands in shared memory, and with the A operand in tensor memory (rows in
// lanes, K packed two bfloat16 a column).  Descriptors are given as (low word, high word): a
// descriptor's start address lives in its low word, the high word is the same for all tiles of a kind.
__device__ __forceinline__ void umma_ss_lohi(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                             uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_ts_lohi(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi,
                                             uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_addr(uint32_t bar_addr) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}
// 32 consecutive columns of this thread's lane written (no wait).
__device__ __forceinline__ void tmem_st32_nowait(uint32_t taddr, const uint32_t* w) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        :: "r"(taddr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]), "r"(w[8]),
           "r"(w[9]), "r"(w[10]), "r"(w[11]), "r"(w[12]), "r"(w[13]), "r"(w[14]), "r"(w[15]), "r"(w[16]), "r"(w[17]),
           "r"(w[18]), "r"(w[19]), "r"(w[20]), "r"(w[21]), "r"(w[22]), "r"(w[23]), "r"(w[24]), "r"(w[25]), "r"(w[26]),
           "r"(w[27]), "r"(w[28]), "r"(w[29]), "r"(w[30]), "r"(w[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// The reverse: 64 consecutive columns of this thread's lane written back.
__device__ __forceinline__ void tmem_st32x2(uint32_t taddr, const float* v) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
            "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
            :: "r"(taddr + h * 32),
               "r"(__float_as_uint(v[h * 32 + 0])), "r"(__float_as_uint(v[h * 32 + 1])), "r"(__float_as_uint(v[h * 32 + 2])),
               "r"(__float_as_uint(v[h * 32 + 3])), "r"(__float_as_uint(v[h * 32 + 4])), "r"(__float_as_uint(v[h * 32 + 5])),
               "r"(__float_as_uint(v[h * 32 + 6])), "r"(__float_as_uint(v[h * 32 + 7])), "r"(__float_as_uint(v[h * 32 + 8])),
               "r"(__float_as_uint(v[h * 32 + 9])), "r"(__float_as_uint(v[h * 32 + 10])), "r"(__float_as_uint(v[h * 32 + 11])),
               "r"(__float_as_uint(v[h * 32 + 12])), "r"(__float_as_uint(v[h * 32 + 13])), "r"(__float_as_uint(v[h * 32 + 14])),
               "r"(__float_as_uint(v[h * 32 + 15])), "r"(__float_as_uint(v[h * 32 + 16])), "r"(__float_as_uint(v[h * 32 + 17])),
               "r"(__float_as_uint(v[h * 32 + 18])), "r"(__float_as_uint(v[h * 32 + 19])), "r"(__float_as_uint(v[h * 32 + 20])),
               "r"(__float_as_uint(v[h * 32 + 21])), "r"(__float_as_uint(v[h * 32 + 22])), "r"(__float_as_uint(v[h * 32 + 23])),
               "r"(__float_as_uint(v[h * 32 + 24])), "r"(__float_as_uint(v[h * 32 + 25])), "r"(__float_as_uint(v[h * 32 + 26])),
               "r"(__float_as_uint(v[h * 32 + 27])), "r"(__float_as_uint(v[h * 32 + 28])), "r"(__float_as_uint(v[h * 32 + 29])),
               "r"(__float_as_uint(v[h * 32 + 30])), "r"(__float_as_uint(v[h * 32 + 31]))
            : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

struct AttnTcArgs {
    __nv_bfloat16* out;
    const int* page_table;
    const int* q_start;
    const int* q_len;
    const int* kv_before;
    int out_row_stride, nqh, nkh, table_cols, window;
    float scale_log2;
    int num_pages;
    int* error_flag;
};

__global__ void __launch_bounds__(FA_THREADS, 2)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, AttnTcArgs a) {
    constexpr int HD = BRAID_HD;
    pdl_trigger();
    // the swizzled tiles want 1024-byte alignment; two CTAs an SM leave no room for slack, so
    // the start of dynamic shared memory is checked instead of rounded up
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0) atomicExch(a.error_flag, 1);
        return;
    }
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + FA_Q_BYTES;                 // [FA_KST]
    uint8_t* sV = sK + FA_KST * FA_KV_BYTES;       // [FA_VST]
    uint64_t* bars = (uint64_t*)(sV + FA_VST * FA_KV_BYTES);
    uint64_t* q_full = bars;                       // [1]
    uint64_t* k_full = q_full + 1;                 // [FA_KST]
    uint64_t* k_empty = k_full + FA_KST;           // [FA_KST]
    uint64_t* v_full = k_empty + FA_KST;           // [FA_VST]
    uint64_t* v_empty = v_full + FA_VST;           // [FA_VST]
    uint64_t* s_full = v_empty + FA_VST;           // [2]
    // two p_ready barriers take turns: the softmax warps may finish tile j + 1 before the MMA warp has
    // looked at tile j's (it issues S of tile j + 1 first, and may then wait for a value tile), and a
    // single barrier two phases ahead reads like one that has not moved
    uint64_t* p_ready = s_full + 2;                // [2]
    uint64_t* pv_done = p_ready + 2;               // [1]
    uint32_t* tmem_slot = (uint32_t*)(pv_done + 1);
    static_assert((1 + 2 * FA_KST + 2 * FA_VST + 5) * 8 + 8 <= FA_BAR_BYTES, "the barriers outgrow their bytes");
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = a.nqh / a.nkh;
    const int hpc = g < FA_BM ? g : FA_BM;
    const int tpc = FA_BM / hpc;
    const int hchunks = (g + hpc - 1) / hpc;
    // CTAs start in the order x, y, z: all kv heads and sequences of the last token tile first, then
    // the tile before, ...: late tokens see the most keys, so the longest CTAs start first and the
    // short ones fill the gaps at the end
    const int seq = blockIdx.y;
    const int kvh = blockIdx.x / hchunks, hchunk = blockIdx.x - kvh * hchunks;
    const int tile = gridDim.z - 1 - blockIdx.z;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < FA_KST; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
        for (int s = 0; s < FA_VST; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
        mbar_init(&p_ready[0], 128); mbar_init(&p_ready[1], 128); mbar_init(pv_done, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, FA_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base + 128;
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
                tma_load_3d(&map_q, q_full, sQ + hb * FA_QBLOCK_BYTES, hb * 64, head0, q_start + tok0);
            const int* table = a.page_table + (size_t)seq * a.table_cols;
            // key and value tiles go out independently, each as soon as its stage is free
            int jk = 0, jv = 0;
            uint32_t idle = 0;
            uint64_t idle_since = 0;
            while (jk < n_tiles || jv < n_tiles) {
                bool moved = false;
                const bool k_turn = jk < n_tiles && mbar_try_wait(&k_empty[jk % FA_KST], (uint32_t)((jk / FA_KST) & 1) ^ 1u);
                const bool v_turn = !k_turn && jv < n_tiles && mbar_try_wait(&v_empty[jv % FA_VST], (uint32_t)((jv / FA_VST) & 1) ^ 1u);
                if (k_turn || v_turn) {
                    const int j = k_turn ? jk : jv;
                    int page = (t_lo + j < a.table_cols) ? table[t_lo + j] : -1;
                    if (page < 0 || page >= a.num_pages) {          // a visible position without a page: the table is broken
                        atomicExch(a.error_flag, 1);
                        page = 0;
                    }
                    const int row = ((page * 2 + (k_turn ? 0 : 1)) * a.nkh + kvh) * FA_PAGE;
                    const int st = k_turn ? jk % FA_KST : jv % FA_VST;
                    uint64_t* bar = k_turn ? &k_full[st] : &v_full[st];
                    uint8_t* dst = (k_turn ? sK : sV) + st * FA_KV_BYTES;
                    mbar_expect_tx(bar, FA_KV_BYTES);
#pragma unroll
                    for (int hb = 0; hb < FA_HB; ++hb) tma_load_2d(&map_kv, bar, dst + hb * FA_KBLOCK_BYTES, hb * 64, row);
                    if (k_turn) ++jk; else ++jv;
                    moved = true;
                }
                if (moved) { idle = 0; idle_since = 0; continue; }
                if (++idle >= TC_SPIN_LIMIT) { *abort_flag = 1; break; }
                if ((idle & 1023u) == 1023u) {              // the same bound as mbar_wait: time on the device's clock
                    if (*abort_flag) break;
                    const uint64_t now = global_timer_ns();
                    if (idle_since == 0) idle_since = now;
                    else if (now - idle_since > TC_WAIT_LIMIT_NS) { *abort_flag = 1; break; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && active) {
            constexpr uint32_t idesc_qk = umma_idesc_bf16(FA_BM, FA_BN);
            constexpr uint32_t idesc_pv = umma_idesc_bf16_b_mn(FA_BM, HD);
            bool ok = mbar_wait(q_full, 0, abort_flag);
            // operand descriptors differ only in their start address (bits 0..13 of the low word, in 16-byte units)
            const uint64_t dq = umma_desc_sw128(smem_u32(sQ));
            const uint64_t dk = umma_desc_sw128(smem_u32(sK));
            const uint64_t dv = umma_desc_sw128_mn(smem_u32(sV), FA_KBLOCK_BYTES);
            const uint32_t q_lo = (uint32_t)dq, k_lo = (uint32_t)dk, v_lo = (uint32_t)dv;
            const uint32_t kq_hi = (uint32_t)(dq >> 32), v_hi = (uint32_t)(dv >> 32);
            const uint32_t bar0 = smem_u32(bars);                        // barrier i lies at bar0 + 8 i
            const uint32_t a_k_empty = bar0 + 8 * (uint32_t)(k_empty - bars), a_v_empty = bar0 + 8 * (uint32_t)(v_empty - bars);
            const uint32_t a_s_full = bar0 + 8 * (uint32_t)(s_full - bars), a_pv_done = bar0 + 8 * (uint32_t)(pv_done - bars);
            auto issue_pv = [&](int i, int st) -> bool {
                if (!mbar_wait(&v_full[st], (uint32_t)((i / FA_VST) & 1), abort_flag)) return false;
                if (!mbar_wait(&p_ready[i & 1], (uint32_t)((i >> 1) & 1), abort_flag)) return false;     // P written, O rescaled
                tc_fence_after();
                const uint32_t vs_lo = v_lo + (uint32_t)((st * FA_KV_BYTES) >> 4);
                const uint32_t tp = tmem_base + (i & 1) * FA_BN;
                umma_ts_lohi(tmem_o, tp, vs_lo, v_hi, idesc_pv, i > 0 ? 1u : 0u);
#pragma unroll
                for (int ks = 1; ks < FA_BN / 16; ++ks)
                    umma_ts_lohi(tmem_o, tp + ks * 8, vs_lo + (uint32_t)((ks * 16 * 128) >> 4), v_hi, idesc_pv, 1u);
                umma_commit_addr(a_pv_done);
                umma_commit_addr(a_v_empty + 8 * st);
                return true;
            };
            int kst = 0, vst = 0;                  // ring stages of key tile j and of value tile j - 1
            for (int j = 0; j < n_tiles && ok; ++j) {
                ok = mbar_wait(&k_full[kst], (uint32_t)((j / FA_KST) & 1), abort_flag);
                // S of tile j goes where S and P of tile j - 2 were: the second product of tile j - 2,
                // which reads that P, has to be complete (it was issued a tile ago, so this wait is short;
                // issue order alone does not keep a product's writes behind its predecessor's reads)
                if (ok && j >= 2) ok = mbar_wait(pv_done, (uint32_t)(j & 1), abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t ks_lo = k_lo + (uint32_t)((kst * FA_KV_BYTES) >> 4);
                const uint32_t ts = tmem_base + (j & 1) * FA_BN;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint32_t qoff = ((ks >> 2) * FA_QBLOCK_BYTES + (ks & 3) * 32) >> 4, koff = ((ks >> 2) * FA_KBLOCK_BYTES + (ks & 3) * 32) >> 4;
                    umma_ss_lohi(ts, q_lo + qoff, kq_hi, ks_lo + koff, kq_hi, idesc_qk, ks > 0 ? 1u : 0u);
                }
                umma_commit_addr(a_s_full + 8 * (j & 1));
                umma_commit_addr(a_k_empty + 8 * kst);
                if (++kst == FA_KST) kst = 0;
                if (j > 0) {
                    ok = issue_pv(j - 1, vst);
                    if (++vst == FA_VST) vst = 0;
                }
            }
            if (ok && n_tiles > 0) issue_pv(n_tiles - 1, vst);
        }
    } else if (active) {
        const int quarter = warp & 3;                          // tensor-memory lanes 32 * quarter ...
        const int r = quarter * 32 + lane;                     // this thread's row
        const int tl = r / hpc, hl = r - tl * hpc;
        const bool valid = tl < n_tok && hl < n_heads;
        const int pos = valid ? pos_min + tl : -1;
        const int lo = (a.window > 0) ? pos - a.window + 1 : 0;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int st = j & 1;
            ok = mbar_wait(&s_full[st], (uint32_t)((j >> 1) & 1), abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            float sv[64];
            tmem_ld32x2(tmem_base + st * FA_BN + lane_addr, sv);
            const int key0 = (t_lo + j) * FA_BN;
            const bool all_visible = (key0 + FA_BN - 1 <= pos_min) && (a.window == 0 || key0 >= pos_max - a.window + 1);
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
            if (all_visible) {
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 64; i += 4) {
                        mx0 = fmaxf(mx0, sv[i]); mx1 = fmaxf(mx1, sv[i + 1]);
                        mx2 = fmaxf(mx2, sv[i + 2]); mx3 = fmaxf(mx3, sv[i + 3]);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 64; i += 4) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + i + e;
                        if (!(key <= pos && key >= lo)) sv[i + e] = -INFINITY;
                    }
                    mx0 = fmaxf(mx0, sv[i]); mx1 = fmaxf(mx1, sv[i + 1]);
                    mx2 = fmaxf(mx2, sv[i + 2]); mx3 = fmaxf(mx3, sv[i + 3]);
                }
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * a.scale_log2;   // scale > 0 commutes with the maximum
            // raise m only when the tile towers over it; -inf + 8 = -inf, so the first finite maximum always does
            const bool raise = mx > m + FA_RAISE;
            const float factor = raise ? fast_exp2(m - mx) : 1.f;                     // exp2(-inf) = 0: nothing was summed yet
            if (raise) m = mx;
            // a row that is no query (past the tile's tokens or heads) sums nothing: exp2(-inf) = 0
            const float ms = (!valid && all_visible) ? INFINITY : ((m == -INFINITY) ? 0.f : m);
            // probabilities, rounded to bfloat16
            float sum0 = 0.f, sum1 = 0.f;
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float p0 = fast_exp2(fmaf(sv[2 * i], a.scale_log2, -ms));
                const float p1 = fast_exp2(fmaf(sv[2 * i + 1], a.scale_log2, -ms));
                sum0 += p0;
                sum1 += p1;
                __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
                pk[i] = *reinterpret_cast<uint32_t*>(&b);
            }
            l = l * factor + (sum0 + sum1);
            tmem_st32_nowait(tmem_base + st * FA_BN + lane_addr, pk);      // over the first half of this row's scores
            if (j > 0) {
                // Every tile, the second product of the tile before is waited for (it was issued a whole
                // softmax ago, so this costs nothing): a parity wait only tells apart a barrier that is
                // at most one phase off, and a thread that looked at pv_done only now and then, or
                // only at the end, could find it two phases behind and take that for done.
                ok = mbar_wait(pv_done, (uint32_t)((j - 1) & 1), abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (__any_sync(0xffffffffu, raise)) {          // tensor-memory loads and stores take the whole warp
                    tc_fence_after();
#pragma unroll
                    for (int h = 0; h < HD / 64; ++h) {
                        float ov[64];
                        tmem_ld32x2(tmem_o + h * 64 + lane_addr, ov);
#pragma unroll
                        for (int i = 0; i < 64; ++i) ov[i] *= factor;
                        tmem_st32x2(tmem_o + h * 64 + lane_addr, ov);
                    }
                }
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&p_ready[st]);
        }
        if (ok && n_tiles > 0) {
            ok = mbar_wait(pv_done, (uint32_t)((n_tiles - 1) & 1), abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                tc_fence_after();
                const float inv = 1.f / l;
                __nv_bfloat16* dst = a.out + (size_t)(q_start + tok0 + tl) * a.out_row_stride + (size_t)(head0 + hl) * HD;
#pragma unroll
                for (int h = 0; h < HD / 64; ++h) {
                    float ov[64];
                    tmem_ld32x2(tmem_o + h * 64 + lane_addr, ov);
                    if (valid) {
#pragma unroll
                        for (int c = 0; c < 64; c += 8) {
                            uint32_t w[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                __nv_bfloat162 b = __floats2bfloat162_rn(ov[c + 2 * i] * inv, ov[c + 2 * i + 1] * inv);
                                w[i] = *reinterpret_cast<uint32_t*>(&b);
                            }
                            *reinterpret_cast<uint4*>(dst + h * 64 + c) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
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
    TcEncodeTiledFn fn = tc_encode_tiled_fn();
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
    if (gx > 65535 || (long long)nkh * hchunks > 0x7fffffffLL || n_seqs > 65535)
        BRAID_REFUSE("attn_tc: the step exceeds the grid limits (%lld token tiles, %d sequences)", gx, n_seqs);
    const long long num_pages = cache_rows / (2LL * nkh * FA_PAGE);
    AttnTcArgs a{(__nv_bfloat16*)out, page_table, q_start, q_len, kv_before, out_row_stride, nqh, nkh, table_cols, window,
                 scale * 1.4426950408889634f, (int)num_pages, error_flag};
    braid_launch(attn_tc_kernel, dim3(nkh * hchunks, n_seqs, (unsigned)gx), dim3(FA_THREADS), FA_SMEM,
                 (cudaStream_t)stream, mq, mkv, a);
    BRAID_LAUNCH_CHECK();
}

#else
extern "C" int braid_attn_tc_supported(void) { return 0; }
#endif
