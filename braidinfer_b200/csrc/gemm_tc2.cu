// bfloat16 matrix product of prompts on pairs of SMs (tcgen05.mma.cta_group::2):
//   out[n, m] = sum_k x[n, k] * w[m, k],   float32 accumulation in tensor memory.
//
// Two CTAs of a cluster compute one [256 weight rows x 256 tokens] output tile.  Each CTA
// loads its own [128 x 64] half of the weight tile and its own [128 x 64] half of the token
// tile per k block (32 KB a stage instead of the 48 KB a CTA of gemm_tc.cu loads for half the
// output), the leader CTA (rank 0) issues one MMA of M = 256, N = 256 that reads both CTAs'
// shared memory, and each CTA's tensor memory receives its 128 rows of the accumulator, all
// 256 token columns.  A third less shared-memory fill and L2 traffic per FLOP than one CTA a
// tile: where the product is bound by power, that is what there is to save.
//
//   warp 0 (both CTAs)  one lane issues the CTA's TMA loads (cta_group::2, no multicast); their
//                       bytes are counted on the leader's `full` barrier of the stage;
//   warp 1              allocates tensor memory (both CTAs, cta_group::2); in the leader one
//                       lane issues the MMAs and commits: `empty` of the stage and `acc_full` of
//                       the accumulator buffer are signalled in both CTAs (commit with
//                       .multicast::cluster, which is no load);
//   warps 2..5 (both)   epilogue of the CTA's 128 rows: store, float32 residual sum, or SwiGLU
//                       (as in gemm_tc.cu); they arrive on the leader's `acc_empty`.  Where the
//                       output can be addressed by TMA, 32 tokens at a time go through a staging
//                       tile in shared memory and leave as one TMA store; the residual sum in
//                       place (out == res) is a TMA reduce-add, so no thread waits for a load of
//                       the residual from global memory.
//
// Persistent: one cluster per pair of SMs walks the tiles in the order of tc_tile_coords.
// Every wait is bounded by time; a wait that runs out sets *error_flag, and the kernel frees
// its tensor memory and returns.
#include "common.cuh"
#include "streamk.cuh"
#include "tcgen05.cuh"

#define T2_BLOCK_M 128          // weight rows of one CTA (256 a pair)
#define T2_BLOCK_N 256          // tokens of a tile; each CTA loads T2_HALF_N of them
#define T2_HALF_N 128
#define T2_BLOCK_K 64
#define T2_UMMA_K 16
#define T2_STAGES 6
#define T2_THREADS 192
#define T2_A_BYTES (T2_BLOCK_M * T2_BLOCK_K * 2)
#define T2_B_BYTES (T2_HALF_N * T2_BLOCK_K * 2)
#define T2_STAGE_BYTES (T2_A_BYTES + T2_B_BYTES)
#define T2_CHUNK 32              // token columns per tensor-memory load, and rows of a staging tile
#define T2_OUT_BYTES (T2_CHUNK * T2_BLOCK_M * 4)          // one staging tile: [32 tokens][128 outputs] float32
#define T2_SMEM_BYTES (T2_STAGES * T2_STAGE_BYTES + 2 * T2_OUT_BYTES + 1024 + 256)
#define T2_TMEM_COLS 512        // two accumulator buffers of 256 columns
#define T2_PEER_BIT_MASK 0xFEFFFFFFu      // a shared::cluster address with the CTA-rank bit cleared: the pair's leader

struct GemmTc2Args {
    void* out;                 // mode 0: [n, ldo] bf16/f32; 1: f32; 2: bf16/f32 [n, ldo]
    const float* res;          // mode 1
    int n_rows, m_out, k_in;   // mode 2: m_out is the number of gate rows (w has 2 * m_out rows)
    long long ldo;
    int out_dtype;
    int m_tiles, n_tiles;      // tiles of 256 weight rows x 256 tokens
    int* error_flag;
};

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// A tile into this CTA's shared memory; its bytes are counted on the barrier of the pair's leader.
__device__ __forceinline__ void tma_load_2d_pair(const CUtensorMap* map, uint64_t* bar, void* dst, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar) & T2_PEER_BIT_MASK), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive, once the MMAs issued so far are complete, on the barrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both) : "memory");
}
// Arrive on the barrier at this offset in the pair's leader.
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, 0;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// At most one group of stores may still be reading its staging tile.
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
struct T2Unit { int m0, n0; };

struct T2Walk {
    const GemmTc2Args& a;
    int u, step;
    __device__ T2Walk(const GemmTc2Args& a_) : a(a_) {
        u = blockIdx.x / 2;
        step = gridDim.x / 2;
    }
    __device__ bool next(T2Unit& t) {
        if (u >= a.m_tiles * a.n_tiles) return false;
        int mt, nt;
        tc_tile_coords(u, a.m_tiles, a.n_tiles, mt, nt);
        t.m0 = mt * 2 * T2_BLOCK_M;
        t.n0 = nt * T2_BLOCK_N;
        u += step;
        return true;
    }
};

template <int MODE, bool TMA_OUT>
__global__ void __launch_bounds__(T2_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                const __grid_constant__ CUtensorMap map_out, GemmTc2Args a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* staging = smem + T2_STAGES * T2_STAGE_BYTES;             // two tiles of T2_OUT_BYTES
    uint64_t* bars = (uint64_t*)(staging + 2 * T2_OUT_BYTES);
    uint64_t* full = bars;                                  // counted in the leader only
    uint64_t* empty = bars + T2_STAGES;                     // one in each CTA, for its own loader
    uint64_t* acc_full = bars + 2 * T2_STAGES;              // [2], one in each CTA, for its own epilogue
    uint64_t* acc_empty = acc_full + 2;                     // [2], counted in the leader: both CTAs' epilogues
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const bool leader = rank == 0;
    pdl_trigger();
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        if (TMA_OUT) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_out) : "memory");
        for (int s = 0; s < T2_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * 128); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, T2_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                       // both CTAs' barriers exist before either signals the other's
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_kb = (a.k_in + T2_BLOCK_K - 1) / T2_BLOCK_K;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // the first ring of weight tiles before the dependency wait: no kernel writes weights
            {
                T2Walk pre(a);
                T2Unit t;
                int n = 0;
                while (n < T2_STAGES && pre.next(t))
                    for (int i = 0; i < total_kb && n < T2_STAGES; ++i, ++n) {
                        if (leader) mbar_expect_tx(&full[n], 2 * T2_STAGE_BYTES);
                        tma_load_2d_pair(&map_w, &full[n], smem + n * T2_STAGE_BYTES, i * T2_BLOCK_K, t.m0 + (int)rank * T2_BLOCK_M);
                    }
            }
            pdl_wait();
            T2Walk walk(a);
            T2Unit t;
            int issued = 0;
            while (ok && walk.next(t)) {
                for (int i = 0; i < total_kb; ++i, ++issued) {
                    uint8_t* sa = smem + stage * T2_STAGE_BYTES;
                    uint8_t* sb = sa + T2_A_BYTES;
                    const int kx = i * T2_BLOCK_K;
                    if (issued >= T2_STAGES) {
                        ok = mbar_wait(&empty[stage], phase ^ 1u, abort_flag);
                        if (!ok) break;
                        if (leader) mbar_expect_tx(&full[stage], 2 * T2_STAGE_BYTES);
                        tma_load_2d_pair(&map_w, &full[stage], sa, kx, t.m0 + (int)rank * T2_BLOCK_M);
                    }
                    tma_load_2d_pair(&map_x, &full[stage], sb, kx, t.n0 + (int)rank * T2_HALF_N);
                    if (++stage == T2_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = umma_idesc_bf16(2 * T2_BLOCK_M, T2_BLOCK_N);
            int stage = 0, buf = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            T2Walk walk(a);
            T2Unit t;
            while (ok && walk.next(t)) {
                ok = mbar_wait(&acc_empty[buf], ((acc_phase >> buf) & 1u) ^ 1u, abort_flag);   // both epilogues have drained it
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * T2_BLOCK_N;
                for (int i = 0; i < total_kb; ++i) {
                    ok = mbar_wait(&full[stage], phase, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * T2_STAGE_BYTES);
                    const uint32_t sb = sa + T2_A_BYTES;
#pragma unroll
                    for (int k = 0; k < T2_BLOCK_K / T2_UMMA_K; ++k) {
                        const uint32_t koff = k * T2_UMMA_K * 2;
                        const uint32_t accum = (i > 0 || k > 0) ? 1u : 0u;
                        umma_bf16_pair(tmem_d, umma_desc_sw128(sa + koff), umma_desc_sw128(sb + koff), idesc, accum);
                    }
                    umma_commit_pair(&empty[stage]);
                    if (++stage == T2_STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit_pair(&acc_full[buf]);
                acc_phase ^= (1u << buf);
                buf ^= 1;
            }
        }
    } else {
        const int quarter = warp & 3;
        const bool issuer = threadIdx.x == 64;             // the one thread that issues and awaits the TMA stores
        pdl_wait();
        int buf = 0;
        uint32_t full_phase = 0, chunk_no = 0;
        bool ok = true;
        T2Walk walk(a);
        T2Unit t;
        while (ok && walk.next(t)) {
            const int m0 = t.m0 + (int)rank * T2_BLOCK_M;                  // this CTA's 128 rows of the pair's 256
            const int m = (MODE == 2) ? (m0 + quarter * 32) / 2 + (lane & 15) : m0 + quarter * 32 + lane;
            ok = mbar_wait(&acc_full[buf], (full_phase >> buf) & 1u, abort_flag);
            if (TMA_OUT) ok = epilogue_all(ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t trow = tmem_base + buf * T2_BLOCK_N + ((uint32_t)(quarter * 32) << 16);
            constexpr int CH = T2_CHUNK;
#pragma unroll 1
            for (int c0 = 0; c0 < T2_BLOCK_N; c0 += CH) {
                if (t.n0 + c0 >= a.n_rows) break;
                float v[CH];
                tmem_ld32(trow + c0, v);
                if (TMA_OUT) {
                    // the staging tile is free once the store before the last one has read it
                    uint8_t* tile = staging + (chunk_no & 1u) * T2_OUT_BYTES;
                    ++chunk_no;
                    if (issuer) bulk_wait_read_1();
                    epilogue_sync();
                    if (MODE == 2) {
                        // [32 tokens][64 outputs] bfloat16; the halves of a warp swap values as below
                        const bool is_up = (lane & 16) != 0;
                        __nv_bfloat16* dst = (__nv_bfloat16*)tile + (is_up ? 64 : 0) + quarter * 16 + (lane & 15);
#pragma unroll
                        for (int p2 = 0; p2 < CH / 2; ++p2) {
                            const float from_up = __shfl_xor_sync(0xffffffffu, v[2 * p2], 16);
                            const float from_gate = __shfl_xor_sync(0xffffffffu, v[2 * p2 + 1], 16);
                            const float g = is_up ? from_gate : v[2 * p2];
                            const float u = is_up ? v[2 * p2 + 1] : from_up;
                            dst[2 * p2 * 64] = __float2bfloat16_rn(__fdividef(g, 1.f + __expf(-g)) * u);
                        }
                    } else if (a.out_dtype == BRAID_F32) {
                        float* dst = (float*)tile + quarter * 32 + lane;
#pragma unroll
                        for (int i = 0; i < CH; ++i) dst[i * T2_BLOCK_M] = v[i];
                    } else {
                        __nv_bfloat16* dst = (__nv_bfloat16*)tile + quarter * 32 + lane;
#pragma unroll
                        for (int i = 0; i < CH; ++i) dst[i * T2_BLOCK_M] = __float2bfloat16_rn(v[i]);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    epilogue_sync();
                    const int x0 = MODE == 2 ? m0 / 2 : m0;
                    if (issuer && x0 < a.m_out) {
                        // rows and columns past the matrix are clipped by the tensor map
                        if (MODE == 1) tma_reduce_add_2d(&map_out, tile, x0, t.n0 + c0);
                        else tma_store_2d(&map_out, tile, x0, t.n0 + c0);
                        bulk_commit();
                    }
                    continue;
                }
                if (MODE == 2) {
                    // rows interleave gate and up in blocks of 16 (see gemm_tc.cu): the halves of a warp swap values
                    const bool is_up = (lane & 16) != 0;
                    const size_t o0 = (size_t)(t.n0 + c0 + (is_up ? 1 : 0)) * a.ldo + m;
#pragma unroll
                    for (int p2 = 0; p2 < CH / 2; ++p2) {
                        const float from_up = __shfl_xor_sync(0xffffffffu, v[2 * p2], 16);
                        const float from_gate = __shfl_xor_sync(0xffffffffu, v[2 * p2 + 1], 16);
                        const float g = is_up ? from_gate : v[2 * p2];
                        const float u = is_up ? v[2 * p2 + 1] : from_up;
                        const float y = __fdividef(g, 1.f + __expf(-g)) * u;
                        const int n = t.n0 + c0 + 2 * p2 + (is_up ? 1 : 0);
                        if (m < a.m_out && n < a.n_rows) {
                            if (a.out_dtype == BRAID_F32) ((float*)a.out)[o0 + (size_t)(2 * p2) * a.ldo] = y;
                            else ((__nv_bfloat16*)a.out)[o0 + (size_t)(2 * p2) * a.ldo] = __float2bfloat16_rn(y);
                        }
                    }
                    continue;
                }
                if (m < a.m_out) {
                    const size_t o0 = (size_t)(t.n0 + c0) * a.ldo + m;
                    if (MODE == 1) {
                        float r[CH];
#pragma unroll
                        for (int i = 0; i < CH; ++i) r[i] = (t.n0 + c0 + i < a.n_rows) ? a.res[o0 + (size_t)i * a.ldo] : 0.f;
#pragma unroll
                        for (int i = 0; i < CH; ++i)
                            if (t.n0 + c0 + i < a.n_rows) ((float*)a.out)[o0 + (size_t)i * a.ldo] = r[i] + v[i];
                    } else {
#pragma unroll
                        for (int i = 0; i < CH; ++i) {
                            if (t.n0 + c0 + i >= a.n_rows) break;
                            if (a.out_dtype == BRAID_F32) ((float*)a.out)[o0 + (size_t)i * a.ldo] = v[i];
                            else ((__nv_bfloat16*)a.out)[o0 + (size_t)i * a.ldo] = __float2bfloat16_rn(v[i]);
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive_leader(&acc_empty[buf]);
            full_phase ^= (1u << buf);
            buf ^= 1;
        }
        if (TMA_OUT && issuer) bulk_wait_all();           // the stores are complete, not only read, before the kernel ends
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(a.error_flag, 1);
    cluster_sync_all();                       // neither CTA frees tensor memory or leaves while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, T2_TMEM_COLS);
    }
}

// rows x k bfloat16 matrix with row stride ld (elements); box = 128 rows x 64, 128-byte swizzle.
static int make_map2(CUtensorMap* map, const void* base, long long rows, long long k, long long ld) {
    TcEncodeTiledFn fn = tc_encode_tiled_fn();
    if (!fn) BRAID_REFUSE("gemm_tc2: the driver does not export cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {T2_BLOCK_K, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) BRAID_REFUSE("gemm_tc2: cuTensorMapEncodeTiled failed with %d (rows=%lld k=%lld ld=%lld)", (int)r, rows, k, ld);
    return BRAID_OK;
}

// The output as TMA sees it: `inner` contiguous elements a row, `rows` rows `ld` elements apart; box = 32 rows x box_inner.
static int make_map_out(CUtensorMap* map, void* base, int out_dtype, long long inner, long long rows, long long ld, int box_inner) {
    TcEncodeTiledFn fn = tc_encode_tiled_fn();
    if (!fn) BRAID_REFUSE("gemm_tc2: the driver does not export cuTensorMapEncodeTiled");
    const int esize = out_dtype == BRAID_F32 ? 4 : 2;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * esize};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, T2_CHUNK};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, out_dtype == BRAID_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base,
                    dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) BRAID_REFUSE("gemm_tc2: cuTensorMapEncodeTiled failed with %d for the output (inner=%lld rows=%lld ld=%lld)", (int)r, inner, rows, ld);
    return BRAID_OK;
}

template <int MODE, bool TMA_OUT>
static int launch_tc2(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mo, const GemmTc2Args& a, int pairs, cudaStream_t s) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc2_kernel<MODE, TMA_OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES);
        if (e != cudaSuccess) { braid_set_error("gemm_tc2: cannot reserve %d bytes of shared memory: %s", T2_SMEM_BYTES, cudaGetErrorString(e)); return (int)e; }
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(T2_THREADS);
    cfg.dynamicSmemBytes = T2_SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = braid_pdl_enabled();
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<MODE, TMA_OUT>, mw, mx, mo, a);
    BRAID_LAUNCH_CHECK();
}

// As braid_gemm_tc with whole tiles (mode 0 store, 1 float32 residual sum, 2 SwiGLU over interleaved
// gate/up rows), for prompts: tiles of 256 weight rows x 256 tokens on pairs of SMs.  The output leaves
// through TMA where it can be addressed so (16-byte aligned base and row stride; the residual sum in
// place; SwiGLU in bfloat16) unless `direct_out` is set; otherwise each thread stores its own elements.
extern "C" int braid_gemm_tc2(const void* x, const void* w, void* out, const float* res, int out_dtype, int mode,
                              int n_rows, int m_out, int k_in, long long ldx, long long ldw, long long ldo,
                              int direct_out, int* error_flag, void* stream) {
    if (n_rows <= 0 || m_out <= 0) return BRAID_OK;
    if (mode < 0 || mode > 2) BRAID_REFUSE("gemm_tc2: unknown epilogue %d", mode);
    if (k_in <= 0) BRAID_REFUSE("gemm_tc2: k=%d must be positive", k_in);
    if ((ldx % 8) || (ldw % 8)) BRAID_REFUSE("gemm_tc2: row strides (%lld, %lld) must be multiples of 8 elements for TMA", ldx, ldw);
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) BRAID_REFUSE("gemm_tc2: operands must be 16-byte aligned for TMA");
    if (mode == 1 && (!res || out_dtype != BRAID_F32)) BRAID_REFUSE("gemm_tc2: the residual epilogue writes float32 and needs res");
    if (out_dtype != BRAID_F32 && out_dtype != BRAID_BF16) BRAID_REFUSE("gemm_tc2: unknown out dtype code %d", out_dtype);
    if (!error_flag) BRAID_REFUSE("gemm_tc2: error_flag is required");
    const int w_rows = (mode == 2) ? 2 * ((m_out + 15) / 16) * 16 : m_out;
    CUtensorMap mw, mx, mo;
    int rc = make_map2(&mw, w, w_rows, k_in, ldw);
    if (rc) return rc;
    rc = make_map2(&mx, x, n_rows, k_in, ldx);
    if (rc) return rc;
    const int esize = out_dtype == BRAID_F32 ? 4 : 2;
    bool tma_out = !direct_out && ((uintptr_t)out & 15) == 0 && (ldo * esize) % 16 == 0 && ldo >= m_out;
    if (mode == 1 && (const void*)res != (const void*)out) tma_out = false;       // the reduce-add sums into what is there
    if (mode == 2 && out_dtype != BRAID_BF16) tma_out = false;
    if (tma_out) {
        rc = make_map_out(&mo, out, out_dtype, m_out, n_rows, ldo, mode == 2 ? T2_BLOCK_M / 2 : T2_BLOCK_M);
        if (rc) return rc;
    } else {
        mo = mx;                                   // never read
    }
    const int m_tiles = (w_rows + 2 * T2_BLOCK_M - 1) / (2 * T2_BLOCK_M);
    const int n_tiles = (n_rows + T2_BLOCK_N - 1) / T2_BLOCK_N;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 1) sms = 148;
    const long long units = (long long)m_tiles * n_tiles;
    const int pairs = (int)(units < sms / 2 ? units : sms / 2);
    GemmTc2Args a{out, res, n_rows, m_out, k_in, ldo, out_dtype, m_tiles, n_tiles, error_flag};
    cudaStream_t s = (cudaStream_t)stream;
    if (tma_out) {
        if (mode == 0) return launch_tc2<0, true>(mw, mx, mo, a, pairs, s);
        if (mode == 1) return launch_tc2<1, true>(mw, mx, mo, a, pairs, s);
        return launch_tc2<2, true>(mw, mx, mo, a, pairs, s);
    }
    if (mode == 0) return launch_tc2<0, false>(mw, mx, mo, a, pairs, s);
    if (mode == 1) return launch_tc2<1, false>(mw, mx, mo, a, pairs, s);
    return launch_tc2<2, false>(mw, mx, mo, a, pairs, s);
}
