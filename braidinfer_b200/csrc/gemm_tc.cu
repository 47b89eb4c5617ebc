// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05) of sm_100a:
//   out[n, m] = sum_k x[n, k] * w[m, k],   float32 accumulation in tensor memory.
//
// The weight matrix is the UMMA "A" operand (128 output features per CTA fill the 128
// lanes of tensor memory), the tokens are the "B" operand (BLOCK_N of them, 16..256),
// so the same kernel streams weights for a handful of decoded tokens and tiles a long
// prompt.  Both operands are K-major in global memory, as model folders store weights
// ([out, in]) and as activations are laid out ([tokens, in]), so neither is transposed.
//
//   warp 0      one lane issues TMA loads (cp.async.bulk.tensor, no multicast) of
//               [128 x 64] weight and [BLOCK_N x 64] token tiles, 128-byte swizzled,
//               into a ring of shared-memory stages, signalling `full` mbarriers;
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (K = 16 each, four
//               per stage) and tcgen05.commit, which frees the stage (`empty`) and at
//               the end signals `acc_full`;
//   warps 2..5  epilogue: tcgen05.ld of their 32 lanes, then one of
//                 0  store in bfloat16 or float32,
//                 1  float32 residual sum: out = res + product,
//                 2  SwiGLU: w interleaves gate and up rows in blocks of 16, so each
//                    epilogue warp holds 16 outputs' gate (lanes 0..15) and up (lanes
//                    16..31) and pairs them with a shuffle; out = silu(gate) * up,
//                 3  float32 partial sums of a run of k blocks ("stream-k"), added up
//                    by a reduce kernel with one of the epilogues above.
//               The tokens may come with a row scale still to be applied (rowscale.cuh: the RMSNorm
//               of the tensor they were made from, left to this product): epilogues 0 and 2, here and in
//               the reduce kernel, multiply each token's results by it.
//
// The kernel is persistent: one CTA per SM walks its share of the work units (output tile
// x slice of k).  The loader runs ahead across units, and with two accumulator buffers
// in tensor memory (whenever 2 x BLOCK_N x accumulators fits its 512 columns) the
// epilogue of one unit overlaps the products of the next.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets *error_flag, tells the
// other warps to stop, and the kernel frees its tensor memory and returns.
//
// Replaces the reference's per-row GEMV ops (kernels/megakernel_ops.hip:168-276 linear,
// :1474-1602 feed-forward, :1783-1842 output head), which run on scalar FMA.
#include "common.cuh"
#include "rowscale.cuh"
#include "streamk.cuh"
#include "tcgen05.cuh"
#include "trace.cuh"

// Slots of a traced launch: 0 entry, 1 barriers and tensor memory set up, 2 first ring of weight
// tiles asked for, 3 dependency wait over, 4 first stage full, 5 last accumulator complete,
// 6 epilogue done, 7 all warps done.
BRAID_TRACE_BUFFER(gemm_tc, 160)

#define TC_BLOCK_M 128
#define TC_BLOCK_K 64
#define TC_UMMA_K 16
#define TC_THREADS 192

struct GemmTcArgs {
    void* out;                 // mode 0: [n, ldo] bf16/f32; 1: f32; 2: bf16/f32 [n, ldo]; 3: f32 [slot][n_rows][128]
    const float* res;          // mode 1
    int n_rows, m_out, k_in;   // mode 2: m_out is the number of gate rows (w has 2 * m_out rows)
    long long ldo;
    int out_dtype;
    int m_tiles, n_tiles;
    int max_segs;              // mode 3: partial slots per CTA
    int* error_flag;
    int tile_begin, tile_end;  // the tiles of the walk (tc_tile_coords) that this launch covers
    RowScaleArgs scale;        // modes 0, 2: a row scale of the tokens, or none; mode 3: see rs_out
    float* rs_out;             // mode 3 with a scale: CTA 0 writes the scale of every row here, for the kernel that adds up
};

template <int BLOCK_N, int MODE>
struct TcCfg {
    static constexpr int kABytes = TC_BLOCK_M * TC_BLOCK_K * 2;
    static constexpr int kBBytes = BLOCK_N * TC_BLOCK_K * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBudget = 200 * 1024;
    static constexpr int kStagesRaw = kBudget / kStageBytes;
    static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
    static constexpr int kAccCols = BLOCK_N;                               // columns of one accumulator buffer
    static constexpr int kAccBufs = (kAccCols * 2 <= 512) ? 2 : 1;          // two: the epilogue overlaps the next tile
    static constexpr int kTmemCols = (kAccCols * kAccBufs) < 32 ? 32 : (kAccCols * kAccBufs);
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment */ + 256 /* barriers */;
};


// Work of a persistent CTA.
//
// Output tiles are numbered in walk order (tc_tile_coords in streamk.cuh); a launch covers tiles
// [tile_begin, tile_end).
//
// Modes 0-2: units u = tile_begin + blockIdx.x, + gridDim.x, ...; a unit is one whole
// [128 x BLOCK_N] output tile.
//
// Mode 3 ("stream-k", for steps whose whole tiles would leave SMs idle: a few tokens, or a few hundred
// with few weight tiles): the
// k blocks of the launch's tiles form one line of (tile_end - tile_begin) * total_kb blocks, cut into
// gridDim.x equal ranges.  A CTA's range is a run of segments (tile, first k block,
// count); it writes the float32 partial product of its j-th segment to slot
// blockIdx.x * max_segs + j, and a reduce kernel adds the slots of a tile
// in ascending CTA order.  Every CTA streams the same number of bytes whatever the shape.
struct TcUnit { int m0, n0, slot, kb_begin, num_kb; };

template <int BLOCK_N, int MODE>
struct TcWalk {
    const GemmTcArgs& a;
    int total_kb;
    long long idx, hi;       // mode 3: position in the line of k blocks
    int u, seg;
    __device__ TcWalk(const GemmTcArgs& a_) : a(a_) {
        total_kb = (a.k_in + TC_BLOCK_K - 1) / TC_BLOCK_K;
        if (MODE == 3) {
            const long long w = (long long)(a.tile_end - a.tile_begin) * total_kb;
            idx = (long long)blockIdx.x * w / gridDim.x;
            hi = (long long)(blockIdx.x + 1) * w / gridDim.x;
        } else {
            idx = hi = 0;
        }
        u = a.tile_begin + blockIdx.x;
        seg = 0;
    }
    __device__ bool next(TcUnit& t) {
        int tile;
        if (MODE == 3) {
            if (idx >= hi) return false;
            const int in_line = (int)(idx / total_kb);
            tile = a.tile_begin + in_line;
            t.kb_begin = (int)(idx - (long long)in_line * total_kb);
            t.num_kb = (int)min((long long)(total_kb - t.kb_begin), hi - idx);
            t.slot = blockIdx.x * a.max_segs + seg;
            idx += t.num_kb;
            ++seg;
        } else {
            if (u >= a.tile_end) return false;
            tile = u;
            t.kb_begin = 0;
            t.num_kb = total_kb;
            t.slot = 0;
            u += gridDim.x;
        }
        int mt, nt;
        tc_tile_coords(tile, a.m_tiles, a.n_tiles, mt, nt);
        t.m0 = mt * TC_BLOCK_M;
        t.n0 = nt * BLOCK_N;
        return true;
    }
};

template <int BLOCK_N, int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmTcArgs a) {
    using Cfg = TcCfg<BLOCK_N, MODE>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + Cfg::kStages * Cfg::kStageBytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + Cfg::kStages;
    uint64_t* acc_full = bars + 2 * Cfg::kStages;          // [kAccBufs]
    uint64_t* acc_empty = acc_full + 2;                    // [kAccBufs]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    __shared__ float rs_s[BLOCK_N];            // row scale of the tile's tokens (modes 0, 2 with a.scale)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef BRAID_TRACE
    __shared__ unsigned long long* trace_row_shared;
    if (threadIdx.x == 0) {
        trace_row_shared = braid_trace_open(gemm_tc, 160);
        BRAID_STAMP(trace_row_shared, 0);
    }
#endif
    pdl_trigger();
    if (threadIdx.x == 0) {                    // the descriptors' own fetch, off the critical path
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
#ifdef BRAID_TRACE
    unsigned long long* const trace_row = trace_row_shared;
    if (threadIdx.x == 0) BRAID_STAMP(trace_row, 1);
#endif

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // Weights are written by no kernel, so the first ring of weight tiles is on its
            // way before the predecessor in the stream has finished; the token tiles of the
            // same stages follow once it has.
            {
                TcWalk<BLOCK_N, MODE> pre(a);
                TcUnit t;
                int n = 0;
                while (n < Cfg::kStages && pre.next(t))
                    for (int i = 0; i < t.num_kb && n < Cfg::kStages; ++i, ++n) {
                        uint8_t* sa = smem + n * Cfg::kStageBytes;
                        mbar_expect_tx(&full[n], Cfg::kStageBytes);
                        const int kx = (t.kb_begin + i) * TC_BLOCK_K;
                        tma_load_2d(&map_w, &full[n], sa, kx, t.m0);
                    }
            }
            BRAID_STAMP(trace_row, 2);
            pdl_wait();
            BRAID_STAMP(trace_row, 3);
            TcWalk<BLOCK_N, MODE> walk(a);
            TcUnit t;
            int issued = 0;                       // k blocks whose weight tile is already in flight
            while (ok && walk.next(t)) {
                for (int i = 0; i < t.num_kb; ++i, ++issued) {
                    uint8_t* sa = smem + stage * Cfg::kStageBytes;
                    uint8_t* sb = sa + Cfg::kABytes;
                    const int kx = (t.kb_begin + i) * TC_BLOCK_K;
                    if (issued >= Cfg::kStages) {
                        ok = mbar_wait(&empty[stage], phase ^ 1u, abort_flag);
                        if (!ok) break;
                        mbar_expect_tx(&full[stage], Cfg::kStageBytes);
                        tma_load_2d(&map_w, &full[stage], sa, kx, t.m0);
                    }
                    tma_load_2d(&map_x, &full[stage], sb, kx, t.n0);
                    if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(TC_BLOCK_M, BLOCK_N);
            int stage = 0, buf = 0;
            uint32_t phase = 0, acc_phase = 0;      // bit b: phase of accumulator buffer b
            bool ok = true;
            TcWalk<BLOCK_N, MODE> walk(a);
            TcUnit t;
            while (ok && walk.next(t)) {
                ok = mbar_wait(&acc_empty[buf], ((acc_phase >> buf) & 1u) ^ 1u, abort_flag);   // the epilogue has drained this buffer
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * Cfg::kAccCols;
                for (int i = 0; i < t.num_kb; ++i) {
                    ok = mbar_wait(&full[stage], phase, abort_flag);
                    if (!ok) break;
                    BRAID_STAMP_ONCE(trace_row, 4);
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
                    const uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
                    for (int k = 0; k < TC_BLOCK_K / TC_UMMA_K; ++k) {
                        const uint32_t koff = k * TC_UMMA_K * 2;     // bytes along the 128-byte row
                        const uint32_t accum = (i > 0 || k > 0) ? 1u : 0u;
                        umma_bf16(tmem_d, umma_desc_sw128(sa + koff), umma_desc_sw128(sb + koff), idesc, accum);
                    }
                    umma_commit(&empty[stage]);
                    if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(&acc_full[buf]);
                acc_phase ^= (1u << buf);
                if (Cfg::kAccBufs == 2) buf ^= 1;
            }
        }
    } else {
        // epilogue warps: warp w may read tensor-memory lanes 32 * (w % 4) ...
        const int quarter = warp & 3;
        pdl_wait();
        int buf = 0;
        uint32_t full_phase = 0;                  // bit b: phase of accumulator buffer b
        bool ok = true;
        TcWalk<BLOCK_N, MODE> walk(a);
        TcUnit t;
        // with a row scale the epilogue threads meet at barriers inside a unit: they then agree on whether
        // a wait ran out, so that none of them waits at a barrier for one that left
        const bool scaled = (MODE == 0 || MODE == 2) && a.scale.shares != nullptr;
        int rs_n0 = -1;
        if (MODE == 3 && a.rs_out && blockIdx.x == 0) {
            // the rows' scales from their shares, once, while these warps have nothing else to do: the kernel
            // that adds the partial sums up then reads one float a row
            for (int j = threadIdx.x - 64; j < a.n_rows; j += 128) a.rs_out[j] = row_scale_of(a.scale, j);
        }
        while (ok && walk.next(t)) {
            // mode 2: every 32 weight rows are 16 gate rows then the 16 up rows of the same outputs,
            // so a warp's lanes 0..15 hold gate and lanes 16..31 hold up of outputs [m - lane % 16 ...]
            const int m = (MODE == 2) ? (t.m0 + quarter * 32) / 2 + (lane & 15) : t.m0 + quarter * 32 + lane;
            if (scaled && t.n0 != rs_n0) {
                epilogue_sync();                              // the last unit's readers are done
                for (int j = threadIdx.x - 64; j < BLOCK_N; j += 128)
                    rs_s[j] = (t.n0 + j < a.n_rows) ? row_scale_of(a.scale, t.n0 + j) : 0.f;
                epilogue_sync();
                rs_n0 = t.n0;
            }
            ok = mbar_wait(&acc_full[buf], (full_phase >> buf) & 1u, abort_flag);
            if (scaled) ok = epilogue_all(ok);
            if (!ok) break;
            if (warp == 2 && lane == 0) BRAID_STAMP(trace_row, 5);
            tc_fence_after();
            const uint32_t trow = tmem_base + buf * Cfg::kAccCols + ((uint32_t)(quarter * 32) << 16);
            constexpr int CH = BLOCK_N >= 32 ? 32 : 16;       // columns per tensor-memory load and wait
#pragma unroll 1
            for (int c0 = 0; c0 < BLOCK_N; c0 += CH) {
                if (t.n0 + c0 >= a.n_rows) break;
                float v[CH];
                if (CH == 32) tmem_ld32(trow + c0, v);
                else tmem_ld16(trow + c0, v);
                if (scaled) {
#pragma unroll
                    for (int i = 0; i < CH; ++i) v[i] *= rs_s[c0 + i];
                }
                if (MODE == 2) {
                    // The halves of a warp swap values; the gate half then finishes the even
                    // columns and the up half the odd ones, so all lanes compute and store.
                    const bool is_up = (lane & 16) != 0;
                    const size_t o0 = (size_t)(t.n0 + c0 + (is_up ? 1 : 0)) * a.ldo + m;
#pragma unroll
                    for (int p2 = 0; p2 < CH / 2; ++p2) {
                        // columns 2 p2 (finished by the gate half) and 2 p2 + 1 (by the up half): every
                        // lane computes, none idles
                        const float from_up = __shfl_xor_sync(0xffffffffu, v[2 * p2], 16);        // gate lanes get up's value
                        const float from_gate = __shfl_xor_sync(0xffffffffu, v[2 * p2 + 1], 16);  // up lanes get gate's value
                        const float g = is_up ? from_gate : v[2 * p2];
                        const float u = is_up ? v[2 * p2 + 1] : from_up;
                        // silu(g) * u with the fast exponential and division: a few ulp, far inside
                        // the bfloat16 rounding of the result, and no slow path for the infinities
                        // that exp(-g) reaches (g / inf = 0 is the right limit)
                        const float y = __fdividef(g, 1.f + __expf(-g)) * u;
                        const int n = t.n0 + c0 + 2 * p2 + (is_up ? 1 : 0);
                        if (m < a.m_out && n < a.n_rows) {
                            if (a.out_dtype == BRAID_F32) ((float*)a.out)[o0 + (size_t)(2 * p2) * a.ldo] = y;
                            else ((__nv_bfloat16*)a.out)[o0 + (size_t)(2 * p2) * a.ldo] = __float2bfloat16_rn(y);
                        }
                    }
                    continue;
                }
                const bool mine = true;
                if (mine && m < a.m_out) {
                    if (MODE == 3) {
                        // slot layout [BLOCK_N][128]: this thread's output feature is column quarter * 32 + lane
                        float* dst = (float*)a.out + ((size_t)t.slot * BLOCK_N + c0) * TC_BLOCK_M + quarter * 32 + lane;
#pragma unroll
                        for (int i = 0; i < CH; ++i)
                            if (t.n0 + c0 + i < a.n_rows) dst[(size_t)i * TC_BLOCK_M] = v[i];
                    } else if (MODE == 1) {
                        // all loads of the residual first: out may be res itself, which would
                        // otherwise chain every load behind the store before it
                        const size_t o0 = (size_t)(t.n0 + c0) * a.ldo + m;
                        float r[CH];
#pragma unroll
                        for (int i = 0; i < CH; ++i) r[i] = (t.n0 + c0 + i < a.n_rows) ? a.res[o0 + (size_t)i * a.ldo] : 0.f;
#pragma unroll
                        for (int i = 0; i < CH; ++i)
                            if (t.n0 + c0 + i < a.n_rows) ((float*)a.out)[o0 + (size_t)i * a.ldo] = r[i] + v[i];
                    } else {
                        const size_t o0 = (size_t)(t.n0 + c0) * a.ldo + m;
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
            mbar_arrive(&acc_empty[buf]);
            full_phase ^= (1u << buf);
            if (Cfg::kAccBufs == 2) buf ^= 1;
        }
    }
    if (warp == 2 && lane == 0) BRAID_STAMP(trace_row, 6);
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) BRAID_STAMP(trace_row, 7);
    if (threadIdx.x == 0 && *abort_flag) atomicExch(a.error_flag, 1);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ------------------------------------------------------------------ stream-k reduce
// Adds up the partial products of the tiles of a stream-k line and finishes them: mode 0 store;
// 1 res + sum (float32); 2 the tile's weight rows interleave gate and up in blocks of 16 (its 128
// rows are 64 outputs), out = silu(gate) * up.  One thread per four consecutive outputs of a
// token; threads are laid over the line's tiles.
template <int MODE>
__global__ void streamk_reduce_kernel(StreamK k, void* __restrict__ out, const float* __restrict__ res,
                                      int m_out, long long ldo, int out_dtype, const float* __restrict__ rs_rows) {
    pdl_trigger();
    constexpr int GROUPS = (MODE == 2) ? 16 : 32;          // groups of four outputs that a tile holds per token
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long per_tile = (long long)k.block_n * GROUPS;
    const int in_line = (int)(i / per_tile);
    if ((long long)in_line * k.total_kb >= k.w) return;
    const int r = (int)(i - (long long)in_line * per_tile);
    const int row = r / GROUPS, g = r - row * GROUPS;
    int mt, nt;
    tc_tile_coords(k.tile_begin + in_line, k.m_tiles, k.n_tiles, mt, nt);
    const int n = nt * k.block_n + row;
    // output feature m and, within the tile's 128 weight rows, the column(s) that hold its sum
    const int m = (MODE == 2) ? mt * 64 + g * 4 : mt * STREAMK_TILE_M + g * 4;
    const int c0 = (MODE == 2) ? mt * STREAMK_TILE_M + (g / 4) * 32 + (g % 4) * 4 : m;
    if (n >= k.n_rows || m >= m_out) return;
    // where the partial sums lie is arithmetic only: done before the wait for the product
    const StreamKSpan sp = streamk_span_of_tile(k, in_line);
    pdl_wait();
    const float rs = (MODE != 1 && rs_rows) ? rs_rows[n] : 1.f;      // asked for with the partial sums: one trip
    float v[4];
    if (MODE == 2) {
        float4 g4, u4;
        streamk_sum4_pair(k, sp, n, c0, c0 + 16, g4, u4);
        g4.x *= rs; g4.y *= rs; g4.z *= rs; g4.w *= rs;
        u4.x *= rs; u4.y *= rs; u4.z *= rs; u4.w *= rs;
        v[0] = g4.x / (1.f + expf(-g4.x)) * u4.x;
        v[1] = g4.y / (1.f + expf(-g4.y)) * u4.y;
        v[2] = g4.z / (1.f + expf(-g4.z)) * u4.z;
        v[3] = g4.w / (1.f + expf(-g4.w)) * u4.w;
    } else {
        const float4 s4 = streamk_sum4(k, sp, n, c0);
        v[0] = s4.x * rs; v[1] = s4.y * rs; v[2] = s4.z * rs; v[3] = s4.w * rs;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        if (m + e >= m_out) break;
        const size_t o = (size_t)n * ldo + m + e;
        if (MODE == 1) ((float*)out)[o] = res[o] + v[e];
        else if (out_dtype == BRAID_F32) ((float*)out)[o] = v[e];
        else ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(v[e]);
    }
}

static int launch_streamk_reduce(const StreamK& k, void* out, const float* res, int m_out, long long ldo, int out_dtype,
                                 int mode, const float* rs_rows, cudaStream_t s) {
    const long long tiles = k.w / k.total_kb;
    const long long total = tiles * k.block_n * (mode == 2 ? 16 : 32);
    const int threads = 128;
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 0x7fffffffLL) BRAID_REFUSE("streamk_reduce: %lld outputs exceed one launch", total);
    if (mode == 0) braid_launch(streamk_reduce_kernel<0>, dim3((int)blocks), dim3(threads), 0, s, k, out, res, m_out, ldo, out_dtype, rs_rows);
    else if (mode == 1) braid_launch(streamk_reduce_kernel<1>, dim3((int)blocks), dim3(threads), 0, s, k, out, res, m_out, ldo, out_dtype, rs_rows);
    else braid_launch(streamk_reduce_kernel<2>, dim3((int)blocks), dim3(threads), 0, s, k, out, res, m_out, ldo, out_dtype, rs_rows);
    BRAID_LAUNCH_CHECK();
}

// ------------------------------------------------------------------ host side
// rows x k bfloat16 matrix with row stride ld (elements); box = box_rows x 64, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long k, long long ld, int box_rows) {
    TcEncodeTiledFn fn = tc_encode_tiled_fn();
    if (!fn) BRAID_REFUSE("gemm_tc: the driver does not export cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TC_BLOCK_K, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) BRAID_REFUSE("gemm_tc: cuTensorMapEncodeTiled failed with %d (rows=%lld k=%lld ld=%lld)", (int)r, rows, k, ld);
    return BRAID_OK;
}

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BLOCK_N, int MODE>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const GemmTcArgs& a, dim3 grid, cudaStream_t s) {
    using Cfg = TcCfg<BLOCK_N, MODE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BLOCK_N, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        if (e != cudaSuccess) { braid_set_error("gemm_tc: cannot reserve %d bytes of shared memory: %s", Cfg::kSmemBytes, cudaGetErrorString(e)); return (int)e; }
        configured = true;
    }
    braid_launch(gemm_tc_kernel<BLOCK_N, MODE>, dim3(grid), dim3(TC_THREADS), Cfg::kSmemBytes, s, mw, mx, a);
    BRAID_LAUNCH_CHECK();
}

template <int MODE>
static int dispatch_tc(int block_n, const CUtensorMap& mw, const CUtensorMap& mx, const GemmTcArgs& a, dim3 grid, cudaStream_t s) {
    switch (block_n) {
        case 16: return launch_tc<16, MODE>(mw, mx, a, grid, s);
        case 32: return launch_tc<32, MODE>(mw, mx, a, grid, s);
        case 64: return launch_tc<64, MODE>(mw, mx, a, grid, s);
        case 128: return launch_tc<128, MODE>(mw, mx, a, grid, s);
        case 256: return launch_tc<256, MODE>(mw, mx, a, grid, s);
    }
    BRAID_REFUSE("gemm_tc: token tile %d is not one of 16, 32, 64, 128, 256", block_n);
}

struct StreamKPlan { int grid, max_segs, total_kb, m_tiles, n_tiles, tile_begin, tiles; long long w, bytes; };

static StreamKPlan plan_stream_k(int n_rows, int w_rows, int k_in, int block_n) {
    StreamKPlan p;
    p.total_kb = (k_in + TC_BLOCK_K - 1) / TC_BLOCK_K;
    p.m_tiles = (w_rows + TC_BLOCK_M - 1) / TC_BLOCK_M;
    p.n_tiles = (n_rows + block_n - 1) / block_n;
    const long long all = (long long)p.m_tiles * p.n_tiles;
    p.tile_begin = 0;                  // the line holds every tile (the kernels take any first tile)
    p.tiles = (int)(all - p.tile_begin);
    p.w = (long long)p.tiles * p.total_kb;
    p.grid = (int)(p.w < sm_count() ? p.w : sm_count());
    if (p.grid <= 0) { p.grid = 0; p.max_segs = 0; p.bytes = 0; return p; }
    const long long per = (p.w + p.grid - 1) / p.grid;
    p.max_segs = (int)((per + p.total_kb - 1) / p.total_kb) + 1;
    p.bytes = (long long)p.grid * p.max_segs * block_n * TC_BLOCK_M * 4;
    return p;
}

static bool valid_block_n(int b) { return b == 16 || b == 32 || b == 64 || b == 128 || b == 256; }

// Bytes of float32 scratch that the stream-k form needs for this shape and token tile
// (-1: not a token tile this kernel has).
extern "C" long long braid_gemm_tc_workspace_bytes(int n_rows, int w_rows, int k_in, int block_n) {
    if (!valid_block_n(block_n) || n_rows <= 0 || w_rows <= 0 || k_in <= 0) return -1;
    return plan_stream_k(n_rows, w_rows, k_in, block_n).bytes;
}

// x: [n_rows, k_in] bf16 (row stride ldx); w: [w_rows, k_in] bf16 (row stride ldw), where
// w_rows = m_out; for the SwiGLU epilogue w_rows = 2 * ceil(m_out / 16) * 16 and the rows are
// interleaved in blocks of 16: block t holds gate rows [16t, 16t+16) then up rows [16t, 16t+16)
// (rows past m_out are zero).  stream_k != 0 balances the
// weight stream over all SMs for any shape (meant for up to a few hundred tokens) and needs
// `workspace` of at least braid_gemm_tc_workspace_bytes() bytes for the same shape and tile
// (`workspace_bytes` says how many it has; too few is refused, never written past).
// block_n names the token tile: 16, 32, 64, 128 or 256.  With stream_k and plan_out != null only
// the partial products are computed; plan_out receives {grid, max_segs, total_kb,
// n_tiles, block_n, w, m_tiles, tile_begin} for the kernel that adds them up (fused_reduce.cu).
// scale_*: a row scale that x still wants (rowscale.cuh), or null shares.  Whole tiles apply it in their
// epilogue; the stream-k form writes every row's scale to rs_rows (n_rows floats, required then) and the
// kernel that adds the partial sums up, here or the caller's, multiplies by it.
extern "C" int braid_gemm_tc(const void* x, const void* w, void* out, const float* res, void* workspace,
                             long long workspace_bytes, int out_dtype, int mode, int n_rows, int m_out, int k_in,
                             long long ldx, long long ldw, long long ldo, int block_n, int stream_k,
                             int* plan_out, const float* scale_shares, int scale_n_shares, long long scale_stride,
                             float scale_width, float scale_eps, float* rs_rows, int* error_flag, void* stream) {
    if (n_rows <= 0 || m_out <= 0) return BRAID_OK;
    if (mode < 0 || mode > 2) BRAID_REFUSE("gemm_tc: unknown epilogue %d", mode);
    if (k_in <= 0) BRAID_REFUSE("gemm_tc: k=%d must be positive", k_in);
    if ((ldx % 8) || (ldw % 8)) BRAID_REFUSE("gemm_tc: row strides (%lld, %lld) must be multiples of 8 elements for TMA", ldx, ldw);
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) BRAID_REFUSE("gemm_tc: operands must be 16-byte aligned for TMA");
    if (mode == 1 && (!res || out_dtype != BRAID_F32)) BRAID_REFUSE("gemm_tc: the residual epilogue writes float32 and needs res");
    if (out_dtype != BRAID_F32 && out_dtype != BRAID_BF16) BRAID_REFUSE("gemm_tc: unknown out dtype code %d", out_dtype);
    if (!error_flag) BRAID_REFUSE("gemm_tc: error_flag is required");
    const int w_rows = (mode == 2) ? 2 * ((m_out + 15) / 16) * 16 : m_out;
    if (!valid_block_n(block_n)) BRAID_REFUSE("gemm_tc: token tile %d is not one of 16, 32, 64, 128, 256", block_n);
    if (stream_k && !workspace) BRAID_REFUSE("gemm_tc: the stream-k form needs a workspace");
    const RowScaleArgs scale{scale_shares, scale_n_shares, scale_stride, scale_width, scale_eps};
    if (const char* why = row_scale_problem(scale, n_rows)) BRAID_REFUSE("gemm_tc: row scale: %s", why);
    if (scale.shares && mode == 1) BRAID_REFUSE("gemm_tc: the residual epilogue takes no row scale");
    if (scale.shares && stream_k && !rs_rows)
        BRAID_REFUSE("gemm_tc: a stream-k product with a row scale needs rs_rows (n_rows floats) for the rows' scales");
    if (stream_k) {
        // the partial sums of every CTA's segments must fit: checked here, on the host, for the very
        // plan the kernel will walk
        const long long need = plan_stream_k(n_rows, w_rows, k_in, block_n).bytes;
        if (need > workspace_bytes)
            BRAID_REFUSE("gemm_tc: the stream-k form of %d rows x %d x %d with token tile %d needs %lld bytes of workspace, "
                         "it was given %lld", n_rows, w_rows, k_in, block_n, need, workspace_bytes);
    }
    cudaStream_t s = (cudaStream_t)stream;

    CUtensorMap mw, mx;
    int rc = make_map(&mw, w, w_rows, k_in, ldw, TC_BLOCK_M);
    if (rc) return rc;
    rc = make_map(&mx, x, n_rows, k_in, ldx, block_n);
    if (rc) return rc;

    const int m_tiles = (w_rows + TC_BLOCK_M - 1) / TC_BLOCK_M;
    const int n_tiles = (n_rows + block_n - 1) / block_n;
    const int all_tiles = m_tiles * n_tiles;
    StreamKPlan p{};
    if (stream_k) p = plan_stream_k(n_rows, w_rows, k_in, block_n);
    const int whole_end = stream_k ? p.tile_begin : all_tiles;       // tiles [0, whole_end) run as whole tiles
    if (whole_end > 0) {
        GemmTcArgs a{out, res, n_rows, m_out, k_in, ldo, out_dtype, m_tiles, n_tiles, 0, error_flag, 0, whole_end, scale, nullptr};
        dim3 grid((unsigned)(whole_end < sm_count() ? whole_end : sm_count()), 1, 1);
        if (mode == 0) rc = dispatch_tc<0>(block_n, mw, mx, a, grid, s);
        else if (mode == 1) rc = dispatch_tc<1>(block_n, mw, mx, a, grid, s);
        else rc = dispatch_tc<2>(block_n, mw, mx, a, grid, s);
        if (rc) return rc;
    }
    if (!stream_k || p.tiles == 0) return BRAID_OK;
    GemmTcArgs a{workspace, nullptr, n_rows, w_rows, k_in, 0, BRAID_F32, p.m_tiles, p.n_tiles, p.max_segs, error_flag,
                 p.tile_begin, p.tile_begin + p.tiles, scale, scale.shares ? rs_rows : nullptr};
    rc = dispatch_tc<3>(block_n, mw, mx, a, dim3(p.grid, 1, 1), s);
    if (rc) return rc;
    if (plan_out) {
        // the caller adds the partial products up itself (fused with what follows the product)
        plan_out[0] = p.grid; plan_out[1] = p.max_segs; plan_out[2] = p.total_kb; plan_out[3] = p.n_tiles;
        plan_out[4] = block_n; plan_out[5] = (int)p.w; plan_out[6] = p.m_tiles; plan_out[7] = p.tile_begin;
        return BRAID_OK;
    }
    StreamK k{(const float*)workspace, p.grid, p.max_segs, p.total_kb, p.n_tiles, n_rows, block_n, p.w, p.m_tiles, p.tile_begin};
    return launch_streamk_reduce(k, out, res, m_out, ldo, out_dtype, mode, scale.shares ? rs_rows : nullptr, s);
}

// Add up the partial products of an earlier stream-k call made with plan_out (the same
// reduce the fused call runs): mode 0 store, 1 res + sum, 2 silu(gate) * up.
extern "C" int braid_streamk_reduce(const float* partial, const int* plan, int n_rows, void* out, const float* res,
                                    int m_out, long long ldo, int out_dtype, int mode, const float* rs_rows, void* stream) {
    if (n_rows <= 0 || m_out <= 0) return BRAID_OK;
    if (mode < 0 || mode > 2) BRAID_REFUSE("streamk_reduce: unknown epilogue %d", mode);
    if (mode == 1 && (!res || out_dtype != BRAID_F32)) BRAID_REFUSE("streamk_reduce: the residual epilogue writes float32 and needs res");
    if (rs_rows && mode == 1) BRAID_REFUSE("streamk_reduce: the residual epilogue takes no row scale");
    return launch_streamk_reduce(streamk_from_plan(partial, plan, n_rows), out, res, m_out, ldo, out_dtype, mode, rs_rows, (cudaStream_t)stream);
}
