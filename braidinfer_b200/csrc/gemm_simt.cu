// Plain matrix product on the CUDA cores: out[n, m] = sum_k x[n, k] * w[m, k].
//
// w is [out_features, in_features] row-major as model folders store it, so y = W x
// (kernels/megakernel_ops.hip:168-216 of the reference; oracle
// crates/braidinfer-runtime/tests/linear_proj_test.rs:13-23).  Products and sums are
// IEEE float32 FMA in a fixed order along k; no tensor cores and no reduced-precision
// mode, which makes this the matrix product of the true 32-bit path.  With bfloat16
// inputs it is the reference that the tensor-core kernel is checked against.
//
// Epilogues: 0 stores the product in `out_dtype`; 1 stores res + product as float32
// (the residual sum; out may be res itself).
#include "common.cuh"

#define SG_BM 64   // output features per block
#define SG_BN 64   // tokens per block
#define SG_BK 16

template <typename T, typename TO, int MODE>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ x, const T* __restrict__ w, TO* __restrict__ out,
                 const float* __restrict__ res, int n_rows, int m_out, int k_in,
                 long long ldx, long long ldw, long long ldo) {
    pdl_trigger();
    pdl_wait();
    __shared__ float xs[SG_BK][SG_BN + 4];
    __shared__ float ws[SG_BK][SG_BM + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;     // tx: outputs, ty: tokens
    const int n0 = blockIdx.y * SG_BN, m0 = blockIdx.x * SG_BM;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < k_in; k0 += SG_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = threadIdx.x + i * 256;        // 0..1023
            const int r = e >> 4, c = e & 15;           // r: row in tile, c: k offset
            const int k = k0 + c;
            const int n = n0 + r, m = m0 + r;
            xs[c][r] = (n < n_rows && k < k_in) ? to_f32(x[(size_t)n * ldx + k]) : 0.f;
            ws[c][r] = (m < m_out && k < k_in) ? to_f32(w[(size_t)m * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < SG_BK; ++kk) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int n = n0 + ty * 4 + i;
        if (n >= n_rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + tx * 4 + j;
            if (m >= m_out) continue;
            const size_t o = (size_t)n * ldo + m;
            if (MODE == 1) out[o] = from_f32<TO>(res[o] + acc[i][j]);
            else out[o] = from_f32<TO>(acc[i][j]);
        }
    }
}

extern "C" int braid_gemm_simt(const void* x, const void* w, void* out, const float* res,
                               int in_dtype, int out_dtype, int mode,
                               int n_rows, int m_out, int k_in,
                               long long ldx, long long ldw, long long ldo, void* stream) {
    if (n_rows <= 0 || m_out <= 0) return BRAID_OK;
    if (k_in <= 0) BRAID_REFUSE("gemm_simt: k=%d must be positive", k_in);
    if (mode == 1 && (out_dtype != BRAID_F32 || res == nullptr)) BRAID_REFUSE("gemm_simt: the residual epilogue writes float32 and needs res");
    if (mode != 0 && mode != 1) BRAID_REFUSE("gemm_simt: unknown epilogue %d", mode);
    dim3 grid((m_out + SG_BM - 1) / SG_BM, (n_rows + SG_BN - 1) / SG_BN);
    if (grid.y > 65535) BRAID_REFUSE("gemm_simt: %d rows exceed the grid limit", n_rows);
    cudaStream_t s = (cudaStream_t)stream;
#define SG_LAUNCH(T, TO, MODE) braid_launch(gemm_simt_kernel<T, TO, MODE>, dim3(grid), dim3(256), 0, s, (const T*)x, (const T*)w, (TO*)out, res, n_rows, m_out, k_in, ldx, ldw, ldo)
    if (in_dtype == BRAID_F32 && out_dtype == BRAID_F32) { if (mode) SG_LAUNCH(float, float, 1); else SG_LAUNCH(float, float, 0); }
    else if (in_dtype == BRAID_BF16 && out_dtype == BRAID_F32) { if (mode) SG_LAUNCH(__nv_bfloat16, float, 1); else SG_LAUNCH(__nv_bfloat16, float, 0); }
    else if (in_dtype == BRAID_BF16 && out_dtype == BRAID_BF16) SG_LAUNCH(__nv_bfloat16, __nv_bfloat16, 0);
    else BRAID_REFUSE("gemm_simt: unsupported dtype codes in=%d out=%d", in_dtype, out_dtype);
#undef SG_LAUNCH
    BRAID_LAUNCH_CHECK();
}
