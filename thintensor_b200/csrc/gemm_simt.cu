// out[s][m][n] = sum over the s-th slice of k of x[m][k] * w[n][k]  (+ bias[n] in s = 0)
//
// The exact matrix product: float32 FMA on CUDA cores, no tensor-core mode of any
// kind, float32 or bfloat16 operands widened exactly.  It is the product of the true
// 32-bit path, the oracle of the tensor-core kernel in tests, and what a bfloat16 model
// falls back to for a weight that its checkpoint stores in float32.  Any m, n, k.
//
// Weights are [out_features, in_features] row-major as checkpoints store them and are
// applied as W x, like torch.mv(W, x) at thinruntime/gpu_runtime.py:10112; the Triton
// counterparts are _matvec_kernel / _matvec_looped_kernel / _matvec_split_k_kernel,
// thinruntime/triton_kernels.py:484-535, 2959-2986, 3022-3083.
#include "common.cuh"

#define GS_BM 64
#define GS_BN 64
#define GS_BK 16
#define GS_THREADS 256

template <typename TX, typename TW>
__global__ void __launch_bounds__(GS_THREADS)
gemm_simt_kernel(const TX* __restrict__ x, long long ldx, const TW* __restrict__ w, long long ldw,
                 const float* __restrict__ bias, float* __restrict__ out, long long ldo, long long split_stride,
                 int m, int n, int k, int k_per_split) {
    __shared__ float xs[GS_BK][GS_BM + 4];
    __shared__ float ws[GS_BK][GS_BN + 4];
    const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
    const int split = blockIdx.z;
    const int k_begin = split * k_per_split;
    const int k_end = min(k, k_begin + k_per_split);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    // loader mapping: 256 threads fetch 64 rows x 16 k = 1024 numbers, 4 consecutive k each
    const int load_row = threadIdx.x >> 2, load_k = (threadIdx.x & 3) * 4;
    for (int kk = k_begin; kk < k_end; kk += GS_BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int kx = kk + load_k + e;
            const int gm = m0 + load_row, gn = n0 + load_row;
            xs[load_k + e][load_row] = (gm < m && kx < k_end) ? tt_to_float(x[(size_t)gm * ldx + kx]) : 0.0f;
            ws[load_k + e][load_row] = (gn < n && kx < k_end) ? tt_to_float(w[(size_t)gn * ldw + kx]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int e = 0; e < GS_BK; ++e) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[e][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[e][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    float* o = out + (size_t)split * split_stride;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= n) continue;
            float v = acc[i][j];
            if (bias && split == 0) v += bias[gn];
            o[(size_t)gm * ldo + gn] = v;
        }
    }
}

// Skinny form for few rows of x (decoding): one warp per output column n and up to 8
// rows of x at a time, lanes stride over k, so the weights are read once per 8 rows.
template <typename TX, typename TW>
__global__ void gemm_rows_kernel(const TX* __restrict__ x, long long ldx, const TW* __restrict__ w, long long ldw,
                                 const float* __restrict__ bias, float* __restrict__ out, long long ldo, int m, int n,
                                 int k) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = blockIdx.x * (blockDim.x >> 5) + warp;
    if (col >= n) return;
    const TW* wrow = w + (size_t)col * ldw;
    for (int m0 = 0; m0 < m; m0 += 8) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
        for (int kk = lane; kk < k; kk += 32) {
            const float wv = tt_to_float(wrow[kk]);
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (m0 + i < m) acc[i] = fmaf(tt_to_float(x[(size_t)(m0 + i) * ldx + kk]), wv, acc[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float total = tt_warp_sum(acc[i]);
            if (lane == 0 && m0 + i < m) out[(size_t)(m0 + i) * ldo + col] = total + (bias ? bias[col] : 0.0f);
        }
    }
}

template <typename TX, typename TW>
static int launch(const void* x, long long ldx, const void* w, long long ldw, const float* bias, float* out,
                  long long ldo, long long split_stride, int m, int n, int k, int splits, cudaStream_t stream) {
    if (m <= 16 && splits == 1) {
        const int warps = 8;
        gemm_rows_kernel<TX, TW><<<(n + warps - 1) / warps, warps * 32, 0, stream>>>((const TX*)x, ldx, (const TW*)w, ldw, bias, out, ldo, m, n, k);
        TT_LAUNCH_CHECK();
    }
    int k_per_split = (k + splits - 1) / splits;
    k_per_split = (k_per_split + GS_BK - 1) / GS_BK * GS_BK;
    const dim3 grid((n + GS_BN - 1) / GS_BN, (m + GS_BM - 1) / GS_BM, splits);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    gemm_simt_kernel<TX, TW><<<grid, GS_THREADS, 0, stream>>>((const TX*)x, ldx, (const TW*)w, ldw, bias, out, ldo, split_stride, m, n, k, k_per_split);
    TT_LAUNCH_CHECK();
}

extern "C" int tt_gemm_simt(const void* x, int x_dtype, long long ldx, const void* w, int w_dtype, long long ldw,
                            const float* bias, float* out, long long ldo, long long split_stride, int m, int n, int k,
                            int splits, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0 || splits < 1 || splits > 64) return (int)cudaErrorInvalidValue;
    if (x_dtype == TT_F32 && w_dtype == TT_F32) return launch<float, float>(x, ldx, w, ldw, bias, out, ldo, split_stride, m, n, k, splits, stream);
    if (x_dtype == TT_BF16 && w_dtype == TT_BF16) return launch<__nv_bfloat16, __nv_bfloat16>(x, ldx, w, ldw, bias, out, ldo, split_stride, m, n, k, splits, stream);
    if (x_dtype == TT_BF16 && w_dtype == TT_F32) return launch<__nv_bfloat16, float>(x, ldx, w, ldw, bias, out, ldo, split_stride, m, n, k, splits, stream);
    if (x_dtype == TT_F32 && w_dtype == TT_BF16) return launch<float, __nv_bfloat16>(x, ldx, w, ldw, bias, out, ldo, split_stride, m, n, k, splits, stream);
    return (int)cudaErrorInvalidValue;
}
