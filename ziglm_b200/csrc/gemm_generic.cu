// Y[M,N] (+)= X[M,K] * W[N,K]^T (+ bias[N]) on the CUDA cores, any sizes.
//
// This is the matrix product of the true 32-bit path (plain FFMA, no reduced
// precision tensor-core mode) and the catch-all for operand types the tensor-core
// kernels do not take.  The reference's products are `y[r] = sum_c W[r,c]*x[c]`
// with float accumulation over widened weights (src/cuda_bridge.cu:963-1018,
// src/math.zig:121-176); it runs one such GEMV per token
// (src/cuda_bridge.cu:1439-1444), this kernel tiles tokens instead.
//
// Each output element is owned by one thread that adds its K products in
// ascending k with fmaf, so a value does not depend on M, on where the row sits
// in the batch, or on the tile it falls in.
#include "common.cuh"

namespace zlm {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TX, typename TW, typename TY, typename TB, bool ACC>
__global__ void __launch_bounds__(256)
gemm_generic_kernel(const TX* __restrict__ X, const TW* __restrict__ W, const TB* __restrict__ bias,
                    TY* __restrict__ Y, int M, int N, int K, long ldx, long ldw, long ldy) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    // loader coordinates: 64 rows x 16 k, four consecutive k per thread
    const int lr = tid >> 2, lk = (tid & 3) * 4;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        {
            const int gm = m0 + lr;
            const TX* src = X + (long)gm * ldx + k0 + lk;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int gk = k0 + lk + i;
                As[lk + i][lr] = (gm < M && gk < K) ? to_float(src[i]) : 0.f;
            }
            const int gn = n0 + lr;
            const TW* wsrc = W + (long)gn * ldw + k0 + lk;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int gk = k0 + lk + i;
                Bs[lk + i][lr] = (gn < N && gk < K) ? to_float(wsrc[i]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Bs[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias) v += to_float(bias[gn]);
            TY* dst = Y + (long)gm * ldy + gn;
            if (ACC) *dst = from_float<TY>(to_float(*dst) + v);
            else *dst = from_float<TY>(v);
        }
    }
}

template <typename TX, typename TW, typename TY, typename TB>
static int launch(const void* X, const void* W, const void* bias, void* Y, int accumulate, int M, int N, int K,
                  long ldx, long ldw, long ldy, cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (accumulate)
        gemm_generic_kernel<TX, TW, TY, TB, true><<<grid, 256, 0, stream>>>(
            (const TX*)X, (const TW*)W, (const TB*)bias, (TY*)Y, M, N, K, ldx, ldw, ldy);
    else
        gemm_generic_kernel<TX, TW, TY, TB, false><<<grid, 256, 0, stream>>>(
            (const TX*)X, (const TW*)W, (const TB*)bias, (TY*)Y, M, N, K, ldx, ldw, ldy);
    return launch_status();
}

template <typename TX, typename TW, typename TY>
static int pick_bias(int bias_dtype, const void* X, const void* W, const void* bias, void* Y, int accumulate, int M,
                     int N, int K, long ldx, long ldw, long ldy, cudaStream_t stream) {
    if (bias == nullptr || bias_dtype == ZLM_F32)
        return launch<TX, TW, TY, float>(X, W, bias, Y, accumulate, M, N, K, ldx, ldw, ldy, stream);
    if (bias_dtype == ZLM_BF16)
        return launch<TX, TW, TY, __nv_bfloat16>(X, W, bias, Y, accumulate, M, N, K, ldx, ldw, ldy, stream);
    return ZLM_ERR_UNSUPPORTED;
}

template <typename TX, typename TW>
static int pick_y(int y_dtype, int bias_dtype, const void* X, const void* W, const void* bias, void* Y,
                  int accumulate, int M, int N, int K, long ldx, long ldw, long ldy, cudaStream_t stream) {
    if (y_dtype == ZLM_F32)
        return pick_bias<TX, TW, float>(bias_dtype, X, W, bias, Y, accumulate, M, N, K, ldx, ldw, ldy, stream);
    if (y_dtype == ZLM_BF16)
        return pick_bias<TX, TW, __nv_bfloat16>(bias_dtype, X, W, bias, Y, accumulate, M, N, K, ldx, ldw, ldy,
                                                 stream);
    return ZLM_ERR_UNSUPPORTED;
}

}  // namespace zlm

using namespace zlm;

// accumulate != 0: Y += X*W^T (+bias); the running sum is read and written in Y's type.
ZLM_EXPORT int zlm_gemm_generic(const void* X, int x_dtype, const void* W, int w_dtype, const void* bias,
                                int bias_dtype, void* Y, int y_dtype, int accumulate, int M, int N, int K,
                                long ldx, long ldw, long ldy, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || ldx < K || ldw < K || ldy < N) return ZLM_ERR_BAD_ARG;
    if (x_dtype == ZLM_F32 && w_dtype == ZLM_F32)
        return pick_y<float, float>(y_dtype, bias_dtype, X, W, bias, Y, accumulate, M, N, K, ldx, ldw, ldy, stream);
    if (x_dtype == ZLM_F32 && w_dtype == ZLM_BF16)
        return pick_y<float, __nv_bfloat16>(y_dtype, bias_dtype, X, W, bias, Y, accumulate, M, N, K, ldx, ldw, ldy,
                                            stream);
    if (x_dtype == ZLM_BF16 && w_dtype == ZLM_F32)
        return pick_y<__nv_bfloat16, float>(y_dtype, bias_dtype, X, W, bias, Y, accumulate, M, N, K, ldx, ldw, ldy,
                                            stream);
    if (x_dtype == ZLM_BF16 && w_dtype == ZLM_BF16)
        return pick_y<__nv_bfloat16, __nv_bfloat16>(y_dtype, bias_dtype, X, W, bias, Y, accumulate, M, N, K, ldx,
                                                    ldw, ldy, stream);
    return ZLM_ERR_UNSUPPORTED;
}
