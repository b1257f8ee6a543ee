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
//
// Three kernels keep that rule.  gemm_generic_kernel tiles 64 tokens x 64 weight
// rows and takes every operand type; float operands with more than 96 tokens go to
// gemm_large_kernel (128 x 128 tiles, 64 outputs a thread); a step of a few tokens would use a sixty-fourth of such a tile and too few
// blocks to draw on the memory system, so float operands with at most 32 tokens go
// to gemm_skinny_kernel, which streams 32 or 128 weight rows a block through a ring
// of asynchronous copies and gives every (row, token) pair to one thread.
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

// ------------------------------------------------------ many tokens, float operands
// Tiles of 128 tokens x 128 weight rows for float operands whose rows start on 16-byte boundaries: 256 threads,
// 8 x 8 outputs a thread (two groups of four tokens, two groups of four rows, so that a thread reads its 16
// operands of a k with four 16-byte loads), K in steps of 16 through two buffers of shared memory: the next
// step's 16-byte global loads are in flight while this step is summed.  Every output is still one thread's sum
// in ascending k, one fused multiply-add each.
constexpr int LM = 128, LN = 128, LK = 16, LLD = 128 + 4;

template <typename TB, bool ACC>
__global__ void __launch_bounds__(256, 2)
gemm_large_kernel(const float* __restrict__ X, const float* __restrict__ W, const TB* __restrict__ bias,
                  float* __restrict__ Y, int M, int N, int K, long ldx, long ldw, long ldy) {
    __shared__ __align__(16) float As[2][LK][LLD];           // [k][token]
    __shared__ __align__(16) float Bs[2][LK][LLD];           // [k][weight row]
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * LM, n0 = blockIdx.x * LN;
    // loader: 128 rows x 16 k = 512 pieces of four k; a thread loads rows lr and lr + 64 at k offset lk
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    // rows beyond M or N repeat the last one; their outputs are not stored
    const float* xsrc[2];
    const float* wsrc[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        xsrc[h] = X + (long)min(m0 + lr + 64 * h, M - 1) * ldx + lk;
        wsrc[h] = W + (long)min(n0 + lr + 64 * h, N - 1) * ldw + lk;
    }
    float4 xa[2], wb[2];
    auto fetch = [&](int k0) {                               // K is a multiple of 4: a piece is whole or absent
        if (k0 + lk < K) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                xa[h] = *reinterpret_cast<const float4*>(xsrc[h] + k0);
                wb[h] = *reinterpret_cast<const float4*>(wsrc[h] + k0);
            }
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) xa[h] = wb[h] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto stage = [&](int buf) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = lr + 64 * h;
            As[buf][lk + 0][r] = xa[h].x; As[buf][lk + 1][r] = xa[h].y;
            As[buf][lk + 2][r] = xa[h].z; As[buf][lk + 3][r] = xa[h].w;
            Bs[buf][lk + 0][r] = wb[h].x; Bs[buf][lk + 1][r] = wb[h].y;
            Bs[buf][lk + 2][r] = wb[h].z; Bs[buf][lk + 3][r] = wb[h].w;
        }
    };

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    fetch(0);
    stage(0);
    __syncthreads();
    int buf = 0;
    for (int k0 = 0; k0 < K; k0 += LK) {
        const bool more = k0 + LK < K;
        if (more) fetch(k0 + LK);
#pragma unroll
        for (int k = 0; k < LK; ++k) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (more) {
            stage(buf ^ 1);                                  // the other buffer was last read one step ago
            __syncthreads();
            buf ^= 1;
        }
    }

#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias) v += to_float(bias[gn]);
            float* dst = Y + (long)gm * ldy + gn;
            if (ACC) *dst = *dst + v;
            else *dst = v;
        }
    }
}

// Float operands whose rows start on 16-byte boundaries, more than 96 tokens.  ZLM_ERR_UNSUPPORTED otherwise.
static int launch_large(const void* X, const void* W, const void* bias, int bias_dtype, void* Y, int accumulate, int M,
                        int N, int K, long ldx, long ldw, long ldy, cudaStream_t stream) {
    if (M <= 96 || (K & 3) || (ldx & 3) || (ldw & 3) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15))
        return ZLM_ERR_UNSUPPORTED;
    if (bias != nullptr && bias_dtype != ZLM_F32 && bias_dtype != ZLM_BF16) return ZLM_ERR_UNSUPPORTED;
    const dim3 grid((N + LN - 1) / LN, (M + LM - 1) / LM);
    const float* x = (const float*)X;
    const float* w = (const float*)W;
    float* y = (float*)Y;
#define ZLM_LARGE(TBV, ACCV)                                                                                         \
    gemm_large_kernel<TBV, ACCV><<<grid, 256, 0, stream>>>(x, w, (const TBV*)bias, y, M, N, K, ldx, ldw, ldy)
    if (bias != nullptr && bias_dtype == ZLM_BF16) {
        if (accumulate) ZLM_LARGE(__nv_bfloat16, true);
        else ZLM_LARGE(__nv_bfloat16, false);
    } else {
        if (accumulate) ZLM_LARGE(float, true);
        else ZLM_LARGE(float, false);
    }
#undef ZLM_LARGE
    return launch_status();
}

// ------------------------------------------------------ few tokens, float operands
// A block of four warps owns 32 * RW weight rows and all M <= (4 / RW) * TT tokens.  Warp w owns the rows of row
// group w % RW (lane l: row l of the group) and the tokens of token group w / RW (TT of them), so a thread carries
// TT running sums.  The K range comes in chunks of SK_BK / RW floats: all threads issue 16-byte asynchronous
// copies of the rows' chunk and of the tokens' chunk into one of SK_STAGES stages, and compute from the oldest
// stage while the younger ones are in flight.  A row of a stage is padded by four floats, so that the 32 lanes'
// 16-byte reads of their rows fall in different banks.
//
// RW = 1 (32 rows a block, up to 32 tokens over the four warps) gives narrow products enough blocks to fill the
// device.  RW = 4 (128 rows a block, up to 8 tokens, every warp with rows of its own) is for wide products with
// few tokens: a weight value is then read from shared memory by one warp instead of four, and it is shared memory
// reads that bound these kernels.
constexpr int SK_WARPS = 4, SK_BK = 128, SK_STAGES = 4;
template <int RW> struct SkChunk { static constexpr int value = SK_BK / RW; };   // floats of K a stage

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* src, int src_bytes) {
    // copies src_bytes (0..16) and fills the rest of the 16 bytes with zeros
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int RW, int TT, typename TB, bool ACC>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(const float* __restrict__ X, const float* __restrict__ W, const TB* __restrict__ bias,
                   float* __restrict__ Y, int M, int N, int K, long ldx, long ldw, long ldy) {
    constexpr int ROWS = 32 * RW;                            // weight rows staged
    constexpr int TOK = (SK_WARPS / RW) * TT;                // token rows staged
    constexpr int BKC = SkChunk<RW>::value, LD = BKC + 4;          // floats of K a stage, and a staged row's pitch
    extern __shared__ __align__(16) float sk_smem[];
    float* Ws = sk_smem;                                     // [SK_STAGES][ROWS][LD]
    float* Xs = sk_smem + SK_STAGES * ROWS * LD;             // [SK_STAGES][TOK][LD]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row_group = warp % RW, token_group = warp / RW;
    const int n0 = blockIdx.x * ROWS;
    const int n_chunks = (K + BKC - 1) / BKC;

    // The pieces of 16 bytes a thread copies are the same in every chunk: piece j of this thread is row
    // tid / PPR + j * RSTEP at float (tid % PPR) * 4 of the chunk.  Row offsets are kept, not recomputed.
    constexpr int PPR = BKC / 4;                             // pieces a row
    constexpr int RSTEP = SK_WARPS * 32 / PPR;               // rows between a thread's pieces
    constexpr int WP = ROWS / RSTEP, XP = (TOK + RSTEP - 1) / RSTEP;
    const int pr = tid / PPR, pc = (tid % PPR) * 4;
    const float* wsrc[WP];
#pragma unroll
    for (int j = 0; j < WP; ++j)                             // rows beyond N repeat the last one and are not stored
        wsrc[j] = W + (long)min(n0 + pr + j * RSTEP, N - 1) * ldw + pc;
    const float* xsrc[XP];
#pragma unroll
    for (int j = 0; j < XP; ++j) xsrc[j] = X + (long)min(pr + j * RSTEP, M - 1) * ldx + pc;

    auto issue = [&](int chunk) {
        const int stage = chunk % SK_STAGES, k0 = chunk * BKC;
        float* ws = Ws + stage * ROWS * LD + pr * LD + pc;
        float* xs = Xs + stage * TOK * LD + pr * LD + pc;
        // pieces beyond K are zeros (K is a multiple of 4: a piece is whole or absent)
        const bool have = k0 + pc < K;
        const int bytes = have ? 16 : 0, at = have ? k0 : 0;
#pragma unroll
        for (int j = 0; j < WP; ++j) cp_async_16(ws + j * RSTEP * LD, wsrc[j] + at, bytes);
#pragma unroll
        for (int j = 0; j < XP; ++j)
            if (pr + j * RSTEP < TOK) cp_async_16(xs + j * RSTEP * LD, xsrc[j] + at, bytes);
    };

    for (int c = 0; c < SK_STAGES - 1; ++c) {
        if (c < n_chunks) issue(c);
        cp_async_commit();
    }
    float acc[TT];
#pragma unroll
    for (int t = 0; t < TT; ++t) acc[t] = 0.f;
    const bool active = token_group * TT < M;                // warps whose tokens do not exist only help copying

    for (int chunk = 0; chunk < n_chunks; ++chunk) {
        cp_async_wait<SK_STAGES - 2>();                      // this thread's copies of the oldest stage have landed
        __syncthreads();                                     // ... and everyone's; the stage computed last is free
        if (chunk + SK_STAGES - 1 < n_chunks) issue(chunk + SK_STAGES - 1);
        cp_async_commit();
        if (active) {
            const float* ws = Ws + (chunk % SK_STAGES) * ROWS * LD + (row_group * 32 + lane) * LD;
            const float* xs = Xs + (chunk % SK_STAGES) * TOK * LD + token_group * TT * LD;
            // the loads of the next four k are issued before the sums of these four: with eight warps an SM
            // nothing else hides the latency of shared memory
            float4 w = *reinterpret_cast<const float4*>(ws);
            float4 x[TT];
#pragma unroll
            for (int t = 0; t < TT; ++t) x[t] = *reinterpret_cast<const float4*>(xs + t * LD);
#pragma unroll
            for (int k = 0; k < BKC; k += 4) {
                float4 wn = w, xn[TT];
#pragma unroll
                for (int t = 0; t < TT; ++t) xn[t] = x[t];
                if (k + 4 < BKC) {
                    wn = *reinterpret_cast<const float4*>(ws + k + 4);
#pragma unroll
                    for (int t = 0; t < TT; ++t) xn[t] = *reinterpret_cast<const float4*>(xs + t * LD + k + 4);
                }
#pragma unroll
                for (int t = 0; t < TT; ++t) {
                    // ascending k, one fused multiply-add each: the order of gemm_generic_kernel
                    acc[t] = fmaf(x[t].x, w.x, acc[t]);
                    acc[t] = fmaf(x[t].y, w.y, acc[t]);
                    acc[t] = fmaf(x[t].z, w.z, acc[t]);
                    acc[t] = fmaf(x[t].w, w.w, acc[t]);
                }
                w = wn;
#pragma unroll
                for (int t = 0; t < TT; ++t) x[t] = xn[t];
            }
        }
    }
    const int gn = n0 + row_group * 32 + lane;
    if (!active || gn >= N) return;
    const float b = bias ? to_float(bias[gn]) : 0.f;
#pragma unroll
    for (int t = 0; t < TT; ++t) {
        const int gm = token_group * TT + t;
        if (gm >= M) break;
        float v = acc[t];
        if (bias) v += b;
        float* dst = Y + (long)gm * ldy + gn;
        if (ACC) *dst = *dst + v;
        else *dst = v;
    }
}

template <int RW, int TT, typename TB, bool ACC>
static int launch_skinny_one(const float* X, const float* W, const void* bias, float* Y, int M, int N, int K, long ldx,
                             long ldw, long ldy, cudaStream_t stream) {
    constexpr int ROWS = 32 * RW, TOK = (SK_WARPS / RW) * TT, LD = SkChunk<RW>::value + 4;
    const int smem = SK_STAGES * (ROWS + TOK) * LD * (int)sizeof(float);
    static bool configured = false;                          // one flag per kernel: this function is its only launcher
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<RW, TT, TB, ACC>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    gemm_skinny_kernel<RW, TT, TB, ACC><<<(N + ROWS - 1) / ROWS, SK_WARPS * 32, smem, stream>>>(
        X, W, (const TB*)bias, Y, M, N, K, ldx, ldw, ldy);
    return launch_status();
}

template <int RW, int TT, typename TB>
static int launch_skinny_tt(const float* X, const float* W, const void* bias, float* Y, int accumulate, int M, int N,
                            int K, long ldx, long ldw, long ldy, cudaStream_t stream) {
    if (accumulate) return launch_skinny_one<RW, TT, TB, true>(X, W, bias, Y, M, N, K, ldx, ldw, ldy, stream);
    return launch_skinny_one<RW, TT, TB, false>(X, W, bias, Y, M, N, K, ldx, ldw, ldy, stream);
}

// Products with at least this many weight rows and at most 8 tokens give every warp rows of its own (RW = 4):
// there are then still more blocks than the device holds at once.
constexpr int SK_WIDE_N = 16384;

// Float operands whose rows start on 16-byte boundaries, at most 32 tokens.  Returns ZLM_ERR_UNSUPPORTED otherwise.
static int launch_skinny(const void* X, const void* W, const void* bias, int bias_dtype, void* Y, int accumulate, int M,
                         int N, int K, long ldx, long ldw, long ldy, cudaStream_t stream) {
    if (M > 8 * SK_WARPS || (K & 3) || (ldx & 3) || (ldw & 3) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15))
        return ZLM_ERR_UNSUPPORTED;
    if (bias != nullptr && bias_dtype != ZLM_F32 && bias_dtype != ZLM_BF16) return ZLM_ERR_UNSUPPORTED;
    const float* x = (const float*)X;
    const float* w = (const float*)W;
    float* y = (float*)Y;
#define ZLM_SKINNY(RWV, TTV)                                                                                         \
    (bias != nullptr && bias_dtype == ZLM_BF16                                                                       \
         ? launch_skinny_tt<RWV, TTV, __nv_bfloat16>(x, w, bias, y, accumulate, M, N, K, ldx, ldw, ldy, stream)        \
         : launch_skinny_tt<RWV, TTV, float>(x, w, bias, y, accumulate, M, N, K, ldx, ldw, ldy, stream))
    if (N >= SK_WIDE_N && M <= 8) {                          // every warp its own rows, all tokens
        if (M <= 1) return ZLM_SKINNY(4, 1);
        if (M <= 2) return ZLM_SKINNY(4, 2);
        if (M <= 4) return ZLM_SKINNY(4, 4);
        return ZLM_SKINNY(4, 8);
    }
    const int tt = (M + SK_WARPS - 1) / SK_WARPS;            // tokens per warp: 1, 2, 4 or 8
    if (tt <= 1) return ZLM_SKINNY(1, 1);
    if (tt <= 2) return ZLM_SKINNY(1, 2);
    if (tt <= 4) return ZLM_SKINNY(1, 4);
    return ZLM_SKINNY(1, 8);
#undef ZLM_SKINNY
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
    if (x_dtype == ZLM_F32 && w_dtype == ZLM_F32 && y_dtype == ZLM_F32 && M <= 8 * SK_WARPS) {
        const int rc = launch_skinny(X, W, bias, bias_dtype, Y, accumulate, M, N, K, ldx, ldw, ldy, stream);
        if (rc != ZLM_ERR_UNSUPPORTED) return rc;
    }
    if (x_dtype == ZLM_F32 && w_dtype == ZLM_F32 && y_dtype == ZLM_F32) {
        const int rc = launch_large(X, W, bias, bias_dtype, Y, accumulate, M, N, K, ldx, ldw, ldy, stream);
        if (rc != ZLM_ERR_UNSUPPORTED) return rc;
    }
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
