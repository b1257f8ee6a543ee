// Embedding gather, RMSNorm (with optional row gather) and the gated activation.
//
// Formulas follow the reference:
//   embedding  x = W_e[token] widened to float, times a scale that is 1 for this
//              architecture                      (src/model.zig:495-503)
//   RMSNorm    ss = sum x_i^2, inv = 1/sqrt(ss/n + eps), y_i = (x_i*inv)*w_i
//              (src/math.zig:850-945; GPU twin src/cuda_bridge.cu:1475-1534)
//   SwiGLU     act_j = silu(g_j)*u_j, silu(z) = z/(1+exp(-z))
//              (src/math.zig:1108-1117, src/cuda_bridge.cu:2271-2285)
// The residual stream is float in both precisions, so the norm always reads
// float and writes the storage type of the next matrix product.
#include "common.cuh"

namespace zlm {

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int d, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const long row = (long)tokens[t] * d;
    float* o = out + (long)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_float(table[row + i]) * scale;
}

// ------------------------------------------------------------------ RMSNorm
// One block per output row.  rows == nullptr: row r of the input; otherwise row
// rows[r] (this is how the final norm runs on the wanted positions only).
template <typename TO> __device__ __forceinline__ void store4(TO* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = v;
}
template <typename TW> __device__ __forceinline__ void load4(const TW* p, float (&w)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&w)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&w)[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    w[0] = a.x; w[1] = a.y; w[2] = b.x; w[3] = b.y;
}

// VEC: the row length is a multiple of 4 and every pointer is 16-byte aligned, so a thread moves four
// elements at a time and keeps up to MAXV groups of its row in registers between the two passes.
template <typename TW, typename TO, bool VEC>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ rows, int d, float eps, float weight_offset) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (long)(rows ? rows[r] : r) * d;
    TO* o = out + (long)r * d;
    if (VEC) {
        constexpr int MAXV = 8;
        float4 keep[MAXV];
        const int n4 = d >> 2;
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < n4) {
                keep[k] = reinterpret_cast<const float4*>(xr)[i];
                ss = fmaf(keep[k].x, keep[k].x, ss); ss = fmaf(keep[k].y, keep[k].y, ss);
                ss = fmaf(keep[k].z, keep[k].z, ss); ss = fmaf(keep[k].w, keep[k].w, ss);
            }
        }
        for (int i = threadIdx.x + MAXV * blockDim.x; i < n4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(xr)[i];
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < n4) {
                float ww[4];
                load4<TW>(w + 4 * i, ww);
                store4<TO>(o + 4 * i, (keep[k].x * inv) * (ww[0] + weight_offset), (keep[k].y * inv) * (ww[1] + weight_offset),
                           (keep[k].z * inv) * (ww[2] + weight_offset), (keep[k].w * inv) * (ww[3] + weight_offset));
            }
        }
        for (int i = threadIdx.x + MAXV * blockDim.x; i < n4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(xr)[i];
            float ww[4];
            load4<TW>(w + 4 * i, ww);
            store4<TO>(o + 4 * i, (v.x * inv) * (ww[0] + weight_offset), (v.y * inv) * (ww[1] + weight_offset),
                       (v.z * inv) * (ww[2] + weight_offset), (v.w * inv) * (ww[3] + weight_offset));
        }
    } else {
        float ss = 0.f;
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float v = xr[i];
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
        for (int i = threadIdx.x; i < d; i += blockDim.x)
            o[i] = from_float<TO>((xr[i] * inv) * (to_float(w[i]) + weight_offset));
    }
}

// --------------------------------------------------------- gated activation
// gu is [T, 2*I].  interleaved == 0: gate in columns [0, I), up in columns [I, 2I);
// interleaved != 0: gate j in column 2j, up j in column 2j+1.
template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ out, long total, int I, int kind,
                                 int interleaved) {
    pdl_launch_dependents();
    pdl_wait();
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long t = idx / I;
    const int j = (int)(idx - t * I);
    const float g = to_float(gu[t * 2 * I + (interleaved ? 2 * j : j)]);
    const float u = to_float(gu[t * 2 * I + (interleaved ? 2 * j + 1 : I + j)]);
    float a;
    if (kind == 0) {
        a = g / (1.0f + expf(-g));                         // silu
    } else {
        const float c = 0.7978845608028654f;               // gelu (tanh form)
        a = 0.5f * g * (1.0f + tanhf(c * (g + 0.044715f * g * g * g)));
    }
    out[idx] = from_float<T>(a * u);
}

// y += x (float), used by parts that cannot fold their residual sum into a product
__global__ void add_kernel(float* __restrict__ y, const float* __restrict__ x, long n) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] += x[i];
}

template <typename TI, typename TO>
__global__ void convert_kernel(const TI* __restrict__ in, TO* __restrict__ out, long n) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_float<TO>(to_float(in[i]));
}

static int norm_threads(int d) {
    int t = 32;
    while (t < 512 && t * 4 < d) t <<= 1;
    return t;
}


// -------------------------------------------------------------- random weights
// Element i of a tensor with key k is a function of (k, i) alone:
//   h = mix64(k + i); a = top 24 bits of h, b = the 24 bits below them;
//   u1 = (a + 1) / 2^24 in (0, 1], angle = 2 pi b / 2^24;
//   z = sqrt(-2 ln u1) * cos(angle)                      (Box-Muller, one of its two values)
//   value = mean + std * z, rounded to the storage type.
// Every floating operation is a single IEEE-rounded +, *, / or sqrt in float (the _rn intrinsics keep
// the compiler from fusing them), and ln, sin and cos are the short polynomials below, so the same
// steps in NumPy give the same bits (ziglm_b200/weights/random_init.py: normal_values).  The
// reference fills its fixtures from one sequential generator (src/synthetic.zig:232-249); a counter
// lets any element be regenerated without the others, on the host or on the device.
__device__ __forceinline__ uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__device__ __forceinline__ float det_sin(float x) {          // x in [0, pi/4]
    const float x2 = __fmul_rn(x, x);
    float p = 2.75573192e-6f;                                 // 1/9!
    p = __fadd_rn(__fmul_rn(p, x2), -1.98412698e-4f);         // -1/7!
    p = __fadd_rn(__fmul_rn(p, x2), 8.33333333e-3f);          // 1/5!
    p = __fadd_rn(__fmul_rn(p, x2), -1.66666667e-1f);         // -1/3!
    p = __fadd_rn(__fmul_rn(p, x2), 1.0f);
    return __fmul_rn(x, p);
}

__device__ __forceinline__ float det_cos(float x) {          // x in [0, pi/4]
    const float x2 = __fmul_rn(x, x);
    float p = -2.75573192e-7f;                                // -1/10!
    p = __fadd_rn(__fmul_rn(p, x2), 2.48015873e-5f);          // 1/8!
    p = __fadd_rn(__fmul_rn(p, x2), -1.38888889e-3f);         // -1/6!
    p = __fadd_rn(__fmul_rn(p, x2), 4.16666667e-2f);          // 1/4!
    p = __fadd_rn(__fmul_rn(p, x2), -0.5f);
    return __fadd_rn(__fmul_rn(p, x2), 1.0f);
}

__device__ __forceinline__ float det_normal(uint64_t key, uint64_t index) {
    const uint64_t h = mix64(key + index);
    const uint32_t n = (uint32_t)(h >> 40) + 1u;              // 1 .. 2^24
    const uint32_t b = (uint32_t)(h >> 16) & 0xFFFFFFu;
    // ln(n / 2^24) = (e - 24) ln 2 + ln m with n = m 2^e, m in (sqrt(1/2), sqrt(2)]
    int e = 31 - __clz(n);
    float m = __fmul_rn((float)n, __int_as_float((127 - e) << 23));      // exact: n < 2^25, a power of two
    if (m > 1.41421354f) { m = __fmul_rn(m, 0.5f); e += 1; }
    const float s = __fdiv_rn(__fadd_rn(m, -1.0f), __fadd_rn(m, 1.0f));
    const float s2 = __fmul_rn(s, s);
    float p = 1.11111111e-1f;                                 // 1/9
    p = __fadd_rn(__fmul_rn(p, s2), 1.42857143e-1f);          // 1/7
    p = __fadd_rn(__fmul_rn(p, s2), 0.2f);
    p = __fadd_rn(__fmul_rn(p, s2), 3.33333333e-1f);
    p = __fadd_rn(__fmul_rn(p, s2), 1.0f);
    const float ln_m = __fmul_rn(__fmul_rn(2.0f, s), p);
    const float ln_u = __fadd_rn(__fmul_rn((float)(e - 24), 0.693147182f), ln_m);
    const float r = __fsqrt_rn(__fmul_rn(-2.0f, ln_u));
    // cos(2 pi b / 2^24) by octants, the argument folded into [0, pi/4]
    const uint32_t oct = b >> 21, rem = b & 0x1FFFFFu;
    const float step = 3.74507039e-7f;                        // 2 pi / 2^24
    const float x = __fmul_rn((float)((oct & 1u) ? 0x200000u - rem : rem), step);
    float c;
    switch (oct) {
        case 0: c = det_cos(x); break;
        case 1: c = det_sin(x); break;
        case 2: c = -det_sin(x); break;
        case 3: c = -det_cos(x); break;
        case 4: c = -det_cos(x); break;
        case 5: c = -det_sin(x); break;
        case 6: c = det_sin(x); break;
        default: c = det_cos(x); break;
    }
    return __fmul_rn(r, c);
}

template <typename TO>
__global__ void fill_normal_kernel(TO* __restrict__ out, long n, uint64_t key, float mean, float std_dev) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
        out[i] = from_float<TO>(__fadd_rn(mean, __fmul_rn(std_dev, det_normal(key, (uint64_t)i))));
}

}  // namespace zlm

using namespace zlm;

ZLM_EXPORT int zlm_embed(const void* table, int table_dtype, const int* tokens, float* out, int T, int d,
                         float scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0) return ZLM_ERR_BAD_ARG;
    const int threads = d >= 1024 ? 256 : 128;
    cudaError_t e;
    if (table_dtype == ZLM_F32)
        e = launch_pdl(embed_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)table, tokens, out, d, scale);
    else if (table_dtype == ZLM_BF16)
        e = launch_pdl(embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)table,
                       tokens, out, d, scale);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

ZLM_EXPORT int zlm_rmsnorm(const float* x, const void* w, int w_dtype, void* out, int out_dtype, const int* rows,
                           int n_rows, int d, float eps, float weight_offset, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0) return ZLM_ERR_BAD_ARG;
    const bool vec = d % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0;
    const int threads = vec ? (d >= 2048 ? 256 : (d >= 512 ? 128 : 64)) : norm_threads(d);
    cudaError_t e;
#define ZLM_NORM(TW, TO)                                                                                       \
    e = vec ? launch_pdl(rmsnorm_kernel<TW, TO, true>, dim3(n_rows), dim3(threads), 0, stream, x, (const TW*)w,  \
                         (TO*)out, rows, d, eps, weight_offset)                                                \
            : launch_pdl(rmsnorm_kernel<TW, TO, false>, dim3(n_rows), dim3(threads), 0, stream, x, (const TW*)w, \
                         (TO*)out, rows, d, eps, weight_offset)
    if (w_dtype == ZLM_F32 && out_dtype == ZLM_F32) ZLM_NORM(float, float);
    else if (w_dtype == ZLM_F32 && out_dtype == ZLM_BF16) ZLM_NORM(float, __nv_bfloat16);
    else if (w_dtype == ZLM_BF16 && out_dtype == ZLM_F32) ZLM_NORM(__nv_bfloat16, float);
    else if (w_dtype == ZLM_BF16 && out_dtype == ZLM_BF16) ZLM_NORM(__nv_bfloat16, __nv_bfloat16);
    else return ZLM_ERR_UNSUPPORTED;
#undef ZLM_NORM
    return e == cudaSuccess ? launch_status() : (int)e;
}

ZLM_EXPORT int zlm_gated_act(const void* gu, void* out, int dtype, int T, int I, int kind, int interleaved,
                             cudaStream_t stream) {
    if (T <= 0) return 0;
    if (I <= 0 || (kind != 0 && kind != 1)) return ZLM_ERR_BAD_ARG;
    const long total = (long)T * I;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(gated_act_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)gu, (float*)out,
                       total, I, kind, interleaved);
    else if (dtype == ZLM_BF16)
        e = launch_pdl(gated_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream,
                       (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, total, I, kind, interleaved);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

ZLM_EXPORT int zlm_add(float* y, const float* x, long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(y, x, n);
    return launch_status();
}

ZLM_EXPORT int zlm_convert(const void* in, int in_dtype, void* out, int out_dtype, long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (in_dtype == ZLM_F32 && out_dtype == ZLM_BF16)
        convert_kernel<float, __nv_bfloat16><<<blocks, 256, 0, stream>>>((const float*)in, (__nv_bfloat16*)out, n);
    else if (in_dtype == ZLM_BF16 && out_dtype == ZLM_F32)
        convert_kernel<__nv_bfloat16, float><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (float*)out, n);
    else
        return ZLM_ERR_UNSUPPORTED;
    return launch_status();
}

// out[i] = mean + std * z(key, i), i < n, z a standard normal value that depends on (key, i) only.
ZLM_EXPORT int zlm_fill_normal(void* out, int out_dtype, long n, unsigned long long key, float mean, float std_dev,
                               cudaStream_t stream) {
    if (n < 0 || (n > 0 && !out)) return ZLM_ERR_BAD_ARG;
    if (n == 0) return 0;
    long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_dtype == ZLM_BF16)
        fill_normal_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>((__nv_bfloat16*)out, n, key, mean, std_dev);
    else if (out_dtype == ZLM_F32)
        fill_normal_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>((float*)out, n, key, mean, std_dev);
    else
        return ZLM_ERR_UNSUPPORTED;
    return launch_status();
}
