// Rotary positions, cache writes and attention over the paged cache: the plain
// kernels that take every head size (a multiple of 8), every number of heads
// and groups, both storage types, prompts, continued prompts and single decoded
// tokens alike.  They are the whole 32-bit path and the fallback of the bf16
// path for head sizes the tensor-core kernels do not cover.
//
// Formulas, as the reference computes them:
//   RoPE     pairs (i, i+rot/2) inside a head: theta = pos*inv_freq[i],
//            h[i]       = a*cos(theta) - b*sin(theta)
//            h[i+rot/2] = a*sin(theta) + b*cos(theta)
//            (src/model.zig:569-597,642-653; src/cuda_bridge.cu:2070-2108)
//            inv_freq comes from a table built once from the configuration (the
//            reference recomputes 1/powf(base, 2i/rot) per thread and ignores the
//            configured base, src/model.zig:405-413).
//   cache    keys are stored rotated (src/model.zig:655, src/kv_cache.zig:63-85)
//   scores   kvh = h / (n_heads/n_kv_heads); s_t = (q_h . K[t,kvh]) * scale
//            (src/model.zig:554,659-678)
//   mask     a token at position p sees keys [start, p], start = 0 or
//            p-window+1 (src/model.zig:660-661); nothing is materialised
//   softmax  m = max s, e = exp(s-m), p = e/sum e in float (src/math.zig:1088-1106)
//   values   o_h = sum_t p_t V[t,kvh,:] (src/model.zig:683-700)
//
// Cache layout: pages of `page_size` positions.  Page p of one layer holds
// [n_kv_heads][page_size][head_dim] for keys and the same for values.  A step
// gives each of its sequences a row of page numbers (`block_table`), so position
// t of sequence b lives in page block_table[b*bt_stride + t/page_size], row
// t%page_size.
#include "common.cuh"

namespace zlm {

// ------------------------------------------------------- rope + cache write
// One block per token.  The cosines and sines of the token's position are formed once in shared
// memory (float32 angles), then the threads walk the heads: q and k heads are rotated in place,
// k (rotated) and v heads are copied to the token's row of the cache pages.
// qkv row layout: [q: n_heads*hd | k: n_kv*hd | v: n_kv*hd]
constexpr int ROPE_MAX_HALF = 256;

template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, long row_stride, int n_heads, int n_kv, int hd, int rot,
                                  const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                  const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                  int bt_stride, T* __restrict__ k_pages, T* __restrict__ v_pages, int page_size,
                                  long page_stride) {
    __shared__ float cos_s[ROPE_MAX_HALF], sin_s[ROPE_MAX_HALF];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rot / 2;
    const bool have_table = inv_freq != nullptr && half > 0;
    if (have_table) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float theta = (float)pos * inv_freq[i];
            sincosf(theta, &sin_s[i], &cos_s[i]);
        }
    }
    __syncthreads();
    T* row0 = qkv + (long)t * row_stride;
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (k_pages != nullptr && n_kv > 0) {
        const int b = seq_of_token[t];
        const int page = block_table[(long)b * bt_stride + pos / page_size];
        const long off = (long)page * page_stride + (long)(pos % page_size) * hd;
        kdst = k_pages + off;       // head h of the cache row lies h * page_size * hd further
        vdst = v_pages + off;
    }
    const long kv_head_stride = (long)page_size * hd;
    // this block's share of the heads, counted over q heads, k heads, v heads in that order
    const int total_heads = n_heads + 2 * n_kv;
    const int per = (total_heads + gridDim.y - 1) / gridDim.y;
    const int h_lo = blockIdx.y * per, h_hi = min(total_heads, h_lo + per);
    const int rot_hi = min(h_hi, n_heads + n_kv);            // heads below this one are rotated
    if (have_table && rot_hi > h_lo) {
        for (int idx = threadIdx.x; idx < (rot_hi - h_lo) * half; idx += blockDim.x) {
            const int head = h_lo + idx / half, i = idx % half;
            T* row = row0 + (long)head * hd;
            const float a = to_float(row[i]);
            const float b2 = to_float(row[i + half]);
            const float c = cos_s[i], sn = sin_s[i];
            const T lo = from_float<T>(a * c - b2 * sn);
            const T hi = from_float<T>(a * sn + b2 * c);
            row[i] = lo;
            row[i + half] = hi;
            if (kdst && head >= n_heads) {
                T* d = kdst + (long)(head - n_heads) * kv_head_stride;
                d[i] = lo;
                d[i + half] = hi;
            }
        }
    }
    if (kdst) {
        // what the rotation left alone of the k heads (everything when there is no table), and the v heads
        const int k_first = have_table ? rot : 0;
        const int k_rest = hd - k_first;
        const int k_lo = max(h_lo, n_heads), k_hi = rot_hi;
        for (int idx = threadIdx.x; idx < (k_hi - k_lo) * k_rest; idx += blockDim.x) {
            const int h = k_lo - n_heads + idx / k_rest, i = k_first + idx % k_rest;
            kdst[(long)h * kv_head_stride + i] = row0[(long)(n_heads + h) * hd + i];
        }
        const int v_lo = max(h_lo, n_heads + n_kv);
        for (int idx = threadIdx.x; idx < (h_hi - v_lo) * hd; idx += blockDim.x) {
            const int h = v_lo - n_heads - n_kv + idx / hd, i = idx % hd;
            vdst[(long)h * kv_head_stride + i] = row0[(long)(n_heads + n_kv + h) * hd + i];
        }
    }
}

// The same for bf16 rows whose heads, halves and strides are multiples of 8 elements: a thread moves
// 16 bytes at a time (8 pairs of the rotation, or 8 elements of a copy), which is what a prompt of
// thousands of tokens needs to run at memory speed.  Same arithmetic, element by element.
__global__ void rope_store_vec_kernel(__nv_bfloat16* __restrict__ qkv, long row_stride, int n_heads, int n_kv, int hd,
                                      int rot, const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                      const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                      int bt_stride, __nv_bfloat16* __restrict__ k_pages,
                                      __nv_bfloat16* __restrict__ v_pages, int page_size, long page_stride) {
    __shared__ float cos_s[ROPE_MAX_HALF], sin_s[ROPE_MAX_HALF];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = positions[t];                       // positions, tables and frequencies are older than the step
    const int half = rot / 2;
    const bool have_table = inv_freq != nullptr && half > 0;
    if (have_table)
        for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sin_s[i], &cos_s[i]);
    __nv_bfloat16* kdst = nullptr;
    __nv_bfloat16* vdst = nullptr;
    if (k_pages != nullptr && n_kv > 0) {
        const int b = seq_of_token[t];
        const int page = block_table[(long)b * bt_stride + pos / page_size];
        const long off = (long)page * page_stride + (long)(pos % page_size) * hd;
        kdst = k_pages + off;
        vdst = v_pages + off;
    }
    __syncthreads();
    pdl_wait();
    __nv_bfloat16* row0 = qkv + (long)t * row_stride;
    const long kv_head_stride = (long)page_size * hd;
    const int total_heads = n_heads + 2 * n_kv;
    const int per = (total_heads + gridDim.y - 1) / gridDim.y;
    const int h_lo = blockIdx.y * per, h_hi = min(total_heads, h_lo + per);
    const int rot_hi = min(h_hi, n_heads + n_kv);
    if (have_table && rot_hi > h_lo) {
        const int units = half / 8;
        for (int idx = threadIdx.x; idx < (rot_hi - h_lo) * units; idx += blockDim.x) {
            const int head = h_lo + idx / units, i0 = (idx % units) * 8;
            __nv_bfloat16* row = row0 + (long)head * hd;
            uint4 lo = *reinterpret_cast<const uint4*>(row + i0);
            uint4 hi = *reinterpret_cast<const uint4*>(row + i0 + half);
            __nv_bfloat162* lp = reinterpret_cast<__nv_bfloat162*>(&lo);
            __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 x = __bfloat1622float2(lp[k]), y = __bfloat1622float2(hp[k]);
                const float c0 = cos_s[i0 + 2 * k], s0 = sin_s[i0 + 2 * k];
                const float c1 = cos_s[i0 + 2 * k + 1], s1 = sin_s[i0 + 2 * k + 1];
                lp[k] = __halves2bfloat162(__float2bfloat16_rn(x.x * c0 - y.x * s0), __float2bfloat16_rn(x.y * c1 - y.y * s1));
                hp[k] = __halves2bfloat162(__float2bfloat16_rn(x.x * s0 + y.x * c0), __float2bfloat16_rn(x.y * s1 + y.y * c1));
            }
            *reinterpret_cast<uint4*>(row + i0) = lo;
            *reinterpret_cast<uint4*>(row + i0 + half) = hi;
            if (kdst && head >= n_heads) {
                __nv_bfloat16* d = kdst + (long)(head - n_heads) * kv_head_stride;
                *reinterpret_cast<uint4*>(d + i0) = lo;
                *reinterpret_cast<uint4*>(d + i0 + half) = hi;
            }
        }
    }
    if (kdst) {
        const int k_first = have_table ? rot : 0;
        const int k_units = (hd - k_first) / 8;
        const int k_lo = max(h_lo, n_heads), k_hi = rot_hi;
        for (int idx = threadIdx.x; idx < (k_hi - k_lo) * k_units; idx += blockDim.x) {
            const int h = k_lo - n_heads + idx / k_units, i = k_first + (idx % k_units) * 8;
            *reinterpret_cast<uint4*>(kdst + (long)h * kv_head_stride + i) =
                *reinterpret_cast<const uint4*>(row0 + (long)(n_heads + h) * hd + i);
        }
        const int v_lo = max(h_lo, n_heads + n_kv), v_units = hd / 8;
        for (int idx = threadIdx.x; idx < (h_hi - v_lo) * v_units; idx += blockDim.x) {
            const int h = v_lo - n_heads - n_kv + idx / v_units, i = (idx % v_units) * 8;
            *reinterpret_cast<uint4*>(vdst + (long)h * kv_head_stride + i) =
                *reinterpret_cast<const uint4*>(row0 + (long)(n_heads + n_kv + h) * hd + i);
        }
    }
}

// ------------------------------------------------------------ attention
// grid (T, n_heads); 128 threads.  Warp w takes the key blocks w, w+4, ... of 32
// keys; lane j scores key j of the block, then the lanes split the head's
// dimensions for the weighted sum of values.  The four partial results are
// merged in warp order, so the result depends only on (start, pos).
constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_HD = 256;

template <typename T, int VEC>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int hd);

template <>
__device__ __forceinline__ float dot_row<float, 4>(const float* __restrict__ q, const float* __restrict__ k, int hd) {
    float acc = 0.f;
    for (int d = 0; d < hd; d += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(k + d);
        acc = fmaf(q[d], kv.x, acc);
        acc = fmaf(q[d + 1], kv.y, acc);
        acc = fmaf(q[d + 2], kv.z, acc);
        acc = fmaf(q[d + 3], kv.w, acc);
    }
    return acc;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16, 8>(const float* __restrict__ q,
                                                           const __nv_bfloat16* __restrict__ k, int hd) {
    float acc = 0.f;
    for (int d = 0; d < hd; d += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(p[i]);
            acc = fmaf(q[d + 2 * i], f.x, acc);
            acc = fmaf(q[d + 2 * i + 1], f.y, acc);
        }
    }
    return acc;
}

template <typename T, int VEC>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_general_kernel(const T* __restrict__ q, long q_row_stride, T* __restrict__ out, int n_heads, int n_kv,
                         int hd, float scale, int window, const int* __restrict__ positions,
                         const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int bt_stride,
                         const T* __restrict__ k_pages, const T* __restrict__ v_pages, int page_size,
                         long page_stride) {
    __shared__ float q_s[ATT_MAX_HD];
    __shared__ float acc_s[ATT_WARPS][ATT_MAX_HD];
    __shared__ float m_s[ATT_WARPS], l_s[ATT_WARPS];

    const int t = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[t];
    const int b = seq_of_token[t];
    const int kvh = h / (n_heads / n_kv);
    const int start = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* bt = block_table + (long)b * bt_stride;

    for (int i = threadIdx.x; i < hd; i += blockDim.x) q_s[i] = to_float(q[(long)t * q_row_stride + (long)h * hd + i]);
    __syncthreads();

    constexpr int NREG = ATT_MAX_HD / 32;
    float acc[NREG];
#pragma unroll
    for (int i = 0; i < NREG; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    const int n_keys = pos - start + 1;
    const int n_blocks = (n_keys + 31) / 32;
    for (int kb = warp; kb < n_blocks; kb += ATT_WARPS) {
        const int j = start + kb * 32 + lane;
        const bool valid = j <= pos;
        float s = -INFINITY;
        long row_off = 0;
        if (valid) {
            const int page = bt[j / page_size];
            row_off = (long)page * page_stride + ((long)kvh * page_size + j % page_size) * hd;
            s = dot_row<T, VEC>(q_s, k_pages + row_off, hd) * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));       // lane 0 of the block is always valid
        const float corr = expf(m - m_new);               // exp(-inf) = 0 on the first block
        const float p = valid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < NREG; ++i) acc[i] *= corr;
        const int n_valid = min(32, pos - (start + kb * 32) + 1);
        for (int jj = 0; jj < n_valid; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long voff = __shfl_sync(0xffffffffu, row_off, jj);
            const T* vrow = v_pages + voff;
#pragma unroll
            for (int i = 0; i < NREG; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] = fmaf(pj, to_float(vrow[d]), acc[i]);
            }
        }
    }

    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int i = 0; i < NREG; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc_s[warp][d] = acc[i];
    }
    __syncthreads();

    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) big = fmaxf(big, m_s[w]);
    float wgt[ATT_WARPS];
    float denom = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
        wgt[w] = m_s[w] == -INFINITY ? 0.f : expf(m_s[w] - big);
        denom += l_s[w] * wgt[w];
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) o += acc_s[w][d] * wgt[w];
        out[((long)t * n_heads + h) * hd + d] = from_float<T>(o / denom);
    }
}

}  // namespace zlm

using namespace zlm;

// Rotates q and k in place inside qkv and copies k (rotated) and v into the cache.
// inv_freq == nullptr: no rotation.  k_pages == nullptr: nothing is stored (a layer
// that reads another layer's cache).
ZLM_EXPORT int zlm_rope_store(void* qkv, int dtype, long row_stride, int T, int n_heads, int n_kv, int hd, int rot,
                              const float* inv_freq, const int* positions, const int* seq_of_token,
                              const int* block_table, int bt_stride, void* k_pages, void* v_pages, int page_size,
                              long page_stride, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || rot < 0 || rot > hd || (rot & 1) || n_heads <= 0 || n_kv < 0 || page_size <= 0)
        return ZLM_ERR_BAD_ARG;
    if (rot / 2 > ROPE_MAX_HALF) return ZLM_ERR_UNSUPPORTED;
    // few tokens (a decode step): the heads of a token are shared out over several blocks
    const int total_heads = n_heads + 2 * n_kv;
    int parts = (296 + T - 1) / T;
    if (parts > total_heads) parts = total_heads;
    if (parts < 1) parts = 1;
    const int per = (total_heads + parts - 1) / parts;
    parts = (total_heads + per - 1) / per;
    const int work = per * (hd / 2);
    const int threads = work >= 2048 ? 256 : (work >= 512 ? 128 : 64);
    dim3 grid(T, parts);
    cudaError_t e;
    if (dtype == ZLM_F32)
        e = launch_pdl(rope_store_kernel<float>, grid, dim3(threads), 0, stream, (float*)qkv, row_stride, n_heads, n_kv,
                       hd, rot, inv_freq, positions, seq_of_token, block_table, bt_stride, (float*)k_pages,
                       (float*)v_pages, page_size, page_stride);
    else if (dtype == ZLM_BF16 && hd % 8 == 0 && rot % 16 == 0 && row_stride % 8 == 0 && page_stride % 8 == 0 &&
             (uintptr_t)qkv % 16 == 0 && (uintptr_t)k_pages % 16 == 0 && (uintptr_t)v_pages % 16 == 0)
        e = launch_pdl(rope_store_vec_kernel, grid, dim3(work >= 256 * 8 ? 256 : (work >= 128 * 8 ? 128 : 64)), 0, stream,
                       (__nv_bfloat16*)qkv, row_stride, n_heads, n_kv, hd, rot, inv_freq, positions, seq_of_token,
                       block_table, bt_stride, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, page_size, page_stride);
    else if (dtype == ZLM_BF16)
        e = launch_pdl(rope_store_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (__nv_bfloat16*)qkv,
                       row_stride, n_heads, n_kv, hd, rot, inv_freq, positions, seq_of_token, block_table, bt_stride,
                       (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, page_size, page_stride);
    else
        return ZLM_ERR_UNSUPPORTED;
    return e == cudaSuccess ? launch_status() : (int)e;
}

ZLM_EXPORT int zlm_attention_general(const void* q, long q_row_stride, void* out, int dtype, int T, int n_heads,
                                     int n_kv, int hd, float scale, int window, const int* positions,
                                     const int* seq_of_token, const int* block_table, int bt_stride,
                                     const void* k_pages, const void* v_pages, int page_size, long page_stride,
                                     cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || page_size <= 0) return ZLM_ERR_BAD_ARG;
    if (hd <= 0 || hd > ATT_MAX_HD || hd % 8) return ZLM_ERR_UNSUPPORTED;
    dim3 grid(T, n_heads);
    if (dtype == ZLM_F32)
        attention_general_kernel<float, 4><<<grid, ATT_WARPS * 32, 0, stream>>>(
            (const float*)q, q_row_stride, (float*)out, n_heads, n_kv, hd, scale, window, positions, seq_of_token,
            block_table, bt_stride, (const float*)k_pages, (const float*)v_pages, page_size, page_stride);
    else if (dtype == ZLM_BF16)
        attention_general_kernel<__nv_bfloat16, 8><<<grid, ATT_WARPS * 32, 0, stream>>>(
            (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, n_heads, n_kv, hd, scale, window, positions,
            seq_of_token, block_table, bt_stride, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
            page_size, page_stride);
    else
        return ZLM_ERR_UNSUPPORTED;
    return launch_status();
}
