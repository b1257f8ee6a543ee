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
// The keys a token sees, [start, pos], are cut into parts of ATT_PART = 256 consecutive keys counted from
// `start`.  Within a part warp w of a block takes the key blocks w and w + 4 of 32 keys: lane j scores key j of
// a block, then the lanes split the head's dimensions for the weighted sum of values; the four warps' partial
// results are merged in warp order into the part's (max, sum, weighted values).  The parts are then folded one
// after another, in ascending order, into the result.  A block works for G query heads that share a key/value
// head (the largest of 4, 2, 1 that divides the group), so a key or value row is read once for all of them.
//
// Two ways to run, with bit-for-bit the same result, because a part's result depends on (start, pos, part)
// alone and the fold is the same arithmetic in the same order:
//   whole   grid (T, n_heads / G, 1): a block computes and folds all parts of its token (prompts: the tokens
//           alone give enough blocks);
//   split   grid (T, n_heads / G, parts): a block computes one part and stores it in scratch memory, and
//           attention_fold_kernel folds a token's parts (steps of few tokens: the parts give the blocks).
constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_HD = 256;
constexpr int ATT_PART = ATT_WARPS * 2 * 32;

// k[d..d+VEC) of one key row as floats
template <typename T, int VEC> __device__ __forceinline__ void load_vec(const T* __restrict__ p, float (&f)[VEC]);
template <> __device__ __forceinline__ void load_vec<float, 4>(const float* __restrict__ p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load_vec<__nv_bfloat16, 8>(const __nv_bfloat16* __restrict__ p, float (&f)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(h[i]);
        f[2 * i] = v.x; f[2 * i + 1] = v.y;
    }
}

// Fold a part (mp, lp, op) into the running (m, l, o): every operation is one rounded multiply, add or fused
// multiply-add, written out so that both kernels that fold do exactly the same.
__device__ __forceinline__ void fold_weights(float m, float mp, float& m_new, float& a, float& b) {
    m_new = fmaxf(m, mp);
    a = expf(m - m_new);                 // exp(-inf) = 0 for the first part
    b = expf(mp - m_new);
}
__device__ __forceinline__ float fold_value(float o, float a, float op, float b) {
    return __fmaf_rn(op, b, __fmul_rn(o, a));
}

template <typename T, int VEC, int G, int NREG>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_general_kernel(const T* __restrict__ q, long q_row_stride, T* __restrict__ out, int n_heads, int n_kv,
                         int hd, float scale, int window, const int* __restrict__ positions,
                         const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int bt_stride,
                         const T* __restrict__ k_pages, const T* __restrict__ v_pages, int page_size,
                         long page_stride, float* __restrict__ part_ml, float* __restrict__ part_o, int max_parts) {
    __shared__ float q_s[G][ATT_MAX_HD];
    __shared__ float acc_s[G][ATT_WARPS][NREG * 32];
    __shared__ float m_s[G][ATT_WARPS], l_s[G][ATT_WARPS];

    const int t = blockIdx.x, h0 = blockIdx.y * G;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = positions[t];
    const int b = seq_of_token[t];
    const int kvh = h0 / (n_heads / n_kv);
    const int start = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_keys = pos - start + 1;
    const int n_parts = (n_keys + ATT_PART - 1) / ATT_PART;
    const bool split = part_o != nullptr;
    const int p_lo = split ? (int)blockIdx.z : 0, p_hi = split ? min(n_parts, (int)blockIdx.z + 1) : n_parts;
    if (p_lo >= n_parts) return;
    const int* bt = block_table + (long)b * bt_stride;

    for (int i = threadIdx.x; i < G * hd; i += blockDim.x)
        q_s[i / hd][i % hd] = to_float(q[(long)t * q_row_stride + (long)(h0 + i / hd) * hd + i % hd]);
    __syncthreads();

    // the running result: thread x owns dimensions x and x + 128 of every head
    float run_m[G], run_l[G], run_o[G][2];
#pragma unroll
    for (int g = 0; g < G; ++g) { run_m[g] = -INFINITY; run_l[g] = 0.f; run_o[g][0] = run_o[g][1] = 0.f; }

    for (int part = p_lo; part < p_hi; ++part) {
        float acc[G][NREG], m[G], l[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
            for (int i = 0; i < NREG; ++i) acc[g][i] = 0.f;
        }
        const int part_first = start + part * ATT_PART;
#pragma unroll 1
        for (int kb = warp; kb < 2 * ATT_WARPS; kb += ATT_WARPS) {
            const int first = part_first + kb * 32;
            if (first > pos) break;                              // uniform per warp
            const int j = first + lane;
            const bool valid = j <= pos;
            float sc[G];
#pragma unroll
            for (int g = 0; g < G; ++g) sc[g] = 0.f;
            long row_off = 0;
            if (valid) {
                const int page = bt[j / page_size];
                row_off = (long)page * page_stride + ((long)kvh * page_size + j % page_size) * hd;
                const T* krow = k_pages + row_off;
                // several 16-byte loads of the row in flight at once: the loop is bound by their latency
#pragma unroll 8
                for (int d = 0; d < hd; d += VEC) {
                    float kv[VEC];
                    load_vec<T, VEC>(krow + d, kv);
#pragma unroll
                    for (int g = 0; g < G; ++g)
#pragma unroll
                        for (int i = 0; i < VEC; ++i) sc[g] = fmaf(q_s[g][d + i], kv[i], sc[g]);
                }
            }
            float pr[G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float sv = valid ? sc[g] * scale : -INFINITY;
                const float m_new = fmaxf(m[g], warp_max(sv));   // lane 0 of the block is always valid
                const float corr = expf(m[g] - m_new);           // exp(-inf) = 0 on the first block
                pr[g] = valid ? expf(sv - m_new) : 0.f;
                l[g] = l[g] * corr + warp_sum(pr[g]);
                m[g] = m_new;
#pragma unroll
                for (int i = 0; i < NREG; ++i) acc[g][i] *= corr;
            }
            const int n_valid = min(32, pos - first + 1);
#pragma unroll 4
            for (int jj = 0; jj < n_valid; ++jj) {
                const long voff = __shfl_sync(0xffffffffu, row_off, jj);
                const T* vrow = v_pages + voff;
                float pj[G];
#pragma unroll
                for (int g = 0; g < G; ++g) pj[g] = __shfl_sync(0xffffffffu, pr[g], jj);
#pragma unroll
                for (int i = 0; i < NREG; ++i) {
                    const int d = lane + 32 * i;
                    if (d < hd) {
                        const float v = to_float(vrow[d]);
#pragma unroll
                        for (int g = 0; g < G; ++g) acc[g][i] = fmaf(pj[g], v, acc[g][i]);
                    }
                }
            }
        }
        __syncthreads();                                         // the part before has been folded
#pragma unroll
        for (int g = 0; g < G; ++g) {
            if (lane == 0) { m_s[g][warp] = m[g]; l_s[g][warp] = l[g]; }
#pragma unroll
            for (int i = 0; i < NREG; ++i) acc_s[g][warp][lane + 32 * i] = acc[g][i];
        }
        __syncthreads();
        // the four warps' results, merged in warp order: the part's (max, sum, weighted values)
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float big = -INFINITY;
#pragma unroll
            for (int w = 0; w < ATT_WARPS; ++w) big = fmaxf(big, m_s[g][w]);
            float wgt[ATT_WARPS];
            float lp = 0.f;
#pragma unroll
            for (int w = 0; w < ATT_WARPS; ++w) {
                wgt[w] = m_s[g][w] == -INFINITY ? 0.f : expf(m_s[g][w] - big);
                lp = __fmaf_rn(l_s[g][w], wgt[w], lp);
            }
            float a, bb, m_new;
            fold_weights(run_m[g], big, m_new, a, bb);
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int d = threadIdx.x + r * ATT_WARPS * 32;
                if (d < hd) {
                    float op = 0.f;
#pragma unroll
                    for (int w = 0; w < ATT_WARPS; ++w) op = __fmaf_rn(acc_s[g][w][d], wgt[w], op);
                    if (split) part_o[(((long)t * n_heads + h0 + g) * max_parts + part) * hd + d] = op;
                    else run_o[g][r] = fold_value(run_o[g][r], a, op, bb);
                }
            }
            if (split) {
                if (threadIdx.x == 0) {
                    float* ml = part_ml + (((long)t * n_heads + h0 + g) * max_parts + part) * 2;
                    ml[0] = big; ml[1] = lp;
                }
            } else {
                run_l[g] = fold_value(run_l[g], a, lp, bb);
                run_m[g] = m_new;
            }
        }
    }
    if (split) return;
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int d = threadIdx.x + r * ATT_WARPS * 32;
            if (d < hd) out[((long)t * n_heads + h0 + g) * hd + d] = from_float<T>(run_o[g][r] / run_l[g]);
        }
}

// grid (T, n_heads), 128 threads: folds the parts a split launch left in scratch memory, in ascending order.
template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_fold_kernel(T* __restrict__ out, int n_heads, int hd, int window, const int* __restrict__ positions,
                      const float* __restrict__ part_ml, const float* __restrict__ part_o, int max_parts) {
    const int t = blockIdx.x, h = blockIdx.y;
    const int pos = positions[t];
    const int start = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_parts = (pos - start + 1 + ATT_PART - 1) / ATT_PART;
    const float* ml = part_ml + ((long)t * n_heads + h) * max_parts * 2;
    const float* po = part_o + ((long)t * n_heads + h) * max_parts * hd;
    float run_m = -INFINITY, run_l = 0.f, run_o[2] = {0.f, 0.f};
    for (int part = 0; part < n_parts; ++part) {
        float a, bb, m_new;
        fold_weights(run_m, ml[2 * part], m_new, a, bb);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int d = threadIdx.x + r * ATT_WARPS * 32;
            if (d < hd) run_o[r] = fold_value(run_o[r], a, po[(long)part * hd + d], bb);
        }
        run_l = fold_value(run_l, a, ml[2 * part + 1], bb);
        run_m = m_new;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int d = threadIdx.x + r * ATT_WARPS * 32;
        if (d < hd) out[((long)t * n_heads + h) * hd + d] = from_float<T>(run_o[r] / run_l);
    }
}

template <typename T, int VEC, int G>
static int launch_attention(const void* q, long q_row_stride, void* out, int T_, int n_heads, int n_kv, int hd, float scale,
                            int window, const int* positions, const int* seq_of_token, const int* block_table,
                            int bt_stride, const void* k_pages, const void* v_pages, int page_size, long page_stride,
                            float* part_ml, float* part_o, int max_parts, cudaStream_t stream) {
    dim3 grid(T_, n_heads / G, part_o ? max_parts : 1);
    if (hd <= 128)
        attention_general_kernel<T, VEC, G, 4><<<grid, ATT_WARPS * 32, 0, stream>>>(
            (const T*)q, q_row_stride, (T*)out, n_heads, n_kv, hd, scale, window, positions, seq_of_token, block_table,
            bt_stride, (const T*)k_pages, (const T*)v_pages, page_size, page_stride, part_ml, part_o, max_parts);
    else
        attention_general_kernel<T, VEC, G, 8><<<grid, ATT_WARPS * 32, 0, stream>>>(
            (const T*)q, q_row_stride, (T*)out, n_heads, n_kv, hd, scale, window, positions, seq_of_token, block_table,
            bt_stride, (const T*)k_pages, (const T*)v_pages, page_size, page_stride, part_ml, part_o, max_parts);
    int rc = launch_status();
    if (rc || !part_o) return rc;
    attention_fold_kernel<T><<<dim3(T_, n_heads), ATT_WARPS * 32, 0, stream>>>((T*)out, n_heads, hd, window, positions,
                                                                           part_ml, part_o, max_parts);
    return launch_status();
}

template <typename T, int VEC>
static int pick_group(int group, const void* q, long q_row_stride, void* out, int T_, int n_heads, int n_kv, int hd,
                      float scale, int window, const int* positions, const int* seq_of_token, const int* block_table,
                      int bt_stride, const void* k_pages, const void* v_pages, int page_size, long page_stride,
                      float* part_ml, float* part_o, int max_parts, cudaStream_t stream) {
#define ZLM_ATT(GV)                                                                                                     \
    launch_attention<T, VEC, GV>(q, q_row_stride, out, T_, n_heads, n_kv, hd, scale, window, positions, seq_of_token,   \
                                 block_table, bt_stride, k_pages, v_pages, page_size, page_stride, part_ml, part_o,     \
                                 max_parts, stream)
    if (group % 4 == 0) return ZLM_ATT(4);
    if (group % 2 == 0) return ZLM_ATT(2);
    return ZLM_ATT(1);
#undef ZLM_ATT
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

// Floats of scratch memory that let zlm_attention_general spread a step of T tokens whose longest visible range
// is max_keys keys over more blocks (0: the step has enough tokens, or one part of keys).
ZLM_EXPORT long zlm_attention_general_scratch(int T, int n_heads, int n_kv, int hd, int max_keys) {
    if (T <= 0 || n_heads <= 0 || n_kv <= 0 || n_heads % n_kv) return 0;
    const int group = n_heads / n_kv, g = group % 4 == 0 ? 4 : (group % 2 == 0 ? 2 : 1);
    const long parts = (max_keys + ATT_PART - 1) / ATT_PART;
    if (parts <= 1 || (long)T * (n_heads / g) >= 2 * 148) return 0;
    return (long)T * n_heads * parts * (hd + 2);
}

// max_keys: the most keys any token of the step sees.  scratch (float, scratch_floats elements; may be null):
// when it holds at least zlm_attention_general_scratch(...) floats and that is not 0, the parts of the keys are
// computed by blocks of their own and folded by a second kernel; the result is bit for bit the same.
ZLM_EXPORT int zlm_attention_general(const void* q, long q_row_stride, void* out, int dtype, int T, int n_heads,
                                     int n_kv, int hd, float scale, int window, const int* positions,
                                     const int* seq_of_token, const int* block_table, int bt_stride,
                                     const void* k_pages, const void* v_pages, int page_size, long page_stride,
                                     int max_keys, float* scratch, long scratch_floats, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || page_size <= 0) return ZLM_ERR_BAD_ARG;
    if (hd <= 0 || hd > ATT_MAX_HD || hd % 8) return ZLM_ERR_UNSUPPORTED;
    float *part_ml = nullptr, *part_o = nullptr;
    int max_parts = 1;
    const long need = zlm_attention_general_scratch(T, n_heads, n_kv, hd, max_keys);
    if (need > 0 && scratch != nullptr && scratch_floats >= need) {
        max_parts = (max_keys + ATT_PART - 1) / ATT_PART;
        if (max_parts > 65535) return ZLM_ERR_UNSUPPORTED;
        part_o = scratch;
        part_ml = scratch + (long)T * n_heads * max_parts * hd;
    }
    const int group = n_heads / n_kv;
    if (dtype == ZLM_F32)
        return pick_group<float, 4>(group, q, q_row_stride, out, T, n_heads, n_kv, hd, scale, window, positions,
                                    seq_of_token, block_table, bt_stride, k_pages, v_pages, page_size, page_stride,
                                    part_ml, part_o, max_parts, stream);
    if (dtype == ZLM_BF16)
        return pick_group<__nv_bfloat16, 8>(group, q, q_row_stride, out, T, n_heads, n_kv, hd, scale, window, positions,
                                            seq_of_token, block_table, bt_stride, k_pages, v_pages, page_size,
                                            page_stride, part_ml, part_o, max_parts, stream);
    return ZLM_ERR_UNSUPPORTED;
}
