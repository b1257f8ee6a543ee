// Attention over the paged bf16 cache on the tensor cores, head sizes 64 and 128.
//
// Two kernels share one inner step.  A page of the cache (64 positions of one
// key/value head) is brought into shared memory by TMA with the 128-byte swizzle,
// through a ring of stages guarded by mbarriers (a producer warp issues the copies,
// four consumer warps compute).  The scores S = Q K^T and the sum O += P V are
// mma.sync m16n8k16 (bf16 in, float out) with ldmatrix reading the swizzled tiles;
// the softmax is the running-maximum form in float, in base 2 with the scale folded
// in.  The formulas are those of the plain kernel in attention.cu (the reference's
// src/model.zig:659-700): scores scaled after the dot product, keys [start, pos]
// visible, softmax with maximum subtraction, weighted sum of values; query head h
// reads key/value head h / (n_heads / n_kv_heads).
//
//   decode   one block per (split, kv head, token).  The rows of the tile are the
//            query heads that share the kv head (up to 16), so the keys and values
//            are read once for all of them.  The four warps take 16 keys each of
//            every page.  The key range of a long sequence is split over blocks;
//            each writes an unnormalised partial result (o, m, l) to scratch and a
//            second kernel merges the splits in order.
//   prefill  one block per (query tile of 64 tokens, head, sequence); each warp owns
//            16 query rows and walks the pages up to its last row's position.
//
// Probabilities are rounded to bf16 before they multiply the values, as the
// tensor-core instruction needs; everything else stays in float.
#include "common.cuh"
#include "tc_common.cuh"

#include <mutex>
#include <unordered_map>

namespace zlm {
using namespace tc;

constexpr int PAGE = 64;
constexpr int ATC_CONSUMERS = 4;
constexpr int ATC_THREADS = (ATC_CONSUMERS + 1) * 32;
constexpr int ERR_ATT_FULL = 11, ERR_ATT_EMPTY = 12;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x on the special function unit (flushes denormals; exact enough before rounding to bf16)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// A [64 keys x HD] tile is HD/64 boxes of 64 rows x 128 bytes, each stored with the
// 128-byte swizzle: the 16-byte chunk c of row r lies at chunk (c ^ (r & 7)).
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int key, int chunk) {
    return base + ((chunk >> 3) << 13) + (key << 7) + ((((chunk & 7) ^ (key & 7))) << 4);
}

template <int HD, int NSTAGES> struct AtcCfg {
    static constexpr int TILE_BYTES = PAGE * HD * 2;             // one page of keys (or values) of one head
    static constexpr int STAGES = NSTAGES;
    static constexpr int SMEM = 1024 + STAGES * 2 * TILE_BYTES + 256;
};
// decode streams the cache and wants many copies in flight; a prompt block is compute-bound and
// leaves room for several blocks per SM instead
template <int HD> using DecodeCfg = AtcCfg<HD, HD == 128 ? 4 : 6>;
template <int HD> using PrefillCfg = AtcCfg<HD, 2>;

// Query fragments of 16 rows straight from global memory: row pointers may differ per row.
template <int HD>
__device__ __forceinline__ void load_q_frags(uint32_t (&qf)[HD / 16][4], const __nv_bfloat16* row_lo,
                                             const __nv_bfloat16* row_hi, int tid4) {
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        const int c = ks * 16 + 2 * tid4;
        qf[ks][0] = row_lo ? *reinterpret_cast<const uint32_t*>(row_lo + c) : 0u;
        qf[ks][1] = row_hi ? *reinterpret_cast<const uint32_t*>(row_hi + c) : 0u;
        qf[ks][2] = row_lo ? *reinterpret_cast<const uint32_t*>(row_lo + c + 8) : 0u;
        qf[ks][3] = row_hi ? *reinterpret_cast<const uint32_t*>(row_hi + c + 8) : 0u;
    }
}

// One step of the running softmax for a warp's 16 rows over NT*8 keys of the page in shared memory.
//   key0        first key (row of the tile) this warp reads
//   gkey0       position in the sequence of that key
//   lim_lo/hi   last visible position of rows gid / gid+8;  start_lo/hi first visible one
//   FULL        every key of the step is visible to every row: no masks are evaluated
template <int HD, int NT, bool FULL>
__device__ __forceinline__ void page_step(const uint32_t (&qf)[HD / 16][4], uint32_t k_tile, uint32_t v_tile, int key0,
                                          int gkey0, int lim_lo, int lim_hi, int start_lo, int start_hi,
                                          float scale_log2, float (&m)[2], float (&l)[2], float (&o)[HD / 8][4],
                                          int lane) {
    const int gid = lane >> 2, tid4 = lane & 3, mi = lane >> 3, r8 = lane & 7;
    float s[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            uint32_t kf[4];
            ldsm_x4(kf, tile_addr(k_tile, key0 + np * 16 + ((mi >> 1) << 3) + r8, 2 * ks + (mi & 1)));
            mma_16816(s[2 * np], qf[ks], kf[0], kf[1]);
            mma_16816(s[2 * np + 1], qf[ks], kf[2], kf[3]);
        }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const bool hi = i >= 2;
            if (FULL) {
                s[nt][i] *= scale_log2;
            } else {
                const int key = gkey0 + nt * 8 + 2 * tid4 + (i & 1);
                const bool vis = key <= (hi ? lim_hi : lim_lo) && key >= (hi ? start_hi : start_lo);
                s[nt][i] = vis ? s[nt][i] * scale_log2 : -INFINITY;
            }
            mx[hi] = fmaxf(mx[hi], s[nt][i]);
        }
    }
    float corr[2], use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m[h], mx[h]);
        use[h] = m_new == -INFINITY ? 0.f : m_new;          // a row that has seen no key yet
        corr[h] = fast_exp2(m[h] - use[h]);                  // 2^(-inf) = 0 the first time
        m[h] = m_new;
        l[h] *= corr[h];
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            s[nt][i] = fast_exp2(s[nt][i] - use[i >> 1]);
            l[i >> 1] += s[nt][i];
        }
    }
    // the running maxima settle after a few pages; the accumulators are rescaled only when one moved
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            o[n][0] *= corr[0]; o[n][1] *= corr[0];
            o[n][2] *= corr[1]; o[n][3] *= corr[1];
        }
    }
#pragma unroll
    for (int kp = 0; kp < NT / 2; ++kp) {
        uint32_t pf[4];
        pf[0] = pack_bf16(s[2 * kp][0], s[2 * kp][1]);
        pf[1] = pack_bf16(s[2 * kp][2], s[2 * kp][3]);
        pf[2] = pack_bf16(s[2 * kp + 1][0], s[2 * kp + 1][1]);
        pf[3] = pack_bf16(s[2 * kp + 1][2], s[2 * kp + 1][3]);
#pragma unroll
        for (int j = 0; j < HD / 16; ++j) {
            uint32_t vf[4];
            ldsm_x4_trans(vf, tile_addr(v_tile, key0 + kp * 16 + ((mi & 1) << 3) + r8, 2 * j + (mi >> 1)));
            mma_16816(o[2 * j], pf, vf[0], vf[1]);
            mma_16816(o[2 * j + 1], pf, vf[2], vf[3]);
        }
    }
}

struct AtcCommon {
    const __nv_bfloat16* q;
    long q_row_stride;
    int n_heads, n_kv;
    float scale_log2;
    int window;
    const int* block_table;
    int bt_stride;
    int* err;
};

// The producer warp: copies the pages [page_lo, page_hi) of one kv head into the ring.
template <int HD, typename C>
__device__ __forceinline__ void produce_pages(const CUtensorMap* tk, const CUtensorMap* tv, const int* bt, int n_kv,
                                              int kvh, int page_lo, int page_hi, uint32_t k0, uint32_t v0,
                                              uint32_t full0, uint32_t empty0, volatile int* abort_flag, int* err) {
    int issued = 0;
    for (int p = page_lo; p < page_hi; ++p, ++issued) {
        const int s = issued % C::STAGES;
        const uint32_t ph = (issued / C::STAGES) & 1;
        if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_flag, err, ERR_ATT_EMPTY)) break;
        const int row = (bt[p] * n_kv + kvh) * PAGE;
        mbar_expect_tx(full0 + 8 * s, 2 * C::TILE_BYTES);
#pragma unroll
        for (int b = 0; b < HD / 64; ++b) {
            tma_load_2d(k0 + s * C::TILE_BYTES + b * 8192, tk, full0 + 8 * s, b * 64, row);
            tma_load_2d(v0 + s * C::TILE_BYTES + b * 8192, tv, full0 + 8 * s, b * 64, row);
        }
    }
    if (*abort_flag) {
        const int first = issued > C::STAGES ? issued - C::STAGES : 0;
        for (int i = first; i < issued; ++i) {
            bool landed = false;
            for (uint32_t n = 0; n < WAIT_POLLS && !landed; ++n)
                landed = mbar_try_wait(full0 + 8 * (i % C::STAGES), (i / C::STAGES) & 1);
            if (!landed && err) atomicCAS(err, 0, ERR_WAIT_DRAIN);
        }
    }
}

// ------------------------------------------------------------------- decode
template <int HD>
__global__ void __launch_bounds__(ATC_THREADS)
attn_decode_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v, AtcCommon a,
                   const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                   float* __restrict__ part_o, float* __restrict__ part_ml) {
    using C = DecodeCfg<HD>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t k0 = base, v0 = base + C::STAGES * C::TILE_BYTES;
    const uint32_t bar = v0 + C::STAGES * C::TILE_BYTES;
    const uint32_t full0 = bar, empty0 = bar + 8 * C::STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + (bar - base) + 16 * C::STAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_splits = gridDim.x, split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const int group = a.n_heads / a.n_kv;
    const int pos = positions[t];
    const int start = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    const int* bt = a.block_table + (long)seq_of_token[t] * a.bt_stride;
    const int first_page = start / PAGE, end_page = pos / PAGE + 1;
    const int per = (end_page - first_page + n_splits - 1) / n_splits;
    const int page_lo = first_page + split * per;
    const int page_hi = min(end_page, page_lo + per);

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, ATC_CONSUMERS);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();                      // the keys and values of this step are written by the kernel before

    const int gid = lane >> 2, tid4 = lane & 3;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.f;

    if (warp == ATC_CONSUMERS) {
        if (lane == 0)
            produce_pages<HD, C>(&tmap_k, &tmap_v, bt, a.n_kv, kvh, page_lo, page_hi, k0, v0, full0, empty0, abort_flag,
                              a.err);
        __syncwarp();
    } else {
        // rows of the tile: the query heads of this kv head (rows beyond the group are zero)
        const __nv_bfloat16* qrow = a.q + (long)t * a.q_row_stride + (long)kvh * group * HD;
        uint32_t qf[HD / 16][4];
        load_q_frags<HD>(qf, gid < group ? qrow + gid * HD : nullptr, gid + 8 < group ? qrow + (gid + 8) * HD : nullptr,
                         tid4);
        int it = 0;
        for (int p = page_lo; p < page_hi; ++p, ++it) {
            const int s = it % C::STAGES;
            if (!mbar_wait(full0 + 8 * s, (it / C::STAGES) & 1, abort_flag, a.err, ERR_ATT_FULL)) break;
            if (p * PAGE >= start && p * PAGE + PAGE - 1 <= pos)
                page_step<HD, 2, true>(qf, k0 + s * C::TILE_BYTES, v0 + s * C::TILE_BYTES, warp * 16, p * PAGE + warp * 16,
                                       pos, pos, start, start, a.scale_log2, m, l, o, lane);
            else
                page_step<HD, 2, false>(qf, k0 + s * C::TILE_BYTES, v0 + s * C::TILE_BYTES, warp * 16, p * PAGE + warp * 16,
                                        pos, pos, start, start, a.scale_log2, m, l, o, lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
            l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
        }
    }
    __syncthreads();            // every page has been consumed: the stage memory is free for the merge

    // merge the four warps (each saw a quarter of the keys), rows < group only
    float* mo = reinterpret_cast<float*>(smem);                       // [4][16][HD]
    float* mm = mo + ATC_CONSUMERS * 16 * HD;                          // [4][16]
    float* ml = mm + ATC_CONSUMERS * 16;                               // [4][16]
    if (warp < ATC_CONSUMERS) {
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            float* r0 = mo + ((warp * 16 + gid) * HD) + n * 8 + 2 * tid4;
            float* r1 = mo + ((warp * 16 + gid + 8) * HD) + n * 8 + 2 * tid4;
            r0[0] = o[n][0]; r0[1] = o[n][1];
            r1[0] = o[n][2]; r1[1] = o[n][3];
        }
        if (tid4 == 0) {
            mm[warp * 16 + gid] = m[0]; mm[warp * 16 + gid + 8] = m[1];
            ml[warp * 16 + gid] = l[0]; ml[warp * 16 + gid + 8] = l[1];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < group * HD; idx += blockDim.x) {
        const int r = idx / HD, d = idx - r * HD;
        float big = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATC_CONSUMERS; ++w) big = fmaxf(big, mm[w * 16 + r]);
        float acc = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < ATC_CONSUMERS; ++w) {
            const float mw = mm[w * 16 + r];
            const float wgt = mw == -INFINITY ? 0.f : exp2f(mw - big);
            acc += mo[(w * 16 + r) * HD + d] * wgt;
            den += ml[w * 16 + r] * wgt;
        }
        const long row = ((long)t * a.n_heads + kvh * group + r) * n_splits + split;
        part_o[row * HD + d] = acc;
        if (d == 0) { part_ml[row * 2] = big; part_ml[row * 2 + 1] = den; }
    }
}

// out[t, h, :] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M), splits in order.
template <int HD>
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  __nv_bfloat16* __restrict__ out, int n_splits) {
    pdl_launch_dependents();
    pdl_wait();
    const long row = blockIdx.x;                    // t * n_heads + h
    float big = -INFINITY;
    for (int s = 0; s < n_splits; ++s) big = fmaxf(big, part_ml[(row * n_splits + s) * 2]);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float acc = 0.f, den = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = part_ml[(row * n_splits + s) * 2];
            const float wgt = ms == -INFINITY ? 0.f : exp2f(ms - big);
            acc += part_o[(row * n_splits + s) * HD + d] * wgt;
            den += part_ml[(row * n_splits + s) * 2 + 1] * wgt;
        }
        out[row * HD + d] = __float2bfloat16_rn(acc / den);
    }
}

// ------------------------------------------------------------- decode, flat
// The same arithmetic with the work laid out flat.  The pages of all (token, kv head) items of the
// step form one sequence of length total; block c takes pages [c * chunk, (c + 1) * chunk) of it,
// chunk = ceil(total / blocks), whatever items they belong to.  The grid is one resident wave (two
// blocks per SM), so that every SM streams the same number of pages whether the batch holds one long
// sequence or many of unequal lengths.  The producer never drains at an item's end.  An item that one
// block reads whole is normalised and stored by that block.  Otherwise each block writes its piece
// (o, m, l) into slot (block + item), which grows along the walk, so blocks + items slots suffice, and
// counts itself on the item's counter; the block that arrives last merges the pieces in slot order and
// sets the counter back to zero.  No block waits for another.
//
// An item also has work that does not grow with its pages: its query rows are fetched and rotated, and its
// result is combined over the warps, written, counted and perhaps merged.  With many short sequences that
// work outweighs the pages, so the sequence that is divided is one of units: every item begins with
// item_cost(HD) empty units (about what its fixed work costs, in pages) followed by one unit per page.
// A block that holds many item starts thereby gets fewer pages.  Page k of item i is the unit
// V_i + item_cost + k, with V_i the units before the item; block c owns the units [c * chunk, (c + 1) * chunk).
constexpr int FLAT_MAX_TOKENS = 4096;
template <int HD> __host__ __device__ constexpr int item_cost() { return 256 / HD; }

// Two stages of 32 KB (four of 16 KB at head size 64): with more, only one of an SM's two blocks fits beside the
// block of the q|k|v product that runs before this kernel, and the second starts cold when that block leaves
// (measured: 3.85 against 3.90 ms a step at batch 8, 8.63 against 8.77 ms at batch 64).
template <int HD> using FlatCfg = AtcCfg<HD, HD == 128 ? 2 : 4>;

struct FlatSizes {
    int merge_floats;      // [4 warps][group][HD] + [4][16] + [4][16]
    int prefix_ints;       // T + 1
    int smem;
};
template <int HD>
static inline FlatSizes flat_sizes(int group, int T) {
    FlatSizes z;
    z.merge_floats = ATC_CONSUMERS * group * HD + 2 * ATC_CONSUMERS * 16;
    z.prefix_ints = T + 1;
    z.smem = 1024 + FlatCfg<HD>::STAGES * 2 * FlatCfg<HD>::TILE_BYTES + 256 + 4 * z.merge_floats + 4 * z.prefix_ints;
    return z;
}

__device__ __forceinline__ void bar_consumers() { asm volatile("bar.sync 1, %0;" ::"n"(ATC_CONSUMERS * 32) : "memory"); }

// Barrier of the consumer warps that also tells every one of them whether any passed true.
__device__ __forceinline__ bool bar_consumers_or(bool v) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred p, 1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r) : "r"((uint32_t)v), "n"(ATC_CONSUMERS * 32) : "memory");
    return r != 0;
}

// What the flat kernel does for the step's new token itself when the rotation and the cache write are
// not left to a kernel before it.  The rows of q are then [q heads | k heads | v heads] as the fused
// projection left them: the block rotates the query heads as it loads them, and the block that reads
// the page of a sequence's newest position rotates the new key, puts key and value into the page in
// shared memory and into the cache.  rot is a multiple of 32 (pairs (i, i + rot/2) stay in one thread).
struct FlatRope {
    int fused;                 // 0: q is rotated and the cache is complete
    int store;                 // this layer owns the cache: write the new key and value
    int rot;                   // rotated width (0: no rotation)
    const float* inv_freq;     // [rot / 2]
    __nv_bfloat16* k_pages;
    __nv_bfloat16* v_pages;
};

// Rotate the fragments of 16 query rows in registers: column c of a fragment pairs with c + rot/2,
// which lies HP = rot/32 fragments further in the same thread and the same register.
template <int HD, int HP>
__device__ __forceinline__ void rotate_q_frags_by(uint32_t (&qf)[HD / 16][4], const float* cs, const float* sn, int tid4) {
#pragma unroll
    for (int ks = 0; ks < HP; ++ks) {
#pragma unroll
        for (int slot = 0; slot < 4; ++slot) {
            const int c = ks * 16 + 2 * tid4 + (slot >= 2 ? 8 : 0);
            const float2 x = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&qf[ks][slot]));
            const float2 y = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&qf[ks + HP][slot]));
            const float c0 = cs[c], s0 = sn[c], c1 = cs[c + 1], s1 = sn[c + 1];
            qf[ks][slot] = pack_bf16(x.x * c0 - y.x * s0, x.y * c1 - y.y * s1);
            qf[ks + HP][slot] = pack_bf16(x.x * s0 + y.x * c0, x.y * s1 + y.y * c1);
        }
    }
}

template <int HD>
__device__ __forceinline__ void rotate_q_frags(uint32_t (&qf)[HD / 16][4], const float* cs, const float* sn, int half,
                                               int tid4) {
    switch (half / 16) {
        case 1: rotate_q_frags_by<HD, 1>(qf, cs, sn, tid4); break;
        case 2: rotate_q_frags_by<HD, 2>(qf, cs, sn, tid4); break;
        case 3: if constexpr (HD >= 96) rotate_q_frags_by<HD, 3>(qf, cs, sn, tid4); break;
        case 4: if constexpr (HD >= 128) rotate_q_frags_by<HD, 4>(qf, cs, sn, tid4); break;
        default: break;
    }
}

template <int HD>
__global__ void __launch_bounds__(ATC_THREADS, 2)
attn_decode_flat_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                        AtcCommon a, FlatRope rope, const int* __restrict__ positions,
                        const int* __restrict__ seq_of_token, int T, int* __restrict__ counters,
                        float* __restrict__ slots, __nv_bfloat16* __restrict__ out) {
    __shared__ float cs_s[HD / 2], sn_s[HD / 2];
    using C = FlatCfg<HD>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t k0 = base, v0 = base + C::STAGES * C::TILE_BYTES;
    const uint32_t bar = v0 + C::STAGES * C::TILE_BYTES;
    const uint32_t full0 = bar, empty0 = bar + 8 * C::STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + (bar - base) + 16 * C::STAGES);
    const int group = a.n_heads / a.n_kv;
    float* mo = reinterpret_cast<float*>(smem + (bar - base) + 256);           // [4][group][HD]
    float* mm = mo + ATC_CONSUMERS * group * HD;                                // [4][16]
    float* ml = mm + ATC_CONSUMERS * 16;                                        // [4][16]
    int* pre = reinterpret_cast<int*>(ml + ATC_CONSUMERS * 16);                 // [T + 1] pages before token t

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, ATC_CONSUMERS);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    // Positions and block tables are written by the host's copy before the step's first kernel, not by
    // the kernel before this one: they may be read before the wait below.
    for (int t = threadIdx.x; t < T; t += blockDim.x) {
        const int pos = positions[t];
        const int start = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
        pre[t + 1] = pos / PAGE + 1 - start / PAGE;
    }
    if (threadIdx.x == 0) pre[0] = 0;
    __syncthreads();
    if (warp == 0) {
        int carry = 0;
        for (int b0 = 0; b0 < T; b0 += 32) {
            int v = b0 + lane < T ? pre[b0 + lane + 1] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int u = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += u;
            }
            if (b0 + lane < T) pre[b0 + lane + 1] = v + carry;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();
    constexpr int IC = item_cost<HD>();
    const long total = ((long)pre[T] + (long)IC * T) * a.n_kv;         // units: pages and the items' fixed work
    const long chunk = max(1L, (total + gridDim.x - 1) / gridDim.x);
    const long g0 = (long)blockIdx.x * chunk, g1 = min(total, g0 + chunk);
    if (g0 >= total) return;
    // the token whose units hold g0: the last t with n_kv * (pre[t] + IC * t) <= g0
    int t0 = 0;
    {
        int lo = 0, hi = T - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (((long)pre[mid] + (long)IC * mid) * a.n_kv <= g0) lo = mid; else hi = mid - 1;
        }
        t0 = lo;
    }
    const int p0 = pre[t0 + 1] - pre[t0];
    const int rem0 = (int)(g0 - ((long)pre[t0] + (long)IC * t0) * a.n_kv);
    const int kvh0 = rem0 / (p0 + IC);
    const long v0_item = g0 - (rem0 - kvh0 * (p0 + IC));               // units before the item (t0, kvh0)

    if (warp == ATC_CONSUMERS) {
        // ---- producer: the whole warp fetches block-table entries, lane 0 issues the copies
        // Only the page that holds a sequence's newest position was written by the kernel before this one
        // (the step's keys and values); every other page is older than the step and is requested at once.
        int t = t0, kvh = kvh0, issued = 0;
        long vi = v0_item;
        bool alive = true;
        bool waited = rope.fused && rope.store;      // the newest key and value are put in by this kernel itself
        while (vi < g1 && t < T && alive) {
            const int p_t = pre[t + 1] - pre[t];
            // this block's pages of the item: the units [g0, g1) that fall on pages
            const int j = (int)min((long)p_t, max(0L, g0 - vi - IC));
            const int seg = (int)min((long)p_t, max(0L, g1 - vi - IC)) - j;
            vi += p_t + IC;
            if (seg <= 0) {
                if (++kvh == a.n_kv) { kvh = 0; ++t; }
                continue;
            }
            const int pos = positions[t];
            const int start = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
            const int* bt = a.block_table + (long)seq_of_token[t] * a.bt_stride + start / PAGE + j;
            const int i_new = p_t - 1 - j;               // index within this run of the page of position pos
            for (int i0 = 0; i0 < seg && alive; i0 += 32) {
                const int mine = i0 + lane < seg ? bt[i0 + lane] : 0;
                const int n = min(32, seg - i0);
                for (int i = 0; i < n; ++i, ++issued) {
                    const int page = __shfl_sync(0xffffffffu, mine, i);
                    int ok = 1;
                    if (lane == 0) {
                        const int s = issued % C::STAGES;
                        const uint32_t ph = (issued / C::STAGES) & 1;
                        ok = mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_flag, a.err, ERR_ATT_EMPTY) ? 1 : 0;
                        if (ok) {
                            if (!waited && i0 + i == i_new) { pdl_wait(); waited = true; }
                            const int row = (page * a.n_kv + kvh) * PAGE;
                            mbar_expect_tx(full0 + 8 * s, 2 * C::TILE_BYTES);
#pragma unroll
                            for (int b = 0; b < HD / 64; ++b) {
                                tma_load_2d(k0 + s * C::TILE_BYTES + b * 8192, &tmap_k, full0 + 8 * s, b * 64, row);
                                tma_load_2d(v0 + s * C::TILE_BYTES + b * 8192, &tmap_v, full0 + 8 * s, b * 64, row);
                            }
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) { alive = false; break; }
                }
            }
            if (++kvh == a.n_kv) { kvh = 0; ++t; }
        }
        if (lane == 0 && *abort_flag) {
            const int first = issued > C::STAGES ? issued - C::STAGES : 0;
            for (int i = first; i < issued; ++i) {
                bool landed = false;
                for (uint32_t n = 0; n < WAIT_POLLS && !landed; ++n)
                    landed = mbar_try_wait(full0 + 8 * (i % C::STAGES), (i / C::STAGES) & 1);
                if (!landed && a.err) atomicCAS(a.err, 0, ERR_WAIT_DRAIN);
            }
        }
        return;
    }

    // ---- consumers
    pdl_wait();
    const int gid = lane >> 2, tid4 = lane & 3;
    // a slot: [group][HD] sums, then [group][2] (maximum, denominator); slots start on 16-byte boundaries
    const long slot_floats = ((long)group * (HD + 2) + 3) / 4 * 4;
    const int half = rope.fused ? rope.rot / 2 : 0;
    int t = t0, kvh = kvh0, it = 0, t_angles = -1;
    long vi = v0_item;
    for (bool first_item = true; ; first_item = false) {
        if (!first_item && ++kvh == a.n_kv) { kvh = 0; ++t; }
        if (vi >= g1 || t >= T) break;
        const int p_t = pre[t + 1] - pre[t];
        const int j = (int)min((long)p_t, max(0L, g0 - vi - IC));
        const int seg = (int)min((long)p_t, max(0L, g1 - vi - IC)) - j;
        const long s_i = vi + IC;                                      // the unit of the item's first page
        vi += p_t + IC;
        if (seg <= 0) continue;
        const int pos = positions[t];
        const int start = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
        const int first_page = start / PAGE;
        if (half > 0 && t != t_angles) {
            // cosines and sines of this token's position (float32 angles, as the separate kernel forms them)
            if (t_angles >= 0) bar_consumers();
            for (int i = threadIdx.x; i < half; i += ATC_CONSUMERS * 32)
                sincosf((float)pos * rope.inv_freq[i], &sn_s[i], &cs_s[i]);
            bar_consumers();
            t_angles = t;
        }
        const __nv_bfloat16* qrow = a.q + (long)t * a.q_row_stride + (long)kvh * group * HD;
        uint32_t qf[HD / 16][4];
        load_q_frags<HD>(qf, gid < group ? qrow + gid * HD : nullptr, gid + 8 < group ? qrow + (gid + 8) * HD : nullptr,
                         tid4);
        if (half > 0) rotate_q_frags<HD>(qf, cs_s, sn_s, half, tid4);
        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        float o[HD / 8][4];
#pragma unroll
        for (int n = 0; n < HD / 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
        for (int i = 0; i < seg; ++i, ++it) {
            const int s = it % C::STAGES;
            bool landed = mbar_wait(full0 + 8 * s, (it / C::STAGES) & 1, abort_flag, a.err, ERR_ATT_FULL);
            const int p = first_page + j + i;
            if (rope.fused && rope.store && j + i == p_t - 1) {
                // The page of position pos: its row pos % 64 is not in the cache yet.  The new key (rotated)
                // and value go into the page in shared memory and into the cache, then everybody reads.
                landed = !bar_consumers_or(!landed);
                if (landed) {
                    const int r = pos % PAGE;
                    const __nv_bfloat16* knew = a.q + (long)t * a.q_row_stride + (long)(a.n_heads + kvh) * HD;
                    const __nv_bfloat16* vnew = knew + (long)a.n_kv * HD;
                    const long crow = ((long)a.block_table[(long)seq_of_token[t] * a.bt_stride + p] * a.n_kv + kvh) * PAGE + r;
                    __nv_bfloat16* kdst = rope.k_pages + crow * HD;
                    __nv_bfloat16* vdst = rope.v_pages + crow * HD;
                    uint8_t* ktile = smem + (k0 + s * C::TILE_BYTES - base);
                    uint8_t* vtile = smem + (v0 + s * C::TILE_BYTES - base);
                    for (int d = threadIdx.x; d < HD; d += ATC_CONSUMERS * 32) {
                        __nv_bfloat16 kv;
                        if (d < 2 * half) {
                            const int ii = d < half ? d : d - half;
                            const float x = __bfloat162float(knew[ii]), y = __bfloat162float(knew[ii + half]);
                            kv = __float2bfloat16_rn(d < half ? x * cs_s[ii] - y * sn_s[ii] : x * sn_s[ii] + y * cs_s[ii]);
                        } else {
                            kv = knew[d];
                        }
                        const __nv_bfloat16 vv = vnew[d];
                        const uint32_t off = tile_addr(0u, r, d >> 3) + (d & 7) * 2;
                        *reinterpret_cast<__nv_bfloat16*>(ktile + off) = kv;
                        *reinterpret_cast<__nv_bfloat16*>(vtile + off) = vv;
                        kdst[d] = kv;
                        vdst[d] = vv;
                    }
                }
                bar_consumers();
            }
            if (!landed) break;
            if (p * PAGE >= start && p * PAGE + PAGE - 1 <= pos)
                page_step<HD, 2, true>(qf, k0 + s * C::TILE_BYTES, v0 + s * C::TILE_BYTES, warp * 16, p * PAGE + warp * 16,
                                       pos, pos, start, start, a.scale_log2, m, l, o, lane);
            else
                page_step<HD, 2, false>(qf, k0 + s * C::TILE_BYTES, v0 + s * C::TILE_BYTES, warp * 16, p * PAGE + warp * 16,
                                        pos, pos, start, start, a.scale_log2, m, l, o, lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
            l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
        }
        // the four warps each saw a quarter of the keys of every page: through shared memory, rows < group only
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) {
            const int d = n * 8 + 2 * tid4;
            if (gid < group) { float* r0 = mo + (warp * group + gid) * HD + d; r0[0] = o[n][0]; r0[1] = o[n][1]; }
            if (gid + 8 < group) { float* r1 = mo + (warp * group + gid + 8) * HD + d; r1[0] = o[n][2]; r1[1] = o[n][3]; }
        }
        if (tid4 == 0) {
            mm[warp * 16 + gid] = m[0]; mm[warp * 16 + gid + 8] = m[1];
            ml[warp * 16 + gid] = l[0]; ml[warp * 16 + gid + 8] = l[1];
        }
        const bool dead = bar_consumers_or(*abort_flag != 0);          // the same answer in every warp
        const int item = t * a.n_kv + kvh;
        const int first_block = (int)(s_i / chunk);
        const int pieces = (int)((s_i + p_t - 1) / chunk) - first_block + 1;
        __nv_bfloat16* orow = out + ((long)t * a.n_heads + (long)kvh * group) * HD;
        if (!dead) {
            float* slot = slots + (long)(blockIdx.x + item) * slot_floats;
            for (int idx = threadIdx.x; idx < group * HD; idx += ATC_CONSUMERS * 32) {
                const int r = idx / HD, d = idx - r * HD;
                float big = -INFINITY;
#pragma unroll
                for (int w = 0; w < ATC_CONSUMERS; ++w) big = fmaxf(big, mm[w * 16 + r]);
                float acc = 0.f, den = 0.f;
#pragma unroll
                for (int w = 0; w < ATC_CONSUMERS; ++w) {
                    const float mw = mm[w * 16 + r];
                    const float wgt = mw == -INFINITY ? 0.f : exp2f(mw - big);
                    acc += mo[(w * group + r) * HD + d] * wgt;
                    den += ml[w * 16 + r] * wgt;
                }
                if (pieces == 1) {
                    orow[r * HD + d] = __float2bfloat16_rn(acc / den);
                } else {
                    slot[idx] = acc;
                    if (d == 0) { slot[group * HD + 2 * r] = big; slot[group * HD + 2 * r + 1] = den; }
                }
            }
        }
        if (pieces > 1 && !dead) {
            bar_consumers();                       // the piece is written: thread 0 has seen every thread's part ...
            bool last = false;
            if (threadIdx.x == 0) {
                __threadfence();                   // ... and makes it visible to the GPU before it counts the piece
                last = atomicAdd(&counters[item], 1) == pieces - 1;
                if (last) counters[item] = 0;      // every piece has arrived: ready for the next call
            }
            last = bar_consumers_or(last);
            if (last) {
                __threadfence();
                const float* first = slots + (long)(first_block + item) * slot_floats;
                const long step = slot_floats;
                if (pieces <= 8) {
                    // The usual case, in one round of loads and without shared memory: a thread takes four
                    // neighbouring sums of a row and, with them, the (m, l) of that row from every piece.
                    for (int f = threadIdx.x; f < group * HD / 4; f += ATC_CONSUMERS * 32) {
                        const int r = f / (HD / 4);
                        float4 v[8];
                        float2 ml2[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            if (u < pieces) {
                                v[u] = __ldcg(reinterpret_cast<const float4*>(first + u * step) + f);
                                ml2[u] = __ldcg(reinterpret_cast<const float2*>(first + u * step + group * HD + 2 * r));
                            } else {
                                v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                                ml2[u] = make_float2(-INFINITY, 0.f);
                            }
                        }
                        float big = -INFINITY;
#pragma unroll
                        for (int u = 0; u < 8; ++u) big = fmaxf(big, ml2[u].x);
                        float den = 0.f;
                        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const float w = ml2[u].x == -INFINITY ? 0.f : exp2f(ml2[u].x - big);
                            den += ml2[u].y * w;
                            acc.x += v[u].x * w; acc.y += v[u].y * w; acc.z += v[u].z * w; acc.w += v[u].w * w;
                        }
                        const float inv = 1.f / den;
                        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
                        __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
                        uint2 packed;
                        packed.x = *reinterpret_cast<uint32_t*>(&lo);
                        packed.y = *reinterpret_cast<uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>(orow + 4 * f) = packed;
                    }
                } else if (pieces <= 2 * HD) {
                    // (m, l) of every piece in one round of loads, turned into weights 2^(m - M) / L in place
                    float* wm = mo;                                    // [group][pieces]
                    float* wl = mo + group * pieces;
                    for (int i = threadIdx.x; i < group * pieces; i += ATC_CONSUMERS * 32) {
                        const int r = i / pieces, sidx = i - r * pieces;
                        const float2 v = __ldcg(reinterpret_cast<const float2*>(first + sidx * step + group * HD + 2 * r));
                        wm[i] = v.x;
                        wl[i] = v.y;
                    }
                    bar_consumers();
                    if (threadIdx.x < group) {
                        const int r = threadIdx.x;
                        float big = -INFINITY, den = 0.f;
                        for (int sidx = 0; sidx < pieces; ++sidx) big = fmaxf(big, wm[r * pieces + sidx]);
                        for (int sidx = 0; sidx < pieces; ++sidx) {
                            const float mv = wm[r * pieces + sidx];
                            den += mv == -INFINITY ? 0.f : wl[r * pieces + sidx] * exp2f(mv - big);
                        }
                        mm[r] = big;
                        ml[r] = 1.f / den;
                    }
                    bar_consumers();
                    for (int i = threadIdx.x; i < group * pieces; i += ATC_CONSUMERS * 32) {
                        const int r = i / pieces;
                        const float mv = wm[i];
                        wm[i] = mv == -INFINITY ? 0.f : exp2f(mv - mm[r]) * ml[r];
                    }
                    bar_consumers();
                    // four neighbouring sums of a row per load, eight pieces in flight
                    for (int f = threadIdx.x; f < group * HD / 4; f += ATC_CONSUMERS * 32) {
                        const int r = f / (HD / 4);
                        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                        for (int s0 = 0; s0 < pieces; s0 += 8) {
                            float4 v[8];
#pragma unroll
                            for (int u = 0; u < 8; ++u)
                                v[u] = s0 + u < pieces ? __ldcg(reinterpret_cast<const float4*>(first + (s0 + u) * step) + f)
                                                       : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const float w = s0 + u < pieces ? wm[r * pieces + s0 + u] : 0.f;
                                acc.x += v[u].x * w; acc.y += v[u].y * w; acc.z += v[u].z * w; acc.w += v[u].w * w;
                            }
                        }
                        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
                        uint2 packed;
                        packed.x = *reinterpret_cast<uint32_t*>(&lo);
                        packed.y = *reinterpret_cast<uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>(orow + 4 * f) = packed;
                    }
                } else {
                    // more pieces than the merge area holds weights for: straight from global memory
                    for (int idx = threadIdx.x; idx < group * HD; idx += ATC_CONSUMERS * 32) {
                        const int r = idx / HD, d = idx - r * HD;
                        const float* ml_r = first + group * HD + 2 * r;
                        float big = -INFINITY;
                        for (int sidx = 0; sidx < pieces; ++sidx) big = fmaxf(big, __ldcg(ml_r + sidx * step));
                        float acc = 0.f, den = 0.f;
                        for (int sidx = 0; sidx < pieces; ++sidx) {
                            const float mv = __ldcg(ml_r + sidx * step);
                            const float wgt = mv == -INFINITY ? 0.f : exp2f(mv - big);
                            acc += __ldcg(first + sidx * step + idx) * wgt;
                            den += __ldcg(ml_r + sidx * step + 1) * wgt;
                        }
                        orow[r * HD + d] = __float2bfloat16_rn(acc / den);
                    }
                }
            }
        }
        bar_consumers();                           // the merge area is free for the next item
        if (dead) break;
    }
}

// ------------------------------------------------------------------ prefill
template <int HD>
__global__ void __launch_bounds__(ATC_THREADS, 2)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v, AtcCommon a,
                    const int* __restrict__ cu_seqlens, const int* __restrict__ past_lens,
                    __nv_bfloat16* __restrict__ out) {
    using C = PrefillCfg<HD>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t k0 = base, v0 = base + C::STAGES * C::TILE_BYTES;
    const uint32_t bar = v0 + C::STAGES * C::TILE_BYTES;
    const uint32_t full0 = bar, empty0 = bar + 8 * C::STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + (bar - base) + 16 * C::STAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y;
    const int tok_begin = cu_seqlens[b], n_new = cu_seqlens[b + 1] - tok_begin;
    // the last query tiles see the most keys: give them the lowest block indices
    const int q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * 64;
    if (q0 >= n_new) return;
    const int past = past_lens[b];
    const int kvh = h / (a.n_heads / a.n_kv);
    const int* bt = a.block_table + (long)b * a.bt_stride;
    const int rows_here = min(64, n_new - q0);
    const int pos_first = past + q0, pos_last = past + q0 + rows_here - 1;
    const int start_first = (a.window > 0 && pos_first - a.window + 1 > 0) ? pos_first - a.window + 1 : 0;
    const int page_lo = start_first / PAGE, page_hi = pos_last / PAGE + 1;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, ATC_CONSUMERS);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();

    if (warp == ATC_CONSUMERS) {
        if (lane == 0)
            produce_pages<HD, C>(&tmap_k, &tmap_v, bt, a.n_kv, kvh, page_lo, page_hi, k0, v0, full0, empty0, abort_flag,
                              a.err);
        return;
    }
    const int gid = lane >> 2, tid4 = lane & 3;
    const int r_lo = q0 + warp * 16 + gid, r_hi = r_lo + 8;          // rows within the sequence's new tokens
    const bool has_lo = r_lo < n_new, has_hi = r_hi < n_new;
    const __nv_bfloat16* qbase = a.q + (long)h * HD;
    uint32_t qf[HD / 16][4];
    load_q_frags<HD>(qf, has_lo ? qbase + (long)(tok_begin + r_lo) * a.q_row_stride : nullptr,
                     has_hi ? qbase + (long)(tok_begin + r_hi) * a.q_row_stride : nullptr, tid4);
    const int lim_lo = has_lo ? past + r_lo : -1, lim_hi = has_hi ? past + r_hi : -1;
    const int st_lo = (a.window > 0 && lim_lo - a.window + 1 > 0) ? lim_lo - a.window + 1 : 0;
    const int st_hi = (a.window > 0 && lim_hi - a.window + 1 > 0) ? lim_hi - a.window + 1 : 0;
    // the warp's rows span positions [w_first, w_last]: pages wholly outside need no work
    const int w_first = past + q0 + warp * 16, w_last = min(pos_last, w_first + 15);
    const int w_start = (a.window > 0 && w_first - a.window + 1 > 0) ? w_first - a.window + 1 : 0;
    const int w_last_start = (a.window > 0 && w_last - a.window + 1 > 0) ? w_last - a.window + 1 : 0;
    const bool w_rows_all = w_first + 15 <= pos_last;        // all 16 rows of the warp are real tokens

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.f;

    int it = 0;
    for (int p = page_lo; p < page_hi; ++p, ++it) {
        const int s = it % C::STAGES;
        if (!mbar_wait(full0 + 8 * s, (it / C::STAGES) & 1, abort_flag, a.err, ERR_ATT_FULL)) break;
        const bool needed = w_first <= pos_last && p * PAGE <= w_last && p * PAGE + PAGE - 1 >= w_start;
        if (needed) {
            // a page every row of the warp sees whole needs no masks (rows beyond the sequence never store)
            const bool full = p * PAGE + PAGE - 1 <= w_first && p * PAGE >= w_last_start && w_rows_all;
            if (full)
                page_step<HD, 8, true>(qf, k0 + s * C::TILE_BYTES, v0 + s * C::TILE_BYTES, 0, p * PAGE, lim_lo, lim_hi,
                                       st_lo, st_hi, a.scale_log2, m, l, o, lane);
            else
                page_step<HD, 8, false>(qf, k0 + s * C::TILE_BYTES, v0 + s * C::TILE_BYTES, 0, p * PAGE, lim_lo, lim_hi,
                                        st_lo, st_hi, a.scale_log2, m, l, o, lane);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * s);
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 1);
        l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 2);
    }
    if (*abort_flag) return;
    const float inv_lo = has_lo ? 1.f / l[0] : 0.f, inv_hi = has_hi ? 1.f / l[1] : 0.f;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        const int d = n * 8 + 2 * tid4;
        if (has_lo)
            *reinterpret_cast<uint32_t*>(out + ((long)(tok_begin + r_lo) * a.n_heads + h) * HD + d) =
                pack_bf16(o[n][0] * inv_lo, o[n][1] * inv_lo);
        if (has_hi)
            *reinterpret_cast<uint32_t*>(out + ((long)(tok_begin + r_hi) * a.n_heads + h) * HD + d) =
                pack_bf16(o[n][2] * inv_hi, o[n][3] * inv_hi);
    }
}

// ------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// The pages of one layer as a matrix [n_pages * n_kv * 64, hd], read in boxes of 64 rows x 64 elements.
static int page_map(CUtensorMap* out, const void* ptr, long rows, int hd) {
    struct Key { const void* p; long rows; int hd; };
    static std::unordered_map<const void*, std::pair<Key, CUtensorMap>> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(ptr);
    if (it != cache.end() && it->second.first.rows == rows && it->second.first.hd == hd) {
        *out = it->second.second;
        return 0;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return ZLM_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)PAGE};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ZLM_ERR_BAD_ARG;
    if (cache.size() > 4096) cache.clear();
    cache[ptr] = {Key{ptr, rows, hd}, m};
    *out = m;
    return 0;
}

static int* att_error_word() {
    static int* word = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        if (cudaMalloc(&word, sizeof(int)) == cudaSuccess) cudaMemset(word, 0, sizeof(int));
        else word = nullptr;
    });
    return word;
}

template <typename Kern>
static int set_smem(Kern kern, int bytes, bool* done) {
    if (*done) return 0;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return (int)e;
    // ask for the largest shared-memory carve-out, so that several blocks fit an SM
    e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return (int)e;
    *done = true;
    return 0;
}

static int fill_common(AtcCommon* a, CUtensorMap* mk, CUtensorMap* mv, const void* q, long q_row_stride, int n_heads,
                       int n_kv, int hd, float scale, int window, const int* block_table, int bt_stride,
                       const void* k_pages, const void* v_pages, long n_pages, int page_size) {
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || page_size != PAGE) return ZLM_ERR_BAD_ARG;
    if (hd != 64 && hd != 128) return ZLM_ERR_UNSUPPORTED;
    if (((uintptr_t)q % 4) || (q_row_stride % 2) || ((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16))
        return ZLM_ERR_UNSUPPORTED;
    int rc = page_map(mk, k_pages, n_pages * n_kv * PAGE, hd);
    if (rc) return rc;
    rc = page_map(mv, v_pages, n_pages * n_kv * PAGE, hd);
    if (rc) return rc;
    a->q = (const __nv_bfloat16*)q;
    a->q_row_stride = q_row_stride;
    a->n_heads = n_heads;
    a->n_kv = n_kv;
    a->scale_log2 = scale * 1.4426950408889634f;
    a->window = window;
    a->block_table = block_table;
    a->bt_stride = bt_stride;
    a->err = att_error_word();
    return 0;
}

}  // namespace zlm

using namespace zlm;

// Decode-style attention: every token is a tile of its own (its query heads grouped by kv head).
// part_o: float [T * n_heads * n_splits * hd], part_ml: float [T * n_heads * n_splits * 2] (scratch).
ZLM_EXPORT int zlm_attention_decode(const void* q, long q_row_stride, void* out, int T, int n_heads, int n_kv, int hd,
                                    float scale, int window, const int* positions, const int* seq_of_token,
                                    const int* block_table, int bt_stride, const void* k_pages, const void* v_pages,
                                    long n_pages, int page_size, int n_splits, float* part_o, float* part_ml,
                                    cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n_splits < 1 || n_splits > 65535) return ZLM_ERR_BAD_ARG;
    if (n_kv > 0 && n_heads / n_kv > 16) return ZLM_ERR_UNSUPPORTED;
    AtcCommon a;
    CUtensorMap mk, mv;
    int rc = fill_common(&a, &mk, &mv, q, q_row_stride, n_heads, n_kv, hd, scale, window, block_table, bt_stride,
                         k_pages, v_pages, n_pages, page_size);
    if (rc) return rc;
    dim3 grid(n_splits, n_kv, T);
    using CFG128 = DecodeCfg<128>;
    using CFG64 = DecodeCfg<64>;
    if (hd == 128) {
        static bool done = false;
        rc = set_smem(attn_decode_kernel<128>, CFG128::SMEM, &done);
        if (rc) return rc;
        cudaError_t e = launch_pdl(attn_decode_kernel<128>, grid, dim3(ATC_THREADS), CFG128::SMEM, stream, mk, mv, a,
                                   positions, seq_of_token, part_o, part_ml);
        if (e == cudaSuccess)
            e = launch_pdl(attn_merge_kernel<128>, dim3(T * n_heads), dim3(128), 0, stream, (const float*)part_o,
                           (const float*)part_ml, (__nv_bfloat16*)out, n_splits);
        if (e != cudaSuccess) return (int)e;
    } else {
        static bool done = false;
        rc = set_smem(attn_decode_kernel<64>, CFG64::SMEM, &done);
        if (rc) return rc;
        cudaError_t e = launch_pdl(attn_decode_kernel<64>, grid, dim3(ATC_THREADS), CFG64::SMEM, stream, mk, mv, a,
                                   positions, seq_of_token, part_o, part_ml);
        if (e == cudaSuccess)
            e = launch_pdl(attn_merge_kernel<64>, dim3(T * n_heads), dim3(64), 0, stream, (const float*)part_o,
                           (const float*)part_ml, (__nv_bfloat16*)out, n_splits);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_status();
}

// Decode attention with the pages of the whole step divided evenly over one resident wave of blocks.
//   n_blocks  0: two blocks (or what fits) per SM; else that many blocks
//   scratch   floats for zlm_attention_decode_flat_scratch(...) of the same arguments
namespace zlm {
template <int HD>
static int flat_blocks(int group, int T, int* smem_out) {
    const FlatSizes z = flat_sizes<HD>(group, T);
    if (smem_out) *smem_out = z.smem;
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    static int max_dynamic = 0;
    if (max_dynamic == 0) {
        // the kernel's static shared memory counts against the same 227 KB
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, attn_decode_flat_kernel<HD>) != cudaSuccess) { cudaGetLastError(); return 0; }
        const int room = 227 * 1024 - (int)fa.sharedSizeBytes;
        if (cudaFuncSetAttribute(attn_decode_flat_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, room) !=
                cudaSuccess ||
            cudaFuncSetAttribute(attn_decode_flat_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared) != cudaSuccess) {
            cudaGetLastError();
            return 0;
        }
        max_dynamic = room;
    }
    if (z.smem > max_dynamic) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_flat_kernel<HD>, ATC_THREADS, z.smem) !=
        cudaSuccess) return 0;
    return sms * min(per_sm, 2);
}
}  // namespace zlm

ZLM_EXPORT int zlm_attention_decode_flat_blocks(int T, int n_heads, int n_kv, int hd) {
    if (T <= 0 || T > FLAT_MAX_TOKENS || n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || n_heads / n_kv > 16) return 0;
    if (hd == 128) return flat_blocks<128>(n_heads / n_kv, T, nullptr);
    if (hd == 64) return flat_blocks<64>(n_heads / n_kv, T, nullptr);
    return 0;
}

// Floats of piece storage the flat kernel needs with n_blocks blocks.  Beside it the caller keeps T * n_kv
// int counters that are zero before the first call; every call that completes leaves them zero.
ZLM_EXPORT long zlm_attention_decode_flat_scratch(int T, int n_heads, int n_kv, int hd, int n_blocks) {
    if (T <= 0 || n_kv <= 0 || n_heads <= 0 || n_blocks <= 0) return 0;
    const long slot = ((long)(n_heads / n_kv) * (hd + 2) + 3) / 4 * 4;
    return ((long)n_blocks + (long)T * n_kv) * slot;
}

ZLM_EXPORT int zlm_attention_decode_flat(const void* q, long q_row_stride, void* out, int T, int n_heads, int n_kv,
                                         int hd, float scale, int window, const int* positions,
                                         const int* seq_of_token, const int* block_table, int bt_stride,
                                         const void* k_pages, const void* v_pages, long n_pages, int page_size,
                                         int n_blocks, int* counters, float* scratch, long scratch_floats,
                                         int rope_fused, int rope_store, int rot, const float* inv_freq,
                                         cudaStream_t stream) {
    if (T <= 0) return 0;
    if (T > FLAT_MAX_TOKENS) return ZLM_ERR_UNSUPPORTED;
    if (n_kv > 0 && n_heads / n_kv > 16) return ZLM_ERR_UNSUPPORTED;
    if (rope_fused && (rot < 0 || rot > hd || rot % 32 || (rot > 0 && !inv_freq))) return ZLM_ERR_UNSUPPORTED;
    FlatRope rope;
    rope.fused = rope_fused ? 1 : 0;
    rope.store = rope_fused && rope_store ? 1 : 0;
    rope.rot = rope_fused ? rot : 0;
    rope.inv_freq = inv_freq;
    rope.k_pages = (__nv_bfloat16*)const_cast<void*>(k_pages);
    rope.v_pages = (__nv_bfloat16*)const_cast<void*>(v_pages);
    AtcCommon a;
    CUtensorMap mk, mv;
    int rc = fill_common(&a, &mk, &mv, q, q_row_stride, n_heads, n_kv, hd, scale, window, block_table, bt_stride,
                         k_pages, v_pages, n_pages, page_size);
    if (rc) return rc;
    const int group = n_heads / n_kv;
    int smem = 0;
    const int resident = hd == 128 ? flat_blocks<128>(group, T, &smem) : flat_blocks<64>(group, T, &smem);
    if (resident <= 0) return ZLM_ERR_UNSUPPORTED;
    if (n_blocks <= 0) n_blocks = resident;
    if (!counters || !scratch || zlm_attention_decode_flat_scratch(T, n_heads, n_kv, hd, n_blocks) > scratch_floats)
        return ZLM_ERR_BAD_ARG;
    cudaError_t e;
    if (hd == 128)
        e = launch_pdl(attn_decode_flat_kernel<128>, dim3(n_blocks), dim3(ATC_THREADS), (size_t)smem, stream, mk, mv, a,
                       rope, positions, seq_of_token, T, counters, scratch, (__nv_bfloat16*)out);
    else
        e = launch_pdl(attn_decode_flat_kernel<64>, dim3(n_blocks), dim3(ATC_THREADS), (size_t)smem, stream, mk, mv, a,
                       rope, positions, seq_of_token, T, counters, scratch, (__nv_bfloat16*)out);
    if (e != cudaSuccess) return (int)e;
    return launch_status();
}

// Prompt attention: B sequences with cu_seqlens[B+1] new tokens each after past_lens[b] cached ones.
ZLM_EXPORT int zlm_attention_prefill(const void* q, long q_row_stride, void* out, int B, int max_new, int n_heads,
                                     int n_kv, int hd, float scale, int window, const int* cu_seqlens,
                                     const int* past_lens, const int* block_table, int bt_stride, const void* k_pages,
                                     const void* v_pages, long n_pages, int page_size, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    AtcCommon a;
    CUtensorMap mk, mv;
    int rc = fill_common(&a, &mk, &mv, q, q_row_stride, n_heads, n_kv, hd, scale, window, block_table, bt_stride,
                         k_pages, v_pages, n_pages, page_size);
    if (rc) return rc;
    dim3 grid((max_new + 63) / 64, n_heads, B);
    if (grid.y > 65535 || grid.z > 65535) return ZLM_ERR_UNSUPPORTED;
    using CFG128 = PrefillCfg<128>;
    using CFG64 = PrefillCfg<64>;
    if (hd == 128) {
        static bool done = false;
        rc = set_smem(attn_prefill_kernel<128>, CFG128::SMEM, &done);
        if (rc) return rc;
        cudaError_t e = launch_pdl(attn_prefill_kernel<128>, grid, dim3(ATC_THREADS), CFG128::SMEM, stream, mk, mv, a,
                                   cu_seqlens, past_lens, (__nv_bfloat16*)out);
        if (e != cudaSuccess) return (int)e;
    } else {
        static bool done = false;
        rc = set_smem(attn_prefill_kernel<64>, CFG64::SMEM, &done);
        if (rc) return rc;
        cudaError_t e = launch_pdl(attn_prefill_kernel<64>, grid, dim3(ATC_THREADS), CFG64::SMEM, stream, mk, mv, a,
                                   cu_seqlens, past_lens, (__nv_bfloat16*)out);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_status();
}

ZLM_EXPORT int zlm_attention_tc_status(int* out) {
    int* w = att_error_word();
    if (!w) { *out = -1; return 0; }
    cudaError_t e = cudaMemcpy(out, w, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
    if (*out != 0) cudaMemset(w, 0, sizeof(int));
    return 0;
}

// Runs the give-up path of the bounded waits once, harmlessly (see wait_selftest_kernel): afterwards
// zlm_attention_tc_status returns 90.  seen: two ints on the device.
ZLM_EXPORT int zlm_attention_tc_wait_selftest(int polls, int* seen, cudaStream_t stream) {
    return tc::run_wait_selftest(att_error_word(), polls, seen, stream);
}

// ------------------------------------------------- decode attention that allocates nothing
// See attention_noalloc.h: the same kernels as zlm_attention_decode, with the split scratch and the
// error word in file-scope device arrays instead of memory the caller (or this library) allocates.
#include "attention_noalloc.h"

namespace zlm {

static __device__ __align__(256) float g_noalloc_scratch[ZLM_NOALLOC_SCRATCH_FLOATS];
static __device__ __align__(256) int g_noalloc_err[64];

struct NoAllocDevice {
    bool ready;
    bool smem_set[2];       // the shared-memory limit of the kernel for head size 64 / 128 has been raised
    float* scratch;
    int* err;
};
static NoAllocDevice g_noalloc_dev[64];
static std::mutex g_noalloc_mu;

// In host code the arrays' names are stand-ins, not device addresses: the address that kernels may use
// comes from cudaGetSymbolAddress, asked once per device with that device current.
static int noalloc_setup(float** scratch, int** err, int hd = 0) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return ZLM_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    NoAllocDevice& d = g_noalloc_dev[dev];
    if (!d.ready) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        d.scratch = static_cast<float*>(p);
        e = cudaGetSymbolAddress(&p, g_noalloc_err);
        if (e != cudaSuccess) return (int)e;
        d.err = static_cast<int*>(p);
        d.ready = true;
    }
    if (hd == 64 && !d.smem_set[0]) {
        e = cudaFuncSetAttribute(attn_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeCfg<64>::SMEM);
        if (e != cudaSuccess) return (int)e;
        d.smem_set[0] = true;
    }
    if (hd == 128 && !d.smem_set[1]) {
        e = cudaFuncSetAttribute(attn_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeCfg<128>::SMEM);
        if (e != cudaSuccess) return (int)e;
        d.smem_set[1] = true;
    }
    *scratch = d.scratch;
    *err = d.err;
    return 0;
}

}  // namespace zlm

ZLM_EXPORT int zlm_attention_decode_noalloc(const void* q, long q_row_stride, void* out, int T, int n_heads, int n_kv,
                                            int hd, float scale, int window, const int* positions,
                                            const int* seq_of_token, const int* block_table, int bt_stride,
                                            const void* k_pages, const void* v_pages, long n_pages, int page_size,
                                            int n_splits, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n_splits < 1 || n_splits > 65535) return ZLM_ERR_BAD_ARG;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || page_size != PAGE) return ZLM_ERR_BAD_ARG;
    if (hd != 64 && hd != 128) return ZLM_ERR_UNSUPPORTED;
    if (n_heads / n_kv > 16) return ZLM_ERR_UNSUPPORTED;
    if (((uintptr_t)q % 4) || (q_row_stride % 2) || ((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16))
        return ZLM_ERR_UNSUPPORTED;
    const long rows = (long)T * n_heads * n_splits;
    if (rows * (hd + 2) > (long)ZLM_NOALLOC_SCRATCH_FLOATS) return ZLM_NOALLOC_ERR_TOO_LARGE;
    float* scratch = nullptr;
    int* err = nullptr;
    int rc = noalloc_setup(&scratch, &err, hd);
    if (rc) return rc;
    float* part_o = scratch;                       // [rows, hd]
    float* part_ml = scratch + rows * hd;          // [rows, 2]
    CUtensorMap mk, mv;
    rc = page_map(&mk, k_pages, n_pages * n_kv * PAGE, hd);
    if (rc) return rc;
    rc = page_map(&mv, v_pages, n_pages * n_kv * PAGE, hd);
    if (rc) return rc;
    AtcCommon a;
    a.q = (const __nv_bfloat16*)q;
    a.q_row_stride = q_row_stride;
    a.n_heads = n_heads;
    a.n_kv = n_kv;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.window = window;
    a.block_table = block_table;
    a.bt_stride = bt_stride;
    a.err = err;
    dim3 grid(n_splits, n_kv, T);
    if (hd == 128) {
        attn_decode_kernel<128><<<grid, ATC_THREADS, DecodeCfg<128>::SMEM, stream>>>(mk, mv, a, positions,
                                                                                     seq_of_token, part_o, part_ml);
        attn_merge_kernel<128><<<T * n_heads, 128, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, n_splits);
    } else {
        attn_decode_kernel<64><<<grid, ATC_THREADS, DecodeCfg<64>::SMEM, stream>>>(mk, mv, a, positions, seq_of_token,
                                                                                   part_o, part_ml);
        attn_merge_kernel<64><<<T * n_heads, 64, 0, stream>>>(part_o, part_ml, (__nv_bfloat16*)out, n_splits);
    }
    return launch_status();
}

// The error word of this entry point's bounded waits (its own, in the library's device memory): *out receives
// 0 or the code of a wait that ran out since the last call, and the word is cleared.  Allocates nothing;
// synchronises the device.
ZLM_EXPORT int zlm_attention_decode_noalloc_status(int* out) {
    float* scratch = nullptr;
    int* err = nullptr;
    int rc = noalloc_setup(&scratch, &err);
    if (rc) return rc;
    cudaError_t e = cudaMemcpy(out, err, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
    if (*out != 0) e = cudaMemset(err, 0, sizeof(int));
    return e == cudaSuccess ? 0 : (int)e;
}

ZLM_EXPORT const char* zlm_attention_decode_noalloc_error(int code) {
    switch (code) {
        case 0: return "ok";
        case ZLM_ERR_BAD_ARG: return "bad argument (head counts, page size or number of splits)";
        case ZLM_ERR_UNSUPPORTED: return "unsupported size (head size 64 or 128, at most 16 query heads per kv head) "
                                         "or misaligned pointers";
        case ZLM_NOALLOC_ERR_TOO_LARGE:
            return "T * n_heads * n_splits * (head_dim + 2) exceeds the built-in scratch of 2 Mi floats; "
                   "use fewer splits or zlm_attention_decode with scratch of your own";
        default: return code > 0 ? "CUDA error (the code is a cudaError_t)" : "unknown code";
    }
}
