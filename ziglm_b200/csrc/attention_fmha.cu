// Prompt attention over the paged bf16 cache on the 5th-generation tensor cores (tcgen05), head sizes
// 64 and 128.
//
// One block per (tile of 128 queries, head, sequence).  The 128 query rows are the M side of both
// products, the accumulators live in tensor memory:
//   S = Q K^T   128 x 128 scores per step of two pages of 64 keys (two buffers, so the next step's
//               scores are computed while the softmax of this step runs),
//   O += P V    128 x head_dim.
// A tcgen05.mma with M = 128 reads its 128 x 16 A operand from shared memory in about 128 cycles
// whatever its N, so steps are as wide as tensor memory allows: N = 128 keys for the scores.
// Roles: warp 0 loads Q once and the K/V pages through a ring of stages with TMA (128-byte swizzle);
// warp 1 issues the tcgen05.mma instructions (K pages are K-major operands, V pages MN-major ones,
// both exactly as the cache stores them); warps 2-5 are the softmax: thread r owns query row r,
// reads its row of S with tcgen05.ld, keeps the running maximum and sum in float (base 2, scale
// folded in), writes the probabilities as bf16 into shared memory as the A operand of P V, and
// rescales O in tensor memory when its maximum has moved by more than 2^8 (a rescale that is
// skipped leaves probabilities up to 256, well inside bf16 and float range, and cancels in O / l).
// The formulas are those of attention.cu (the reference's src/model.zig:659-700): scores scaled
// after the dot product, keys [start, pos] visible, softmax with maximum subtraction, weighted sum.
// Every mbarrier wait is bounded and reports through an error word.
#include "common.cuh"
#include "tc_common.cuh"

#include <mutex>
#include <unordered_map>

namespace zlm {
using namespace tc;

constexpr int FM_BQ = 128;           // queries per block
constexpr int FM_PAGE = 64;          // keys per page
constexpr int FM_NP = 2;             // pages per step
constexpr int FM_KEYS = FM_PAGE * FM_NP;
constexpr int FM_THREADS = 192;      // TMA warp, MMA warp, four softmax warps
constexpr int ERR_FM_ALIGN = 20, ERR_FM_Q = 21, ERR_FM_KV = 22, ERR_FM_S = 23, ERR_FM_P = 24, ERR_FM_O = 25, ERR_FM_EMPTY = 26;

template <int HD> struct FmCfg {
    static constexpr int STAGES = 2;
    static constexpr int Q_BYTES = FM_BQ * HD * 2;
    static constexpr int PAGE_BYTES = FM_PAGE * HD * 2;          // one page of keys (or of values)
    static constexpr int KV_BYTES = FM_NP * PAGE_BYTES;          // the keys (or values) of one step
    static constexpr int P_BYTES = FM_BQ * FM_KEYS * 2;
    // The kernel checks that its shared memory starts on a 1024-byte boundary (the swizzled tiles need
    // it) and reports an error if it does not.
    static constexpr int SMEM = Q_BYTES + STAGES * 2 * KV_BYTES + P_BYTES + 128;
    static constexpr int S_COL = HD;                             // TMEM columns: O first, then two S buffers
    static constexpr int TMEM_COLS = HD + 2 * FM_KEYS <= 256 ? 256 : 512;
};

// One lane polls the barrier for its warp; 128 threads polling at once slow the barrier unit down.
__device__ __forceinline__ bool warp_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code,
                                               int lane) {
    int ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, err, code) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

struct FmArgs {
    __nv_bfloat16* out;
    int n_heads, n_kv;
    float scale_log2;
    int window;
    const int* block_table;
    int bt_stride;
    const int* cu_seqlens;
    const int* past_lens;
    int* err;
};

template <int HD>
__global__ void __launch_bounds__(FM_THREADS, 1)
fmha_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, FmArgs a) {
    using C = FmCfg<HD>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    uint8_t* smem = smem_raw;
    if (base & 1023u) {                                  // the swizzled tiles need this alignment
        if (threadIdx.x == 0 && a.err) atomicCAS(a.err, 0, ERR_FM_ALIGN);
        return;
    }
    const uint32_t q_smem = base;
    const uint32_t k_smem = q_smem + C::Q_BYTES;
    const uint32_t v_smem = k_smem + C::STAGES * C::KV_BYTES;
    const uint32_t p_smem = v_smem + C::STAGES * C::KV_BYTES;
    const uint32_t bar = p_smem + C::P_BYTES;
    // barriers
    const uint32_t q_full = bar;
    const uint32_t kv_full0 = bar + 8, kv_empty0 = kv_full0 + 8 * C::STAGES;
    const uint32_t s_full0 = kv_empty0 + 8 * C::STAGES, s_empty0 = s_full0 + 16;
    const uint32_t p_full = s_empty0 + 16, p_empty = p_full + 8;     // one P buffer: phase j belongs to page j
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + (p_empty + 8 - base));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, h = blockIdx.y;
    const int tok_begin = a.cu_seqlens[b], n_new = a.cu_seqlens[b + 1] - tok_begin;
    // the last query tiles see the most keys: give them the lowest block indices
    const int q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * FM_BQ;
    if (q0 >= n_new) return;
    const int past = a.past_lens[b];
    const int kvh = h / (a.n_heads / a.n_kv);
    const int* bt = a.block_table + (long)b * a.bt_stride;
    const int rows_here = min(FM_BQ, n_new - q0);
    const int pos_first = past + q0, pos_last = past + q0 + rows_here - 1;
    const int start_first = (a.window > 0 && pos_first - a.window + 1 > 0) ? pos_first - a.window + 1 : 0;
    const int page_lo = start_first / FM_PAGE, page_hi = pos_last / FM_PAGE + 1;
    const int n_pages = page_hi - page_lo;
    const int n_blocks = (n_pages + FM_NP - 1) / FM_NP;           // steps of two pages; the last may hold one

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_q);
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
        mbar_init(q_full, 1);
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(kv_full0 + 8 * s, 1);
            mbar_init(kv_empty0 + 8 * s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(s_full0 + 8 * i, 1);
            mbar_init(s_empty0 + 8 * i, 4);      // one arrival per softmax warp
        }
        mbar_init(p_full, 4);
        mbar_init(p_empty, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_holder), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    pdl_launch_dependents();
    pdl_wait();                       // queries, keys and values of this step are written by earlier kernels

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_expect_tx(q_full, C::Q_BYTES);
#pragma unroll
            for (int x = 0; x < HD / 64; ++x)
                tma_load_2d(q_smem + x * (FM_BQ * 128), &tmap_q, q_full, h * HD + x * 64, tok_begin + q0);
            int issued = 0;
            for (int j = 0; j < n_blocks; ++j, ++issued) {
                const int s = j % C::STAGES;
                if (!mbar_wait(kv_empty0 + 8 * s, ((j / C::STAGES) & 1) ^ 1u, abort_flag, a.err, ERR_FM_EMPTY)) break;
                const int np = min(FM_NP, n_pages - j * FM_NP);
                mbar_expect_tx(kv_full0 + 8 * s, np * 2 * C::PAGE_BYTES);
                for (int pg = 0; pg < np; ++pg) {
                    const int row = (bt[page_lo + j * FM_NP + pg] * a.n_kv + kvh) * FM_PAGE;
#pragma unroll
                    for (int x = 0; x < HD / 64; ++x) {
                        // keys: per 64-dim chunk the pages lie one after the other, so the step's keys are rows
                        // 0..127 of one K-major tile; values: page after page, each an MN-major tile of its own
                        tma_load_2d(k_smem + s * C::KV_BYTES + (x * FM_NP + pg) * (FM_PAGE * 128), &tmap_k,
                                    kv_full0 + 8 * s, x * 64, row);
                        tma_load_2d(v_smem + s * C::KV_BYTES + pg * C::PAGE_BYTES + x * (FM_PAGE * 128), &tmap_v,
                                    kv_full0 + 8 * s, x * 64, row);
                    }
                }
            }
            if (*abort_flag) {
                // let copies in flight land before the block gives up its shared memory
                for (uint32_t i = 0; i < WAIT_POLLS; ++i)
                    if (mbar_try_wait(q_full, 0)) break;
                const int first = issued > C::STAGES ? issued - C::STAGES : 0;
                for (int j = first; j < issued; ++j) {
                    bool landed = false;
                    for (uint32_t i = 0; i < WAIT_POLLS && !landed; ++i)
                        landed = mbar_try_wait(kv_full0 + 8 * (j % C::STAGES), (j / C::STAGES) & 1);
                    if (!landed && a.err) atomicCAS(a.err, 0, ERR_WAIT_DRAIN);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s2 = idesc_bf16(FM_BQ, FM_KEYS);         // S: 128 x 128 keys, K = head_dim
            constexpr uint32_t idesc_s1 = idesc_bf16(FM_BQ, FM_PAGE);         // a last step of one page
            constexpr uint32_t idesc_o = idesc_bf16_b_mn(FM_BQ, HD);          // O: 128 x head_dim, K = 16 keys
            const uint32_t tmem_o = tmem_base;
            bool alive = mbar_wait(q_full, 0, abort_flag, a.err, ERR_FM_Q);
            for (int j = 0; j <= n_blocks && alive; ++j) {
                if (j < n_blocks) {
                    // scores of page j into S buffer j & 1
                    const int s = j % C::STAGES, sb = j & 1;
                    if (!mbar_wait(kv_full0 + 8 * s, (j / C::STAGES) & 1, abort_flag, a.err, ERR_FM_KV)) break;
                    if (!mbar_wait(s_empty0 + 8 * sb, ((j >> 1) & 1) ^ 1u, abort_flag, a.err, ERR_FM_S)) break;
                    tc_fence_after_sync();
                    const uint32_t tmem_s = tmem_base + C::S_COL + sb * FM_KEYS;
                    const uint32_t idesc_s = n_pages - j * FM_NP >= FM_NP ? idesc_s2 : idesc_s1;
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ++ks) {
                        const uint64_t da = smem_desc_sw128(q_smem + (ks >> 2) * (FM_BQ * 128) + (ks & 3) * 32);
                        const uint64_t db = smem_desc_sw128(k_smem + s * C::KV_BYTES + (ks >> 2) * (FM_KEYS * 128) + (ks & 3) * 32);
                        umma_bf16(tmem_s, da, db, idesc_s, ks != 0 ? 1u : 0u);
                    }
                    umma_commit(s_full0 + 8 * sb);
                }
                if (j >= 1) {
                    // O += P V for page j - 1, once the softmax has written P
                    const int jj = j - 1, s = jj % C::STAGES;
                    if (!mbar_wait(p_full, jj & 1, abort_flag, a.err, ERR_FM_P)) break;
                    tc_fence_after_sync();
                    const int np = min(FM_NP, n_pages - jj * FM_NP);
                    for (int pg = 0; pg < np; ++pg) {
#pragma unroll
                        for (int ks = 0; ks < FM_PAGE / 16; ++ks) {
                            const uint64_t da = smem_desc_sw128(p_smem + pg * (FM_BQ * 128) + ks * 32);
                            const uint64_t db = smem_desc_sw128_mn(v_smem + s * C::KV_BYTES + pg * C::PAGE_BYTES + ks * 2048,
                                                                   FM_PAGE * 128);
                            umma_bf16(tmem_o, da, db, idesc_o, (jj | pg | ks) != 0 ? 1u : 0u);
                        }
                    }
                    umma_commit(kv_empty0 + 8 * s);      // the page's stage is free
                    umma_commit(p_empty);                // so is the P buffer, and O holds pages 0..jj
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- softmax
        const int q = warp & 3;
        const int r = q * 32 + lane;                                  // query row of this thread
        const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
        const bool real = q0 + r < n_new;
        // rows beyond the sequence's tokens compute like its last row and are never stored
        const int pos = real ? past + q0 + r : pos_last;
        const int start = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
        float m = -INFINITY, l = 0.f;
        bool alive = true;
        for (int j = 0; j < n_blocks; ++j) {
            const int sb = j & 1;
            alive = warp_mbar_wait(s_full0 + 8 * sb, (j >> 1) & 1, abort_flag, a.err, ERR_FM_S, lane);
            if (!alive) break;
            tc_fence_after_sync();
            const int np = min(FM_NP, n_pages - j * FM_NP);
            float sc[FM_KEYS];
#pragma unroll
            for (int c = 0; c < FM_KEYS / 32; ++c) {
                if (c * 32 < np * FM_PAGE) {
                    uint32_t v[32];
                    tmem_ld32(t_lane + C::S_COL + sb * FM_KEYS + c * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) sc[c * 32 + i] = __uint_as_float(v[i]);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) sc[c * 32 + i] = 0.f;     // a page that is not there: masked below
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_empty0 + 8 * sb);             // this S buffer may be overwritten
            const int key0 = (page_lo + j * FM_NP) * FM_PAGE;
            const int key_end = key0 + np * FM_PAGE - 1;               // last key this step really holds
            const bool full = np == FM_NP && key0 >= start && key_end <= pos;
            float mx = -INFINITY;
            if (full) {
#pragma unroll
                for (int i = 0; i < FM_KEYS; ++i) {
                    sc[i] *= a.scale_log2;
                    mx = fmaxf(mx, sc[i]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < FM_KEYS; ++i) {
                    const int key = key0 + i;
                    sc[i] = (key <= pos && key >= start && key <= key_end) ? sc[i] * a.scale_log2 : -INFINITY;
                    mx = fmaxf(mx, sc[i]);
                }
            }
            // the reference maximum moves only when the true one has grown by more than 8 (in base 2)
            float corr = 1.0f;
            if (mx > m + 8.0f) {
                corr = exp2f(m - mx);                                   // 0 the first time (m = -inf)
                m = mx;
            }
            const float use = m == -INFINITY ? 0.f : m;
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < FM_KEYS; ++i) {
                float p;
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(sc[i] - use));
                sc[i] = p;
                sum += p;
            }
            l = l * corr + sum;
            // Page j-1 must be in O, and its probabilities read, before O is rescaled or P overwritten.
            // The softmax waited for page j-2 one step ago, so the parity of this phase is unambiguous.
            if (j > 0) {
                alive = warp_mbar_wait(p_empty, (j - 1) & 1, abort_flag, a.err, ERR_FM_O, lane);
                if (!alive) break;
                tc_fence_after_sync();
            }
            // rescale O when some row of the warp moved its reference (never for the first page: O is empty)
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld32(t_lane + c * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
                    tmem_st32(t_lane + c * 32, v);
                }
                tmem_st_wait();
                tc_fence_before_sync();
            }
            // P as the A operand of the next product: per page a tile of 128 rows x 64 keys (128 bytes a
            // row, 8 chunks, swizzled)
            uint8_t* prow = smem + (p_smem - base) + r * 128;
#pragma unroll
            for (int c = 0; c < FM_KEYS / 8; ++c) {
                if (c * 8 >= np * FM_PAGE) break;
                uint4 pk;
                __nv_bfloat162 t0 = __floats2bfloat162_rn(sc[c * 8 + 0], sc[c * 8 + 1]);
                __nv_bfloat162 t1 = __floats2bfloat162_rn(sc[c * 8 + 2], sc[c * 8 + 3]);
                __nv_bfloat162 t2 = __floats2bfloat162_rn(sc[c * 8 + 4], sc[c * 8 + 5]);
                __nv_bfloat162 t3 = __floats2bfloat162_rn(sc[c * 8 + 6], sc[c * 8 + 7]);
                pk.x = *reinterpret_cast<uint32_t*>(&t0); pk.y = *reinterpret_cast<uint32_t*>(&t1);
                pk.z = *reinterpret_cast<uint32_t*>(&t2); pk.w = *reinterpret_cast<uint32_t*>(&t3);
                *reinterpret_cast<uint4*>(prow + (c >> 3) * (FM_BQ * 128) + (((c & 7) ^ (r & 7)) << 4)) = pk;
            }
            fence_proxy_async();                                       // visible to the tensor core's reads
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        // O holds every page: normalise and store this thread's row
        if (alive) {
            alive = warp_mbar_wait(p_empty, (n_blocks - 1) & 1, abort_flag, a.err, ERR_FM_O, lane);
        }
        if (alive) {
            tc_fence_after_sync();
            const float inv = 1.0f / l;
            __nv_bfloat16* orow = a.out + ((long)(tok_begin + q0 + r) * a.n_heads + h) * HD;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(t_lane + c * 32, v);
                tmem_ld_wait();
                if (real) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 pk;
                        __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(v[g * 8 + 0]) * inv, __uint_as_float(v[g * 8 + 1]) * inv);
                        __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(v[g * 8 + 2]) * inv, __uint_as_float(v[g * 8 + 3]) * inv);
                        __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(v[g * 8 + 4]) * inv, __uint_as_float(v[g * 8 + 5]) * inv);
                        __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(v[g * 8 + 6]) * inv, __uint_as_float(v[g * 8 + 7]) * inv);
                        pk.x = *reinterpret_cast<uint32_t*>(&t0); pk.y = *reinterpret_cast<uint32_t*>(&t1);
                        pk.z = *reinterpret_cast<uint32_t*>(&t2); pk.w = *reinterpret_cast<uint32_t*>(&t3);
                        *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = pk;
                    }
                }
            }
        }
        __syncwarp();
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn fm_encode_fn() {
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

// A bf16 matrix [rows, cols] with row stride ld, read in boxes of box_rows x 64 elements (128-byte swizzle).
static int fm_map(CUtensorMap* out, const void* ptr, long rows, long cols, long ld, int box_rows) {
    struct Key {
        const void* p; long rows, cols, ld; int box;
        bool operator==(const Key& o) const { return p == o.p && rows == o.rows && cols == o.cols && ld == o.ld && box == o.box; }
    };
    struct Hash {
        size_t operator()(const Key& k) const {
            size_t h = std::hash<const void*>()(k.p);
            h = h * 1000003u ^ (size_t)k.rows; h = h * 1000003u ^ (size_t)k.cols;
            h = h * 1000003u ^ (size_t)k.ld; h = h * 1000003u ^ (size_t)k.box;
            return h;
        }
    };
    static std::unordered_map<Key, CUtensorMap, Hash> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    Key k{ptr, rows, cols, ld, box_rows};
    auto it = cache.find(k);
    if (it == cache.end()) {
        EncodeTiledFn fn = fm_encode_fn();
        if (!fn) return ZLM_ERR_UNSUPPORTED;
        cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
        cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
        cuuint32_t estr[2] = {1, 1};
        CUtensorMap m;
        CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return ZLM_ERR_BAD_ARG;
        if (cache.size() > 16384) cache.clear();
        it = cache.emplace(k, m).first;
    }
    *out = it->second;
    return 0;
}

static int* fm_error_word() {
    static int* word = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        if (cudaMalloc(&word, sizeof(int)) == cudaSuccess) cudaMemset(word, 0, sizeof(int));
        else word = nullptr;
    });
    return word;
}

template <int HD>
static int fm_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FmArgs& a, dim3 grid,
                     cudaStream_t stream) {
    static bool done = false;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(fmha_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             FmCfg<HD>::SMEM);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(fmha_prefill_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    cudaError_t e = launch_pdl(fmha_prefill_kernel<HD>, grid, dim3(FM_THREADS), FmCfg<HD>::SMEM, stream, mq, mk, mv, a);
    return e == cudaSuccess ? launch_status() : (int)e;
}

}  // namespace zlm

using namespace zlm;

// Prompt attention: B sequences with cu_seqlens[B+1] new tokens each after past_lens[b] cached ones.
// q: bf16 [T, q_row_stride], the query heads first in each row; out: bf16 [T, n_heads * hd].
ZLM_EXPORT int zlm_attention_prefill_fmha(const void* q, long q_row_stride, long total_tokens, void* out, int B,
                                          int max_new, int n_heads, int n_kv, int hd, float scale, int window,
                                          const int* cu_seqlens, const int* past_lens, const int* block_table,
                                          int bt_stride, const void* k_pages, const void* v_pages, long n_pages,
                                          int page_size, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || page_size != FM_PAGE || total_tokens <= 0) return ZLM_ERR_BAD_ARG;
    if (hd != 64 && hd != 128) return ZLM_ERR_UNSUPPORTED;
    if (((uintptr_t)q % 16) || (q_row_stride % 8) || ((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16) ||
        ((uintptr_t)out % 16))
        return ZLM_ERR_UNSUPPORTED;
    dim3 grid((max_new + FM_BQ - 1) / FM_BQ, n_heads, B);
    if (grid.y > 65535 || grid.z > 65535) return ZLM_ERR_UNSUPPORTED;
    CUtensorMap mq, mk, mv;
    int rc = fm_map(&mq, q, total_tokens, (long)n_heads * hd, q_row_stride, FM_BQ);
    if (rc) return rc;
    rc = fm_map(&mk, k_pages, n_pages * n_kv * FM_PAGE, hd, hd, FM_PAGE);
    if (rc) return rc;
    rc = fm_map(&mv, v_pages, n_pages * n_kv * FM_PAGE, hd, hd, FM_PAGE);
    if (rc) return rc;
    FmArgs a;
    a.out = (__nv_bfloat16*)out;
    a.n_heads = n_heads;
    a.n_kv = n_kv;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.window = window;
    a.block_table = block_table;
    a.bt_stride = bt_stride;
    a.cu_seqlens = cu_seqlens;
    a.past_lens = past_lens;
    a.err = fm_error_word();
    return hd == 128 ? fm_launch<128>(mq, mk, mv, a, grid, stream) : fm_launch<64>(mq, mk, mv, a, grid, stream);
}

ZLM_EXPORT int zlm_attention_fmha_status(int* out) {
    int* w = fm_error_word();
    if (!w) { *out = -1; return 0; }
    cudaError_t e = cudaMemcpy(out, w, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
    if (*out != 0) cudaMemset(w, 0, sizeof(int));
    return 0;
}
