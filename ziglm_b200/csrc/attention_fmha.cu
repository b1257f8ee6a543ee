// Prompt attention over the paged bf16 cache on the 5th-generation tensor cores (tcgen05), head sizes
// 64 and 128.
//
// One block per (256 consecutive queries, head, sequence): two tiles of 128 query rows that share
// the K/V pages the block loads.  The 128 rows of a tile are the M side of both products and the
// accumulators live in tensor memory:
//   S_t = Q_t K^T    128 x 128 scores per step of two pages of 64 keys,
//   O_t += P_t V     128 x head_dim, with P_t (bf16) read from tensor memory, where it overwrites S_t.
// Roles: warp 0 loads Q once and the K and V pages through two rings of stages with TMA (128-byte
// swizzle; a K stage is free as soon as the scores are computed, a V stage after P V); warp 1 issues
// the tcgen05.mma instructions (K pages are K-major operands, V pages MN-major ones, both exactly as
// the cache stores them) in the order  P_0 V, S_0 of the next step, P_1 V, S_1 of the next step, so
// that the tensor core works for one tile while the softmax of the other runs; warps 2-5 are the
// softmax of tile 0 and warps 6-9 of tile 1: thread r owns query row r, reads its row of S with
// tcgen05.ld (all 128 scores issued together and waited for once; the row stays in registers between
// the maximum and the exponentials), keeps the running maximum and sum in float (base 2, scale folded
// in), writes the probabilities with tcgen05.st, and rescales O in tensor memory when its maximum has moved by more
// than 2^8 (a rescale that is skipped leaves probabilities up to 256, well inside bf16 and float
// range, and cancels in O / l).  The tensor core runs its instructions in the order of issue, so when
// S_t of a step is there, P_t V of the step before is complete: the softmax may touch O_t and
// overwrite the old probabilities without another wait.
// The formulas are those of attention.cu (the reference's src/model.zig:659-700): scores scaled
// after the dot product, keys [start, pos] visible, softmax with maximum subtraction, weighted sum.
// Every mbarrier wait is bounded and reports through an error word.
#include "common.cuh"
#include "tc_common.cuh"

#include <mutex>
#include <unordered_map>

namespace zlm {
using namespace tc;

constexpr int FM_BQ = 128;           // query rows of a tile
constexpr int FM_TILES = 2;          // tiles of a block
constexpr int FM_ROWS = FM_BQ * FM_TILES;
constexpr int FM_PAGE = 64;          // keys per page
constexpr int FM_NP = 2;             // pages per step
constexpr int FM_KEYS = FM_PAGE * FM_NP;
constexpr int FM_THREADS = 320;      // TMA warp, MMA warp, four softmax warps per tile
constexpr int ERR_FM_ALIGN = 20, ERR_FM_Q = 21, ERR_FM_KV = 22, ERR_FM_S = 23, ERR_FM_P = 24, ERR_FM_O = 25, ERR_FM_EMPTY = 26;

template <int HD> struct FmCfg {
    static constexpr int NK = 2, NV = 2;                         // stages of the K ring and of the V ring
    static constexpr int Q_BYTES = FM_BQ * HD * 2;               // one tile of queries
    static constexpr int PAGE_BYTES = FM_PAGE * HD * 2;          // one page of keys (or of values)
    static constexpr int KV_BYTES = FM_NP * PAGE_BYTES;          // the keys (or values) of one step
    // The kernel checks that its shared memory starts on a 1024-byte boundary (the swizzled tiles need
    // it) and reports an error if it does not.
    static constexpr int SMEM = FM_TILES * Q_BYTES + (NK + NV) * KV_BYTES + 256;
    static constexpr int O_COL = 0;                              // TMEM columns: O_0, O_1, then S_0, S_1
    static constexpr int S_COL = FM_TILES * HD;
    static constexpr int TMEM_COLS = 512;
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

// The softmax of one query row over a step of NP pages: S from tensor memory, P (bf16) back over its first
// half.  Returns the factor by which the running sum was rescaled; updates m (reference maximum, base 2) and l.
template <int HD, int NP>
__device__ __forceinline__ float softmax_row(uint32_t t_s, uint32_t t_o, bool full, int lo_vis, int hi_vis, float scale,
                                             float neg_big, int lt, float& m, float& l) {
    constexpr int N = NP * FM_PAGE;
    uint32_t v[N];
#pragma unroll
    for (int c = 0; c < N / 32; ++c) tmem_ld32(t_s + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
    tmem_ld_wait();
    float mx8[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) mx8[i] = neg_big;
    if (full) {
#pragma unroll
        for (int i = 0; i < N; ++i) mx8[i & 7] = fmaxf(mx8[i & 7], __uint_as_float(v[i]));
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) {
            if (i < lo_vis || i > hi_vis) v[i] = __float_as_uint(neg_big);      // stays masked below
            mx8[i & 7] = fmaxf(mx8[i & 7], __uint_as_float(v[i]));
        }
    }
    const float mx_raw = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])),
                               fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
    const float mx = mx_raw == neg_big ? -INFINITY : mx_raw * scale;       // the scale is positive
    // the reference maximum moves only when the true one has grown by more than 8 (in base 2)
    float corr = 1.0f;
    if (mx > m + 8.0f) {
        corr = exp2f(m - mx);                                   // 0 the first time (m = -inf)
        m = mx;
    }
    const float use = m == -INFINITY ? 0.f : m;
    // rescale O when some row of the warp moved its reference (never in the first step: O is empty)
    if (lt > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(t_o + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
            tmem_st32(t_o + c * 32, o);
        }
    }
    // stage by stage over the row: neighbouring instructions never depend on one another
    float sum8[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) sum8[i] = 0.f;
#pragma unroll
    for (int c = 0; c < N / 32; ++c) {
        float x[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = fmaf(__uint_as_float(v[c * 32 + i]), scale, -use);   // masked: about -3e38
#pragma unroll
        for (int i = 0; i < 32; ++i) asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(x[i]) : "f"(x[i]));
#pragma unroll
        for (int i = 0; i < 32; ++i) sum8[i & 7] += x[i];
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 pp = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
            pk[i] = *reinterpret_cast<uint32_t*>(&pp);
        }
        tmem_st16(t_s + c * 16, pk);
    }
    l = l * corr + (((sum8[0] + sum8[1]) + (sum8[2] + sum8[3])) + ((sum8[4] + sum8[5]) + (sum8[6] + sum8[7])));
    return corr;
}

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
    const uint32_t k_smem = q_smem + FM_TILES * C::Q_BYTES;
    const uint32_t v_smem = k_smem + C::NK * C::KV_BYTES;
    const uint32_t bar = v_smem + C::NV * C::KV_BYTES;
    // barriers
    const uint32_t q_full = bar;
    const uint32_t k_full0 = bar + 8, k_empty0 = k_full0 + 8 * C::NK;
    const uint32_t v_full0 = k_empty0 + 8 * C::NK, v_empty0 = v_full0 + 8 * C::NV;
    const uint32_t s_full0 = v_empty0 + 8 * C::NV;                   // [tile]: the scores of a step are there
    const uint32_t p_full0 = s_full0 + 8 * FM_TILES;                 // [tile]: the probabilities are written
    const uint32_t o_full0 = p_full0 + 8 * FM_TILES;                 // [tile]: the last P V is complete
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + (o_full0 + 8 * FM_TILES - base));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.y, h = blockIdx.x;
    const int tok_begin = a.cu_seqlens[b], n_new = a.cu_seqlens[b + 1] - tok_begin;
    // The last query tiles see the most keys.  Blocks start in the order of their indices (x fastest), so the
    // tile is the slowest index and counts down: the longest blocks of all heads and sequences start first and
    // the short ones fill the SMs' last gaps (at 2,048 tokens and 32 heads the step otherwise ends 13 tile-units
    // after it began instead of 8).  Heads are the fastest index: the heads of a kv group read the same pages
    // at about the same time.
    const int q0 = ((int)gridDim.z - 1 - (int)blockIdx.z) * FM_ROWS;
    if (q0 >= n_new) return;
    const int past = a.past_lens[b];
    const int kvh = h / (a.n_heads / a.n_kv);
    const int* bt = a.block_table + (long)b * a.bt_stride;
    // The two tiles: their rows, the positions they span and the pages those see.  Tile 0 always has rows;
    // tile 1 has none when the sequence ends inside tile 0.
    int rows_t[FM_TILES], pos_last_t[FM_TILES], step_lo[FM_TILES], step_hi[FM_TILES];
    int page_lo = 0, page_hi = 0;
#pragma unroll
    for (int t = 0; t < FM_TILES; ++t) {
        rows_t[t] = max(0, min(FM_BQ, n_new - q0 - t * FM_BQ));
        const int pf = past + q0 + t * FM_BQ;
        pos_last_t[t] = pf + max(rows_t[t], 1) - 1;
        const int sf = (a.window > 0 && pf - a.window + 1 > 0) ? pf - a.window + 1 : 0;
        const int plo = sf / FM_PAGE, phi = pos_last_t[t] / FM_PAGE + 1;
        if (t == 0) { page_lo = plo; page_hi = phi; }
        else if (rows_t[t] > 0) page_hi = phi;
        step_lo[t] = (plo - page_lo) / FM_NP;
        step_hi[t] = rows_t[t] > 0 ? (phi - page_lo + FM_NP - 1) / FM_NP : 0;
        if (rows_t[t] == 0) step_lo[t] = 0;
    }
    const int n_pages = page_hi - page_lo;
    const int n_steps = (n_pages + FM_NP - 1) / FM_NP;            // steps of two pages; the last may hold one

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_q);
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
        mbar_init(q_full, 1);
        for (int s = 0; s < C::NK; ++s) { mbar_init(k_full0 + 8 * s, 1); mbar_init(k_empty0 + 8 * s, 1); }
        for (int s = 0; s < C::NV; ++s) { mbar_init(v_full0 + 8 * s, 1); mbar_init(v_empty0 + 8 * s, 1); }
        for (int t = 0; t < FM_TILES; ++t) {
            mbar_init(s_full0 + 8 * t, 1);
            mbar_init(p_full0 + 8 * t, 4);       // one arrival per softmax warp of the tile
            mbar_init(o_full0 + 8 * t, 1);
        }
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
            // rows beyond the sequence's tokens are read all the same (another sequence's, or zeros past the
            // end of the matrix): they compute like real rows and are never stored
            mbar_expect_tx(q_full, FM_TILES * C::Q_BYTES);
#pragma unroll
            for (int t = 0; t < FM_TILES; ++t)
#pragma unroll
                for (int x = 0; x < HD / 64; ++x)
                    tma_load_2d(q_smem + t * C::Q_BYTES + x * (FM_BQ * 128), &tmap_q, q_full, h * HD + x * 64,
                                tok_begin + q0 + t * FM_BQ);
            int issued = 0;
            bool alive = true;
            for (int j = 0; j < n_steps && alive; ++j, ++issued) {
                const int np = min(FM_NP, n_pages - j * FM_NP);
                int rows[FM_NP];
                for (int pg = 0; pg < np; ++pg) rows[pg] = (bt[page_lo + j * FM_NP + pg] * a.n_kv + kvh) * FM_PAGE;
                // keys: per 64-dim chunk the pages lie one after the other, so the step's keys are rows 0..127 of
                // one K-major tile; values: page after page, each an MN-major tile of its own
                const int sk = j % C::NK;
                if (!mbar_wait(k_empty0 + 8 * sk, ((j / C::NK) & 1) ^ 1u, abort_flag, a.err, ERR_FM_EMPTY)) break;
                mbar_expect_tx(k_full0 + 8 * sk, np * C::PAGE_BYTES);
                for (int pg = 0; pg < np; ++pg)
#pragma unroll
                    for (int x = 0; x < HD / 64; ++x)
                        tma_load_2d(k_smem + sk * C::KV_BYTES + (x * FM_NP + pg) * (FM_PAGE * 128), &tmap_k,
                                    k_full0 + 8 * sk, x * 64, rows[pg]);
                const int sv = j % C::NV;
                if (!mbar_wait(v_empty0 + 8 * sv, ((j / C::NV) & 1) ^ 1u, abort_flag, a.err, ERR_FM_EMPTY)) {
                    alive = false;
                    ++issued;                         // the keys of this step are in flight
                    break;
                }
                mbar_expect_tx(v_full0 + 8 * sv, np * C::PAGE_BYTES);
                for (int pg = 0; pg < np; ++pg)
#pragma unroll
                    for (int x = 0; x < HD / 64; ++x)
                        tma_load_2d(v_smem + sv * C::KV_BYTES + pg * C::PAGE_BYTES + x * (FM_PAGE * 128), &tmap_v,
                                    v_full0 + 8 * sv, x * 64, rows[pg]);
            }
            if (*abort_flag) {
                // let copies in flight land before the block gives up its shared memory
                for (uint32_t i = 0; i < WAIT_POLLS; ++i)
                    if (mbar_try_wait(q_full, 0)) break;
                for (int ring = 0; ring < 2; ++ring) {
                    const int n = ring == 0 ? C::NK : C::NV;
                    const uint32_t full0 = ring == 0 ? k_full0 : v_full0;
                    const int first = issued > n ? issued - n : 0;
                    for (int j = first; j < issued; ++j) {
                        bool landed = false;
                        for (uint32_t i = 0; i < WAIT_POLLS && !landed; ++i)
                            landed = mbar_try_wait(full0 + 8 * (j % n), (j / n) & 1);
                    }
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
            bool alive = mbar_wait(q_full, 0, abort_flag, a.err, ERR_FM_Q);
            // step j: for each tile first P V of step j - 1, then the scores of step j
            for (int j = 0; j <= n_steps && alive; ++j) {
#pragma unroll
                for (int t = 0; t < FM_TILES; ++t) {
                    if (!alive) break;
                    const int jj = j - 1;
                    if (jj >= step_lo[t] && jj < step_hi[t]) {
                        const int sv = jj % C::NV, lt = jj - step_lo[t];
                        if (!mbar_wait(v_full0 + 8 * sv, (jj / C::NV) & 1, abort_flag, a.err, ERR_FM_KV) ||
                            !mbar_wait(p_full0 + 8 * t, lt & 1, abort_flag, a.err, ERR_FM_P)) {
                            alive = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const int np = min(FM_NP, n_pages - jj * FM_NP);
                        const uint32_t tmem_o = tmem_base + C::O_COL + t * HD;
                        const uint32_t tmem_p = tmem_base + C::S_COL + t * FM_KEYS;
                        for (int pg = 0; pg < np; ++pg) {
#pragma unroll
                            for (int ks = 0; ks < FM_PAGE / 16; ++ks) {
                                const uint64_t db = smem_desc_sw128_mn(
                                    v_smem + sv * C::KV_BYTES + pg * C::PAGE_BYTES + ks * 2048, FM_PAGE * 128);
                                umma_bf16_ts(tmem_o, tmem_p + pg * (FM_PAGE / 2) + ks * 8, db, idesc_o,
                                             (lt | pg | ks) != 0 ? 1u : 0u);
                            }
                        }
                        if (jj == step_hi[t] - 1) umma_commit(o_full0 + 8 * t);
                    }
                    if (j >= step_lo[t] && j < step_hi[t]) {
                        const int sk = j % C::NK;
                        if (!mbar_wait(k_full0 + 8 * sk, (j / C::NK) & 1, abort_flag, a.err, ERR_FM_KV)) {
                            alive = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t tmem_s = tmem_base + C::S_COL + t * FM_KEYS;
                        const uint32_t idesc_s = n_pages - j * FM_NP >= FM_NP ? idesc_s2 : idesc_s1;
#pragma unroll
                        for (int ks = 0; ks < HD / 16; ++ks) {
                            const uint64_t da = smem_desc_sw128(q_smem + t * C::Q_BYTES + (ks >> 2) * (FM_BQ * 128) + (ks & 3) * 32);
                            const uint64_t db = smem_desc_sw128(k_smem + sk * C::KV_BYTES + (ks >> 2) * (FM_KEYS * 128) + (ks & 3) * 32);
                            umma_bf16(tmem_s, da, db, idesc_s, ks != 0 ? 1u : 0u);
                        }
                        umma_commit(s_full0 + 8 * t);
                    }
                }
                if (!alive) break;
                // both tiles have issued what they read of these stages
                if (j >= 1) umma_commit(v_empty0 + 8 * ((j - 1) % C::NV));
                if (j < n_steps) umma_commit(k_empty0 + 8 * (j % C::NK));
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- softmax
        const int t = (warp - 2) >> 2;                                // tile of this warp
        const int q = warp & 3;                                       // TMEM lane quarter this warp may touch
        const int r = q * 32 + lane;                                  // query row of this thread within the tile
        const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
        const uint32_t t_s = t_lane + C::S_COL + t * FM_KEYS;
        const uint32_t t_o = t_lane + C::O_COL + t * HD;
        const bool real = r < rows_t[t];
        // rows beyond the sequence's tokens compute like its last row and are never stored
        const int pos = real ? past + q0 + t * FM_BQ + r : pos_last_t[t];
        const int start = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
        const float scale = a.scale_log2;
        const float neg_big = -3.0e38f;                               // stands for a masked score before scaling
        float m = -INFINITY, l = 0.f;
        bool alive = true;
        for (int j = step_lo[t]; j < step_hi[t]; ++j) {
            const int lt = j - step_lo[t];
            alive = warp_mbar_wait(s_full0 + 8 * t, lt & 1, abort_flag, a.err, ERR_FM_S, lane);
            if (!alive) break;
            tc_fence_after_sync();
            const int np = min(FM_NP, n_pages - j * FM_NP);
            const int key0 = (page_lo + j * FM_NP) * FM_PAGE;
            const int key_end = key0 + np * FM_PAGE - 1;               // last key this step really holds
            const bool full = key0 >= start && key_end <= pos;
            const int lo_vis = max(start, key0) - key0, hi_vis = min(pos, key_end) - key0;   // visible keys [lo, hi]
            // One reading of the row: the loads of all its scores are issued together and waited for once
            // (a tcgen05.ld and its wait cost about as much as the arithmetic on 32 scores), the row stays in
            // registers between the maximum and the exponentials, and the stores of P are waited for once.
            float corr;
            if (np == FM_NP)
                corr = softmax_row<HD, FM_NP>(t_s, t_o, full, lo_vis, hi_vis, scale, neg_big, lt, m, l);
            else
                corr = softmax_row<HD, 1>(t_s, t_o, full, lo_vis, hi_vis, scale, neg_big, lt, m, l);
            (void)corr;
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full0 + 8 * t);
        }
        // O holds every step: normalise and store this thread's row
        if (alive && step_hi[t] > step_lo[t])
            alive = warp_mbar_wait(o_full0 + 8 * t, 0, abort_flag, a.err, ERR_FM_O, lane);
        if (alive && step_hi[t] > step_lo[t]) {
            tc_fence_after_sync();
            const float inv = 1.0f / l;
            __nv_bfloat16* orow = a.out + ((long)(tok_begin + q0 + t * FM_BQ + r) * a.n_heads + h) * HD;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(t_o + c * 32, v);
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
    if (!(scale > 0.f)) return ZLM_ERR_UNSUPPORTED;            // the row maximum is taken before scaling
    if (((uintptr_t)q % 16) || (q_row_stride % 8) || ((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16) ||
        ((uintptr_t)out % 16))
        return ZLM_ERR_UNSUPPORTED;
    dim3 grid(n_heads, B, (max_new + FM_ROWS - 1) / FM_ROWS);
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

// Runs the give-up path of the bounded waits once, harmlessly (see wait_selftest_kernel): afterwards
// zlm_attention_fmha_status returns 90.  seen: two ints on the device.
ZLM_EXPORT int zlm_attention_fmha_wait_selftest(int polls, int* seen, cudaStream_t stream) {
    return tc::run_wait_selftest(fm_error_word(), polls, seen, stream);
}
