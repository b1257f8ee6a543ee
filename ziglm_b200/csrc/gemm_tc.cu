// Y[T, N] (+)= X[T, K] * W[N, K]^T (+ bias) in bf16 on the 5th-generation tensor cores.
//
// One kernel serves prompts and decode steps.  The weight rows are the M side of
// the tensor-core instruction (tiles of 128 rows), the tokens are its N side
// (tiles of 16 to 256 tokens), so a decode step of a few tokens still fills the
// instruction and the kernel's job becomes streaming the weights once.  Per tile:
//   warp 0   issues TMA loads of 128x64 weight and BNx64 token tiles (128-byte
//            swizzle) into a ring of shared-memory stages, signalled by mbarriers;
//   warp 1   issues tcgen05.mma (M=128, N=BN, K=16, bf16 -> float) from the stages
//            into an accumulator in tensor memory, and frees a stage with
//            tcgen05.commit when its instructions have read it;
//   warps 2-9 read the accumulator with tcgen05.ld, add the bias, stage the tile in
//            shared memory and hand it to one TMA store (float or bf16 output) or one
//            TMA reduce-add (sum into a float output: the residual stream).  In the
//            gated mode the weight rows alternate gate and up rows and the epilogue
//            writes act(gate) * up, so the activation never makes a trip to memory.
// When there are too few tiles to occupy the GPU (a decode step against a
// 4096-row weight), the K range is split over the CTAs of a thread-block cluster;
// their partial accumulators are summed in rank order through distributed shared
// memory, so the result does not depend on timing and needs no scratch in global
// memory.  Every mbarrier wait is bounded and reports through an error word.
// Steps of more than 64 tokens run a second kernel (gemm_pair_kernel, further down) in which the two
// CTAs of a cluster work as one on tiles of 256 weight rows x 256 tokens (tcgen05 cta_group::2); its
// epilogue is the same code (store_tile).
//
// The reference multiplies with one CUDA-core GEMV per token
// (src/cuda_bridge.cu:963-989,1439-1444); this kernel is what replaces it.
#include "common.cuh"
#include "tc_common.cuh"

#include <cstdlib>
#include <mutex>
#include <unordered_map>

namespace zlm {
using namespace tc;

constexpr int TC_BM = 128;          // weight rows per tile (UMMA M)
constexpr int TC_BK = 64;           // K elements per stage: one 128-byte swizzle row
constexpr int TC_UMMA_K = 16;
constexpr int TC_EPI_WARPS = 8;                 // two per TMEM lane quarter: they take alternate 16-token chunks
constexpr int TC_THREADS = (2 + TC_EPI_WARPS) * 32;
constexpr int A_BYTES = TC_BM * TC_BK * 2;

enum OutMode { OUT_F32 = 0, OUT_F32_ACC = 1, OUT_BF16 = 2, OUT_BF16_GLU = 3, OUT_BF16_GEGLU = 4 };

struct TcArgs {
    const void* bias;
    int bias_dtype;
    void* Y;
    long ldy;
    int T, N, K;
    int kb_total;        // K blocks of 64 in all
    int kb_per_split;    // K blocks per CTA of a cluster
    int splits;
    int ksplit;          // paired CTAs, accumulating products: parts a tile's K range is cut into (each part adds its sum)
    int grid_x;          // blocks (clusters when K is split) that share the tiles
    int tma_store;       // the output goes through shared memory and a TMA store / reduce
    int glu_kind;        // gated mode: 0 silu, 1 tanh gelu
    // RMSNorm split over two products (steps of a few tokens, see zlm_gemm_tc_norm):
    // this product finishes the residual sum and leaves x * gain as bf16 and the sums of squares per tile row
    const void* norm_gain;      // [N] gain of the norm that follows, or null
    int norm_gain_dtype;
    float norm_offset;          // added to the gain (1 for the architectures that store gain - 1)
    __nv_bfloat16* norm_hb;     // [T, ld_hb] bf16(x_new * gain)
    long ld_hb;
    float* norm_ssq;            // [T, norm_p] sums of x_new^2 over the 128 features of tile row p
    int norm_p;
    // this product reads x * gain and scales every output row by 1 / sqrt(mean x^2 + eps)
    const float* scale_ssq;     // [T, scale_p] or null
    int scale_p;
    float scale_eps;
    int* err;
};

// Tokens staged per TMA store: the box height of the output's tensor map.
__host__ __device__ constexpr int sub_rows(int bn) { return (bn == 16 || bn == 64) ? 16 : 32; }

template <int BN, int DEEP = 0> struct TcCfg {
    // Narrow tiles (decode steps) keep few stages, so that three or four blocks fit an SM: the blocks of
    // the next product become resident while this one drains and request their weight tiles early.
    // DEEP: the gated product of a decode step runs as one tile of a megabyte of weights per block, at
    // most two blocks per SM; what bounds it is the bytes each block has in flight, so it takes a fourth
    // stage (measured: five and more cost the next product its early residence).
    static constexpr int STAGES = BN <= 32 ? (DEEP ? DEEP : 3) : (BN == 128 ? 5 : 4);
    static constexpr int B_BYTES = BN * TC_BK * 2;
    static constexpr int ACC_COLS = BN;                            // columns of one accumulator
    static constexpr int COLS = 2 * BN < 32 ? 32 : 2 * BN;         // two accumulators: a power of two >= 32
    static constexpr int SUB = sub_rows(BN);                       // tokens staged per TMA store
    static constexpr int NBUF = BN >= 128 ? 2 : 1;                 // staging buffers: a store drains while the next fills
    static constexpr int SUB_BYTES = SUB * TC_BM * 4;
    static constexpr int STAGING = NBUF * SUB_BYTES;
    static constexpr int SMEM = 1024 + STAGES * (A_BYTES + B_BYTES) + STAGING + 256;
};

// silu(g) = g / (1 + exp(-g)), or the tanh form of gelu; fast exponentials (the result is rounded to bf16)
template <bool GELU>
__device__ __forceinline__ float gated_activation(float g) {
    if (GELU) {
        // tanh(z) = 1 - 2 / (exp(2z) + 1)
        const float z = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        const float th = 1.0f - __fdividef(2.0f, __expf(2.0f * z) + 1.0f);
        return 0.5f * g * (1.0f + th);
    }
    return __fdividef(g, 1.0f + __expf(-g));
}

__device__ __forceinline__ void grid_dependents_may_launch() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// One accumulator (128 weight rows x BN tokens, in tensor memory at t_acc) to the output.  The eight epilogue
// warps of a block call this together; sub_idx counts the sub-tiles the block has stored so far.
template <class C, int BN, int MODE>
__device__ __forceinline__ void store_tile(const TcArgs& a, const CUtensorMap* tmap_y, uint32_t t_acc, int row0, int tok0,
                                           const float* inv_s, uint8_t* stage_base, uint32_t stage_out, int& sub_idx,
                                           bool add_bias = true) {
    constexpr bool GLU = MODE == OUT_BF16_GLU || MODE == OUT_BF16_GEGLU;
    constexpr int OUT_COLS = GLU ? TC_BM / 2 : TC_BM;              // output features of a tile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q = warp & 3;                     // TMEM lane quarter this warp may read
    const int egroup = (warp - 2) >> 2;         // which of the two warps of that quarter
    const int f_local = q * 32 + lane;
    const bool writer = !GLU || (lane & 1) == 0;
    const int col = GLU ? f_local >> 1 : f_local;
    const uint32_t t_lane = t_acc + ((uint32_t)(q * 32) << 16);

    const int f = row0 + f_local;
    float bias_v = 0.f;
    if (a.bias != nullptr && f < a.N && add_bias)
        bias_v = a.bias_dtype == ZLM_F32 ? reinterpret_cast<const float*>(a.bias)[f]
                                        : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.bias)[f]);
    const int out_f = GLU ? f >> 1 : f;
    const int out_n = GLU ? a.N >> 1 : a.N;
    // The staging area is sized for float32 sub-tiles of 128 features; a bf16 sub-tile is half of that and a
    // gated one a quarter, so the same bytes hold two or four times as many sub-tiles on their way out, and a
    // tile of few sub-tiles never waits for a store to have read its buffer.
    constexpr int OUT_BYTES = (MODE == OUT_F32 || MODE == OUT_F32_ACC) ? 4 : 2;
    constexpr int SUB_STRIDE = C::SUB * OUT_COLS * OUT_BYTES;
    constexpr int NB = BN > C::SUB ? C::STAGING / SUB_STRIDE : C::NBUF;    // a tile of one sub-tile has no use for more
    static_assert(NB >= C::NBUF && SUB_STRIDE % 128 == 0, "staging buffers");
#pragma unroll 1
    for (int c = 0; c < BN / 16; ++c) {
        if (tok0 + c * 16 >= a.T) break;            // whole chunk beyond the last token (uniform per block)
        const int sub_row = (c * 16) % C::SUB;       // row of this chunk inside the staged sub-tile
        const int buf = sub_idx % NB;
        float* stage_f = reinterpret_cast<float*>(stage_base + buf * SUB_STRIDE);
        __nv_bfloat16* stage_h = reinterpret_cast<__nv_bfloat16*>(stage_f);
        if (a.tma_store && sub_row == 0 && sub_idx >= NB) {
            // the store that last used this buffer must have read it before it is overwritten
            if (warp == 2 && lane == 0) tma_store_wait_read_keep<NB - 1>();
            asm volatile("bar.sync 1, 256;" ::: "memory");
        }
        uint32_t v[16];
        const bool mine = (c & 1) == egroup;           // the other warp of this quarter takes the other chunks
        if (mine) {
            tmem_ld16(t_lane + c * 16, v);
            tmem_ld_wait();
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (!mine) break;
            float val = __uint_as_float(v[j]);
            if (a.scale_ssq != nullptr) val *= inv_s[(c * 16 + j) & 63];
            val += bias_v;
            if (GLU) {
                // even lanes hold a gate row, the next lane the matching up row
                const float up = __shfl_down_sync(0xffffffffu, val, 1);
                const float g = val;
                val = gated_activation<MODE == OUT_BF16_GEGLU>(g) * up;
            }
            if (a.tma_store) {
                if (writer) {
                    if (MODE == OUT_F32 || MODE == OUT_F32_ACC) stage_f[(sub_row + j) * OUT_COLS + col] = val;
                    else stage_h[(sub_row + j) * OUT_COLS + col] = __float2bfloat16_rn(val);
                }
            } else {
                const int tok = tok0 + c * 16 + j;
                if (writer && tok < a.T && out_f < out_n) {
                    if (MODE == OUT_BF16 || GLU)
                        reinterpret_cast<__nv_bfloat16*>(a.Y)[(long)tok * a.ldy + out_f] = __float2bfloat16_rn(val);
                    else if (MODE == OUT_F32_ACC)   // one adder per element: the order is fixed
                        atomicAdd(reinterpret_cast<float*>(a.Y) + (long)tok * a.ldy + out_f, val);
                    else
                        reinterpret_cast<float*>(a.Y)[(long)tok * a.ldy + out_f] = val;
                }
            }
        }
        const bool last_of_sub = sub_row + 16 == C::SUB || c == BN / 16 - 1 || tok0 + (c + 1) * 16 >= a.T;
        if (a.tma_store && last_of_sub) {
            fence_proxy_async();                    // the staged rows become visible to the TMA engine
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (warp == 2 && lane == 0) {
                const int x = GLU ? row0 >> 1 : row0;
                const int y = tok0 + c * 16 - sub_row;
                if (MODE == OUT_F32_ACC) tma_reduce_add_2d(tmap_y, stage_out + buf * SUB_STRIDE, x, y);
                else tma_store_2d(tmap_y, stage_out + buf * SUB_STRIDE, x, y);
                tma_store_commit();
            }
        }
        if (a.tma_store && last_of_sub) ++sub_idx;
    }
}

// Persistent: block b works on tiles b, b + gridDim.x, ...  The accumulator in tensor memory is
// double-buffered, so the epilogue of one tile runs while the next tile's products are issued.
template <int BN, int MODE, int DEEP>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               const __grid_constant__ CUtensorMap tmap_y, TcArgs a) {
    using C = TcCfg<BN, DEEP>;
    constexpr int STAGES = C::STAGES;
    constexpr bool GLU = MODE == OUT_BF16_GLU || MODE == OUT_BF16_GEGLU;
    constexpr int OUT_COLS = GLU ? TC_BM / 2 : TC_BM;              // output features of a tile
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t a_base = base;
    const uint32_t b_base = base + STAGES * A_BYTES;
    const uint32_t stage_out = b_base + STAGES * C::B_BYTES;        // the output sub-tile on its way to TMA
    const uint32_t bar_base = stage_out + C::STAGING;
    // barriers: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]; then the TMEM address and the abort flag
    const uint32_t full0 = bar_base, empty0 = bar_base + 8 * STAGES;
    const uint32_t acc_full0 = bar_base + 16 * STAGES, acc_empty0 = acc_full0 + 16;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + (bar_base - base) + 16 * STAGES + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    float* partial = reinterpret_cast<float*>(smem);   // split-K only (one tile per block): [BN][128] floats

    __shared__ float inv_s[64];                     // row scales of a product that completes a norm
    __shared__ float norm_red[2][4][4];             // sums of squares: [epilogue half][token of a group][warp]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = a.splits > 1 ? cluster_rank() : 0u;
    const int kb0 = (int)rank * a.kb_per_split;
    int n_kb = a.kb_total - kb0;
    if (n_kb > a.kb_per_split) n_kb = a.kb_per_split;
    if (n_kb < 0) n_kb = 0;
    const int tok_tiles = (a.T + BN - 1) / BN;
    const int n_tiles = ((a.N + TC_BM - 1) / TC_BM) * tok_tiles;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_w);
        prefetch_tmap(&tmap_x);
        if (a.tma_store) prefetch_tmap(&tmap_y);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, TC_EPI_WARPS);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_holder), C::COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    grid_dependents_may_launch();
    bool first_cluster_barrier_done = false;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // weights do not depend on the kernel before this one: their first tiles are
            // requested before waiting for it, the tokens' tiles after
            int pre = 0;
            if ((int)blockIdx.x < n_tiles) {
                const int row0 = ((int)blockIdx.x / tok_tiles) * TC_BM;
                pre = n_kb < STAGES ? n_kb : STAGES;
                for (int kb = 0; kb < pre; ++kb) {
                    mbar_expect_tx(full0 + 8 * kb, A_BYTES + C::B_BYTES);
                    tma_load_2d(a_base + kb * A_BYTES, &tmap_w, full0 + 8 * kb, (kb0 + kb) * TC_BK, row0);
                }
            }
            grid_dependency_wait();
            int it = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
                const int row0 = (tile / tok_tiles) * TC_BM, tok0 = (tile % tok_tiles) * BN;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= pre) {
                        if (!mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1u, abort_flag, a.err, ERR_WAIT_EMPTY)) {
                            alive = false;
                            break;
                        }
                        mbar_expect_tx(full0 + 8 * s, A_BYTES + C::B_BYTES);
                        tma_load_2d(a_base + s * A_BYTES, &tmap_w, full0 + 8 * s, (kb0 + kb) * TC_BK, row0);
                    }
                    tma_load_2d(b_base + s * C::B_BYTES, &tmap_x, full0 + 8 * s, (kb0 + kb) * TC_BK, tok0);
                }
            }
            if (*abort_flag) {
                // give copies that are still in flight time to land before shared memory is given up
                const int issued = it > pre ? it : pre;
                const int first = issued > STAGES ? issued - STAGES : 0;
                for (int k = first; k < issued; ++k) {
                    bool landed = false;
                    for (uint32_t i = 0; i < WAIT_POLLS && !landed; ++i)
                        landed = mbar_try_wait(full0 + 8 * (k % STAGES), (k / STAGES) & 1);
                    if (!landed && a.err) atomicCAS(a.err, 0, ERR_WAIT_DRAIN);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16(TC_BM, BN);
            int it = 0, local = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x, ++local) {
                const int ab = local & 1;
                // the epilogue must have emptied this accumulator (two tiles ago)
                if (!mbar_wait(acc_empty0 + 8 * ab, ((local >> 1) & 1) ^ 1u, abort_flag, a.err, ERR_WAIT_ACCUM)) break;
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + ab * C::ACC_COLS;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(full0 + 8 * s, (it / STAGES) & 1, abort_flag, a.err, ERR_WAIT_FULL)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after_sync();
#pragma unroll
                    for (int k = 0; k < TC_BK / TC_UMMA_K; ++k) {
                        const uint64_t da = smem_desc_sw128(a_base + s * A_BYTES + k * TC_UMMA_K * 2);
                        const uint64_t db = smem_desc_sw128(b_base + s * C::B_BYTES + k * TC_UMMA_K * 2);
                        umma_bf16(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty0 + 8 * s);
                }
                umma_commit(acc_full0 + 8 * ab);
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue
        grid_dependency_wait();                     // the output may still be read by the kernel before this one
        if (a.scale_ssq != nullptr) {
            // one token tile (the host makes sure): 1 / sqrt(mean x^2 + eps) of its tokens, partial sums in order
            const int et = (int)threadIdx.x - 64;
            if (et < BN && et < 64) {
                float inv = 1.0f;
                if (et < a.T) {
                    float ss = 0.f;
                    for (int p = 0; p < a.scale_p; ++p) ss += a.scale_ssq[(long)et * a.scale_p + p];
                    inv = 1.0f / sqrtf(ss / (float)a.K + a.scale_eps);
                }
                inv_s[et] = inv;
            }
        }
        const int q = warp & 3;                     // TMEM lane quarter this warp may read
        const int egroup = (warp - 2) >> 2;         // which of the two warps of that quarter
        const int f_local = q * 32 + lane;
        const bool writer = !GLU || (lane & 1) == 0;
        const int col = GLU ? f_local >> 1 : f_local;
        uint8_t* stage_base = smem + (stage_out - base);
        int sub_idx = 0;                            // sub-tiles stored so far by this block
        const uint32_t part_addr = smem_u32(partial);
        int local = 0;
        if (a.splits > 1) {
            // ---- K is split over the cluster: one tile per block.  Every rank parks its partial
            // accumulator in its own shared memory; then rank r sums, in rank order, a slice of the
            // tile's token columns over all ranks and writes that slice.
            const int tile = blockIdx.x;
            const int row0 = (tile / tok_tiles) * TC_BM, tok0 = (tile % tok_tiles) * BN;
            if (n_kb > 0) mbar_wait(acc_full0, 0, abort_flag, a.err, ERR_WAIT_ACCUM);
            asm volatile("bar.sync 2, 256;" ::: "memory");
            const bool good = *abort_flag == 0;
            tc_fence_after_sync();
            const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
            if (good) {
#pragma unroll 1
                for (int c = egroup; c < BN / 16; c += 2) {
                    uint32_t v[16];
                    tmem_ld16(t_lane + c * 16, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) partial[(c * 16 + j) * TC_BM + f_local] = __uint_as_float(v[j]);
                }
            }
            cluster_sync_arrive_wait();
            first_cluster_barrier_done = true;
            const int f = row0 + f_local;
            float bias_v = 0.f;
            if (a.bias != nullptr && f < a.N)
                bias_v = a.bias_dtype == ZLM_F32 ? reinterpret_cast<const float*>(a.bias)[f]
                                                : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.bias)[f]);
            const int out_f = GLU ? f >> 1 : f;
            const int out_n = GLU ? a.N >> 1 : a.N;
            const int per = (BN + a.splits - 1) / a.splits;
            const int c_lo = (int)rank * per, c_hi = min(BN, c_lo + per);
            uint32_t remote[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) remote[r] = r < a.splits ? map_to_rank(part_addr, (uint32_t)r) : 0u;
            // Up to EB tokens of this warp at a time (tiles of 64 tokens and more): their partials are all requested before the first sum,
            // their additions to the residual all issued before the first result is used, so the latencies of
            // the cluster's shared memory and of the returning atomics are paid once per group, not per token.
            constexpr int EB = BN >= 64 ? 2 : 1;          // narrow tiles keep their registers: three blocks an SM
            if constexpr (EB == 1) {
                for (int cc = c_lo + egroup; cc < c_hi && good; cc += 2) {
                    const int tok = tok0 + cc;
                    if (tok >= a.T) break;
                    float part[8];
    #pragma unroll
                    for (int r = 0; r < 8; ++r)
                        part[r] = r < a.splits ? ld_cluster_f32(remote[r] + 4u * (cc * TC_BM + f_local)) : 0.f;
                    float val = part[0];
    #pragma unroll
                    for (int r = 1; r < 8; ++r) val += part[r];
                    if (a.scale_ssq != nullptr) val *= inv_s[cc];
                    val += bias_v;
                    if (GLU) {
                        const float up = __shfl_down_sync(0xffffffffu, val, 1);
                        const float g = val;
                        val = gated_activation<MODE == OUT_BF16_GEGLU>(g) * up;
                    }
                    if (writer && out_f < out_n) {
                        if (MODE == OUT_BF16 || GLU)
                            reinterpret_cast<__nv_bfloat16*>(a.Y)[(long)tok * a.ldy + out_f] = __float2bfloat16_rn(val);
                        else if (MODE == OUT_F32_ACC && a.norm_gain == nullptr)   // one adder per element: the order is fixed
                            atomicAdd(reinterpret_cast<float*>(a.Y) + (long)tok * a.ldy + out_f, val);
                        else if (MODE != OUT_F32_ACC)
                            reinterpret_cast<float*>(a.Y)[(long)tok * a.ldy + out_f] = val;
                    }
                    if (MODE == OUT_F32_ACC && a.norm_gain != nullptr) {
                        // The only adder of this element sees the finished residual value: it leaves x * gain for
                        // the product after the norm, and the tile's 128 features of this token give one partial
                        // sum of squares (four warps of this half of the epilogue, summed in warp order).
                        float xn = 0.f;
                        if (out_f < out_n) {
                            xn = atomicAdd(reinterpret_cast<float*>(a.Y) + (long)tok * a.ldy + out_f, val) + val;
                            const float g = a.norm_gain_dtype == ZLM_F32
                                                ? reinterpret_cast<const float*>(a.norm_gain)[out_f]
                                                : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.norm_gain)[out_f]);
                            a.norm_hb[(long)tok * a.ld_hb + out_f] = __float2bfloat16_rn(xn * (g + a.norm_offset));
                        }
                        const float sq = warp_sum(xn * xn);
                        if (lane == 0) norm_red[egroup][0][q] = sq;
                        if (egroup == 0) asm volatile("bar.sync 3, 128;" ::: "memory");
                        else asm volatile("bar.sync 4, 128;" ::: "memory");
                        if (q == 0 && lane == 0)
                            a.norm_ssq[(long)tok * a.norm_p + tile / tok_tiles] =
                                ((norm_red[egroup][0][0] + norm_red[egroup][0][1]) + norm_red[egroup][0][2]) + norm_red[egroup][0][3];
                        if (egroup == 0) asm volatile("bar.sync 3, 128;" ::: "memory");
                        else asm volatile("bar.sync 4, 128;" ::: "memory");
                    }
                }
            } else {
                for (int cc0 = c_lo + egroup; cc0 < c_hi && good; cc0 += 2 * EB) {
                    if (tok0 + cc0 >= a.T) break;
                    bool live[EB];
                    float val[EB];
                    float part[EB][8];
    #pragma unroll
                    for (int u = 0; u < EB; ++u) {
                        const int cc = cc0 + 2 * u;
                        live[u] = cc < c_hi && tok0 + cc < a.T;          // the same for every thread of this half
    #pragma unroll
                        for (int r = 0; r < 8; ++r)
                            part[u][r] = (live[u] && r < a.splits) ? ld_cluster_f32(remote[r] + 4u * (cc * TC_BM + f_local)) : 0.f;
                    }
    #pragma unroll
                    for (int u = 0; u < EB; ++u) {
                        const int cc = cc0 + 2 * u;
                        float v = part[u][0];
    #pragma unroll
                        for (int r = 1; r < 8; ++r) v += part[u][r];     // in rank order
                        if (a.scale_ssq != nullptr) v *= inv_s[cc & 63];
                        v += bias_v;
                        if (GLU) {
                            const float up = __shfl_down_sync(0xffffffffu, v, 1);
                            const float g = v;
                            v = gated_activation<MODE == OUT_BF16_GEGLU>(g) * up;
                        }
                        val[u] = v;
                    }
                    float before[EB];
    #pragma unroll
                    for (int u = 0; u < EB; ++u) {
                        const int tok = tok0 + cc0 + 2 * u;
                        before[u] = 0.f;
                        if (!live[u] || !writer || out_f >= out_n) continue;
                        if (MODE == OUT_BF16 || GLU)
                            reinterpret_cast<__nv_bfloat16*>(a.Y)[(long)tok * a.ldy + out_f] = __float2bfloat16_rn(val[u]);
                        else if (MODE == OUT_F32_ACC && a.norm_gain == nullptr)   // one adder per element: the order is fixed
                            atomicAdd(reinterpret_cast<float*>(a.Y) + (long)tok * a.ldy + out_f, val[u]);
                        else if (MODE == OUT_F32_ACC)
                            before[u] = atomicAdd(reinterpret_cast<float*>(a.Y) + (long)tok * a.ldy + out_f, val[u]);
                        else
                            reinterpret_cast<float*>(a.Y)[(long)tok * a.ldy + out_f] = val[u];
                    }
                    if (MODE == OUT_F32_ACC && a.norm_gain != nullptr) {
                        // The only adder of an element sees the finished residual value: it leaves x * gain for
                        // the product after the norm, and the tile's 128 features of a token give one partial
                        // sum of squares (four warps of this half of the epilogue, summed in warp order).
                        float g = 0.f;
                        if (out_f < out_n)
                            g = (a.norm_gain_dtype == ZLM_F32
                                     ? reinterpret_cast<const float*>(a.norm_gain)[out_f]
                                     : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.norm_gain)[out_f])) + a.norm_offset;
    #pragma unroll
                        for (int u = 0; u < EB; ++u) {
                            float xn = 0.f;
                            if (live[u] && out_f < out_n) {
                                xn = before[u] + val[u];
                                a.norm_hb[(long)(tok0 + cc0 + 2 * u) * a.ld_hb + out_f] = __float2bfloat16_rn(xn * g);
                            }
                            const float sq = warp_sum(xn * xn);
                            if (lane == 0) norm_red[egroup][u][q] = sq;
                        }
                        if (egroup == 0) asm volatile("bar.sync 3, 128;" ::: "memory");
                        else asm volatile("bar.sync 4, 128;" ::: "memory");
                        if (q == 0 && lane < EB && cc0 + 2 * lane < c_hi && tok0 + cc0 + 2 * lane < a.T)
                            a.norm_ssq[(long)(tok0 + cc0 + 2 * lane) * a.norm_p + tile / tok_tiles] =
                                ((norm_red[egroup][lane][0] + norm_red[egroup][lane][1]) + norm_red[egroup][lane][2]) +
                                norm_red[egroup][lane][3];
                        if (egroup == 0) asm volatile("bar.sync 3, 128;" ::: "memory");
                        else asm volatile("bar.sync 4, 128;" ::: "memory");
                    }
                }
            }
        } else
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
            const int row0 = (tile / tok_tiles) * TC_BM, tok0 = (tile % tok_tiles) * BN;
            const int ab = local & 1;
            if (n_kb > 0) mbar_wait(acc_full0 + 8 * ab, (local >> 1) & 1, abort_flag, a.err, ERR_WAIT_ACCUM);
            asm volatile("bar.sync 2, 256;" ::: "memory");     // the four warps go on together or not at all
            if (*abort_flag) break;
            tc_fence_after_sync();
            store_tile<C, BN, MODE>(a, &tmap_y, tmem_base + ab * C::ACC_COLS, row0, tok0, inv_s, stage_base, stage_out,
                                    sub_idx);
            // this accumulator may be overwritten by the tile after next
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * ab);
        }
        if (a.tma_store && a.splits == 1 && warp == 2 && lane == 0) tma_store_wait_read();
        __syncwarp();
    }

    if (a.splits > 1) {
        // every thread of every rank passes two cluster barriers: after the partials are written
        // (rank 0's epilogue passes the first one inside its loop) and after they are read
        if (!first_cluster_barrier_done) cluster_sync_arrive_wait();
        cluster_sync_arrive_wait();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::COLS);
    }
}


// ------------------------------------------------------------- prompts: two CTAs per tile
// For steps of more than 128 tokens the two CTAs of a cluster work as one (tcgen05 cta_group::2) on tiles of
// 256 weight rows x 256 tokens.  Each CTA loads its own 128 weight rows and its own 128 of the tile's tokens,
// so a stage is 32 KB instead of 48 and the ring holds six of them for the same product; the leader (rank 0)
// issues one instruction for both tensor cores.  Each CTA's tensor memory receives the accumulator of its own
// 128 weight rows for all 256 tokens, and its epilogue warps write it as in the kernel above.  Barriers: the
// stage-full barriers live in the leader and count the bytes of both CTAs' loads; stage-empty and
// accumulator-full barriers exist in both CTAs and are signalled by one tcgen05.commit to both; the
// accumulator-empty barriers live in the leader and collect the epilogue warps of both.
struct PairCfg {
    static constexpr int BN = 256;
    static constexpr int STAGES = 6;
    static constexpr int B_BYTES = (BN / 2) * TC_BK * 2;           // this CTA's half of the tile's tokens
    static constexpr int ACC_COLS = BN;
    static constexpr int COLS = 2 * BN;
    static constexpr int SUB = sub_rows(BN);
    static constexpr int NBUF = 2;
    static constexpr int SUB_BYTES = SUB * TC_BM * 4;
    static constexpr int STAGING = NBUF * SUB_BYTES;
    static constexpr int SMEM = 1024 + STAGES * (A_BYTES + B_BYTES) + STAGING + 256;
};

template <int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                 const __grid_constant__ CUtensorMap tmap_y, TcArgs a) {
    using C = PairCfg;
    constexpr int STAGES = C::STAGES, BN = C::BN;
    constexpr uint32_t STAGE_TX = 2u * (A_BYTES + C::B_BYTES);      // both CTAs' loads of one stage
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t a_base = base;
    const uint32_t b_base = base + STAGES * A_BYTES;
    const uint32_t stage_out = b_base + STAGES * C::B_BYTES;
    const uint32_t bar_base = stage_out + C::STAGING;
    const uint32_t full0 = bar_base, empty0 = bar_base + 8 * STAGES;
    const uint32_t acc_full0 = bar_base + 16 * STAGES, acc_empty0 = acc_full0 + 16;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + (bar_base - base) + 16 * STAGES + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                           // 0 leads
    const bool leader = rank == 0;
    const int pair = (int)(blockIdx.x >> 1), n_pairs = (int)(gridDim.x >> 1);
    const int tok_tiles = (a.T + BN - 1) / BN;
    const int n_tiles = ((a.N + 2 * TC_BM - 1) / (2 * TC_BM)) * tok_tiles;
    // A unit of work is a tile, or one of ksplit parts of its K range where the tiles alone would leave most
    // pairs idle (accumulating products of a few hundred tokens: every part adds its sum to the output).
    const int kb_per = (a.kb_total + a.ksplit - 1) / a.ksplit;
    const int n_units = n_tiles * a.ksplit;
    const uint32_t lead_full0 = map_to_rank(full0, 0u);
    const uint32_t lead_acc_empty0 = map_to_rank(acc_empty0, 0u);

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_w);
        prefetch_tmap(&tmap_x);
        if (a.tma_store) prefetch_tmap(&tmap_y);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 2 * TC_EPI_WARPS);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(tmem_holder), C::COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_arrive_wait();            // both CTAs' barriers exist before either signals the other's
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    grid_dependents_may_launch();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            const int my_rows = (int)rank * TC_BM, my_toks = (int)rank * (BN / 2);
            int pre = 0;
            if (pair < n_units) {
                // weights do not depend on the kernel before this one
                const int row0 = ((pair % n_tiles) / tok_tiles) * 2 * TC_BM + my_rows;
                const int kb_lo = (pair / n_tiles) * kb_per;
                const int n_kb = min(kb_per, a.kb_total - kb_lo);
                pre = n_kb < STAGES ? n_kb : STAGES;
                for (int kb = 0; kb < pre; ++kb) {
                    if (leader) mbar_expect_tx(full0 + 8 * kb, STAGE_TX);
                    tma_load_2d_pair(a_base + kb * A_BYTES, &tmap_w, lead_full0 + 8 * kb, (kb_lo + kb) * TC_BK, row0);
                }
            }
            grid_dependency_wait();
            int it = 0;
            bool alive = true;
            for (int unit = pair; unit < n_units && alive; unit += n_pairs) {
                const int tile = unit % n_tiles;
                const int row0 = (tile / tok_tiles) * 2 * TC_BM + my_rows;
                const int tok0 = (tile % tok_tiles) * BN + my_toks;
                const int kb_lo = (unit / n_tiles) * kb_per;
                const int n_kb = min(kb_per, a.kb_total - kb_lo);
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= pre) {
                        if (!mbar_wait(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1u, abort_flag, a.err, ERR_WAIT_EMPTY)) {
                            alive = false;
                            break;
                        }
                        if (leader) mbar_expect_tx(full0 + 8 * s, STAGE_TX);
                        tma_load_2d_pair(a_base + s * A_BYTES, &tmap_w, lead_full0 + 8 * s, (kb_lo + kb) * TC_BK, row0);
                    }
                    tma_load_2d_pair(b_base + s * C::B_BYTES, &tmap_x, lead_full0 + 8 * s, (kb_lo + kb) * TC_BK, tok0);
                }
            }
            if (*abort_flag && leader) {
                // the leader's barriers count both CTAs' copies: give those in flight time to land before either
                // CTA gives up its shared memory (the other CTA waits at the cluster barrier below)
                const int issued = it > pre ? it : pre;
                const int first = issued > STAGES ? issued - STAGES : 0;
                for (int k = first; k < issued; ++k) {
                    bool landed = false;
                    for (uint32_t i = 0; i < WAIT_POLLS && !landed; ++i)
                        landed = mbar_try_wait(full0 + 8 * (k % STAGES), (k / STAGES) & 1);
                    if (!landed && a.err) atomicCAS(a.err, 0, ERR_WAIT_DRAIN);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer (the leader's)
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = idesc_bf16(2 * TC_BM, BN);
            int it = 0, local = 0;
            bool alive = true;
            for (int unit = pair; unit < n_units && alive; unit += n_pairs, ++local) {
                const int n_kb = min(kb_per, a.kb_total - (unit / n_tiles) * kb_per);
                const int ab = local & 1;
                // the epilogues of both CTAs must have emptied this accumulator (two units ago)
                if (!mbar_wait(acc_empty0 + 8 * ab, ((local >> 1) & 1) ^ 1u, abort_flag, a.err, ERR_WAIT_ACCUM)) break;
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + ab * C::ACC_COLS;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(full0 + 8 * s, (it / STAGES) & 1, abort_flag, a.err, ERR_WAIT_FULL)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after_sync();
#pragma unroll
                    for (int k = 0; k < TC_BK / TC_UMMA_K; ++k) {
                        const uint64_t da = smem_desc_sw128(a_base + s * A_BYTES + k * TC_UMMA_K * 2);
                        const uint64_t db = smem_desc_sw128(b_base + s * C::B_BYTES + k * TC_UMMA_K * 2);
                        umma_bf16_pair(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit_pair(empty0 + 8 * s, 3);
                }
                if (alive) umma_commit_pair(acc_full0 + 8 * ab, 3);
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- epilogue (both CTAs)
        grid_dependency_wait();                     // the output may still be read by the kernel before this one
        uint8_t* stage_base = smem + (stage_out - base);
        int sub_idx = 0, local = 0;
        for (int unit = pair; unit < n_units; unit += n_pairs, ++local) {
            const int tile = unit % n_tiles;
            const int row0 = (tile / tok_tiles) * 2 * TC_BM + (int)rank * TC_BM, tok0 = (tile % tok_tiles) * BN;
            const int ab = local & 1;
            mbar_wait(acc_full0 + 8 * ab, (local >> 1) & 1, abort_flag, a.err, ERR_WAIT_ACCUM);
            asm volatile("bar.sync 2, 256;" ::: "memory");     // the eight warps go on together or not at all
            if (*abort_flag) break;
            tc_fence_after_sync();
            if (row0 < a.N)                                    // an odd number of row tiles leaves the last pair half empty
                store_tile<C, BN, MODE>(a, &tmap_y, tmem_base + ab * C::ACC_COLS, row0, tok0, nullptr, stage_base,
                                        stage_out, sub_idx, unit < n_tiles);      // the first part adds the bias
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_acc_empty0 + 8 * ab);
        }
        if (a.tma_store && warp == 2 && lane == 0) tma_store_wait_read();
        __syncwarp();
    }

    // neither CTA leaves while the other may still signal its barriers or read its shared memory
    tc_fence_before_sync();
    cluster_sync_arrive_wait();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, C::COLS);
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

// A matrix [rows, cols] with row stride ld (elements).  Operands (bf16) are read in boxes of box_rows x 64
// with the 128-byte swizzle; outputs (kind 1 bf16, 2 float) are written in boxes of box_rows x box_cols, unswizzled.
static int make_map(CUtensorMap* m, const void* ptr, long rows, long cols, long ld, int box_rows, int box_cols,
                    int kind) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return ZLM_ERR_UNSUPPORTED;
    const int es = kind == 2 ? 4 : 2;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * es};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, kind == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                    const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    kind == 0 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    kind == 0 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : ZLM_ERR_BAD_ARG;
}

struct MapKey {
    const void* ptr; long rows, cols, ld; int box, box_cols, kind;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box == o.box &&
               box_cols == o.box_cols && kind == o.kind;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        h = h * 1000003u ^ (size_t)k.rows; h = h * 1000003u ^ (size_t)k.cols;
        h = h * 1000003u ^ (size_t)k.ld; h = h * 1000003u ^ (size_t)k.box;
        h = h * 1000003u ^ (size_t)(k.box_cols * 4 + k.kind);
        return h;
    }
};

// Descriptors depend on (address, shape, box) only, so they are built once and kept.
static int cached_map(CUtensorMap* out, const void* ptr, long rows, long cols, long ld, int box,
                      int box_cols = TC_BK, int kind = 0) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    MapKey k{ptr, rows, cols, ld, box, box_cols, kind};
    auto it = cache.find(k);
    if (it == cache.end()) {
        CUtensorMap m;
        int rc = make_map(&m, ptr, rows, cols, ld, box, box_cols, kind);
        if (rc) return rc;
        if (cache.size() > 65536) cache.clear();
        it = cache.emplace(k, m).first;
    }
    *out = it->second;
    return 0;
}

static int* error_word() {
    static int* word = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        if (cudaMalloc(&word, sizeof(int)) == cudaSuccess) cudaMemset(word, 0, sizeof(int));
        else word = nullptr;
    });
    return word;
}

template <int BN, int MODE, int DEEP = 0>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& my, const TcArgs& a,
                     cudaStream_t stream) {
    using C = TcCfg<BN, DEEP>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, MODE, DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             C::SMEM);
        if (e != cudaSuccess) return (int)e;
        // ask for the largest shared-memory carve-out, so that two blocks of the narrow tiles fit an SM
        e = cudaFuncSetAttribute(gemm_tc_kernel<BN, MODE, DEEP>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.grid_x, 1, a.splits);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = C::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // may start while its predecessor drains
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = a.splits;
    cfg.attrs = attr;
    cfg.numAttrs = a.splits > 1 ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, MODE, DEEP>, mw, mx, my, a);
    return e == cudaSuccess ? launch_status() : (int)e;
}

template <int BN>
static int pick_mode(int mode, const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& my, const TcArgs& a,
                     cudaStream_t s) {
    switch (mode) {
        case OUT_F32: return launch_tc<BN, OUT_F32>(mw, mx, my, a, s);
        case OUT_F32_ACC: return launch_tc<BN, OUT_F32_ACC>(mw, mx, my, a, s);
        case OUT_BF16_GLU:
            if (BN <= 32 && a.splits == 1 && a.grid_x <= 2 * 148) return launch_tc<BN, OUT_BF16_GLU, 4>(mw, mx, my, a, s);
            return launch_tc<BN, OUT_BF16_GLU>(mw, mx, my, a, s);
        case OUT_BF16_GEGLU:
            if (BN <= 32 && a.splits == 1 && a.grid_x <= 2 * 148) return launch_tc<BN, OUT_BF16_GEGLU, 4>(mw, mx, my, a, s);
            return launch_tc<BN, OUT_BF16_GEGLU>(mw, mx, my, a, s);
        default: return launch_tc<BN, OUT_BF16>(mw, mx, my, a, s);
    }
}


// How many clusters of two can be resident at once (the SMs of a pair share a TPC); asked once.
template <int MODE>
static int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& my, TcArgs a,
                       int pair_tiles, cudaStream_t stream) {
    using C = PairCfg;
    static int resident = 0;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = C::SMEM;
    cfg.stream = stream;
    cfg.attrs = attr;
    if (resident == 0) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return (int)e;
        int dev = 0, sms = 0, n = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2) sms = 148;
        cfg.gridDim = dim3(sms & ~1);
        cfg.numAttrs = 1;
        e = cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<MODE>, &cfg);
        if (e != cudaSuccess || n <= 0) {
            cudaGetLastError();
            return ZLM_ERR_UNSUPPORTED;
        }
        resident = n < sms / 2 ? n : sms / 2;
    }
    // an accumulating product whose tiles would occupy less than half of the pairs is also cut along K
    a.ksplit = 1;
    if (MODE == OUT_F32_ACC && 2 * pair_tiles <= resident) {
        int k = resident / pair_tiles;
        if (k > 8) k = 8;
        if (k > a.kb_total / 8) k = a.kb_total / 8;            // at least eight K blocks a part
        if (k < 1) k = 1;
        const int per = (a.kb_total + k - 1) / k;
        a.ksplit = (a.kb_total + per - 1) / per;               // no empty part
    }
    const int units = pair_tiles * a.ksplit;
    const int pairs = units < resident ? units : resident;
    a.grid_x = 2 * pairs;
    cfg.gridDim = dim3(a.grid_x);
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<MODE>, mw, mx, my, a);
    return e == cudaSuccess ? launch_status() : (int)e;
}

static int pick_pair_mode(int mode, const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& my, const TcArgs& a,
                          int pair_tiles, cudaStream_t s) {
    switch (mode) {
        case OUT_F32: return launch_pair<OUT_F32>(mw, mx, my, a, pair_tiles, s);
        case OUT_F32_ACC: return launch_pair<OUT_F32_ACC>(mw, mx, my, a, pair_tiles, s);
        case OUT_BF16_GLU: return launch_pair<OUT_BF16_GLU>(mw, mx, my, a, pair_tiles, s);
        case OUT_BF16_GEGLU: return launch_pair<OUT_BF16_GEGLU>(mw, mx, my, a, pair_tiles, s);
        default: return launch_pair<OUT_BF16>(mw, mx, my, a, pair_tiles, s);
    }
}

}  // namespace zlm

using namespace zlm;

// X: bf16 [T, K] (row stride ldx), W: bf16 [N, K] (row stride ldw), Y: float or bf16 [T, N] (row stride ldy).
// glu: 0 = plain product; 1 / 2 = the rows of W (and the entries of bias) alternate gate and up rows and Y is
//      bf16 [T, N/2] holding silu(gate) * up (1) or tanh-gelu(gate) * up (2), the bias added before the activation.
// splits: 0 = choose, else the number of CTAs a tile's K range is split over (1..8); 1 also keeps steps of more
//      than 128 tokens on the one-CTA kernel (0 gives them to the kernel that pairs two CTAs per tile).
// Refuses (ZLM_ERR_UNSUPPORTED) strides or addresses TMA cannot read; the caller falls back.
//
// An RMSNorm between two products of a step of at most 64 tokens can ride on them instead of being a kernel of
// its own.  The product before it (accumulate into the float32 residual, K split over a cluster so that one
// thread finishes each element) is given norm_gain / norm_hb / norm_ssq: it also writes bf16(x * gain) to
// norm_hb [T, ld_hb] and, per token and tile row of 128 features, the sum of x^2 to norm_ssq [T, ceil(N/128)].
// *norm_fused says whether it did (it does not when the launch it chooses has no cluster; nothing is written
// then and the caller runs the norm kernel).  The product after it takes X = norm_hb and scale_ssq / scale_p /
// scale_eps: every output row t is multiplied by 1 / sqrt(sum_p scale_ssq[t, p] / K + eps) before the bias.
ZLM_EXPORT int zlm_gemm_tc_norm(const void* X, const void* W, const void* bias, int bias_dtype, void* Y, int y_dtype,
                                int accumulate, int glu, int T, int N, int K, long ldx, long ldw, long ldy, int splits,
                                const void* norm_gain, int norm_gain_dtype, float norm_offset, void* norm_hb,
                                long ld_hb, float* norm_ssq, int* norm_fused, const float* scale_ssq, int scale_p,
                                float scale_eps, cudaStream_t stream) {
    if (norm_fused) *norm_fused = 0;
    if (T <= 0 || N <= 0) return 0;
    if (scale_ssq != nullptr && (T > 64 || scale_p <= 0)) return ZLM_ERR_BAD_ARG;
    if (norm_gain != nullptr && (!accumulate || glu || !norm_hb || !norm_ssq || !norm_fused || ld_hb < N))
        return ZLM_ERR_BAD_ARG;
    const int n_out = glu ? N / 2 : N;
    if (K <= 0 || ldx < K || ldw < K || ldy < n_out || splits < 0 || splits > 8 || glu < 0 || glu > 2)
        return ZLM_ERR_BAD_ARG;
    if (accumulate && y_dtype != ZLM_F32) return ZLM_ERR_BAD_ARG;
    if (glu && ((N & 1) || y_dtype != ZLM_BF16)) return ZLM_ERR_BAD_ARG;
    if ((ldx % 8) || (ldw % 8) || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return ZLM_ERR_UNSUPPORTED;
    // more than 64 tokens and at least two tiles of weight rows: two CTAs per tile of 256 rows x 256 tokens (with 65
    // to 128 tokens half of the tile is empty, which costs less than leaving the K split and the second SM out)
    const bool paired = T > 64 && splits == 0 && N > TC_BM && scale_ssq == nullptr;
    const int bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : (T <= 128 && !paired) ? 128 : 256;
    TcArgs a;
    a.bias = bias; a.bias_dtype = bias_dtype; a.Y = Y; a.ldy = ldy; a.T = T; a.N = N; a.K = K;
    a.kb_total = (K + TC_BK - 1) / TC_BK;
    a.glu_kind = glu == 2 ? 1 : 0;
    a.ksplit = 1;
    a.err = error_word();
    a.norm_gain = nullptr; a.norm_gain_dtype = norm_gain_dtype; a.norm_offset = norm_offset;
    a.norm_hb = (__nv_bfloat16*)norm_hb; a.ld_hb = ld_hb; a.norm_ssq = norm_ssq; a.norm_p = (N + TC_BM - 1) / TC_BM;
    a.scale_ssq = scale_ssq; a.scale_p = scale_p; a.scale_eps = scale_eps;
    const int tiles = ((N + TC_BM - 1) / TC_BM) * ((T + bn - 1) / bn);
    int s = splits;
    if (s == 0) {
        s = 1;
        if (bn <= 64 && tiles < 148) {
            s = (296 + tiles - 1) / tiles;                    // enough CTAs for two per SM
            // the gated product pays for CTAs beyond one resident wave (measured at 128 tiles: 2 beats 3)
            if (glu && s > 1 && tiles * s > 296) --s;
            // 32 and 64 tokens: a rank's share of the reduction over the cluster grows with the tile.  Measured
            // inside decode steps of 32 and 64 sequences (8B shapes): a product that stores does best with five
            // ranks (48 tiles), one that adds with seven rather than eight (32 tiles).
            if (bn >= 32 && s > (accumulate ? 7 : 5)) s = accumulate ? 7 : 5;
            if (s > 8) s = 8;
            const int most = a.kb_total / 4 > 0 ? a.kb_total / 4 : 1;   // at least 4 K blocks per CTA
            if (s > most) s = most;
        }
    }
    if (bn > 64) s = 1;                                       // the partial tile must fit the stage memory
    if (s > a.kb_total) s = a.kb_total;
    a.kb_per_split = (a.kb_total + s - 1) / s;
    s = (a.kb_total + a.kb_per_split - 1) / a.kb_per_split;   // every rank gets at least one block
    a.splits = s;
    if (norm_gain != nullptr && s > 1 && T <= bn) {           // a cluster and one token tile: the norm rides along
        a.norm_gain = norm_gain;
        *norm_fused = 1;
    }
    // one tile per block when K is split; otherwise as many blocks as fit the GPU share the tiles
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0)
            sm_count = 148;
    }
    const int per_sm = bn <= 64 ? 2 : 1;
    a.grid_x = (s > 1 || tiles < sm_count * per_sm) ? tiles : sm_count * per_sm;
    CUtensorMap mw, mx, my;
    int rc = cached_map(&mw, W, N, K, ldw, TC_BM);
    if (rc) return rc;
    rc = cached_map(&mx, X, T, K, ldx, bn);
    if (rc) return rc;
    const int mode = glu == 1 ? OUT_BF16_GLU
                     : glu == 2 ? OUT_BF16_GEGLU
                                : (y_dtype == ZLM_BF16 ? OUT_BF16 : (accumulate ? OUT_F32_ACC : OUT_F32));
    // the output goes through TMA when its rows start on 16-byte boundaries; else the threads store directly
    const int es = y_dtype == ZLM_BF16 ? 2 : 4;
    a.tma_store = ((uintptr_t)Y % 16 == 0) && ((ldy * es) % 16 == 0);
    if (a.tma_store) {
        rc = cached_map(&my, Y, T, n_out, ldy, sub_rows(bn), glu ? TC_BM / 2 : TC_BM, es == 2 ? 1 : 2);
        if (rc) return rc;
    } else {
        my = mx;                                              // never dereferenced
    }
    if (paired) {
        CUtensorMap mxh;
        rc = cached_map(&mxh, X, T, K, ldx, bn / 2);
        if (rc) return rc;
        const int pair_tiles = ((N + 2 * TC_BM - 1) / (2 * TC_BM)) * ((T + bn - 1) / bn);
        rc = pick_pair_mode(mode, mw, mxh, my, a, pair_tiles, stream);
        if (rc != ZLM_ERR_UNSUPPORTED) return rc;
    }
    switch (bn) {
        case 16: return pick_mode<16>(mode, mw, mx, my, a, stream);
        case 32: return pick_mode<32>(mode, mw, mx, my, a, stream);
        case 64: return pick_mode<64>(mode, mw, mx, my, a, stream);
        case 128: return pick_mode<128>(mode, mw, mx, my, a, stream);
        default: return pick_mode<256>(mode, mw, mx, my, a, stream);
    }
}

ZLM_EXPORT int zlm_gemm_tc(const void* X, const void* W, const void* bias, int bias_dtype, void* Y, int y_dtype,
                           int accumulate, int glu, int T, int N, int K, long ldx, long ldw, long ldy, int splits,
                           cudaStream_t stream) {
    return zlm_gemm_tc_norm(X, W, bias, bias_dtype, Y, y_dtype, accumulate, glu, T, N, K, ldx, ldw, ldy, splits, nullptr,
                            ZLM_F32, 0.f, nullptr, 0, nullptr, nullptr, nullptr, 0, 0.f, stream);
}

// Reads and clears the error word the kernels report bounded-wait failures through (synchronises the device).
ZLM_EXPORT int zlm_gemm_tc_status(int* out) {
    int* w = error_word();
    if (!w) { *out = -1; return 0; }
    cudaError_t e = cudaMemcpy(out, w, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
    if (*out != 0) cudaMemset(w, 0, sizeof(int));
    return 0;
}

// Runs the give-up path of the bounded waits once, harmlessly (see wait_selftest_kernel): afterwards
// zlm_gemm_tc_status returns 90.  seen: two ints on the device.
ZLM_EXPORT int zlm_gemm_tc_wait_selftest(int polls, int* seen, cudaStream_t stream) {
    return run_wait_selftest(error_word(), polls, seen, stream);
}
