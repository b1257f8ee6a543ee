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
//   warps 2-5 read the accumulator with tcgen05.ld and write the output: plain
//            store (float or bf16), or sum into a float output (the residual stream).
// When there are too few tiles to occupy the GPU (a decode step against a
// 4096-row weight), the K range is split over the CTAs of a thread-block cluster;
// their partial accumulators are summed in rank order through distributed shared
// memory, so the result does not depend on timing and needs no scratch in global
// memory.  Every mbarrier wait is bounded and reports through an error word.
//
// The reference multiplies with one CUDA-core GEMV per token
// (src/cuda_bridge.cu:963-989,1439-1444); this kernel is what replaces it.
#include "common.cuh"
#include "tc_common.cuh"

#include <mutex>
#include <unordered_map>

namespace zlm {
using namespace tc;

constexpr int TC_BM = 128;          // weight rows per tile (UMMA M)
constexpr int TC_BK = 64;           // K elements per stage: one 128-byte swizzle row
constexpr int TC_UMMA_K = 16;
constexpr int TC_THREADS = 192;
constexpr int A_BYTES = TC_BM * TC_BK * 2;

enum OutMode { OUT_F32 = 0, OUT_F32_ACC = 1, OUT_BF16 = 2 };

struct TcArgs {
    const void* bias;
    int bias_dtype;
    void* Y;
    long ldy;
    int T, N, K;
    int kb_total;        // K blocks of 64 in all
    int kb_per_split;    // K blocks per CTA of a cluster
    int splits;
    int* err;
};

template <int BN> struct TcCfg {
    static constexpr int STAGES = BN <= 16 ? 6 : (BN <= 32 ? 5 : 4);
    static constexpr int B_BYTES = BN * TC_BK * 2;
    static constexpr int COLS = BN < 32 ? 32 : BN;                 // TMEM columns: a power of two >= 32
    static constexpr int SMEM = 1024 + STAGES * (A_BYTES + B_BYTES) + 256;
};

template <int BN, int MODE>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, TcArgs a) {
    using C = TcCfg<BN>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t a_base = base;
    const uint32_t b_base = base + STAGES * A_BYTES;
    const uint32_t bar_base = b_base + STAGES * C::B_BYTES;
    // barriers: full[STAGES], empty[STAGES], accum; then the TMEM address and the abort flag
    const uint32_t full0 = bar_base, empty0 = bar_base + 8 * STAGES, accum_bar = bar_base + 16 * STAGES;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + (bar_base - base) + 16 * STAGES + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    float* partial = reinterpret_cast<float*>(smem);           // reused after the main loop: [BN][128] floats

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * TC_BM;
    const int tok0 = blockIdx.y * BN;
    const uint32_t rank = a.splits > 1 ? cluster_rank() : 0u;
    const int kb0 = (int)rank * a.kb_per_split;
    int n_kb = a.kb_total - kb0;
    if (n_kb > a.kb_per_split) n_kb = a.kb_per_split;
    if (n_kb < 0) n_kb = 0;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_w);
        prefetch_tmap(&tmap_x);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(accum_bar, 1);
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

    bool ok = true;
    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int issued = 0;
            for (int kb = 0; kb < n_kb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_flag, a.err, ERR_WAIT_EMPTY)) break;
                mbar_expect_tx(full0 + 8 * s, A_BYTES + C::B_BYTES);
                tma_load_2d(a_base + s * A_BYTES, &tmap_w, full0 + 8 * s, (kb0 + kb) * TC_BK, row0);
                tma_load_2d(b_base + s * C::B_BYTES, &tmap_x, full0 + 8 * s, (kb0 + kb) * TC_BK, tok0);
                ++issued;
            }
            if (*abort_flag) {
                // give copies that are still in flight time to land before shared memory is given up
                const int first = issued > STAGES ? issued - STAGES : 0;
                for (int kb = first; kb < issued; ++kb) {
                    bool landed = false;
                    for (uint32_t i = 0; i < WAIT_POLLS && !landed; ++i)
                        landed = mbar_try_wait(full0 + 8 * (kb % STAGES), (kb / STAGES) & 1);
                    if (!landed && a.err) atomicCAS(a.err, 0, ERR_WAIT_DRAIN);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16(TC_BM, BN);
            for (int kb = 0; kb < n_kb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait(full0 + 8 * s, ph, abort_flag, a.err, ERR_WAIT_FULL)) break;
                tc_fence_after_sync();
#pragma unroll
                for (int k = 0; k < TC_BK / TC_UMMA_K; ++k) {
                    const uint64_t da = smem_desc_sw128(a_base + s * A_BYTES + k * TC_UMMA_K * 2);
                    const uint64_t db = smem_desc_sw128(b_base + s * C::B_BYTES + k * TC_UMMA_K * 2);
                    umma_bf16(tmem_base, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                }
                umma_commit(empty0 + 8 * s);
            }
            umma_commit(accum_bar);
        }
        __syncwarp();
    } else {
        // ----------------------------------- epilogue warps wait for the accumulator
        ok = n_kb == 0 || mbar_wait(accum_bar, 0, abort_flag, a.err, ERR_WAIT_ACCUM);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after_sync();
    }

    const int q = warp & 3;                     // TMEM lane quarter this warp may read
    const int f_local = q * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);

    if (a.splits > 1) {
        if (warp >= 2 && rank != 0) {
            // partial accumulators of the other ranks go to their own shared memory
#pragma unroll 1
            for (int c = 0; c < BN / 16; ++c) {
                uint32_t v[16];
                if (ok && n_kb > 0) {
                    tmem_ld16(t_lane + c * 16, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0u;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) partial[(c * 16 + j) * TC_BM + f_local] = __uint_as_float(v[j]);
            }
        }
        cluster_sync();
    }

    if (warp >= 2 && rank == 0 && ok) {
        const int f = row0 + f_local;
        float bias_v = 0.f;
        if (a.bias != nullptr && f < a.N)
            bias_v = a.bias_dtype == ZLM_F32 ? reinterpret_cast<const float*>(a.bias)[f]
                                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.bias)[f]);
        const uint32_t part_addr = smem_u32(partial);
#pragma unroll 1
        for (int c = 0; c < BN / 16; ++c) {
            if (tok0 + c * 16 >= a.T) break;            // whole chunk beyond the last token (uniform per warp)
            uint32_t v[16];
            if (n_kb > 0) {
                tmem_ld16(t_lane + c * 16, v);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0u;
            }
            for (uint32_t r = 1; r < (uint32_t)a.splits; ++r) {
                const uint32_t remote = map_to_rank(part_addr, r);
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    v[j] = __float_as_uint(__uint_as_float(v[j]) +
                                           ld_cluster_f32(remote + 4u * ((c * 16 + j) * TC_BM + f_local)));
            }
            if (f < a.N) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = tok0 + c * 16 + j;
                    if (tok < a.T) {
                        const float val = __uint_as_float(v[j]) + bias_v;
                        if (MODE == OUT_BF16) {
                            reinterpret_cast<__nv_bfloat16*>(a.Y)[(long)tok * a.ldy + f] = __float2bfloat16_rn(val);
                        } else {
                            float* dst = reinterpret_cast<float*>(a.Y) + (long)tok * a.ldy + f;
                            *dst = MODE == OUT_F32_ACC ? *dst + val : val;
                        }
                    }
                }
            }
        }
    }

    if (a.splits > 1) cluster_sync();            // the other ranks keep their shared memory until rank 0 has read it
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::COLS);
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

// A bf16 matrix [rows, cols] with row stride ld (elements), read in boxes of box_rows x 64.
static int make_map(CUtensorMap* m, const void* ptr, long rows, long cols, long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return ZLM_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : ZLM_ERR_BAD_ARG;
}

struct MapKey {
    const void* ptr; long rows, cols, ld; int box;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box == o.box;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        h = h * 1000003u ^ (size_t)k.rows; h = h * 1000003u ^ (size_t)k.cols;
        h = h * 1000003u ^ (size_t)k.ld; h = h * 1000003u ^ (size_t)k.box;
        return h;
    }
};

// Descriptors depend on (address, shape, box) only, so they are built once and kept.
static int cached_map(CUtensorMap* out, const void* ptr, long rows, long cols, long ld, int box) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    MapKey k{ptr, rows, cols, ld, box};
    auto it = cache.find(k);
    if (it == cache.end()) {
        CUtensorMap m;
        int rc = make_map(&m, ptr, rows, cols, ld, box);
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

template <int BN, int MODE>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const TcArgs& a, cudaStream_t stream) {
    using C = TcCfg<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             C::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a.N + TC_BM - 1) / TC_BM, (a.T + BN - 1) / BN, a.splits);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = C::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = a.splits;
    cfg.attrs = attr;
    cfg.numAttrs = a.splits > 1 ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, MODE>, mw, mx, a);
    return e == cudaSuccess ? launch_status() : (int)e;
}

template <int BN>
static int pick_mode(int mode, const CUtensorMap& mw, const CUtensorMap& mx, const TcArgs& a, cudaStream_t s) {
    switch (mode) {
        case OUT_F32: return launch_tc<BN, OUT_F32>(mw, mx, a, s);
        case OUT_F32_ACC: return launch_tc<BN, OUT_F32_ACC>(mw, mx, a, s);
        default: return launch_tc<BN, OUT_BF16>(mw, mx, a, s);
    }
}

}  // namespace zlm

using namespace zlm;

// X: bf16 [T, K] (row stride ldx), W: bf16 [N, K] (row stride ldw), Y: float or bf16 [T, N] (row stride ldy).
// splits: 0 = choose, else the number of CTAs a tile's K range is split over (1..8).
// Refuses (ZLM_ERR_UNSUPPORTED) strides or addresses TMA cannot take; the caller falls back.
ZLM_EXPORT int zlm_gemm_tc(const void* X, const void* W, const void* bias, int bias_dtype, void* Y, int y_dtype,
                           int accumulate, int T, int N, int K, long ldx, long ldw, long ldy, int splits,
                           cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || ldx < K || ldw < K || ldy < N || splits < 0 || splits > 8) return ZLM_ERR_BAD_ARG;
    if (accumulate && y_dtype != ZLM_F32) return ZLM_ERR_BAD_ARG;
    if ((ldx % 8) || (ldw % 8) || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return ZLM_ERR_UNSUPPORTED;
    const int bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
    TcArgs a;
    a.bias = bias; a.bias_dtype = bias_dtype; a.Y = Y; a.ldy = ldy; a.T = T; a.N = N; a.K = K;
    a.kb_total = (K + TC_BK - 1) / TC_BK;
    a.err = error_word();
    const int tiles = ((N + TC_BM - 1) / TC_BM) * ((T + bn - 1) / bn);
    int s = splits;
    if (s == 0) {
        s = 1;
        if (bn <= 64 && tiles < 148) {
            s = (296 + tiles - 1) / tiles;                    // enough CTAs for two per SM
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
    CUtensorMap mw, mx;
    int rc = cached_map(&mw, W, N, K, ldw, TC_BM);
    if (rc) return rc;
    rc = cached_map(&mx, X, T, K, ldx, bn);
    if (rc) return rc;
    const int mode = y_dtype == ZLM_BF16 ? OUT_BF16 : (accumulate ? OUT_F32_ACC : OUT_F32);
    switch (bn) {
        case 16: return pick_mode<16>(mode, mw, mx, a, stream);
        case 32: return pick_mode<32>(mode, mw, mx, a, stream);
        case 64: return pick_mode<64>(mode, mw, mx, a, stream);
        case 128: return pick_mode<128>(mode, mw, mx, a, stream);
        default: return pick_mode<256>(mode, mw, mx, a, stream);
    }
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
