// Sampling on the device: argmax, and the reference's sampler chain.
//
// The reference samples on the host (src/sampler.zig:31-157): optional
// repetition/presence penalties over the last ids, logits * (1/T), softmax, sort by
// probability, keep top_k, cut below min_p * p_max (at least one stays), cut once
// the running probability reaches top_p, then draw r = u * sum(kept) and take the
// first kept candidate whose running sum reaches r.  Greedy is the plain argmax
// (src/sampler.zig:159-170; device twin src/cuda_bridge.cu:2946-3062).  Here one
// block of 1024 threads handles one row of logits:
//   * argmax scans every id (the reference's CPU argmax skips id 0, its GPU one does
//     not); the lowest id wins ties.
//   * with top_k in [1, 1024] the k best candidates are selected exactly (radix select
//     on the scaled logits, ties to the lower id), sorted by (probability descending,
//     id ascending) and cut and drawn from in that order by one thread, in the same
//     float operations as the plain statement of the chain.
//   * with top_k == 0 the candidates stay in id order: min_p is a threshold, the
//     draw is a running sum over ids.  top_p < 1 keeps the reference's nucleus (the
//     shortest prefix, by descending probability and ascending id, whose probability
//     reaches top_p): the scaled logit of its last member is found by a radix select
//     over probability mass, summed in 2^-44 fixed point so that the sums do not depend
//     on the order of the additions.
// The uniform number of a draw is a pure function of (seed, counter) of the row, so
// a sequence draws the same whatever else is in its batch.
#include "common.cuh"

namespace zlm {

constexpr int SAMPLE_THREADS = 1024;
constexpr int MAX_TOP_K = 1024;

// splitmix64, the integer hash behind the per-row uniform draw
__host__ __device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long counter) {
    const unsigned long long h = mix64(seed ^ mix64(counter));
    return (float)(h >> 40) * (1.0f / 16777216.0f);   // 24 bits, [0, 1)
}

// order-preserving map from float to unsigned
__device__ __forceinline__ unsigned orderable(float f) {
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// exclusive prefix sum of one int per thread over the block (blockDim.x == 1024)
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_totals, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) warp_totals[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = warp_totals[lane];
        int winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        warp_totals[lane] = winc - w;
        if (lane == 31) *total = winc;
    }
    __syncthreads();
    return warp_totals[warp] + inc - v;
}

__device__ __forceinline__ float block_exclusive_scan_f(float v, float* warp_totals, float* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) warp_totals[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        float w = warp_totals[lane];
        float winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += n;
        }
        warp_totals[lane] = winc - w;
        if (lane == 31) *total = winc;
    }
    __syncthreads();
    return warp_totals[warp] + inc - v;
}

// ------------------------------------------------------------------- argmax
// A row of a large vocabulary is half a megabyte: one block walking it alone is bound by its own load
// latency.  ARGMAX_PARTS blocks take a slice each and leave their best (value, id) in a device array of the
// library; the block that arrives last at the row's counter picks among them and sets the counter back to zero
// (no block waits for another; nothing is allocated).  The lowest id wins ties, also across slices.
constexpr int ARGMAX_PARTS = 32;
constexpr int ARGMAX_THREADS = 256;
constexpr int ARGMAX_MAX_ROWS = 4096;           // rows per launch; the host loops over more
static __device__ float g_argmax_val[ARGMAX_MAX_ROWS * ARGMAX_PARTS];
static __device__ int g_argmax_idx[ARGMAX_MAX_ROWS * ARGMAX_PARTS];
static __device__ int g_argmax_count[ARGMAX_MAX_ROWS];

__device__ __forceinline__ void better(float& best, int& bi, float ov, int oi) {
    if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
}

__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_kernel(const float* __restrict__ logits, int V, long row_stride, int* __restrict__ out) {
    __shared__ float vals[ARGMAX_THREADS / 32];
    __shared__ int idxs[ARGMAX_THREADS / 32];
    __shared__ int last_s;
    const int r = blockIdx.y, part = blockIdx.x;
    const float* row = logits + (long)r * row_stride;
    const int per = (V + ARGMAX_PARTS - 1) / ARGMAX_PARTS;
    const int lo = min(V, part * per), hi = min(V, lo + per);
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += ARGMAX_THREADS) {
        const float v = row[i];
        if (v > best || bi == 0x7fffffff) { best = v; bi = i; }       // ids rise within a thread: ties keep the lower
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        better(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (lane == 0) { vals[warp] = best; idxs[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = lane < ARGMAX_THREADS / 32 ? vals[lane] : -INFINITY;
        bi = lane < ARGMAX_THREADS / 32 ? idxs[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            better(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
        if (lane == 0) {
            g_argmax_val[r * ARGMAX_PARTS + part] = best;
            g_argmax_idx[r * ARGMAX_PARTS + part] = bi;
            __threadfence();
            last_s = atomicAdd(&g_argmax_count[r], 1) == ARGMAX_PARTS - 1;
        }
        __syncwarp();
        if (last_s) {                       // read by the warp that wrote it
            __threadfence();
            best = __ldcg(&g_argmax_val[r * ARGMAX_PARTS + lane]);
            bi = __ldcg(&g_argmax_idx[r * ARGMAX_PARTS + lane]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                better(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
            if (lane == 0) {
                out[r] = bi;
                g_argmax_count[r] = 0;
            }
        }
    }
}

// ------------------------------------------------------------------- sample
struct SampleArgs {
    float inv_temperature;
    int top_k;
    float top_p;
    float min_p;
    float repetition_penalty;
    float presence_penalty;
    int window;           // ids of history per row (0: none); history is [rows, window], -1 = empty
};

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(float* __restrict__ logits, int V, long row_stride, SampleArgs a, const int* __restrict__ history,
              const long long* __restrict__ rng, int* __restrict__ out) {
    __shared__ float fscratch[33];
    __shared__ int iscratch[32];
    __shared__ int itotal;
    __shared__ float ftotal;
    __shared__ int hist[256];
    __shared__ unsigned prefix_s;
    __shared__ int remaining_s;
    __shared__ float cand_z[MAX_TOP_K];
    __shared__ int cand_id[MAX_TOP_K];
    __shared__ int n_cand;

    const int tid = threadIdx.x;
    float* row = logits + (long)blockIdx.x * row_stride;

    // 0. penalties, once per occurrence in the window, in window order
    if (a.window > 0 && (a.repetition_penalty != 1.0f || a.presence_penalty != 0.0f)) {
        const int* h = history + (long)blockIdx.x * a.window;
        if (tid < a.window) {
            const int tok = h[tid];
            bool first = tok >= 0 && tok < V;
            for (int j = 0; j < tid && first; ++j) first = h[j] != tok;
            if (first) {
                float l = row[tok];
                for (int j = tid; j < a.window; ++j) {
                    if (h[j] != tok) continue;
                    l = l > 0.f ? l / a.repetition_penalty : l * a.repetition_penalty;
                    l -= a.presence_penalty;
                }
                row[tok] = l;
            }
        }
        __syncthreads();
    }

    // 1. scaled logits, their max, the softmax denominator
    float m = -INFINITY;
    for (int i = tid; i < V; i += SAMPLE_THREADS) m = fmaxf(m, row[i] * a.inv_temperature);
    m = block_max(m, fscratch);
    // contiguous chunks from here on, so that running sums follow the id order
    const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int lo = min(V, tid * chunk), hi = min(V, lo + chunk);
    float part = 0.f;
    for (int i = lo; i < hi; ++i) part += expf(row[i] * a.inv_temperature - m);
    float denom;
    block_exclusive_scan_f(part, fscratch, &ftotal);
    denom = ftotal;
    __syncthreads();

    const float u = uniform01((unsigned long long)rng[2 * blockIdx.x], (unsigned long long)rng[2 * blockIdx.x + 1]);

    if (a.top_k <= 0) {
        // candidates in id order; min_p is a threshold on the probability
        const float thresh = a.min_p > 0.f ? (1.0f / denom) * a.min_p : -1.f;
        // top_p < 1: the nucleus.  kth = key of the scaled logit of its last member; every id with a larger key
        // is in, of the ids with that key the first tie_keep in id order.  (All keys pass when top_p is 1.)
        unsigned kth = 0u;
        int tie_keep = 0x7fffffff;
        if (a.top_p < 1.0f) {
            __shared__ unsigned long long mass[256];     // probability mass per bucket of a pass, in units of 2^-44
            const double one = 17592186044416.0;                                            // 2^44
            const unsigned long long want = (unsigned long long)((double)a.top_p * one);
            __shared__ unsigned long long above_s;       // mass of the ids above the prefix found so far
            __shared__ int found_s;                      // the nucleus ends inside the eligible ids
            if (tid == 0) { prefix_s = 0u; above_s = 0ull; found_s = 1; }
            __syncthreads();
            for (int pass = 0; pass < 4 && found_s; ++pass) {
                const int shift = 24 - 8 * pass;
                if (tid < 256) mass[tid] = 0ull;
                __syncthreads();
                const unsigned prefix = prefix_s;
                const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
                for (int i = tid; i < V; i += SAMPLE_THREADS) {
                    const float z = row[i] * a.inv_temperature;
                    const unsigned key = orderable(z);
                    if ((key & mask) != prefix) continue;
                    const float pr = expf(z - m) / denom;
                    if (pr >= thresh) atomicAdd(&mass[(key >> shift) & 0xff], (unsigned long long)((double)pr * one));
                }
                __syncthreads();
                if (tid == 0) {
                    unsigned long long cum = above_s;
                    int b = 255;
                    for (; b >= 0; --b) {
                        if (cum + mass[b] >= want) break;
                        cum += mass[b];
                    }
                    if (b < 0) found_s = 0;              // even all eligible ids stay below top_p: all are kept
                    else { prefix_s = prefix | ((unsigned)b << shift); above_s = cum; }
                }
                __syncthreads();
            }
            if (found_s) {
                kth = prefix_s;
                // ids with the key kth have the same probability: as many of them as it takes to reach top_p
                const float z_k = [&] {
                    const unsigned u = (kth & 0x80000000u) ? (kth & 0x7fffffffu) : ~kth;
                    return __uint_as_float(u);
                }();
                const unsigned long long each = (unsigned long long)((double)(expf(z_k - m) / denom) * one);
                const unsigned long long need = want > above_s ? want - above_s : 0ull;
                tie_keep = each > 0ull ? (int)min((unsigned long long)0x7fffffff, (need + each - 1ull) / each) : 0x7fffffff;
                if (tie_keep < 1) tie_keep = 1;
            }
            __syncthreads();
        }
        // rank of this thread's first tie among the ties of the row, in id order
        int my_ties = 0;
        if (tie_keep != 0x7fffffff)
            for (int i = lo; i < hi; ++i) {
                const float z = row[i] * a.inv_temperature;
                if (orderable(z) == kth && expf(z - m) / denom >= thresh) ++my_ties;
            }
        int tie_rank = tie_keep != 0x7fffffff ? block_exclusive_scan(my_ties, iscratch, &itotal) : 0;
        __syncthreads();
        const int tie_rank0 = tie_rank;
        auto kept_prob = [&](int i, int& rank) -> float {
            const float z = row[i] * a.inv_temperature;
            const float pr = expf(z - m) / denom;
            if (!(pr >= thresh)) return -1.f;
            const unsigned key = orderable(z);
            if (key > kth) return pr;
            if (key == kth) return rank++ < tie_keep ? pr : -1.f;
            return -1.f;
        };
        float kept = 0.f;
        for (int i = lo; i < hi; ++i) {
            const float pr = kept_prob(i, tie_rank);
            if (pr >= 0.f) kept += pr;
        }
        const float before = block_exclusive_scan_f(kept, fscratch, &ftotal);
        const float r = u * ftotal;
        // the first id whose running sum reaches r: the thread whose chunk crosses r walks it
        if (tid == 0) { itotal = -1; n_cand = -1; }
        __syncthreads();
        int found = -1, last_kept = -1;
        float run = before;
        tie_rank = tie_rank0;
        for (int i = lo; i < hi; ++i) {
            const float pr = kept_prob(i, tie_rank);
            if (pr >= 0.f) {
                last_kept = i;
                run += pr;
                if (found < 0 && r <= run) found = i;
            }
        }
        if (found >= 0) atomicMin((unsigned*)&itotal, (unsigned)found);   // -1 is the largest unsigned
        if (last_kept >= 0) atomicMax(&n_cand, last_kept);
        __syncthreads();
        if (tid == 0) out[blockIdx.x] = itotal >= 0 ? itotal : max(n_cand, 0);
        return;
    }

    // 2. exact top-k: radix select of the k-th largest scaled logit
    const int k = min(min(a.top_k, MAX_TOP_K), V);
    if (tid == 0) { prefix_s = 0u; remaining_s = k; }
    __syncthreads();
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const unsigned prefix = prefix_s;
        const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = tid; i < V; i += SAMPLE_THREADS) {
            const unsigned key = orderable(row[i] * a.inv_temperature);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int rem = remaining_s;
            int b = 255;
            for (; b > 0; --b) {
                if (hist[b] >= rem) break;
                rem -= hist[b];
            }
            prefix_s = prefix | ((unsigned)b << shift);
            remaining_s = rem;
        }
        __syncthreads();
    }
    const unsigned kth = prefix_s;          // key of the k-th largest; remaining_s ties of it are kept
    const int ties_needed = remaining_s;
    if (tid == 0) n_cand = 0;
    __syncthreads();
    int my_ties = 0;
    for (int i = lo; i < hi; ++i) {
        const float z = row[i] * a.inv_temperature;
        const unsigned key = orderable(z);
        if (key > kth) {
            const int slot = atomicAdd(&n_cand, 1);
            cand_z[slot] = z;
            cand_id[slot] = i;
        } else if (key == kth) {
            ++my_ties;
        }
    }
    const int tie_rank = block_exclusive_scan(my_ties, iscratch, &itotal);
    __syncthreads();
    const int n_above = n_cand;
    {
        int rank = tie_rank;
        for (int i = lo; i < hi && rank < ties_needed; ++i) {
            const float z = row[i] * a.inv_temperature;
            if (orderable(z) == kth) {
                cand_z[n_above + rank] = z;
                cand_id[n_above + rank] = i;
                ++rank;
            }
        }
    }
    __syncthreads();
    for (int i = k + tid; i < MAX_TOP_K; i += SAMPLE_THREADS) { cand_z[i] = -INFINITY; cand_id[i] = 0x7fffffff; }
    __syncthreads();

    // 3. bitonic sort by (z descending, id ascending)
    for (int size = 2; size <= MAX_TOP_K; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const int i = tid;
            const int j = i ^ stride;
            if (j > i) {
                const bool up = (i & size) == 0;
                const float zi = cand_z[i], zj = cand_z[j];
                const int ii = cand_id[i], ij = cand_id[j];
                const bool i_first = zi > zj || (zi == zj && ii < ij);   // i belongs before j
                if (i_first != up) {
                    cand_z[i] = zj; cand_z[j] = zi;
                    cand_id[i] = ij; cand_id[j] = ii;
                }
            }
            __syncthreads();
        }
    }

    // 4. cut and draw, one thread, in the order and the float operations of the chain
    if (tid == 0) {
        int n = k;
        const float p0 = expf(cand_z[0] - m) / denom;
        if (a.min_p > 0.f) {
            const float thresh = p0 * a.min_p;
            for (int i = 0; i < n; ++i) {
                if (expf(cand_z[i] - m) / denom < thresh) { n = max(1, i); break; }
            }
        }
        if (a.top_p < 1.0f) {
            float cum = 0.f;
            for (int i = 0; i < n; ++i) {
                cum += expf(cand_z[i] - m) / denom;
                if (cum >= a.top_p) { n = i + 1; break; }
            }
        }
        float total = 0.f;
        for (int i = 0; i < n; ++i) total += expf(cand_z[i] - m) / denom;
        const float r = u * total;
        float run = 0.f;
        int pick = cand_id[0];
        for (int i = 0; i < n; ++i) {
            run += expf(cand_z[i] - m) / denom;
            if (r <= run) { pick = cand_id[i]; break; }
        }
        out[blockIdx.x] = pick;
    }
}

// ------------------------------------------------------- sample, many blocks per row
// The chain with 1 <= top_k <= 64 on a large vocabulary.  SP_PARTS blocks take a slice of the row each: they
// apply the penalties of the ids in their slice, keep the scaled logits of the slice in shared memory, find
// its maximum, its sum of exponentials and its k best candidates exactly (radix select in shared memory,
// ties to the lower id), and leave them in scratch.  The global k best are among those: the block that
// arrives last at the row's counter sorts the SP_PARTS * k candidates by (logit descending, id ascending),
// forms the row's maximum and denominator from the slices' and cuts and draws as sample_kernel does.
constexpr int SP_PARTS = 32;
constexpr int SP_THREADS = 256;
constexpr int SP_KMAX = 64;
constexpr int SP_SORT = SP_PARTS * SP_KMAX;          // 2048 candidates, a power of two

__global__ void __launch_bounds__(SP_THREADS)
sample_parts_kernel(float* __restrict__ logits, int V, long row_stride, SampleArgs a, const int* __restrict__ history,
                    const long long* __restrict__ rng, int* __restrict__ out, int* __restrict__ counters,
                    float* __restrict__ pmax, float* __restrict__ psum, float* __restrict__ cz, int* __restrict__ cid) {
    extern __shared__ float dyn[];
    __shared__ float fscratch[33];
    __shared__ int iscratch[32];
    __shared__ int itotal;
    __shared__ int hist[256];
    __shared__ unsigned prefix_s;
    __shared__ int remaining_s;
    __shared__ int n_cand;
    __shared__ int last_s;
    const int tid = threadIdx.x, r = blockIdx.y, part = blockIdx.x;
    float* row = logits + (long)r * row_stride;
    const int per = (V + SP_PARTS - 1) / SP_PARTS;
    const int lo = min(V, part * per), hi = min(V, lo + per), n = hi - lo;
    float* z = dyn;                                       // [per] scaled logits of the slice

    // 0. penalties of the ids of this slice, once per id, occurrences in window order (as sample_kernel)
    if (a.window > 0 && (a.repetition_penalty != 1.0f || a.presence_penalty != 0.0f)) {
        const int* h = history + (long)r * a.window;
        if (tid < a.window) {
            const int tok = h[tid];
            bool first = tok >= lo && tok < hi;
            for (int j = 0; j < tid && first; ++j) first = h[j] != tok;
            if (first) {
                float l = row[tok];
                for (int j = tid; j < a.window; ++j) {
                    if (h[j] != tok) continue;
                    l = l > 0.f ? l / a.repetition_penalty : l * a.repetition_penalty;
                    l -= a.presence_penalty;
                }
                row[tok] = l;
            }
        }
        __syncthreads();
    }
    // 1. the slice, its maximum and its sum of exponentials
    float m = -INFINITY;
    for (int i = tid; i < n; i += SP_THREADS) {
        const float v = row[lo + i] * a.inv_temperature;
        z[i] = v;
        m = fmaxf(m, v);
    }
    m = block_max(m, fscratch);
    float part_sum = 0.f;
    for (int i = tid; i < n; i += SP_THREADS) part_sum += expf(z[i] - m);
    part_sum = block_sum(part_sum, fscratch);
    // 2. the k best of the slice, exactly
    const int k = min(a.top_k, n);
    if (tid == 0) { prefix_s = 0u; remaining_s = k; }
    __syncthreads();
    for (int pass = 0; pass < 4 && k > 0; ++pass) {
        const int shift = 24 - 8 * pass;
        hist[tid] = 0;
        __syncthreads();
        const unsigned prefix = prefix_s;
        const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = tid; i < n; i += SP_THREADS) {
            const unsigned key = orderable(z[i]);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int rem = remaining_s;
            int b = 255;
            for (; b > 0; --b) {
                if (hist[b] >= rem) break;
                rem -= hist[b];
            }
            prefix_s = prefix | ((unsigned)b << shift);
            remaining_s = rem;
        }
        __syncthreads();
    }
    const unsigned kth = prefix_s;
    const int ties_needed = remaining_s;
    float* my_cz = cz + ((long)r * SP_PARTS + part) * SP_KMAX;
    int* my_cid = cid + ((long)r * SP_PARTS + part) * SP_KMAX;
    if (tid == 0) n_cand = 0;
    __syncthreads();
    // contiguous runs per thread, so that ties are taken in id order
    const int run = (n + SP_THREADS - 1) / SP_THREADS;
    const int t_lo = min(n, tid * run), t_hi = min(n, t_lo + run);
    int my_ties = 0;
    for (int i = t_lo; i < t_hi && k > 0; ++i) {
        const unsigned key = orderable(z[i]);
        if (key > kth) {
            const int slot = atomicAdd(&n_cand, 1);
            my_cz[slot] = z[i];
            my_cid[slot] = lo + i;
        } else if (key == kth) {
            ++my_ties;
        }
    }
    // exclusive scan of the ties over the 256 threads (8 warps)
    int tie_rank;
    {
        const int lane = tid & 31, warp = tid >> 5;
        int inc = my_ties;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += v;
        }
        __syncthreads();
        if (lane == 31) iscratch[warp] = inc;
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; ++w) before += iscratch[w];
        tie_rank = before + inc - my_ties;
    }
    __syncthreads();
    const int n_above = n_cand;
    {
        int rank = tie_rank;
        for (int i = t_lo; i < t_hi && rank < ties_needed; ++i) {
            if (orderable(z[i]) == kth) {
                my_cz[n_above + rank] = z[i];
                my_cid[n_above + rank] = lo + i;
                ++rank;
            }
        }
    }
    for (int i = k + tid; i < SP_KMAX; i += SP_THREADS) { my_cz[i] = -INFINITY; my_cid[i] = 0x7fffffff; }
    if (tid == 0) { pmax[r * SP_PARTS + part] = m; psum[r * SP_PARTS + part] = part_sum; }
    __threadfence();
    __syncthreads();
    if (tid == 0) last_s = atomicAdd(&counters[r], 1) == SP_PARTS - 1;
    __syncthreads();
    if (!last_s) return;
    __threadfence();

    // ---- the last block of the row: maximum and denominator of the row, in slice order
    float* sz = dyn;                                       // [SP_SORT]
    int* sid = reinterpret_cast<int*>(dyn + SP_SORT);      // [SP_SORT]
    float row_max, denom;
    {
        float mp = tid < SP_PARTS ? __ldcg(&pmax[r * SP_PARTS + tid]) : -INFINITY;
        row_max = block_max(mp, fscratch);
        float sp = tid < SP_PARTS ? __ldcg(&psum[r * SP_PARTS + tid]) * expf(mp - row_max) : 0.f;
        denom = block_sum(sp, fscratch);
    }
    for (int i = tid; i < SP_SORT; i += SP_THREADS) {
        sz[i] = __ldcg(&cz[(long)r * SP_SORT + i]);
        sid[i] = __ldcg(&cid[(long)r * SP_SORT + i]);
    }
    __syncthreads();
    for (int size = 2; size <= SP_SORT; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = tid; i < SP_SORT; i += SP_THREADS) {
                const int j = i ^ stride;
                if (j > i) {
                    const bool up = (i & size) == 0;
                    const float zi = sz[i], zj = sz[j];
                    const int ii = sid[i], ij = sid[j];
                    const bool i_first = zi > zj || (zi == zj && ii < ij);
                    if (i_first != up) { sz[i] = zj; sz[j] = zi; sid[i] = ij; sid[j] = ii; }
                }
            }
            __syncthreads();
        }
    }
    if (tid == 0) {
        const float u = uniform01((unsigned long long)rng[2 * r], (unsigned long long)rng[2 * r + 1]);
        int nn = min(a.top_k, V);
        const float p0 = expf(sz[0] - row_max) / denom;
        if (a.min_p > 0.f) {
            const float thresh = p0 * a.min_p;
            for (int i = 0; i < nn; ++i) {
                if (expf(sz[i] - row_max) / denom < thresh) { nn = max(1, i); break; }
            }
        }
        if (a.top_p < 1.0f) {
            float cum = 0.f;
            for (int i = 0; i < nn; ++i) {
                cum += expf(sz[i] - row_max) / denom;
                if (cum >= a.top_p) { nn = i + 1; break; }
            }
        }
        float total = 0.f;
        for (int i = 0; i < nn; ++i) total += expf(sz[i] - row_max) / denom;
        const float rr = u * total;
        float running = 0.f;
        int pick = sid[0];
        for (int i = 0; i < nn; ++i) {
            running += expf(sz[i] - row_max) / denom;
            if (rr <= running) { pick = sid[i]; break; }
        }
        out[r] = pick;
        counters[r] = 0;
    }
}

}  // namespace zlm

using namespace zlm;

// Floats of scratch zlm_sample_parts needs for `rows` rows (any content).  Beside it the caller keeps one int
// counter per row that is zero before the first call; every call leaves the counters zero.
ZLM_EXPORT long zlm_sample_parts_scratch(int rows) {
    if (rows <= 0) return 0;
    return (long)rows * (2 * SP_PARTS + 2 * SP_SORT);
}

// The chain for 1 <= top_k <= 64 with many blocks per row; ZLM_ERR_UNSUPPORTED for other options (the caller
// uses zlm_sample).  Same arguments as zlm_sample, then the scratch.
ZLM_EXPORT int zlm_sample_parts(float* logits, int rows, int V, long row_stride, float temperature, int top_k,
                                float top_p, float min_p, float repetition_penalty, float presence_penalty,
                                const int* history, int window, const long long* rng, int* out, int* counters,
                                float* scratch, long scratch_floats, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (V <= 0 || row_stride < V || !(temperature > 0.f) || window < 0 || window > SP_THREADS) return ZLM_ERR_BAD_ARG;
    const int per = (V + SP_PARTS - 1) / SP_PARTS;
    if (top_k < 1 || top_k > SP_KMAX || per > 8192 || V < 4 * SP_PARTS) return ZLM_ERR_UNSUPPORTED;
    if (!counters || !scratch || scratch_floats < zlm_sample_parts_scratch(rows)) return ZLM_ERR_BAD_ARG;
    SampleArgs a;
    a.inv_temperature = 1.0f / temperature;
    a.top_k = top_k;
    a.top_p = top_p;
    a.min_p = min_p;
    a.repetition_penalty = repetition_penalty;
    a.presence_penalty = presence_penalty;
    a.window = history ? window : 0;
    float* pmax = scratch;
    float* psum = pmax + (long)rows * SP_PARTS;
    float* cz = psum + (long)rows * SP_PARTS;
    int* cid = reinterpret_cast<int*>(cz + (long)rows * SP_SORT);
    const size_t smem = sizeof(float) * (size_t)(per > 2 * SP_SORT ? per : 2 * SP_SORT);
    sample_parts_kernel<<<dim3(SP_PARTS, rows), SP_THREADS, smem, stream>>>(logits, V, row_stride, a, history, rng, out,
                                                                         counters, pmax, psum, cz, cid);
    return launch_status();
}


ZLM_EXPORT int zlm_argmax(const float* logits, int rows, int V, long row_stride, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (V <= 0 || row_stride < V) return ZLM_ERR_BAD_ARG;
    static_assert(ARGMAX_PARTS == 32, "the last block reads one partial result per lane");
    for (int r0 = 0; r0 < rows; r0 += ARGMAX_MAX_ROWS) {
        const int n = rows - r0 < ARGMAX_MAX_ROWS ? rows - r0 : ARGMAX_MAX_ROWS;
        argmax_kernel<<<dim3(ARGMAX_PARTS, n), ARGMAX_THREADS, 0, stream>>>(logits + (long)r0 * row_stride, V, row_stride,
                                                                           out + r0);
    }
    return launch_status();
}

// logits are modified in place when penalties are on.  rng: [rows][2] = (seed, counter).
ZLM_EXPORT int zlm_sample(float* logits, int rows, int V, long row_stride, float temperature, int top_k, float top_p,
                          float min_p, float repetition_penalty, float presence_penalty, const int* history,
                          int window, const long long* rng, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (V <= 0 || row_stride < V || !(temperature > 0.f) || top_k < 0 || window < 0 || window > SAMPLE_THREADS)
        return ZLM_ERR_BAD_ARG;
    if (top_k > MAX_TOP_K) return ZLM_ERR_UNSUPPORTED;
    SampleArgs a;
    a.inv_temperature = 1.0f / temperature;
    a.top_k = top_k;
    a.top_p = top_p;
    a.min_p = min_p;
    a.repetition_penalty = repetition_penalty;
    a.presence_penalty = presence_penalty;
    a.window = history ? window : 0;
    sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, V, row_stride, a, history, rng, out);
    return launch_status();
}
