// Sampling from float logits [R, V].
//
//   argmax       the greedy token (tensorline/engine.py:43-44, batch_engine.py:386); the lowest
//                index wins a tie.
//   sample       softmax(logits / T) in float (tensorline/engine.py:45); nucleus top-p as in
//                engine.py:46-50: with tokens sorted by falling probability, a token is kept
//                while the mass before it is < top_p; the kept ones are renormalised.  The draw is
//                an inverse-CDF pick in vocabulary order from a uniform u in [0,1) that the host
//                derives from (seed, request, token index), so a request's tokens do not depend on
//                what else is in the batch.
//
// A row is sampled by one thread-block cluster (up to 8 blocks, each with a slice of the vocabulary);
// the blocks exchange their partial results through distributed shared memory.  The weights
// e_i = exp(l_i/T - max) are computed once and kept in shared memory.  There is no sort: the smallest
// kept weight is found by a four-pass radix selection on the float bit pattern (positive floats order
// like integers), each pass a histogram of probability mass by digit (11 bits, then three times 7).  Masses are summed as 64-bit
// fixed-point integers, so every sum is exact and does not depend on the order of additions: the same
// logits, temperature, top-p and uniform number give the same token whatever the launch looks like.
// Tokens of exactly equal weight are kept or dropped together (a sort would split them by position).
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define SAMPLE_THREADS 1024

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int ld, int V, int* __restrict__ out) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float* row = logits + (size_t)blockIdx.x * ld;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) { bv[wid] = best; bi[wid] = idx; }
    __syncthreads();
    if (wid == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        best = lane < nw ? bv[lane] : -INFINITY;
        idx = lane < nw ? bi[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
    }
}

// Wide vocabularies: a row is cut into ARGMAX_SLICES slices, one block each, whose winners go to
// `partial` [R, ARGMAX_SLICES] (value, index) and are merged by one warp per row.  One block per row would
// read 600 KB alone and take tens of microseconds, far longer than anything else after the output head.
#define ARGMAX_SLICES 32

__global__ void __launch_bounds__(256)
argmax_slice_kernel(const float* __restrict__ logits, int ld, int V, float* __restrict__ pval, int* __restrict__ pidx) {
    __shared__ float bv[8];
    __shared__ int bi[8];
    const int r = blockIdx.y, sl = blockIdx.x;
    const int per = (V + ARGMAX_SLICES - 1) / ARGMAX_SLICES;
    const int b = sl * per, e = min(V, b + per);
    const float* row = logits + (size_t)r * ld;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    grid_dependency_wait();
    grid_dependency_trigger();
    for (int i = b + threadIdx.x; i < e; i += blockDim.x) {
        const float v = row[i];
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) { bv[wid] = best; bi[wid] = idx; }
    __syncthreads();
    if (wid == 0) {
        best = lane < 8 ? bv[lane] : -INFINITY;
        idx = lane < 8 ? bi[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) { pval[r * ARGMAX_SLICES + sl] = best; pidx[r * ARGMAX_SLICES + sl] = idx; }
    }
}

__global__ void argmax_merge_kernel(const float* __restrict__ pval, const int* __restrict__ pidx, int* __restrict__ out) {
    const int r = blockIdx.x, lane = threadIdx.x;
    grid_dependency_wait();
    grid_dependency_trigger();
    float best = pval[r * ARGMAX_SLICES + lane];
    int idx = pidx[r * ARGMAX_SLICES + lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if (lane == 0) out[r] = idx == 0x7fffffff ? 0 : idx;
}

// `partial`: scratch of R * 2 * ARGMAX_SLICES 32-bit words for wide rows; null (or a narrow row) takes the
// one-block-per-row kernel.
TL_EXPORT int tl_argmax(const float* logits, int ld, int R, int V, int* out, void* partial, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (partial == nullptr || V < 8192 || R > 65535) {
        argmax_kernel<<<R, SAMPLE_THREADS, 0, stream>>>(logits, ld, V, out);
        return tl_launch_status();
    }
    float* pval = (float*)partial;
    int* pidx = (int*)partial + (size_t)R * ARGMAX_SLICES;
    const int e = launch_after_wait(argmax_slice_kernel, dim3(ARGMAX_SLICES, R), dim3(256), 0, stream, logits, ld, V, pval, pidx);
    if (e) return e;
    return launch_after_wait(argmax_merge_kernel, dim3(R), dim3(32), 0, stream, (const float*)pval, (const int*)pidx, out);
}

#define DRAW_THREADS 512
#define DRAW_MAX_CLUSTER 8
#define RADIX_BINS 192                                   // >= TOP_DIGITS and 128, a multiple of 32
#define RADIX_PASSES 4
#define MASS_SCALE 1099511627776.0f                      // 2^40: weights in (0, 1] as 64-bit fixed point
// A weight with a non-zero fixed-point mass lies in [2^-40, 1], so its top digit (bits 31..21: the exponent
// and two bits of the fraction) lies in [TOP_DIGIT_LO, TOP_DIGIT_HI].  The first pass, which sees every
// weight and a few dozen hot digits, adds into a histogram per warp with 32-bit atomics (low word, carry
// and high word apart; 64-bit shared-memory atomics under that contention were most of the kernel's time).
#define TOP_DIGIT_LO ((127 - 40) * 4)
#define TOP_DIGIT_HI (127 * 4)
#define TOP_DIGITS (TOP_DIGIT_HI - TOP_DIGIT_LO + 1)

typedef unsigned long long u64;

struct DrawShared {
    u64 hist[RADIX_BINS];                                // this block's mass by digit; later the cluster's
    u64 merged[RADIX_PASSES][RADIX_BINS];                // rank 0: the cluster's histogram of each pass
    u64 wsum[DRAW_THREADS / 32];
    unsigned int top_lo[DRAW_THREADS / 32][TOP_DIGITS];  // first pass: per-warp mass by top digit, low and high words
    unsigned int top_hi[DRAW_THREADS / 32][TOP_DIGITS];
    u64 x_sum[DRAW_MAX_CLUSTER];                         // x_*: one slot per rank, written by that rank
    u64 x_kept[DRAW_MAX_CLUSTER];
    float x_max[DRAW_MAX_CLUSTER];
    float x_best[DRAW_MAX_CLUSTER];
    int x_best_idx[DRAW_MAX_CLUSTER];
    u64 lane_sum[32];
    u64 sel_above;
    int sel_bin;
    float red[33];
    int redi[33];
};

__device__ __forceinline__ u64 fixed_mass(float e) { return __float2ull_rz(e * MASS_SCALE); }

__device__ __forceinline__ u64 warp_sum_u64(u64 v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over the block; every thread gets it.
__device__ __forceinline__ u64 block_sum_u64(u64 v, u64* wsum) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    v = warp_sum_u64(v);
    __syncthreads();
    if (lane == 0) wsum[wid] = v;
    __syncthreads();
    u64 t = 0;
    for (int w = 0; w < DRAW_THREADS / 32; ++w) t += wsum[w];
    return t;
}

// One (row, cluster).  CACHED: the block's weights are kept in shared memory behind DrawShared.
template <bool CACHED>
__global__ void __launch_bounds__(DRAW_THREADS)
draw_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
            const float* __restrict__ top_p, const float* __restrict__ uniform, int* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char draw_smem[];
    DrawShared& s = *reinterpret_cast<DrawShared*>(draw_smem);
    float* cache = reinterpret_cast<float*>(draw_smem + sizeof(DrawShared));
    cg::cluster_group cluster = cg::this_cluster();
    const int C = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
    const int r = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
    const float* row = logits + (size_t)r * ld;
    const int slice = (V + C - 1) / C;
    const int b = min(V, rank * slice), e_ = min(V, b + slice), n = e_ - b;
    const float temp = temperature[r];

    if (temp <= 0.f) {                                   // a greedy row inside a sampled batch
        float best = -INFINITY; int idx = 0x7fffffff;
        for (int i = b + tid; i < e_; i += DRAW_THREADS) {
            const float v = row[i];
            if (v > best || (v == best && i < idx)) { best = v; idx = i; }
        }
        const float bm = block_max(best, s.red);
        if (tid == 0) s.redi[0] = 0x7fffffff;
        __syncthreads();
        if (best == bm && idx != 0x7fffffff) atomicMin(&s.redi[0], idx);
        __syncthreads();
        if (tid < C) {
            *cluster.map_shared_rank(&s.x_best[rank], tid) = bm;
            *cluster.map_shared_rank(&s.x_best_idx[rank], tid) = s.redi[0];
        }
        cluster.sync();
        if (rank == 0 && tid == 0) {
            float v = -INFINITY; int w = 0x7fffffff;
            for (int k = 0; k < C; ++k)
                if (s.x_best[k] > v || (s.x_best[k] == v && s.x_best_idx[k] < w)) { v = s.x_best[k]; w = s.x_best_idx[k]; }
            out[r] = w == 0x7fffffff ? 0 : w;
        }
        return;
    }

    // zero the histograms that peers add into, before anyone can get there
    for (int k = tid; k < RADIX_PASSES * RADIX_BINS; k += DRAW_THREADS) (&s.merged[0][0])[k] = 0;

    const float inv_t = 1.0f / temp;
    float mx = -INFINITY;
    for (int i = b + tid; i < e_; i += DRAW_THREADS) mx = fmaxf(mx, row[i] * inv_t);
    mx = block_max(mx, s.red);
    if (tid < C) *cluster.map_shared_rank(&s.x_max[rank], tid) = mx;
    cluster.sync();
    mx = s.x_max[0];
    for (int k = 1; k < C; ++k) mx = fmaxf(mx, s.x_max[k]);

    auto weight = [&](int i) -> float {                  // i: index within the slice
        if (CACHED) return cache[i];
        return expf(row[b + i] * inv_t - mx);
    };
    u64 z = 0;
    for (int i = tid; i < n; i += DRAW_THREADS) {
        const float e = expf(row[b + i] * inv_t - mx);
        if (CACHED) cache[i] = e;
        z += fixed_mass(e);
    }
    z = block_sum_u64(z, s.wsum);
    if (tid < C) *cluster.map_shared_rank(&s.x_sum[rank], tid) = z;
    cluster.sync();
    z = 0;
    for (int k = 0; k < C; ++k) z += s.x_sum[k];

    // The smallest kept weight.  A weight x is kept iff mass{e > x} < target; the kept ones are the
    // top of the order, so the digit of the smallest one is the lowest non-empty bin whose mass above
    // is still < target.
    unsigned int thr_bits = 0u;                          // keep everything
    const float tp = top_p[r];
    if (tp < 1.0f) {
        u64 target = (u64)((double)tp * (double)z);
        if (target < 1) target = 1;                      // the largest weight is always kept
        u64 above = 0;
        unsigned int prefix = 0;
        for (int pass = 0; pass < RADIX_PASSES; ++pass) {
            const int shift = 21 - 7 * pass;             // passes 1..3: bits 20..14, 13..7, 6..0
            for (int k = tid; k < RADIX_BINS; k += DRAW_THREADS) s.hist[k] = 0;
            if (pass == 0) {
                for (int k = tid; k < (DRAW_THREADS / 32) * TOP_DIGITS; k += DRAW_THREADS) {
                    (&s.top_lo[0][0])[k] = 0;
                    (&s.top_hi[0][0])[k] = 0;
                }
                __syncthreads();
                unsigned int* lo = s.top_lo[tid >> 5];
                unsigned int* hi = s.top_hi[tid >> 5];
                for (int i = tid; i < n; i += DRAW_THREADS) {
                    const float e = weight(i);
                    const u64 q = fixed_mass(e);
                    if (q) {
                        const int d = min(max((int)(__float_as_uint(e) >> 21) - TOP_DIGIT_LO, 0), TOP_DIGITS - 1);
                        const unsigned int ql = (unsigned int)q, qh = (unsigned int)(q >> 32);
                        const unsigned int old = atomicAdd(&lo[d], ql);
                        const unsigned int up = qh + (old + ql < old ? 1u : 0u);
                        if (up) atomicAdd(&hi[d], up);
                    }
                }
                __syncthreads();
                for (int k = tid; k < TOP_DIGITS; k += DRAW_THREADS) {
                    u64 t = 0;
                    for (int w = 0; w < DRAW_THREADS / 32; ++w) t += ((u64)s.top_hi[w][k] << 32) + s.top_lo[w][k];
                    s.hist[k] = t;
                }
            } else {
                __syncthreads();
                for (int i = tid; i < n; i += DRAW_THREADS) {
                    const float e = weight(i);
                    const unsigned int bits = __float_as_uint(e);
                    if ((bits >> (shift + 7)) == prefix) {
                        const u64 q = fixed_mass(e);
                        if (q) atomicAdd(&s.hist[(bits >> shift) & 127u], q);
                    }
                }
            }
            __syncthreads();
            u64* total = cluster.map_shared_rank(&s.merged[pass][0], 0);
            for (int k = tid; k < RADIX_BINS; k += DRAW_THREADS)
                if (s.hist[k]) atomicAdd(&total[k], s.hist[k]);
            cluster.sync();
            for (int k = tid; k < RADIX_BINS; k += DRAW_THREADS) s.hist[k] = total[k];
            __syncthreads();
            if (tid < 32) {                              // lane L owns RADIX_BINS / 32 bins in a row
                u64 mine = 0;
                for (int k = 0; k < RADIX_BINS / 32; ++k) mine += s.hist[lane * (RADIX_BINS / 32) + k];
                s.lane_sum[lane] = mine;
                __syncwarp();
                u64 run = above;
                for (int l = lane + 1; l < 32; ++l) run += s.lane_sum[l];
                int cand = 0x7fffffff;
                u64 cand_above = 0;
                for (int k = RADIX_BINS / 32 - 1; k >= 0; --k) {
                    const int bin = lane * (RADIX_BINS / 32) + k;
                    const u64 h = s.hist[bin];
                    if (h && run < target) { cand = bin; cand_above = run; }
                    run += h;
                }
                int lowest = cand;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) lowest = min(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
                if (cand == lowest && cand != 0x7fffffff) { s.sel_bin = cand; s.sel_above = cand_above; }
                if (lowest == 0x7fffffff && lane == 0) { s.sel_bin = 0; s.sel_above = above; }
            }
            __syncthreads();
            prefix = pass == 0 ? (unsigned int)(s.sel_bin + TOP_DIGIT_LO) : (prefix << 7) | (unsigned int)s.sel_bin;
            above = s.sel_above;
        }
        thr_bits = prefix;
    }

    // inverse CDF over the kept tokens in vocabulary order; thread t owns a contiguous range of the slice
    const int per = (n + DRAW_THREADS - 1) / DRAW_THREADS;
    const int tb = min(n, tid * per), te = min(n, tb + per);
    u64 mine = 0;
    for (int i = tb; i < te; ++i) {
        const float e = weight(i);
        if (__float_as_uint(e) >= thr_bits) mine += fixed_mass(e);
    }
    // exclusive scan over the block's threads
    u64 incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    __syncthreads();
    if (lane == 31) s.wsum[tid >> 5] = incl;
    __syncthreads();
    u64 before = incl - mine, block_total = 0;
    for (int w = 0; w < DRAW_THREADS / 32; ++w) {
        if (w < (tid >> 5)) before += s.wsum[w];
        block_total += s.wsum[w];
    }
    if (tid < C) *cluster.map_shared_rank(&s.x_kept[rank], tid) = block_total;
    cluster.sync();
    u64 base = 0, total = 0;
    for (int k = 0; k < C; ++k) {
        if (k < rank) base += s.x_kept[k];
        total += s.x_kept[k];
    }
    const u64 goal = (u64)((double)uniform[r] * (double)total);      // < total, since u < 1
    before += base;
    if (mine && goal >= before && goal < before + mine) {              // exactly one thread of the cluster
        u64 run = before;
        for (int i = tb; i < te; ++i) {
            const float e = weight(i);
            if (__float_as_uint(e) >= thr_bits) {
                run += fixed_mass(e);
                if (run > goal) { out[r] = b + i; break; }
            }
        }
    }
}

TL_EXPORT int tl_sample(const float* logits, int ld, int R, int V, const float* temperature,
                        const float* top_p, const float* uniform, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (R > 65535 || V <= 0) return 1;
    int C = 1;
    while (C < DRAW_MAX_CLUSTER && V / (2 * C) >= 2048) C *= 2;
    const int slice = (V + C - 1) / C;
    const size_t limit = 227 * 1024;
    const bool cached = sizeof(DrawShared) + (size_t)slice * 4 <= limit;
    const size_t smem = sizeof(DrawShared) + (cached ? (size_t)slice * 4 : 0);
    static bool attr_done_on[TL_MAX_DEVICES] = {};
    const int dev = tl_device_index();
    if (dev < 0) return 1;
    bool& attr_done = attr_done_on[dev];
    if (!attr_done) {
        cudaError_t e = cudaFuncSetAttribute(draw_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(draw_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(DrawShared));
        if (e != cudaSuccess) return (int)e;
        attr_done = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(C, R);
    cfg.blockDim = dim3(DRAW_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cached
        ? cudaLaunchKernelEx(&cfg, draw_kernel<true>, logits, ld, V, temperature, top_p, uniform, out)
        : cudaLaunchKernelEx(&cfg, draw_kernel<false>, logits, ld, V, temperature, top_p, uniform, out);
    if (e != cudaSuccess) return (int)e;
    return tl_launch_status();
}
