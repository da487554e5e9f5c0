// Sampling from float logits [R, V], one block per row.
//
//   argmax       the greedy token (tensorline/engine.py:43-44, batch_engine.py:386); the lowest
//                index wins a tie.
//   sample       softmax(logits / T) in float (tensorline/engine.py:45); nucleus top-p as in
//                engine.py:46-50: with tokens sorted by falling probability, a token is kept
//                while the mass before it is < top_p; the kept ones are renormalised.  The draw is
//                an inverse-CDF pick in vocabulary order from a uniform u in [0,1) that the host
//                derives from (seed, request, token index), so a request's tokens do not depend on
//                what else is in the batch.  No sort: the smallest kept probability is found by a
//                bisection on the float bit pattern (positive floats order like integers).
#include "common.cuh"

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

TL_EXPORT int tl_argmax(const float* logits, int ld, int R, int V, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    argmax_kernel<<<R, SAMPLE_THREADS, 0, stream>>>(logits, ld, V, out);
    return tl_launch_status();
}

// Rows with temperature <= 0 get the argmax.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
              const float* __restrict__ top_p, const float* __restrict__ uniform, int* __restrict__ out) {
    __shared__ float red[33];
    __shared__ float scan[SAMPLE_THREADS];
    __shared__ int pick;
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)r * ld;
    const float temp = temperature[r];
    if (temp <= 0.f) {                                  // greedy row inside a sampled batch
        float best = -INFINITY; int idx = 0x7fffffff;
        for (int i = tid; i < V; i += blockDim.x) {
            const float v = row[i];
            if (v > best || (v == best && i < idx)) { best = v; idx = i; }
        }
        const float bm = block_max(best, red);
        int cand = (best == bm) ? idx : 0x7fffffff;
        // smallest index among the threads that hold the maximum
        __shared__ int mi;
        if (tid == 0) mi = 0x7fffffff;
        __syncthreads();
        atomicMin(&mi, cand);
        __syncthreads();
        if (tid == 0) out[r] = mi;
        return;
    }
    const float inv_t = 1.0f / temp;
    float mx = -INFINITY;
    for (int i = tid; i < V; i += blockDim.x) mx = fmaxf(mx, row[i] * inv_t);
    mx = block_max(mx, red);
    float z = 0.f;
    for (int i = tid; i < V; i += blockDim.x) z += expf(row[i] * inv_t - mx);
    z = block_sum(z, red);

    // smallest kept weight (weights e_i = exp(l_i/T - max) lie in (0, 1])
    unsigned int thr_bits = 0u;                          // keep everything
    const float tp = top_p[r];
    if (tp < 1.0f) {
        const float target = tp * z;
        unsigned int lo = 0u, hi = 0x3f800000u;          // bit patterns of 0.0f and 1.0f
        // find the smallest tau with mass{e > tau} < target
        while (lo < hi) {
            const unsigned int mid = lo + ((hi - lo) >> 1);
            const float tau = __uint_as_float(mid);
            float mass = 0.f;
            for (int i = tid; i < V; i += blockDim.x) {
                const float e = expf(row[i] * inv_t - mx);
                if (e > tau) mass += e;
            }
            mass = block_sum(mass, red);
            if (mass < target) hi = mid; else lo = mid + 1;
        }
        thr_bits = lo;
    }
    const float thr = __uint_as_float(thr_bits);

    // inverse CDF over the kept tokens in vocabulary order; thread t owns a contiguous range
    const int per = (V + blockDim.x - 1) / blockDim.x;
    const int b = tid * per, e_ = min(V, b + per);
    float part = 0.f;
    for (int i = b; i < e_; ++i) {
        const float e = expf(row[i] * inv_t - mx);
        if (e >= thr) part += e;
    }
    scan[tid] = part;
    if (tid == 0) pick = -1;
    __syncthreads();
    if (tid == 0) {                                      // serial scan over 1024 partial sums
        float run = 0.f;
        for (int k = 0; k < (int)blockDim.x; ++k) { const float v = scan[k]; scan[k] = run; run += v; }
        red[0] = run;
    }
    __syncthreads();
    const float total = red[0];
    const float goal = uniform[r] * total;
    const float before = scan[tid];
    if (part > 0.f && goal >= before && goal < before + part) {
        float run = before;
        int found = -1, last = -1;
        for (int i = b; i < e_; ++i) {
            const float e = expf(row[i] * inv_t - mx);
            if (e >= thr) {
                last = i;
                run += e;
                if (run > goal) { found = i; break; }
            }
        }
        atomicMax(&pick, found >= 0 ? found : last);
    }
    __syncthreads();
    if (tid == 0) {
        int ans = pick;
        if (ans < 0) {                                   // rounding at the far end: last kept token
            for (int i = V - 1; i >= 0; --i)
                if (expf(row[i] * inv_t - mx) >= thr) { ans = i; break; }
        }
        out[r] = ans < 0 ? 0 : ans;
    }
}

TL_EXPORT int tl_sample(const float* logits, int ld, int R, int V, const float* temperature,
                        const float* top_p, const float* uniform, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    sample_kernel<<<R, SAMPLE_THREADS, 0, stream>>>(logits, ld, V, temperature, top_p, uniform, out);
    return tl_launch_status();
}
