// Embedding gather, residual-add + RMSNorm, SwiGLU activation.
//
// Each kernel has a plain reference in tests/plain/qwen2_plain.py.  Formulas:
//   embedding   x[t,:] = E[ids[t],:]                       (tensorline/paged.py:240)
//   add+RMSNorm x += r;  h = cast(x * rsqrt(mean(x^2)+eps)) * w   (tensorline/fused.py:19-32;
//               the cast to the activation type comes before the weight multiply, fused.py:32)
//   SwiGLU      m = silu(g) * u,  silu(z) = z / (1 + e^-z), from the fused gate|up product
// The residual stream x is float in both engines, so the residual sum is a 32-bit sum.
#include "common.cuh"

// 1 if this library was compiled as the checking build (-DTL_CHECK=1).
TL_EXPORT int tl_check_build() { return TL_CHECKING; }

// ------------------------------------------------------------------ embedding
template <typename TW>
__global__ void embed_kernel(float* __restrict__ x, const TW* __restrict__ table,
                             const int* __restrict__ ids, int H) {
    const int t = blockIdx.x;
    grid_dependency_wait();
    grid_dependency_trigger();
    const TW* row = table + (size_t)ids[t] * H;
    float* out = x + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = to_f<TW>(row[i]);
}

TL_EXPORT int tl_embed(void* x, const void* table, int table_dtype, const int* ids, int T, int H,
                       cudaStream_t stream) {
    if (T <= 0) return 0;
    if (table_dtype == TL_F32)
        launch_after_wait(embed_kernel<float>, dim3(T), dim3(256), 0, stream, (float*)x, (const float*)table, ids, H);
    else
        launch_after_wait(embed_kernel<bf16>, dim3(T), dim3(256), 0, stream, (float*)x, (const bf16*)table, ids, H);
    return tl_launch_status();
}

// ------------------------------------------------------------------ residual add + RMSNorm
// One block per output row.  rows == nullptr: row i of x; else row rows[i] (x is then only
// read, as for the final norm on the rows that want logits).
template <typename TA, typename TW>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TA* __restrict__ r,
                                   const TW* __restrict__ w, TA* __restrict__ out,
                                   const int* __restrict__ rows, int H, float eps, int write_x) {
    __shared__ float red[33];
    const int i = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[i] : i) * H;
    float* xr = x + src;
    const TA* rr = r ? r + src : nullptr;
    TA* o = out + (size_t)i * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = xr[c];
        if (rr) {
            v = v + to_f<TA>(rr[c]);
            if (write_x) xr[c] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = xr[c];
        if (rr && !write_x) v = v + to_f<TA>(rr[c]);
        const float n = to_f<TA>(from_f<TA>(v * rstd));          // cast first, then the weight
        o[c] = from_f<TA>(n * to_f<TW>(w[c]));
    }
}

// The fast path: H a multiple of 4, each thread keeps its NV chunks of 4 values in registers, so
// every load of the row is in flight at once and x, r are read exactly once.  Same arithmetic.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[4]) {
        const uint2 t = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[4]) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 t;
        t.x = *reinterpret_cast<uint32_t*>(&a); t.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = t;
    }
};

// `partial` (instead of r): the addend is still in pieces, [splits][rows of x][H] float, as a split-K product
// leaves them; they are summed in split order and rounded to the activation type first, which is what a
// separate reduction pass would have handed over as r.
template <typename TA, typename TW, int NV, bool PIECES>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ x, const TA* __restrict__ r,
                                       const TW* __restrict__ w, TA* __restrict__ out,
                                       const int* __restrict__ rows, int H, float eps, int write_x,
                                       const float* __restrict__ partial, int splits, size_t plane) {
    __shared__ float red[33];
    const int i = blockIdx.x, nvec = H >> 2;
    float v[NV][4], wv[NV][4];
    // The weights are nobody's output.  A launch of few rows (a decode step) reads them before the wait for the
    // kernel in front, so only the row itself is fetched after it; a launch of many rows keeps all its loads
    // together behind the wait (the wait would otherwise stand between two memory latencies in every block).
    const bool early = gridDim.x <= 128;
    if (early) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < nvec) Vec4<TW>::load(w + 4 * c, wv[k]);
        }
    }
    grid_dependency_wait();
    grid_dependency_trigger();
    const size_t src = (size_t)(rows ? rows[i] : i) * H;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < nvec) {
            Vec4<float>::load(x + src + 4 * c, v[k]);
            if (!early) Vec4<TW>::load(w + 4 * c, wv[k]);
        }
    }
    if (PIECES) {                                        // an instantiation of its own: the plain one keeps its registers
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < nvec) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                for (int sp = 0; sp < splits; ++sp) {
                    float pv[4];
                    Vec4<float>::load(partial + sp * plane + src + 4 * c, pv);
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[e] += pv[e];
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) v[k][e] = v[k][e] + to_f<TA>(from_f<TA>(acc[e]));
                if (write_x) Vec4<float>::store(x + src + 4 * c, v[k]);
            }
        }
    } else if (r) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < nvec) {
                float rv[4];
                Vec4<TA>::load(r + src + 4 * c, rv);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[k][e] = v[k][e] + rv[e];
                if (write_x) Vec4<float>::store(x + src + 4 * c, v[k]);
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k)
        if (threadIdx.x + k * blockDim.x < nvec)
#pragma unroll
            for (int e = 0; e < 4; ++e) ss = fmaf(v[k][e], v[k][e], ss);
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < nvec) {
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = to_f<TA>(from_f<TA>(v[k][e] * rstd)) * wv[k][e];
            Vec4<TA>::store(out + (size_t)i * H + 4 * c, o);
        }
    }
}

template <typename TA, typename TW>
static int launch_add_rmsnorm(void* x, const void* r, const void* w, void* out, const int* rows, int R, int H,
                              float eps, int write_x, const float* partial, int splits, size_t plane, cudaStream_t stream) {
    const int nvec = H >> 2;
    const bool vec = (H & 3) == 0 && nvec <= 8192 &&
                     ((((uintptr_t)x | (uintptr_t)r | (uintptr_t)w | (uintptr_t)out | (uintptr_t)partial) & 15) == 0);
    if (partial && !vec) return 1;                       // pieces only on the vector path; the caller sums them first
#define VLAUNCH(NV) { int th = ((nvec + NV - 1) / NV + 31) / 32 * 32; \
        if (partial) launch_after_wait(add_rmsnorm_vec_kernel<TA, TW, NV, true>, dim3(R), dim3(th), 0, stream, (float*)x, (const TA*)r, (const TW*)w, (TA*)out, rows, H, eps, write_x, partial, splits, plane); \
        else launch_after_wait(add_rmsnorm_vec_kernel<TA, TW, NV, false>, dim3(R), dim3(th), 0, stream, (float*)x, (const TA*)r, (const TW*)w, (TA*)out, rows, H, eps, write_x, partial, splits, plane); }
    if (!vec) add_rmsnorm_kernel<TA, TW><<<R, 256, 0, stream>>>((float*)x, (const TA*)r, (const TW*)w, (TA*)out, rows, H, eps, write_x);
    else if (nvec <= 1024) VLAUNCH(1)
    else if (nvec <= 2048) VLAUNCH(2)
    else if (nvec <= 4096) VLAUNCH(4)
    else VLAUNCH(8)
#undef VLAUNCH
    return 0;
}

TL_EXPORT int tl_add_rmsnorm(void* x, const void* r, const void* w, int w_dtype, void* out, int act_dtype,
                             const int* rows, int R, int H, float eps, int write_x, const float* partial, int splits,
                             long long plane, cudaStream_t stream) {
    if (R <= 0) return 0;
    int e;
    if (act_dtype == TL_F32) {
        if (w_dtype == TL_F32) e = launch_add_rmsnorm<float, float>(x, r, w, out, rows, R, H, eps, write_x, partial, splits, (size_t)plane, stream);
        else e = launch_add_rmsnorm<float, bf16>(x, r, w, out, rows, R, H, eps, write_x, partial, splits, (size_t)plane, stream);
    } else {
        if (w_dtype == TL_F32) e = launch_add_rmsnorm<bf16, float>(x, r, w, out, rows, R, H, eps, write_x, partial, splits, (size_t)plane, stream);
        else e = launch_add_rmsnorm<bf16, bf16>(x, r, w, out, rows, R, H, eps, write_x, partial, splits, (size_t)plane, stream);
    }
    return e ? e : tl_launch_status();
}

// ------------------------------------------------------------------ SwiGLU activation
// gu is [T, 2*I], out [T, I].  Gate and up columns alternate in blocks of `blk` columns: out column c has its
// gate at (c / blk) * 2 blk + c % blk and its up value blk columns further.  blk = I is the plain layout
// (gate in [0, I), up in [I, 2I)); blk = 64 is what a product against interleaved weight rows leaves.
template <typename TA>
__global__ void silu_mul_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int I, int blk, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I;
        const int c = (int)(idx - t * I);
        const int gc = (c / blk) * 2 * blk + c % blk;
        const float g = to_f<TA>(gu[t * 2 * I + gc]);
        const float u = to_f<TA>(gu[t * 2 * I + gc + blk]);
        if constexpr (sizeof(TA) == 4) out[idx] = (g / (1.0f + expf(-g))) * u;     // the 32-bit engine: exact division
        else                           out[idx] = from_f<TA>(tl_silu_mul(g, u));
    }
}

// 8 values (16 bytes of bfloat16) per thread and chunk: requires I % 8 == 0 and blk % 8 == 0.  grid (column
// groups, tokens): no division per element; with many tokens a thread takes two chunks a block's width apart,
// so four 16-byte loads are in flight before the first is used; with few it takes one, for more blocks.
template <int CHUNKS>
__global__ void __launch_bounds__(256) silu_mul_vec8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int I, int blk) {
    const size_t t = blockIdx.y;
    const int c0 = (blockIdx.x * 256 * CHUNKS + threadIdx.x) * 8;
    grid_dependency_wait();
    grid_dependency_trigger();
    const bf16* row = gu + t * 2 * (size_t)I;
    uint4 gv[CHUNKS], uv[CHUNKS];
    int cs[CHUNKS];
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) cs[k] = c0 + k * 256 * 8;
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
        if (cs[k] < I) {
            const int gc = (cs[k] / blk) * 2 * blk + cs[k] % blk;
            gv[k] = *reinterpret_cast<const uint4*>(row + gc);
            uv[k] = *reinterpret_cast<const uint4*>(row + gc + blk);
        }
    }
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
        if (cs[k] >= I) continue;
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv[k]);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv[k]);
        uint4 ov;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float g0 = __low2float(g2[e]), g1 = __high2float(g2[e]);
            const float u0 = __low2float(u2[e]), u1 = __high2float(u2[e]);
            o2[e] = __floats2bfloat162_rn(tl_silu_mul(g0, u0), tl_silu_mul(g1, u1));
        }
        *reinterpret_cast<uint4*>(out + t * I + cs[k]) = ov;
    }
}

TL_EXPORT int tl_silu_mul(const void* gu, void* out, int act_dtype, int T, int I, int blk, cudaStream_t stream) {
    const size_t total = (size_t)T * I;
    if (total == 0) return 0;
    if (blk <= 0 || I % blk) return 1;
    const int threads = 256;
    if (act_dtype == TL_BF16 && (I & 7) == 0 && (blk & 7) == 0 && T <= 65535 && ((((uintptr_t)gu | (uintptr_t)out) & 15) == 0)) {
        if (T >= 256)
            return launch_after_wait(silu_mul_vec8_kernel<2>, dim3((unsigned)((I / 8 + 511) / 512), (unsigned)T), dim3(threads), 0, stream,
                                     (const bf16*)gu, (bf16*)out, I, blk);
        return launch_after_wait(silu_mul_vec8_kernel<1>, dim3((unsigned)((I / 8 + 255) / 256), (unsigned)T), dim3(threads), 0, stream,
                                 (const bf16*)gu, (bf16*)out, I, blk);
    }
    const size_t cap = (size_t)tl_num_sms() * 16;
    const int blocks = (int)((total + threads - 1) / threads < cap ? (total + threads - 1) / threads : cap);
    if (act_dtype == TL_F32)
        silu_mul_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, I, blk, total);
    else
        silu_mul_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, I, blk, total);
    return tl_launch_status();
}
