// Bias add + rotary position encoding + write of keys and values into cache pages, one kernel.
//
// Input: the fused q|k|v projection of every token of the step, [T, (nq + 2 nkv) * d].
// For each token:  q and k get their bias and the rotate-half rotation
//     a = x[i], b = x[i + rot/2]:  x[i] = a cos - b sin,  x[i + rot/2] = b cos + a sin
// (tensorline/fused.py:47-51), angle = pos * inv_freq[i] in float, accurate sincosf;
// dimensions past `rot` (partial rotary) pass through.  q is written back in place, the rotated
// k and the biased v go to the page `table[slot][pos / page]` at offset `pos % page`
// (tensorline/paged.py:202, :252-253).  Pages are laid out [page, kv head, offset, d] so that one
// head's part of a page is contiguous.
//
// Two options of other position encodings and mixers are arguments, not copies of the kernel: the pairing of
// the rotated dimensions (`interleaved`: pair i is dimensions (2i, 2i + 1) instead of (i, i + rot/2)), and an
// RMS norm of every q and k head over its d dimensions with a weight of its own (`q_norm`, `k_norm`, `norm_eps`),
// applied after the bias and before the rotation, statistics in float.
#include "common.cuh"

// grid (T, heads): one block per (token, head), one thread per pair of dimensions, so that all loads
// of a token are in flight together (a decode step has few tokens; latency, not bandwidth, is its cost).
template <typename TA, typename TW>
__global__ void rope_kv_kernel(TA* __restrict__ qkv, const TW* __restrict__ bias,
                               const int* __restrict__ pos, const int* __restrict__ req_slot,
                               const int* __restrict__ table, int max_pages, int page_size,
                               const float* __restrict__ inv_freq, int rot, int nq, int nkv, int d,
                               TA* __restrict__ k_pages, TA* __restrict__ v_pages, int interleaved,
                               const float* __restrict__ q_norm, const float* __restrict__ k_norm, float norm_eps,
                               const TlLimits L) {
    __shared__ float red[33];
    const int t = blockIdx.x, hh = blockIdx.y;
    const int p = pos[t];
    const int half = d >> 1, rhalf = rot >> 1;
    TA* row = qkv + (size_t)t * (nq + 2 * nkv) * d + (size_t)hh * d;
    TA* dst = row;                                               // q is rotated in place
    if (hh >= nq) {
        const int slot = tl_checked(req_slot[t], L.table_rows, L, TL_K_ROPE);
        const int page = tl_checked(table[(size_t)slot * max_pages + tl_checked(p / page_size, max_pages, L, TL_K_ROPE)],
                                    L.total_pages, L, TL_K_ROPE);
        const int kh = hh < nq + nkv ? hh - nq : hh - nq - nkv;
        dst = (hh < nq + nkv ? k_pages : v_pages) +
              (((size_t)page * nkv + kh) * page_size + (p % page_size)) * d;
    }
    const bool rotate_head = hh < nq + nkv;
    const float* nw = !rotate_head ? nullptr : (hh < nq ? q_norm : k_norm);
    float rstd = 1.0f;
    if (nw) {                                                    // RMS over the head: sum of squares of the biased values
        float ss = 0.f;
        for (int e = threadIdx.x; e < d; e += blockDim.x) {
            float v = to_f<TA>(row[e]);
            if (bias) v += to_f<TW>(bias[hh * d + e]);
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, red);
        rstd = 1.0f / sqrtf(ss / (float)d + norm_eps);
    }
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        int e1, e2;
        if (i < rhalf) { e1 = interleaved ? 2 * i : i; e2 = interleaved ? 2 * i + 1 : i + rhalf; }
        else           { e1 = rot + 2 * (i - rhalf); e2 = e1 + 1; }
        float a = to_f<TA>(row[e1]);
        float b = to_f<TA>(row[e2]);
        if (bias) { a += to_f<TW>(bias[hh * d + e1]); b += to_f<TW>(bias[hh * d + e2]); }
        if (nw) {                                                // cast before the weight, as the layer norms do
            a = to_f<TA>(from_f<TA>(a * rstd)) * nw[e1];
            b = to_f<TA>(from_f<TA>(b * rstd)) * nw[e2];
        }
        if (rotate_head && i < rhalf) {
            float s, c;
            sincosf(__fmul_rn((float)p, inv_freq[i]), &s, &c);
            const float ra = __fmul_rn(a, c) - __fmul_rn(b, s);
            const float rb = __fmul_rn(b, c) + __fmul_rn(a, s);
            a = ra; b = rb;
        }
        dst[e1] = from_f<TA>(a);
        dst[e2] = from_f<TA>(b);
    }
}

__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 x = *reinterpret_cast<const float4*>(p), y = *reinterpret_cast<const float4*>(p + 4);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
    const uint4 x = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
    for (int k = 0; k < 4; ++k) { v[2 * k] = __low2float(h[k]); v[2 * k + 1] = __high2float(h[k]); }
}

// The bfloat16 fast path (full rotary, d % 16 == 0): one block per token; the token's d/2 cosines and
// sines are computed once into shared memory and shared by all heads; each thread moves 8 + 8 values
// (two 16-byte loads, two 16-byte stores).  Same arithmetic as the kernel above.
template <typename TW, bool PIECES>
__global__ void rope_kv_vec_kernel(bf16* __restrict__ qkv, const TW* __restrict__ bias,
                                   const int* __restrict__ pos, const int* __restrict__ req_slot,
                                   const int* __restrict__ table, int max_pages, int page_size,
                                   const float* __restrict__ inv_freq, int nq, int nkv, int d,
                                   bf16* __restrict__ k_pages, bf16* __restrict__ v_pages, int heads,
                                   const float* __restrict__ pieces, int splits, size_t plane, const TlLimits L) {
    // `pieces` [splits][T][(nq + 2 nkv) d] float: the projection as a split-K product left it.  The pieces are
    // summed in split order and rounded to bfloat16 first, as the separate summing pass would have stored them
    // in qkv; q still goes to qkv, which is then output only.
    extern __shared__ float cs[];                                // cos[half], sin[half]
    const int t = blockIdx.x;
    const int p = pos[t];
    const int half = d >> 1, per_head = half >> 3;               // threads per head
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf(__fmul_rn((float)p, inv_freq[i]), &s, &c);
        cs[i] = c; cs[half + i] = s;
    }
    size_t page_base = 0;
    if (heads > nq) {
        const int slot = tl_checked(req_slot[t], L.table_rows, L, TL_K_ROPE);
        const int page = tl_checked(table[(size_t)slot * max_pages + tl_checked(p / page_size, max_pages, L, TL_K_ROPE)],
                                    L.total_pages, L, TL_K_ROPE);
        page_base = ((size_t)page * nkv * page_size + (p % page_size)) * d;
    }
    grid_dependency_wait();                              // angles and the page are ready when the projection ends
    grid_dependency_trigger();
    __syncthreads();
    bf16* row = qkv + (size_t)t * (nq + 2 * nkv) * d;
    for (int item = threadIdx.x; item < heads * per_head; item += blockDim.x) {
        const int hh = item / per_head, i0 = (item - hh * per_head) * 8;
        float a[8], b[8];
        if (PIECES) {                                    // an instantiation of its own: the plain one keeps its registers
#pragma unroll
            for (int k = 0; k < 8; ++k) { a[k] = 0.f; b[k] = 0.f; }
            const float* src = pieces + (size_t)t * (nq + 2 * nkv) * d + hh * d + i0;
            for (int sp = 0; sp < splits; ++sp, src += plane) {
                const float4 a0 = *reinterpret_cast<const float4*>(src), a1 = *reinterpret_cast<const float4*>(src + 4);
                const float4 b0 = *reinterpret_cast<const float4*>(src + half), b1 = *reinterpret_cast<const float4*>(src + half + 4);
                a[0] += a0.x; a[1] += a0.y; a[2] += a0.z; a[3] += a0.w; a[4] += a1.x; a[5] += a1.y; a[6] += a1.z; a[7] += a1.w;
                b[0] += b0.x; b[1] += b0.y; b[2] += b0.z; b[3] += b0.w; b[4] += b1.x; b[5] += b1.y; b[6] += b1.z; b[7] += b1.w;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                a[k] = __bfloat162float(__float2bfloat16_rn(a[k]));
                b[k] = __bfloat162float(__float2bfloat16_rn(b[k]));
            }
        } else {
            const uint4 av = *reinterpret_cast<const uint4*>(row + hh * d + i0);
            const uint4 bv = *reinterpret_cast<const uint4*>(row + hh * d + half + i0);
            const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                a[2 * k] = __low2float(a2[k]); a[2 * k + 1] = __high2float(a2[k]);
                b[2 * k] = __low2float(b2[k]); b[2 * k + 1] = __high2float(b2[k]);
            }
        }
        if (bias) {                                      // 8 + 8 consecutive values: vector loads (i0 and d are multiples of 8)
            float ba[8], bb[8];
            load8(bias + hh * d + i0, ba);
            load8(bias + hh * d + half + i0, bb);
#pragma unroll
            for (int k = 0; k < 8; ++k) { a[k] += ba[k]; b[k] += bb[k]; }
        }
        if (hh < nq + nkv) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float c = cs[i0 + k], s = cs[half + i0 + k];
                const float ra = __fmul_rn(a[k], c) - __fmul_rn(b[k], s);
                const float rb = __fmul_rn(b[k], c) + __fmul_rn(a[k], s);
                a[k] = ra; b[k] = rb;
            }
        }
        uint4 ao, bo;
        __nv_bfloat162* ao2 = reinterpret_cast<__nv_bfloat162*>(&ao);
        __nv_bfloat162* bo2 = reinterpret_cast<__nv_bfloat162*>(&bo);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            ao2[k] = __floats2bfloat162_rn(a[2 * k], a[2 * k + 1]);
            bo2[k] = __floats2bfloat162_rn(b[2 * k], b[2 * k + 1]);
        }
        bf16* dst = row + hh * d;
        if (hh >= nq) {
            const int kh = hh < nq + nkv ? hh - nq : hh - nq - nkv;
            dst = (hh < nq + nkv ? k_pages : v_pages) + page_base + (size_t)kh * page_size * d;
        }
        *reinterpret_cast<uint4*>(dst + i0) = ao;
        *reinterpret_cast<uint4*>(dst + half + i0) = bo;
    }
}

TL_EXPORT int tl_rope_kv_write(void* qkv, int act_dtype, const void* bias, int bias_dtype,
                               const int* pos, const int* req_slot, const int* table, int max_pages,
                               int page_size, const float* inv_freq, int rot, int nq, int nkv, int d,
                               void* k_pages, void* v_pages, int write_kv, int T, const float* pieces, int splits,
                               long long plane, int interleaved, const float* q_norm, const float* k_norm,
                               float norm_eps, int table_rows, int total_pages, int* fault, cudaStream_t stream) {
    const TlLimits L{table_rows, total_pages, fault};
    if (T <= 0) return 0;
    if (rot < 0 || rot > d || (rot & 1) || (d & 1)) return 1;     // cudaErrorInvalidValue
    const int heads = write_kv ? nq + 2 * nkv : nq;
    if (heads > 65535) return 1;
    const bool aligned = ((((uintptr_t)qkv | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)pieces | (uintptr_t)bias) & 15) == 0);
    if ((q_norm == nullptr) != (k_norm == nullptr)) return 1;
    const bool plain = !interleaved && q_norm == nullptr;         // the fast path: rotate-half pairs, no q/k norm
    if (pieces && !(plain && act_dtype == TL_BF16 && rot == d && (d & 15) == 0 && aligned)) return 1;   // pieces: the fast path only
    if (plain && act_dtype == TL_BF16 && rot == d && (d & 15) == 0 && aligned) {
        const int items = heads * (d / 16);
        const int threads = items < 1024 ? ((items + 31) / 32) * 32 : 1024;
        const size_t smem = (size_t)d * sizeof(float);
#define VROPE(TW, P) launch_after_wait(rope_kv_vec_kernel<TW, P>, dim3(T), dim3(threads), smem, stream, (bf16*)qkv, (const TW*)bias, \
            pos, req_slot, table, max_pages, page_size, inv_freq, nq, nkv, d, (bf16*)k_pages, (bf16*)v_pages, heads, pieces, splits, (size_t)plane, L)
        if (bias_dtype == TL_F32) return pieces ? VROPE(float, true) : VROPE(float, false);
        return pieces ? VROPE(bf16, true) : VROPE(bf16, false);
#undef VROPE
    }
    dim3 grid(T, heads);
    const int half = d / 2;
    const int threads = half < 256 ? ((half + 31) / 32) * 32 : 256;
#define LAUNCH(TA, TW) rope_kv_kernel<TA, TW><<<grid, threads, 0, stream>>>( \
        (TA*)qkv, (const TW*)bias, pos, req_slot, table, max_pages, page_size, inv_freq, rot, nq, nkv, d, \
        (TA*)k_pages, (TA*)v_pages, interleaved, q_norm, k_norm, norm_eps, L)
    if (act_dtype == TL_F32) { if (bias_dtype == TL_F32) LAUNCH(float, float); else LAUNCH(float, bf16); }
    else                     { if (bias_dtype == TL_F32) LAUNCH(bf16, float);  else LAUNCH(bf16, bf16); }
#undef LAUNCH
    return tl_launch_status();
}
