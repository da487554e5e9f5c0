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
#include "common.cuh"

template <typename TA, typename TW>
__global__ void rope_kv_kernel(TA* __restrict__ qkv, const TW* __restrict__ bias,
                               const int* __restrict__ pos, const int* __restrict__ req_slot,
                               const int* __restrict__ table, int max_pages, int page_size,
                               const float* __restrict__ inv_freq, int rot, int nq, int nkv, int d,
                               TA* __restrict__ k_pages, TA* __restrict__ v_pages, int write_kv) {
    const int t = blockIdx.x;
    const int p = pos[t];
    const int half = d >> 1, rhalf = rot >> 1;
    const int heads = write_kv ? nq + 2 * nkv : nq;
    TA* row = qkv + (size_t)t * (nq + 2 * nkv) * d;
    size_t page_base = 0;
    if (write_kv) {
        const int page = table[(size_t)req_slot[t] * max_pages + p / page_size];
        page_base = ((size_t)page * nkv * page_size + (p % page_size)) * d;   // head 0 of this token
    }
    for (int item = threadIdx.x; item < heads * half; item += blockDim.x) {
        const int hh = item / half, i = item - hh * half;
        int e1, e2;
        const bool rotate = (hh < nq + nkv) && (i < rhalf);
        if (i < rhalf) { e1 = i; e2 = i + rhalf; }
        else           { e1 = rot + 2 * (i - rhalf); e2 = e1 + 1; }
        float a = to_f<TA>(row[hh * d + e1]);
        float b = to_f<TA>(row[hh * d + e2]);
        if (bias) { a += to_f<TW>(bias[hh * d + e1]); b += to_f<TW>(bias[hh * d + e2]); }
        if (rotate) {
            float s, c;
            sincosf(__fmul_rn((float)p, inv_freq[i]), &s, &c);
            const float ra = __fmul_rn(a, c) - __fmul_rn(b, s);
            const float rb = __fmul_rn(b, c) + __fmul_rn(a, s);
            a = ra; b = rb;
        }
        if (hh < nq) {
            row[hh * d + e1] = from_f<TA>(a);
            row[hh * d + e2] = from_f<TA>(b);
        } else {
            const int kh = hh < nq + nkv ? hh - nq : hh - nq - nkv;
            TA* dst = (hh < nq + nkv ? k_pages : v_pages) + page_base + (size_t)kh * page_size * d;
            dst[e1] = from_f<TA>(a);
            dst[e2] = from_f<TA>(b);
        }
    }
}

TL_EXPORT int tl_rope_kv_write(void* qkv, int act_dtype, const void* bias, int bias_dtype,
                               const int* pos, const int* req_slot, const int* table, int max_pages,
                               int page_size, const float* inv_freq, int rot, int nq, int nkv, int d,
                               void* k_pages, void* v_pages, int write_kv, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot < 0 || rot > d || (rot & 1) || (d & 1)) return 1;     // cudaErrorInvalidValue
    const int items = (nq + 2 * nkv) * (d / 2);
    int threads = items < 256 ? ((items + 31) / 32) * 32 : 256;
#define LAUNCH(TA, TW) rope_kv_kernel<TA, TW><<<T, threads, 0, stream>>>( \
        (TA*)qkv, (const TW*)bias, pos, req_slot, table, max_pages, page_size, inv_freq, rot, nq, nkv, d, \
        (TA*)k_pages, (TA*)v_pages, write_kv)
    if (act_dtype == TL_F32) { if (bias_dtype == TL_F32) LAUNCH(float, float); else LAUNCH(float, bf16); }
    else                     { if (bias_dtype == TL_F32) LAUNCH(bf16, float);  else LAUNCH(bf16, bf16); }
#undef LAUNCH
    return tl_launch_status();
}
