// Paged causal grouped-query attention, one warp per (token, query head).
//
// This is the exact-order kernel: the true 32-bit engine uses it for prompts and for decoding,
// and the tests use it (in bfloat16 too) as the on-device reference of the tensor-core kernels.
// A query at position p of a request reads the keys at positions lo..p of that request from the
// cache pages, lo = 0 or p - window + 1 (tensorline/paged.py:237; tensorline/paged_attn.py:43).
// s = (q . k) * scale, softmax over keys in float, o = P V (tensorline/paged_attn.py:46-57).
//
// Keys are taken in tiles of 32 aligned to absolute position 0, each lane owning one key of the
// tile, with a running maximum and sum.  The order of every addition depends only on the
// query's position and the window, never on how the step was cut or batched, so the result for
// a position is bit-identical under every schedule.
#include "common.cuh"

#define ATT_MAX_D 512

template <typename TA>
__global__ void attn_tokenwise_kernel(const TA* __restrict__ q, int q_stride, TA* __restrict__ out,
                                      const TA* __restrict__ k_pages, const TA* __restrict__ v_pages,
                                      const int* __restrict__ table, int max_pages, int page_size,
                                      const int* __restrict__ pos, const int* __restrict__ req_slot,
                                      int nq, int nkv, int d, int window, float scale, const TlLimits L) {
    __shared__ float qs[ATT_MAX_D];
    const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
    const int kh = h / (nq / nkv);
    const int p = pos[t];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int* tab = table + (size_t)tl_checked(req_slot[t], L.table_rows, L, TL_K_TOKENWISE) * max_pages;
    const TA* qrow = q + (size_t)t * q_stride + (size_t)h * d;
    for (int e = lane; e < d; e += 32) qs[e] = to_f<TA>(qrow[e]);
    __syncwarp();

    constexpr int MAXC = ATT_MAX_D / 32;
    float acc[MAXC];
#pragma unroll
    for (int c = 0; c < MAXC; ++c) acc[c] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int j0 = (lo / 32) * 32; j0 <= p; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = (j >= lo) && (j <= p);
        size_t row = 0;
        float s = -INFINITY;
        if (valid) {
            const int page = tl_checked(tab[tl_checked(j / page_size, max_pages, L, TL_K_TOKENWISE)], L.total_pages, L, TL_K_TOKENWISE);
            row = (((size_t)page * nkv + kh) * page_size + (j % page_size)) * d;
            const TA* kr = k_pages + row;
            float dot = 0.f;
            for (int e = 0; e < d; ++e) dot = fmaf(qs[e], to_f<TA>(kr[e]), dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float alpha = expf(m - m_new);            // 0 on the first tile (m = -inf)
        const float pj = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(pj);
#pragma unroll
        for (int c = 0; c < MAXC; ++c) acc[c] *= alpha;
        const int n_here = min(32, p - j0 + 1);
        for (int jj = 0; jj < n_here; ++jj) {
            const float pb = __shfl_sync(0xffffffffu, pj, jj);
            const unsigned long long rb = __shfl_sync(0xffffffffu, (unsigned long long)row, jj);
            if (pb != 0.f) {                             // uniform over the warp
                const TA* vr = v_pages + rb;
#pragma unroll
                for (int c = 0; c < MAXC; ++c) {
                    const int e = lane + 32 * c;
                    if (e < d) acc[c] = fmaf(pb, to_f<TA>(vr[e]), acc[c]);
                }
            }
        }
        m = m_new;
    }
    TA* orow = out + ((size_t)t * nq + h) * d;
    const float inv = 1.0f / l;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
        const int e = lane + 32 * c;
        if (e < d) orow[e] = from_f<TA>(acc[c] * inv);
    }
}

TL_EXPORT int tl_attn_tokenwise(const void* q, int q_stride, void* out, int act_dtype,
                                const void* k_pages, const void* v_pages, const int* table, int max_pages,
                                int page_size, const int* pos, const int* req_slot, int T, int nq, int nkv,
                                int d, int window, float scale, int table_rows, int total_pages, int* fault,
                                cudaStream_t stream) {
    const TlLimits L{table_rows, total_pages, fault};
    if (T <= 0) return 0;
    if (d > ATT_MAX_D || nq % nkv) return 1;
    dim3 grid(T, nq);
    if (act_dtype == TL_F32)
        attn_tokenwise_kernel<float><<<grid, 32, 0, stream>>>((const float*)q, q_stride, (float*)out,
            (const float*)k_pages, (const float*)v_pages, table, max_pages, page_size, pos, req_slot,
            nq, nkv, d, window, scale, L);
    else
        attn_tokenwise_kernel<bf16><<<grid, 32, 0, stream>>>((const bf16*)q, q_stride, (bf16*)out,
            (const bf16*)k_pages, (const bf16*)v_pages, table, max_pages, page_size, pos, req_slot,
            nq, nkv, d, window, scale, L);
    return tl_launch_status();
}
