// Tensor-core paged attention in bfloat16, compiled for one head size (-DHEAD_DIM=d, d % 16 == 0).
//
//   tl_attn_prefill   causal grouped-query flash attention for a step that holds prompt portions
//                     (and, beside them, single decoded tokens).  Replaces the padded SDPA calls of
//                     tensorline/paged.py:263-274: fresh prompts, resumed portions and decoded
//                     tokens all read K and V from the pages, where this step's own tokens were
//                     written first (paged.py:252-253).
//   tl_attn_decode    split-KV paged decode attention: one query token per request, the keys of a
//                     request cut into `splits` ranges that run as separate blocks, float partials
//                     (max, sum, unnormalised output) in scratch memory, merged by
//   tl_attn_combine.  Replaces tensorline/paged_attn.py:25-58, which is serial over the context.
//
// Both put the g = nq / nkv query heads that share a KV head into the rows of the MMA tile, so K
// and V of a KV head are read once for the whole group (tensorline/paged_attn.py:33-35).  Scores,
// running max, sum and the output accumulator are float; P is rounded to bfloat16 for the P V
// product (paged_attn.py:56).  Pages are [page, kv head, offset, d]: a head's part of a page is
// contiguous.  Tensor-core path: mma.sync.m16n8k16 (bf16 in, f32 accumulate) fed by ldmatrix from
// shared-memory tiles that cp.async fills; rows of a tile are padded by 16 bytes, which keeps
// ldmatrix free of bank conflicts for every head size.
#include "common.cuh"
#include <cuda.h>

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size>"
#endif
#if HEAD_DIM % 16 != 0 || HEAD_DIM < 16 || HEAD_DIM > 256
#error "HEAD_DIM must be a multiple of 16 in [16, 256]"
#endif

namespace {

constexpr int D = HEAD_DIM;
constexpr int DP = D + 8;              // padded row, elements
constexpr int CH = D / 8;              // 16-byte chunks per row
constexpr int KBLK = D / 16;           // k-blocks of Q K^T
constexpr int BM = 64;                 // query rows per block (prefill)
constexpr int BN = 64;                 // keys per tile
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;      // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct AttnArgs {
    const bf16* q; int q_stride;       // q rows: token t at q + t * q_stride, head h at + h * D
    bf16* out;                         // [T, nq * D]
    const bf16* k_pages; const bf16* v_pages;
    const int* table; int max_pages; int page_size;
    const int* q_start; const int* start_pos; const int* slots;
    int B, nq, nkv, window;
    float scale_log2;                  // scale * log2(e)
    // decode only
    int chunk, splits;
    float* part_o; float* part_ml;     // [B, nq, splits, D] and [B, nq, splits, 2]
    // prefill only: the tiles in the order in which blocks take them, (request << 16 | tile), longest first over
    // all requests; null: one request after the other from the end
    const int* order;
    TlLimits lim;                      // for the checking build; zeros: nothing known, nothing checked
    // TMA decode with the rotary step folded in: `q` points at the step's q|k|v rows as the projection left them (row stride
    // q_stride, k of KV head h at column (nq + h) * D, v at (nq + nkv + h) * D).  The block applies bias and rotation to its
    // query heads on the way to shared memory; the block whose key range holds the token's own position does the same for
    // the new key and value, writes them to their page (rope_write) and puts them into its own tiles.  Null inv_freq: not folded.
    const float* rope_inv_freq; const void* rope_bias; int rope_bias_f32; int rope_write;
    // tracing build (the TMA decode kernel): stamps 0 block start, 1 dependency wait returned, 2 first stage landed, 3 last
    // stage landed, 4 block end, 5 last stage worked through, 6 at the cluster barrier, 7 past it
    TlTrace trace;
    bf16* k_pages_w; bf16* v_pages_w;
};

// Eight values at i0.. and the eight at D/2 + i0.. of one head's row: + bias, rotated (rotate-half pairs, angle of pair i in
// cs[i] = cos, cs[D/2 + i] = sin) unless `rotate` is false, rounded to bfloat16.  The arithmetic of rope_kv_vec_kernel.
// av, bv: the sixteen values as loaded (the caller issues the loads of all its items before it works on the first).
__device__ __forceinline__ void rope_pairs(const uint4 av, const uint4 bv, const void* bias, int bias_f32, int bias_off, int i0, const float* cs,
                                           bool rotate, uint4& lo, uint4& hi) {
    constexpr int half = HEAD_DIM / 2;
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bv);
    float a[8], b[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        a[2 * k] = __low2float(a2[k]); a[2 * k + 1] = __high2float(a2[k]);
        b[2 * k] = __low2float(b2[k]); b[2 * k + 1] = __high2float(b2[k]);
    }
    if (bias) {
        if (bias_f32) {
            const float* bp = (const float*)bias + bias_off;
#pragma unroll
            for (int k = 0; k < 8; ++k) { a[k] += bp[i0 + k]; b[k] += bp[half + i0 + k]; }
        } else {
            const bf16* bp = (const bf16*)bias + bias_off;
#pragma unroll
            for (int k = 0; k < 8; ++k) { a[k] += __bfloat162float(bp[i0 + k]); b[k] += __bfloat162float(bp[half + i0 + k]); }
        }
    }
    if (rotate) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float c = cs[i0 + k], sn = cs[half + i0 + k];
            const float ra = __fmul_rn(a[k], c) - __fmul_rn(b[k], sn);
            const float rb = __fmul_rn(b[k], c) + __fmul_rn(a[k], sn);
            a[k] = ra; b[k] = rb;
        }
    }
    uint32_t pa[4], pb[4];                                // by value: the results stay in registers at the caller
#pragma unroll
    for (int k = 0; k < 4; ++k) { pa[k] = pack_bf16(a[2 * k], a[2 * k + 1]); pb[k] = pack_bf16(b[2 * k], b[2 * k + 1]); }
    lo = make_uint4(pa[0], pa[1], pa[2], pa[3]);
    hi = make_uint4(pb[0], pb[1], pb[2], pb[3]);
}

// A [ROWS][DP] tile of keys (or values) of one KV head is filled by 128 threads in chunks of 16
// bytes.  Which chunk a thread copies never changes, so its place inside a page, its page
// within the tile and its place in shared memory are worked out once (`TileMap`); a tile then costs
// one table read, one multiply-add and one cp.async per chunk.
template <int ROWS>
struct TileMap {
    static constexpr int ITERS = (ROWS * CH + 127) / 128;
    uint32_t src[ITERS];               // key << 26 | page within tile << 20 | element offset inside the page
    uint32_t dst[ITERS];               // element offset inside the shared tile; 0xFFFFFFFF: no chunk
    __device__ __forceinline__ void init(int tid, int page_size) {
#pragma unroll
        for (int i = 0; i < ITERS; ++i) {
            const int idx = tid + 128 * i;
            const int key = idx / CH, c = idx - key * CH;
            src[i] = ((uint32_t)key << 26) | ((uint32_t)(key / page_size) << 20) |
                     (uint32_t)((key % page_size) * D + c * 8);
            dst[i] = idx < ROWS * CH ? (uint32_t)(key * DP + c * 8) : 0xFFFFFFFFu;
        }
    }
};

// Loads keys [key0, key0 + ROWS) (key0 a multiple of ROWS, ROWS a multiple of the page size) into
// `dst`; keys past `last_key` are zeros.  `tab` points at the table entry of key0's page: the
// request's table row in global memory, or a copy of the block's part of it in shared memory.
// `pages` points at the KV head's part of page 0.
template <int ROWS>
__device__ __forceinline__ void load_kv_tile(bf16* dst, const bf16* pages, const int* tab, size_t page_stride,
                                             int key0, int last_key, const TileMap<ROWS>& map, const TlLimits& L, int kernel) {
    const int keys_valid = last_key - key0;               // keys 0..keys_valid of the tile exist
#pragma unroll
    for (int i = 0; i < TileMap<ROWS>::ITERS; ++i) {
        if ((ROWS * CH) % 128 != 0 && map.dst[i] == 0xFFFFFFFFu) continue;
        const int key = map.src[i] >> 26;
        const bool valid = key <= keys_valid;
        const bf16* src = pages;
        if (valid) src = pages + (size_t)tl_checked(tab[(map.src[i] >> 20) & 63], L.total_pages, L, kernel) * page_stride + (map.src[i] & 0xFFFFF);
        cp_async16(dst + map.dst[i], src, valid);
    }
}

// S[16 x (8*NB)] += Q[16 x D] K^T for the keys of `sK` starting at tile row `key_off`.
template <int NB>
__device__ __forceinline__ void qk_tile(float (&s)[NB][4], const bf16* sQ_rows, const bf16* sK, int key_off, int lane) {
#pragma unroll
    for (int kb = 0; kb < KBLK; ++kb) {
        uint32_t a[4];
        ldsm_x4(a, sQ_rows + ((lane & 7) + ((lane >> 3) & 1) * 8) * DP + kb * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int nb = 0; nb < NB; nb += 2) {
            uint32_t b[4];
            ldsm_x4(b, sK + (key_off + nb * 8 + (lane & 7) + (lane >> 4) * 8) * DP + kb * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16(s[nb], a, b[0], b[1]);
            mma_bf16(s[nb + 1], a, b[2], b[3]);
        }
    }
}

// The same with the Q fragments already in registers.
template <int NB>
__device__ __forceinline__ void qk_tile_regs(float (&s)[NB][4], const uint32_t (&qf)[KBLK][4], const bf16* sK,
                                             int key_off, int lane) {
#pragma unroll
    for (int kb = 0; kb < KBLK; ++kb) {
#pragma unroll
        for (int nb = 0; nb < NB; nb += 2) {
            uint32_t b[4];
            ldsm_x4(b, sK + (key_off + nb * 8 + (lane & 7) + (lane >> 4) * 8) * DP + kb * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16(s[nb], qf[kb], b[0], b[1]);
            mma_bf16(s[nb + 1], qf[kb], b[2], b[3]);
        }
    }
}

// O[16 x D] += P[16 x (8*NB)] V for the keys of `sV` starting at tile row `key_off`.
template <int NB>
__device__ __forceinline__ void pv_tile(float (&o)[D / 8][4], const float (&p)[NB][4], const bf16* sV, int key_off, int lane) {
#pragma unroll
    for (int kb = 0; kb < NB / 2; ++kb) {
        uint32_t a[4];
        a[0] = pack_bf16(p[2 * kb][0], p[2 * kb][1]);
        a[1] = pack_bf16(p[2 * kb][2], p[2 * kb][3]);
        a[2] = pack_bf16(p[2 * kb + 1][0], p[2 * kb + 1][1]);
        a[3] = pack_bf16(p[2 * kb + 1][2], p[2 * kb + 1][3]);
#pragma unroll
        for (int nb = 0; nb < D / 8; nb += 2) {
            uint32_t b[4];
            ldsm_x4_trans(b, sV + (key_off + kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * DP + nb * 8 + (lane >> 4) * 8);
            mma_bf16(o[nb], a, b[0], b[1]);
            mma_bf16(o[nb + 1], a, b[2], b[3]);
        }
    }
}

__device__ __forceinline__ float fast_exp2(float x) {          // 2^x, hardware approximation (about 2 ulp); -inf gives 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Masks, scales and exponentiates one thread's share of S (rows ra = lane/4 and ra + 8), updates the
// running max m[2] (kept in scaled units), the per-thread partial sums l[2] and rescales O.
// key0: position of S column 0.  MASKED = false: the caller knows every key of the tile is visible
// to every row of the warp, and the comparisons are skipped.
template <int NB, bool MASKED>
__device__ __forceinline__ void softmax_step(float (&s)[NB][4], float (&o)[D / 8][4], float (&m)[2], float (&l)[2],
                                             const int (&pos_r)[2], const int (&lo_r)[2], int key0, float scale_log2,
                                             int lane) {
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            if (MASKED) {
                const int j = key0 + nb * 8 + (lane & 3) * 2 + (e & 1);
                if (!(j <= pos_r[r] && j >= lo_r[r])) s[nb][e] = -INFINITY;
            }
            mx[r] = fmaxf(mx[r], s[nb][e]);
        }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        mx[r] *= scale_log2;                                        // the scale is positive: max commutes with it
    }
    // Once the running maxima have settled, a tile leaves them as they are and nothing needs rescaling.
    const bool grew = __any_sync(0xffffffffu, mx[0] > m[0] || mx[1] > m[1]);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const float m_new = fmaxf(m[r], mx[r]);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;     // a row with no visible key yet
        if (grew) {
            const float alpha = fast_exp2(m[r] - m_use);            // m = -inf gives 0
            m[r] = m_new;
            l[r] *= alpha;
#pragma unroll
            for (int nb = 0; nb < D / 8; ++nb) { o[nb][2 * r] *= alpha; o[nb][2 * r + 1] *= alpha; }
        }
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const float p0 = fast_exp2(fmaf(s[nb][2 * r], scale_log2, -m_use));
            const float p1 = fast_exp2(fmaf(s[nb][2 * r + 1], scale_log2, -m_use));
            s[nb][2 * r] = p0; s[nb][2 * r + 1] = p1;
            l[r] += p0 + p1;
        }
    }
}

// ------------------------------------------------------------------------------------ prefill
// PBN: keys per tile.  32 leaves room for three blocks per SM (more warps to hide the latencies of the
// MMA / ldmatrix chains); 64 serves pages of 64 tokens.
template <int PBN>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const AttnArgs A) {
    constexpr int BN = PBN;                                // shadows the decode tile size inside this kernel
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);          // [BM][DP]
    bf16* sK = sQ + BM * DP;                               // [2][BN][DP]
    bf16* sV = sK + 2 * BN * DP;                           // [2][BN][DP]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kh = blockIdx.x % A.nkv, g = A.nq / A.nkv;   // blocks in order of falling length over all KV heads

    // Blocks are handed out in index order and a tile's work grows with its position in the request
    // (causal), so the tiles are taken from the end: the longest ones start first.
    int tile = (int)(gridDim.x / A.nkv) - 1 - (int)(blockIdx.x / A.nkv), b = 0;
    if (A.order != nullptr) {
        const int packed = A.order[blockIdx.x / A.nkv];
        b = packed >> 16; tile = packed & 0xFFFF;
    } else {
        for (; b < A.B; ++b) {
            const int nt = ((A.q_start[b + 1] - A.q_start[b]) * g + BM - 1) / BM;
            if (tile < nt) break;
            tile -= nt;
        }
    }
    if (b >= A.B) return;
    const int qs = A.q_start[b], qlen = A.q_start[b + 1] - qs, sp = A.start_pos[b];
    const int rows_total = qlen * g, row0 = tile * BM;
    const int row_end = min(row0 + BM, rows_total);
    const int* tab = A.table + (size_t)tl_checked(A.slots[b], A.lim.table_rows, A.lim, TL_K_PREFILL) * A.max_pages;
    const int pos_hi = sp + (row_end - 1) / g;
    tl_checked(pos_hi / A.page_size, A.max_pages, A.lim, TL_K_PREFILL);     // the last table entry this tile reads
    const int pos_first = sp + row0 / g;
    const int key_lo = A.window > 0 ? max(0, pos_first - A.window + 1) : 0;
    const int kt_lo = key_lo / BN, kt_hi = pos_hi / BN;

    for (int idx = tid; idx < BM * CH; idx += 128) {       // Q tile: row = (token, head of the group)
        const int r = idx / CH, c = idx - r * CH;
        const int R = row0 + r;
        const bool valid = R < rows_total;
        const bf16* src = A.q;
        if (valid) src = A.q + (size_t)(qs + R / g) * A.q_stride + (size_t)(kh * g + R % g) * D + c * 8;
        cp_async16(sQ + r * DP + c * 8, src, valid);
    }
    TileMap<BN> map;
    map.init(tid, A.page_size);
    const size_t page_stride = (size_t)A.nkv * A.page_size * D;
    const int ppt = BN / A.page_size;                       // pages per tile
    const bf16* kbase = A.k_pages + (size_t)kh * A.page_size * D;
    const bf16* vbase = A.v_pages + (size_t)kh * A.page_size * D;
    load_kv_tile(sK, kbase, tab + kt_lo * ppt, page_stride, kt_lo * BN, pos_hi, map, A.lim, TL_K_PREFILL);
    load_kv_tile(sV, vbase, tab + kt_lo * ppt, page_stride, kt_lo * BN, pos_hi, map, A.lim, TL_K_PREFILL);
    cp_async_commit();

    int pos_r[2], lo_r[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int R = row0 + warp * 16 + (lane >> 2) + r * 8;
        pos_r[r] = R < rows_total ? sp + R / g : -1;       // -1: no key is visible, the row stays empty
        lo_r[r] = A.window > 0 ? max(0, pos_r[r] - A.window + 1) : 0;
    }
    // the warp's own rows: first and last valid one (positions rise with the row index)
    const int wr_first = row0 + warp * 16, wr_last = min(wr_first + 15, rows_total - 1);
    const bool w_valid = wr_first < rows_total;
    const int w_pos_hi = sp + wr_last / g;
    const int w_lo = A.window > 0 ? max(0, sp + wr_first / g - A.window + 1) : 0;
    float o[D / 8][4];
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) { o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int kt = kt_lo; kt <= kt_hi; ++kt) {
        const int buf = (kt - kt_lo) & 1;
        cp_async_wait<0>();
        __syncthreads();                                   // tile kt is in; everyone is done with tile kt-1
        if (kt < kt_hi) {
            load_kv_tile(sK + (buf ^ 1) * BN * DP, kbase, tab + (kt + 1) * ppt, page_stride, (kt + 1) * BN, pos_hi, map, A.lim, TL_K_PREFILL);
            load_kv_tile(sV + (buf ^ 1) * BN * DP, vbase, tab + (kt + 1) * ppt, page_stride, (kt + 1) * BN, pos_hi, map, A.lim, TL_K_PREFILL);
        }
        cp_async_commit();
        // skip tiles wholly outside this warp's rows (above the diagonal or behind the window)
        if (!w_valid || kt * BN > w_pos_hi || kt * BN + BN - 1 < w_lo) continue;
        float s[BN / 8][4];
#pragma unroll
        for (int nb = 0; nb < BN / 8; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
        qk_tile<BN / 8>(s, sQ + warp * 16 * DP, sK + buf * BN * DP, 0, lane);
        // the tile's keys are all visible to all rows of the warp: below every row's position, inside
        // every row's window
        const bool full = (kt * BN + BN - 1 <= sp + wr_first / g) &&
                          (A.window <= 0 || kt * BN >= max(0, w_pos_hi - A.window + 1));
        if (full) softmax_step<BN / 8, false>(s, o, m, l, pos_r, lo_r, kt * BN, A.scale_log2, lane);
        else      softmax_step<BN / 8, true>(s, o, m, l, pos_r, lo_r, kt * BN, A.scale_log2, lane);
        pv_tile<BN / 8>(o, s, sV + buf * BN * DP, 0, lane);
    }
    cp_async_wait<0>();

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float lr = l[r];
        lr += __shfl_xor_sync(0xffffffffu, lr, 1);
        lr += __shfl_xor_sync(0xffffffffu, lr, 2);
        const int R = row0 + warp * 16 + (lane >> 2) + r * 8;
        if (R >= rows_total) continue;
        const float inv = lr > 0.f ? 1.0f / lr : 0.f;
        bf16* dst = A.out + ((size_t)(qs + R / g) * A.nq + (kh * g + R % g)) * D + (lane & 3) * 2;
#pragma unroll
        for (int nb = 0; nb < D / 8; ++nb)
            *reinterpret_cast<uint32_t*>(dst + nb * 8) = pack_bf16(o[nb][2 * r] * inv, o[nb][2 * r + 1] * inv);
    }
}

// ------------------------------------------------------------------------------------ decode
#ifndef TL_DEC_STAGES
#define TL_DEC_STAGES 3
#endif
constexpr int DEC_STAGES = TL_DEC_STAGES;
constexpr int DECODE_KV_SMEM = 2 * DEC_STAGES * BN * DP * 2;
constexpr int DECODE_MERGE_SMEM = (4 * 16 * D + 4 * 16 * 2) * 4;
constexpr int DECODE_TAB_OFFSET = 16 * DP * 2 + (DECODE_KV_SMEM > DECODE_MERGE_SMEM ? DECODE_KV_SMEM : DECODE_MERGE_SMEM);
constexpr int DECODE_MAX_TAB = 1024;                    // table entries a block may copy (4 KB: head size 256 leaves no more)

// grid (splits * m_tiles, nkv, B); 4 warps; each stage is 64 keys, 16 per warp.
__global__ void __launch_bounds__(128) attn_decode_kernel(const AttnArgs A) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);          // [16][DP]
    bf16* sK = sQ + 16 * DP;                               // [STAGES][BN][DP]
    bf16* sV = sK + DEC_STAGES * BN * DP;                  // [STAGES][BN][DP]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = A.nq / A.nkv, m_tiles = (g + 15) / 16;
    const int split = blockIdx.x / m_tiles, mt = blockIdx.x % m_tiles;
    const int kh = blockIdx.y, b = blockIdx.z;
    const int pos = A.start_pos[b], len = pos + 1;
    const int lo = A.window > 0 ? max(0, len - A.window) : 0;
    const int base = (lo / BN) * BN;
    const int k_begin = base + split * A.chunk;
    if (k_begin >= len) return;                            // an empty split: the combine step skips it too
    const int k_end = min(len, k_begin + A.chunk);
    const int n_stage = (k_end - k_begin + BN - 1) / BN;
    const int* gtab = A.table + (size_t)tl_checked(A.slots[b], A.lim.table_rows, A.lim, TL_K_DECODE) * A.max_pages;
    const int qrow = A.q_start[b];
    // this block's part of the request's block table, copied once
    int* stab = reinterpret_cast<int*>(smem_raw + DECODE_TAB_OFFSET);
    const int ppt = BN / A.page_size, first_page = k_begin / A.page_size;
    const int n_pages = (k_end - 1) / A.page_size - first_page + 1;
    for (int i = tid; i < n_stage * ppt; i += 128)
        stab[i] = i < n_pages ? gtab[tl_checked(first_page + i, A.max_pages, A.lim, TL_K_DECODE)] : 0;
    TileMap<BN> map;
    map.init(tid, A.page_size);
    const size_t page_stride = (size_t)A.nkv * A.page_size * D;
    const bf16* kbase = A.k_pages + (size_t)kh * A.page_size * D;
    const bf16* vbase = A.v_pages + (size_t)kh * A.page_size * D;

    // Positions and block tables were written before the step's first kernel; the queries and the newest keys
    // and values come from the kernel just before this one.
    grid_dependency_wait();
    grid_dependency_trigger();
    for (int idx = tid; idx < 16 * CH; idx += 128) {
        const int r = idx / CH, c = idx - r * CH;
        const int hg = mt * 16 + r;
        const bool valid = hg < g;
        const bf16* src = A.q;
        if (valid) src = A.q + (size_t)qrow * A.q_stride + (size_t)(kh * g + hg) * D + c * 8;
        cp_async16(sQ + r * DP + c * 8, src, valid);
    }
    cp_async_commit();                                     // group 0: the queries
    __syncthreads();                                       // the table copy is visible
#pragma unroll
    for (int st = 0; st < DEC_STAGES - 1; ++st) {
        if (st < n_stage) {
            load_kv_tile(sK + st * BN * DP, kbase, stab + st * ppt, page_stride, k_begin + st * BN, k_end - 1, map, A.lim, TL_K_DECODE);
            load_kv_tile(sV + st * BN * DP, vbase, stab + st * ppt, page_stride, k_begin + st * BN, k_end - 1, map, A.lim, TL_K_DECODE);
        }
        cp_async_commit();
    }
    cp_async_wait<DEC_STAGES - 1>();                       // the queries are in
    __syncthreads();
    uint32_t qf[KBLK][4];                                  // Q fragments stay in registers for the whole range
#pragma unroll
    for (int kb = 0; kb < KBLK; ++kb)
        ldsm_x4(qf[kb], sQ + ((lane & 7) + ((lane >> 3) & 1) * 8) * DP + kb * 16 + (lane >> 4) * 8);
    const int pos_r[2] = {k_end - 1, k_end - 1};           // every row sees all keys of the range
    const int lo_r[2] = {max(lo, k_begin), max(lo, k_begin)};
    float o[D / 8][4];
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) { o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int st = 0; st < n_stage; ++st) {
        cp_async_wait<DEC_STAGES - 2>();
        __syncthreads();
        if (st + DEC_STAGES - 1 < n_stage) {
            const int nst = st + DEC_STAGES - 1, nb_ = nst % DEC_STAGES;
            load_kv_tile(sK + nb_ * BN * DP, kbase, stab + nst * ppt, page_stride, k_begin + nst * BN, k_end - 1, map, A.lim, TL_K_DECODE);
            load_kv_tile(sV + nb_ * BN * DP, vbase, stab + nst * ppt, page_stride, k_begin + nst * BN, k_end - 1, map, A.lim, TL_K_DECODE);
        }
        cp_async_commit();
        const int buf = st % DEC_STAGES;
        const int key0 = k_begin + st * BN + warp * 16;    // this warp's 16 keys of the stage
        if (key0 >= k_end) continue;
        float s[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
        qk_tile_regs<2>(s, qf, sK + buf * BN * DP, warp * 16, lane);
        if (key0 + 16 <= k_end && key0 >= lo) softmax_step<2, false>(s, o, m, l, pos_r, lo_r, key0, A.scale_log2, lane);
        else                                  softmax_step<2, true>(s, o, m, l, pos_r, lo_r, key0, A.scale_log2, lane);
        pv_tile<2>(o, s, sV + buf * BN * DP, warp * 16, lane);
    }
    cp_async_wait<0>();
    __syncthreads();                                       // the stage buffers become the merge area

    // merge the four warps: each holds (m, l, O) over its own keys, same fragment layout
    float* mO = reinterpret_cast<float*>(sK);              // [4][16][D]
    float* mML = mO + 4 * 16 * D;                          // [4][16][2]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float lr = l[r];
        lr += __shfl_xor_sync(0xffffffffu, lr, 1);
        lr += __shfl_xor_sync(0xffffffffu, lr, 2);
        const int row = (lane >> 2) + r * 8;
        if ((lane & 3) == 0) { mML[(warp * 16 + row) * 2] = m[r]; mML[(warp * 16 + row) * 2 + 1] = lr; }
#pragma unroll
        for (int nb = 0; nb < D / 8; ++nb) {
            float* dst = mO + (warp * 16 + row) * D + nb * 8 + (lane & 3) * 2;
            dst[0] = o[nb][2 * r]; dst[1] = o[nb][2 * r + 1];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < 16 * D; idx += 128) {
        const int row = idx / D, col = idx - row * D;
        const int hg = mt * 16 + row;
        if (hg >= g) continue;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, mML[(w * 16 + row) * 2]);
        float acc = 0.f, lt = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = mML[(w * 16 + row) * 2];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - mm);
            acc += f * mO[(w * 16 + row) * D + col];
            lt += f * mML[(w * 16 + row) * 2 + 1];
        }
        const int head = kh * g + hg;
        if (A.splits == 1) {
            A.out[((size_t)qrow * A.nq + head) * D + col] = __float2bfloat16_rn(lt > 0.f ? acc / lt : 0.f);
        } else {
            const size_t pi = ((size_t)b * A.nq + head) * A.splits + split;
            A.part_o[pi * D + col] = acc;
            if (col == 0) { A.part_ml[pi * 2] = mm; A.part_ml[pi * 2 + 1] = lt; }
        }
    }
}

#if HEAD_DIM % 64 == 0
// ------------------------------------------------------------------------------------ decode, TMA variant
// The same split-KV decode attention with K and V brought in by TMA: a page's part for one KV head is a
// contiguous [page, d] slab of the cache, so one thread issues a few tensor copies per 64-key stage
// (128-byte swizzle, no per-thread address arithmetic) and the 128 threads only wait on the stage's
// mbarrier.  Taken for head sizes that are multiples of 64 and pages of at least 8 tokens (a page's box
// then starts on a 1024-byte boundary of the swizzle pattern); everything after the loads is the code
// of the kernel above, reading the swizzled tile instead of the padded one.
constexpr int TMA_TILE_BYTES = BN * D * 2;                       // K or V of one stage
constexpr int TMA_Q_OFFSET = 2 * DEC_STAGES * TMA_TILE_BYTES;
constexpr int TMA_BAR_OFFSET = TMA_Q_OFFSET + ((16 * DP * 2 + 15) / 16) * 16;
constexpr int TMA_CS_OFFSET = TMA_BAR_OFFSET + 128;              // room for 2 * DEC_STAGES barriers and a flag; then cos, sin [D]
// Where the other blocks of a cluster put their shares of this block's columns (CLUSTER): [key range][16 rows][columns of this
// block] floats, at most 16 (D + 16) in all, then (m, l) [key range][16 rows], for up to 16 key ranges.  Not in the stage buffers: a block that has
// finished writes here while this one may still be loading keys.
constexpr int TMA_RECV_OFFSET = TMA_CS_OFFSET + D * 4;
constexpr int TMA_MAX_RANGES = 16;                               // key ranges of a cluster: 8 is the portable size, 16 this GPU's
// The receive area is as large as the launch's number of ranges asks (none without a cluster), the table copy follows it:
// with 8 ranges and a table of up to 400 pages two blocks still share an SM.
__host__ __device__ constexpr int tma_recv_ml_offset(int ranges) { return TMA_RECV_OFFSET + 16 * (D + ranges) * 4; }
__host__ __device__ constexpr int tma_tab_offset(int ranges) {
    return ranges > 0 ? tma_recv_ml_offset(ranges) + ranges * 16 * 2 * 4 : TMA_RECV_OFFSET;
}
#ifndef TL_TMA_COPY_WARPS
#define TL_TMA_COPY_WARPS 2
#endif
constexpr int TMA_COPY_WARPS = TL_TMA_COPY_WARPS;
constexpr int TMA_DEC_THREADS = 128 + 32 * TMA_COPY_WARPS;       // four compute warps and the copy warps
static_assert(2 * DEC_STAGES * 8 + 8 <= 128, "the barrier area holds at most 7 stages");
constexpr int TMA_MERGE_OK = (TMA_Q_OFFSET >= DECODE_MERGE_SMEM + 6 * 16 * 4) ? 1 : 0;
static_assert(tma_tab_offset(TMA_MAX_RANGES) + DECODE_MAX_TAB * 4 + 1024 <= 227 * 1024, "the decode block does not fit an SM's shared memory");
static_assert(TMA_MERGE_OK == 1, "the stage buffers must hold the merge area");
constexpr long long TMA_WAIT_CYCLES = 4000000000LL;

__device__ __forceinline__ const bf16* swz_ptr(const unsigned char* tile, int key, int c) {
    return reinterpret_cast<const bf16*>(tile + (c >> 3) * (BN * 128) + key * 128 + (((c & 7) ^ (key & 7)) << 4));
}
__device__ __forceinline__ bool mbar_try_wait_tma(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded: gives up after about two seconds, records the fact and lets the block leave.
__device__ __forceinline__ bool mbar_wait_tma(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
    if (mbar_try_wait_tma(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_wait_tma(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > TMA_WAIT_CYCLES) {
            *abort_flag = 1;
            if (status) atomicCAS(status, 0, 20);
            return false;
        }
    }
}

__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");   // not .aligned: lanes of a warp may arrive apart
}
// The same shared-memory location in block `rank` of this cluster.
__device__ __forceinline__ float* cluster_peer_rw(float* p, int rank) {
    uint64_t out;
    asm volatile("mapa.u64 %0, %1, %2;" : "=l"(out) : "l"(reinterpret_cast<uint64_t>(p)), "r"(rank));
    return reinterpret_cast<float*>(out);
}

// CLUSTER: the blocks of one (request, KV head) - one per key range - form a thread-block cluster and merge their
// partial results through distributed shared memory (every block finishes a slice of the head dimension), so
// nothing goes through global memory and no combine kernel follows.  Needs 2 to 8 key ranges and at most 16
// query heads per KV head (one row tile).  A block whose key range is empty takes part with weight zero.
template <bool CLUSTER>
__global__ void __launch_bounds__(TMA_DEC_THREADS)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const AttnArgs A, int* status) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    bf16* sQ = reinterpret_cast<bf16*>(tiles + TMA_Q_OFFSET);              // [16][DP], padded rows
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + TMA_BAR_OFFSET);  // [DEC_STAGES]: the stage's copies have landed
    uint64_t* empty = full + DEC_STAGES;                                   // [DEC_STAGES]: the four compute warps are done with it
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + DEC_STAGES);
    int* stab = reinterpret_cast<int*>(tiles + tma_tab_offset(CLUSTER ? A.splits : 0));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) tl_stamp(A.trace, 0);
    const int g = A.nq / A.nkv, m_tiles = (g + 15) / 16;
    const int split = blockIdx.x / m_tiles, mt = blockIdx.x % m_tiles;
    const int kh = blockIdx.y, b = blockIdx.z;
    const int pos = A.start_pos[b], len = pos + 1;
    const int lo = A.window > 0 ? max(0, len - A.window) : 0;
    const int base = (lo / BN) * BN;
    const int k_begin = base + split * A.chunk;
    if (!CLUSTER && k_begin >= len) return;
    const int k_end = max(k_begin, min(len, k_begin + A.chunk));
    const int n_stage = (k_end - k_begin + BN - 1) / BN;  // 0: an empty range (CLUSTER only)
    const int* gtab = A.table + (size_t)tl_checked(A.slots[b], A.lim.table_rows, A.lim, TL_K_DECODE_TMA) * A.max_pages;
    const int qrow = A.q_start[b];
    const int ppt = BN / A.page_size, first_page = k_begin / A.page_size;
    const int n_pages = (k_end - 1) / A.page_size - first_page + 1;
    for (int i = tid; i < n_stage * ppt; i += TMA_DEC_THREADS)
        stab[i] = i < n_pages ? tl_checked(gtab[tl_checked(first_page + i, A.max_pages, A.lim, TL_K_DECODE_TMA)], A.lim.total_pages,
                                           A.lim, TL_K_DECODE_TMA) : 0;
    if (tid == 0) {
        for (int s_ = 0; s_ < DEC_STAGES; ++s_) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(full + s_)), "r"(TMA_COPY_WARPS));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(empty + s_)), "r"(4));
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid == 128) {                                      // a copy thread fetches the two descriptors meanwhile
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    const bool fold = A.rope_inv_freq != nullptr;          // bias and rotation of q, k, v happen here, not in a kernel before
    // When this kernel itself makes and writes the token's own key and value, the pages hold nothing that the kernel in
    // front writes (what is in them is from earlier steps, whose kernels have all finished before this one may start): the
    // copy warps then request the first stages at once, while the kernel in front is still at its last tiles.
    const bool early = fold && A.rope_write;
    float* cs = reinterpret_cast<float*>(tiles + TMA_CS_OFFSET);
    if (warp < 4 && fold) {                                // the token's angles, once for all its heads: positions and
        for (int i = tid; i < D / 2; i += 128) {           // frequencies are not the kernel in front's, so before the wait
            float sn, c;
            sincosf(__fmul_rn((float)pos, A.rope_inv_freq[i]), &sn, &c);
            cs[i] = c; cs[D / 2 + i] = sn;
        }
    }
    __syncthreads();                                       // table copy, barriers and angles are visible
    // The token's own key and value: made by the block whose range holds its position, written to their page by one of the
    // blocks of that range (the first row tile), and kept in registers to be put into this block's tiles when that stage
    // has landed (the page in memory still holds what was there before).
    const bool has_new = fold && A.rope_write && n_stage > 0 && pos >= k_begin && pos < k_end;
    const int st_new = has_new ? (pos - k_begin) / BN : -1, r_new = (pos - k_begin) % BN;
    uint4 new_lo = make_uint4(0, 0, 0, 0), new_hi = new_lo;
    int new_i0 = -1, new_is_v = 0;
    if (has_new && warp < 4) {
        constexpr int PER = D / 16;
        if (tid >= 64 && tid < 64 + PER) { new_i0 = (tid - 64) * 8; new_is_v = 0; }
        else if (tid >= 96 && tid < 96 + PER) { new_i0 = (tid - 96) * 8; new_is_v = 1; }
    }
    if (warp < 4 || !early) {
        grid_dependency_wait();                            // queries and the newest keys and values: the kernel before
        if (tid == 0) tl_stamp(A.trace, 1);
        grid_dependency_trigger();
    }
    if (warp < 4 && !fold) {
        for (int idx = tid; idx < 16 * CH; idx += 128) {
            const int r = idx / CH, c = idx - r * CH;
            const int hg = mt * 16 + r;
            const bool valid = hg < g;
            const bf16* src = A.q;
            if (valid) src = A.q + (size_t)qrow * A.q_stride + (size_t)(kh * g + hg) * D + c * 8;
            cp_async16(sQ + r * DP + c * 8, src, valid);
        }
        cp_async_commit();
    }
    if (warp < 4 && fold) {
        // the loads of the new key's or value's item go out before the query items are worked on: one round trip, not two
        const int new_col = (A.nq + (new_is_v ? A.nkv : 0) + kh) * D;
        uint4 nav = make_uint4(0, 0, 0, 0), nbv = nav;
        if (new_i0 >= 0) {
            const bf16* nrow = A.q + (size_t)qrow * A.q_stride + new_col;
            nav = *reinterpret_cast<const uint4*>(nrow + new_i0); nbv = *reinterpret_cast<const uint4*>(nrow + D / 2 + new_i0);
        }
        constexpr int PER = D / 16;                        // items of 8 + 8 values a head
        for (int item = tid; item < 16 * PER; item += 128) {
            const int r = item / PER, i0 = (item - r * PER) * 8, hg = mt * 16 + r;
            uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
            if (hg < g) {
                const int head = kh * g + hg;
                const bf16* row = A.q + (size_t)qrow * A.q_stride + (size_t)head * D;
                rope_pairs(*reinterpret_cast<const uint4*>(row + i0), *reinterpret_cast<const uint4*>(row + D / 2 + i0),
                           A.rope_bias, A.rope_bias_f32, head * D, i0, cs, true, lo, hi);
            }
            *reinterpret_cast<uint4*>(sQ + r * DP + i0) = lo;
            *reinterpret_cast<uint4*>(sQ + r * DP + D / 2 + i0) = hi;
        }
        if (new_i0 >= 0) {
            rope_pairs(nav, nbv, A.rope_bias, A.rope_bias_f32, new_col, new_i0, cs, !new_is_v, new_lo, new_hi);
            if (mt == 0) {
                const int page = stab[pos / A.page_size - first_page];
                bf16* dst = (new_is_v ? A.v_pages_w : A.k_pages_w) + (((size_t)page * A.nkv + kh) * A.page_size + pos % A.page_size) * D;
                *reinterpret_cast<uint4*>(dst + new_i0) = new_lo;
                *reinterpret_cast<uint4*>(dst + D / 2 + new_i0) = new_hi;
            }
        }
    }

    // The copy warps: a TMA copy takes about 95 cycles to issue, whether the boxes of a stage come from one thread
    // or from the lanes of one warp instruction, and a stage is 2 * (64 / page) * (D / 64) boxes (16 for pages of
    // 16 tokens and head size 128: 1,550 cycles, more than the four compute warps need for the stage).  So the
    // boxes are dealt out to TMA_COPY_WARPS warps, each with its own share of the stage's bytes on the barrier.
    if (warp >= 4) {
        const int w = warp - 4;
        constexpr int DB = D / 64;
        const int per_tensor = ppt * DB, total = 2 * per_tensor;
        const int mine = (total - w + TMA_COPY_WARPS - 1) / TMA_COPY_WARPS;       // boxes w, w + TMA_COPY_WARPS, ...
        const uint32_t box_bytes = (uint32_t)A.page_size * 128u;
        for (int st = 0; st < n_stage; ++st) {
            const int buf = st % DEC_STAGES;
            if (st >= DEC_STAGES && !mbar_wait_tma(empty + buf, ((st / DEC_STAGES) - 1) & 1, abort_flag, status)) break;
            unsigned char* kt = tiles + buf * 2 * TMA_TILE_BYTES;
            if (lane == 0)
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(full + buf)), "r"(mine * box_bytes) : "memory");
            __syncwarp();
            for (int k = lane; k < mine; k += 32) {
                const int idx = w + k * TMA_COPY_WARPS;
                const int is_v = idx >= per_tensor, rem = idx - is_v * per_tensor;
                const int pg = rem / DB, db = rem - pg * DB;
                const int row = (stab[st * ppt + pg] * A.nkv + kh) * A.page_size;
                const uint32_t dst = smem_u32(kt + is_v * TMA_TILE_BYTES + db * (BN * 128) + pg * A.page_size * 128);
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                             ::"r"(dst), "l"(is_v ? &map_v : &map_k), "r"(smem_u32(full + buf)), "r"(db * 64), "r"(row) : "memory");
            }
        }
        __syncthreads();                                   // meets the compute warps after their last stage
        __syncthreads();                                   // and after they have laid out their partial results
        if (CLUSTER) cluster_barrier();                    // every thread of the cluster takes part in its barrier
        return;
    }
    cp_async_wait<0>();
    asm volatile("bar.sync 1, 128;" ::: "memory");         // the queries are in (the four compute warps only)
    (void)r_new;
    uint32_t qf[KBLK][4];
#pragma unroll
    for (int kb = 0; kb < KBLK; ++kb)
        ldsm_x4(qf[kb], sQ + ((lane & 7) + ((lane >> 3) & 1) * 8) * DP + kb * 16 + (lane >> 4) * 8);
    const int pos_r[2] = {k_end - 1, k_end - 1};
    const int lo_r[2] = {max(lo, k_begin), max(lo, k_begin)};
    float o[D / 8][4];
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) { o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int st = 0; st < n_stage; ++st) {
        const int buf = st % DEC_STAGES;
        if (!mbar_wait_tma(full + buf, (st / DEC_STAGES) & 1, abort_flag, status)) break;
        if (tid == 0 && st == 0) tl_stamp(A.trace, 2);
        if (tid == 0 && st == n_stage - 1) tl_stamp(A.trace, 3);
        if (st == st_new) {                                // the stage with the token's own position: its new key and value
            if (new_i0 >= 0) {
                unsigned char* tile = tiles + buf * 2 * TMA_TILE_BYTES + (new_is_v ? TMA_TILE_BYTES : 0);
                const int c_lo = new_i0 >> 3, c_hi = (D / 2 + new_i0) >> 3;
                *reinterpret_cast<uint4*>(tile + (c_lo >> 3) * (BN * 128) + r_new * 128 + (((c_lo & 7) ^ (r_new & 7)) << 4)) = new_lo;
                *reinterpret_cast<uint4*>(tile + (c_hi >> 3) * (BN * 128) + r_new * 128 + (((c_hi & 7) ^ (r_new & 7)) << 4)) = new_hi;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // before a later TMA copy into the same buffer
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        const int key0 = k_begin + st * BN + warp * 16;    // this warp's 16 keys of the stage
        if (key0 >= k_end) {                               // none of them exist: hand the buffer back at once
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(empty + buf)) : "memory");
            continue;
        }
        const unsigned char* kt = tiles + buf * 2 * TMA_TILE_BYTES;
        const unsigned char* vt = kt + TMA_TILE_BYTES;
        float s[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
        for (int kb = 0; kb < KBLK; ++kb) {                // S = Q K^T on this warp's 16 keys
            uint32_t bfr[4];
            ldsm_x4(bfr, swz_ptr(kt, warp * 16 + (lane & 7) + (lane >> 4) * 8, kb * 2 + ((lane >> 3) & 1)));
            mma_bf16(s[0], qf[kb], bfr[0], bfr[1]);
            mma_bf16(s[1], qf[kb], bfr[2], bfr[3]);
        }
        if (key0 + 16 <= k_end && key0 >= lo) softmax_step<2, false>(s, o, m, l, pos_r, lo_r, key0, A.scale_log2, lane);
        else                                  softmax_step<2, true>(s, o, m, l, pos_r, lo_r, key0, A.scale_log2, lane);
        uint32_t a[4];
        a[0] = pack_bf16(s[0][0], s[0][1]); a[1] = pack_bf16(s[0][2], s[0][3]);
        a[2] = pack_bf16(s[1][0], s[1][1]); a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int nb = 0; nb < D / 8; nb += 2) {            // O += P V
            uint32_t bfr[4];
            ldsm_x4_trans(bfr, swz_ptr(vt, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, nb + (lane >> 4)));
            mma_bf16(o[nb], a, bfr[0], bfr[1]);
            mma_bf16(o[nb + 1], a, bfr[2], bfr[3]);
        }
        __syncwarp();                                      // every lane has read the stage
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(empty + buf)) : "memory");
    }
    if (tid == 0) tl_stamp(A.trace, 5);
    __syncthreads();                                       // the stage buffers become the merge area
    if (*abort_flag) {
        __syncthreads();
        if (CLUSTER) cluster_barrier();                    // the others must not wait for this block for ever
        return;
    }

    float* mO = reinterpret_cast<float*>(tiles);           // [4][16][D]   every warp's part (its 16 keys of every stage)
    float* mML = mO + 4 * 16 * D;                          // [4][16][2]
    float* sF = mML + 4 * 16 * 2;                          // [4][16]      a warp's weight in the block's result
    float* sMM = sF + 4 * 16;                              // [16]         the block's running maximum and sum
    float* sLT = sMM + 16;                                 // [16]
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float lr = l[r];
        lr += __shfl_xor_sync(0xffffffffu, lr, 1);
        lr += __shfl_xor_sync(0xffffffffu, lr, 2);
        const int row = (lane >> 2) + r * 8;
        if (mt * 16 + row >= g) continue;                  // a row beyond the group: nothing reads it
        if ((lane & 3) == 0) { mML[(warp * 16 + row) * 2] = m[r]; mML[(warp * 16 + row) * 2 + 1] = lr; }
#pragma unroll
        for (int nb = 0; nb < D / 8; ++nb) {
            float* dst = mO + (warp * 16 + row) * D + nb * 8 + (lane & 3) * 2;
            *reinterpret_cast<float2*>(dst) = make_float2(o[nb][2 * r], o[nb][2 * r + 1]);
        }
    }
    __syncthreads();
    if (tid < 16 && mt * 16 + tid < g) {                   // the four warps' weights, once a row
        const int row = tid;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, mML[(w * 16 + row) * 2]);
        float lt = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = mML[(w * 16 + row) * 2];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - mm);
            sF[w * 16 + row] = f;
            lt += f * mML[(w * 16 + row) * 2 + 1];
        }
        sMM[row] = mm; sLT[row] = lt;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const int ns = A.splits, cpc = (D + ns - 1) / ns;      // CLUSTER: block s finishes columns [s * cpc, + cpc)
    float* recvO = reinterpret_cast<float*>(tiles + TMA_RECV_OFFSET);
    float* recvML = reinterpret_cast<float*>(tiles + tma_recv_ml_offset(A.splits));
    const int rows = min(16, g - mt * 16);
    for (int col = tid; col < D; col += 128) {             // a column a thread: the block's result, sent where it is finished
        float* dst_o = nullptr;
        if (CLUSTER) {
            const int owner = col / cpc;
            dst_o = cluster_peer_rw(recvO + (split * 16) * cpc + (col - owner * cpc), owner);
        }
        for (int row = 0; row < rows; ++row) {
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) acc += sF[w * 16 + row] * mO[(w * 16 + row) * D + col];
            const int head = kh * g + mt * 16 + row;
            if (CLUSTER) {
                dst_o[row * cpc] = acc;
            } else if (A.splits == 1) {
                const float lt = sLT[row];
                A.out[((size_t)qrow * A.nq + head) * D + col] = __float2bfloat16_rn(lt > 0.f ? acc / lt : 0.f);
            } else {
                const size_t pi = ((size_t)b * A.nq + head) * A.splits + split;
                A.part_o[pi * D + col] = acc;
                if (col == 0) { A.part_ml[pi * 2] = sMM[row]; A.part_ml[pi * 2 + 1] = sLT[row]; }
            }
        }
    }
    if (CLUSTER) {
        for (int i = tid; i < ns * 16; i += 128) {         // (m, l) of every row to every block
            const int owner = i >> 4, row = i & 15;
            if (row < rows) {
                float* dst = cluster_peer_rw(recvML + (split * 16 + row) * 2, owner);
                dst[0] = sMM[row]; dst[1] = sLT[row];
            }
        }
        if (tid == 0) tl_stamp(A.trace, 6);
        cluster_barrier();                                 // all shares have arrived; nobody touches another block's memory after this
        if (tid == 0) tl_stamp(A.trace, 7);
        for (int idx = tid; idx < rows * cpc; idx += 128) {
            const int row = idx / cpc, c = idx - row * cpc, col = split * cpc + c;
            if (col >= D) continue;
            float ms[TMA_MAX_RANGES], ls[TMA_MAX_RANGES], os[TMA_MAX_RANGES];
            float mm = -INFINITY;
#pragma unroll
            for (int sp = 0; sp < TMA_MAX_RANGES; ++sp) {
                if (sp < ns) {
                    ms[sp] = recvML[(sp * 16 + row) * 2]; ls[sp] = recvML[(sp * 16 + row) * 2 + 1];
                    os[sp] = recvO[(sp * 16 + row) * cpc + c];
                    mm = fmaxf(mm, ms[sp]);
                }
            }
            float acc = 0.f, lt = 0.f;
#pragma unroll
            for (int sp = 0; sp < TMA_MAX_RANGES; ++sp) {
                if (sp < ns) {
                    const float f = ms[sp] == -INFINITY ? 0.f : exp2f(ms[sp] - mm);
                    acc += f * os[sp]; lt += f * ls[sp];
                }
            }
            A.out[((size_t)qrow * A.nq + kh * g + row) * D + col] = __float2bfloat16_rn(lt > 0.f ? acc / lt : 0.f);
        }
    }
    if (tid == 0) tl_stamp(A.trace, 4);
}
#endif  // HEAD_DIM % 64 == 0

// grid (nq, B): merges the partials of the non-empty splits of one (request, head).
__global__ void attn_combine_kernel(const AttnArgs A) {
    const int head = blockIdx.x, b = blockIdx.y;
    const int len = A.start_pos[b] + 1;
    const int lo = A.window > 0 ? max(0, len - A.window) : 0;
    const int base = (lo / BN) * BN;
    const int ns = min(A.splits, (len - base + A.chunk - 1) / A.chunk);
    const size_t p0 = ((size_t)b * A.nq + head) * A.splits;
    __shared__ float wgt[128];                             // a split's weight exp2(m_s - m); at most 128 splits
    __shared__ float inv_total;
    grid_dependency_wait();
    grid_dependency_trigger();
    const int qrow = A.q_start[b];
    if (ns > 128) {                                        // more splits than the weight table holds: one by one
        float mm = -INFINITY;
        for (int sp = 0; sp < ns; ++sp) mm = fmaxf(mm, A.part_ml[(p0 + sp) * 2]);
        float lt = 0.f;
        for (int sp = 0; sp < ns; ++sp) {
            const float ms = A.part_ml[(p0 + sp) * 2];
            lt += (ms == -INFINITY ? 0.f : exp2f(ms - mm)) * A.part_ml[(p0 + sp) * 2 + 1];
        }
        const float inv = lt > 0.f ? 1.0f / lt : 0.f;
        for (int col = threadIdx.x; col < D; col += blockDim.x) {
            float acc = 0.f;
            for (int sp = 0; sp < ns; ++sp) {
                const float ms = A.part_ml[(p0 + sp) * 2];
                acc += (ms == -INFINITY ? 0.f : exp2f(ms - mm)) * A.part_o[(p0 + sp) * D + col];
            }
            A.out[((size_t)qrow * A.nq + head) * D + col] = __float2bfloat16_rn(acc * inv);
        }
        return;
    }
    if (threadIdx.x < 32) {                                // all (m, l) pairs are requested at once: up to four a lane
        const int lane = threadIdx.x;
        float ms[4], ls[4];
        float mm = -INFINITY;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int sp = lane + 32 * k;
            ms[k] = -INFINITY; ls[k] = 0.f;
            if (sp < ns) {
                const float2 ml = *reinterpret_cast<const float2*>(A.part_ml + (p0 + sp) * 2);
                ms[k] = ml.x; ls[k] = ml.y;
            }
            mm = fmaxf(mm, ms[k]);
        }
        mm = warp_max(mm);
        float lt = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int sp = lane + 32 * k;
            const float f = ms[k] == -INFINITY ? 0.f : exp2f(ms[k] - mm);
            if (sp < ns) wgt[sp] = f;
            lt += f * ls[k];
        }
        lt = warp_sum(lt);
        if (lane == 0) inv_total = lt > 0.f ? 1.0f / lt : 0.f;
    }
    __syncthreads();
    const float inv = inv_total;
    for (int col = threadIdx.x; col < D; col += blockDim.x) {
        float acc = 0.f;
#pragma unroll 8
        for (int sp = 0; sp < ns; ++sp) acc += wgt[sp] * A.part_o[(p0 + sp) * D + col];
        A.out[((size_t)qrow * A.nq + head) * D + col] = __float2bfloat16_rn(acc * inv);
    }
}

template <int PBN> constexpr int prefill_smem() { return (BM + 4 * PBN) * DP * 2; }
constexpr int DECODE_SMEM_MAX = DECODE_TAB_OFFSET + DECODE_MAX_TAB * 4;

bool g_attr_done[TL_MAX_DEVICES] = {};        // kernel attributes belong to a device: each one is set up at its first call
int set_attrs() {
    const int dev = tl_device_index();
    if (dev < 0) return 1;
    if (g_attr_done[dev]) return 0;
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, prefill_smem<32>());
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, prefill_smem<64>());
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DECODE_SMEM_MAX);
    if (e != cudaSuccess) return (int)e;
    g_attr_done[dev] = true;
    return 0;
}

}  // namespace

TL_EXPORT int tl_attn_head_dim() { return D; }
// 1 if this library was compiled as the checking build (-DTL_CHECK=1).
TL_EXPORT int tl_check_build() { return TL_CHECKING; }
// Block-table entries a decode block may copy: chunk / page_size of a decode call may not exceed it.
TL_EXPORT int tl_attn_decode_max_table() { return DECODE_MAX_TAB; }


// total_tiles = sum over requests of ceil(q_len * g / 64), computed by the caller.
TL_EXPORT int tl_attn_prefill(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                              const int* table, int max_pages, int page_size, const int* q_start,
                              const int* start_pos, const int* slots, int B, int nq, int nkv, int window,
                              float scale, int total_tiles, const int* order, int table_rows, int total_pages, int* fault,
                              cudaStream_t stream) {
    if (total_tiles <= 0 || B <= 0) return 0;
    if (nq % nkv || BN % page_size) return 1;
    int e = set_attrs();
    if (e) return e;
    AttnArgs A{};
    A.q = (const bf16*)q; A.q_stride = q_stride; A.out = (bf16*)out;
    A.k_pages = (const bf16*)k_pages; A.v_pages = (const bf16*)v_pages;
    A.table = table; A.max_pages = max_pages; A.page_size = page_size;
    A.order = order;
    A.lim = TlLimits{table_rows, total_pages, fault};
    A.q_start = q_start; A.start_pos = start_pos; A.slots = slots;
    A.B = B; A.nq = nq; A.nkv = nkv; A.window = window; A.scale_log2 = scale * LOG2E;
    dim3 grid((unsigned)total_tiles * (unsigned)nkv);
    if (page_size <= 32) attn_prefill_kernel<32><<<grid, 128, prefill_smem<32>(), stream>>>(A);
    else                 attn_prefill_kernel<64><<<grid, 128, prefill_smem<64>(), stream>>>(A);
    return tl_launch_status();
}

// One query token per request (row q_start[b]).  `chunk` (a multiple of 64) keys per split; with
// splits > 1 the partials go to part_o [B, nq, splits, D] and part_ml [B, nq, splits, 2] (float)
// and tl_attn_combine must follow on the same stream.
TL_EXPORT int tl_attn_decode(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                             const int* table, int max_pages, int page_size, const int* q_start,
                             const int* start_pos, const int* slots, int B, int nq, int nkv, int window,
                             float scale, int chunk, int splits, float* part_o, float* part_ml,
                             int table_rows, int total_pages, int* fault, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (nq % nkv || BN % page_size || chunk % BN || splits < 1 || (splits > 1 && (!part_o || !part_ml))) return 1;
    int e = set_attrs();
    if (e) return e;
    AttnArgs A{};
    A.q = (const bf16*)q; A.q_stride = q_stride; A.out = (bf16*)out;
    A.k_pages = (const bf16*)k_pages; A.v_pages = (const bf16*)v_pages;
    A.table = table; A.max_pages = max_pages; A.page_size = page_size;
    A.q_start = q_start; A.start_pos = start_pos; A.slots = slots;
    A.B = B; A.nq = nq; A.nkv = nkv; A.window = window; A.scale_log2 = scale * LOG2E;
    A.chunk = chunk; A.splits = splits; A.part_o = part_o; A.part_ml = part_ml;
    A.lim = TlLimits{table_rows, total_pages, fault};
    const int g = nq / nkv, m_tiles = (g + 15) / 16;
    dim3 grid(splits * m_tiles, nkv, B);
    if (grid.z > 65535) return 1;
    const int tab_entries = chunk / page_size;            // of the longest range a block can have
    if (tab_entries > DECODE_MAX_TAB) return 1;
    e = launch_after_wait(attn_decode_kernel, grid, dim3(128), DECODE_TAB_OFFSET + tab_entries * 4, stream, A);
    if (e || splits == 1) return e;
    dim3 cgrid(nq, B);
    return launch_after_wait(attn_combine_kernel, cgrid, dim3(D < 128 ? ((D + 31) / 32) * 32 : 128), 0, stream, A);
}

#if HEAD_DIM % 64 == 0
namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
bool g_tma_attr_done[TL_MAX_DEVICES] = {};

// The cache tensor [pages, nkv, page, D] as rows of D elements; a box is one page of one KV head, 64 wide.
int make_pages_map(CUtensorMap* map, const void* base, long long rows, int page_size) {
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 101;
}
}  // namespace
#endif

// tl_attn_decode with K and V loaded by TMA.  Needs a head size that is a multiple of 64, pages of 8 to 64
// tokens, and `total_pages` (first dimension of the cache tensors).  `status`: device int for a wait that
// ran out (may be null).  Returns 2 if this build or these sizes do not take the TMA path.
namespace {
struct RopeFold { const float* inv_freq; const void* bias; int bias_f32; int write_kv; };

TlTraceHost g_trace;
int decode_tma_impl(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                    long long total_pages, const int* table, int max_pages, int page_size,
                    const int* q_start, const int* start_pos, const int* slots, int B, int nq, int nkv,
                    int window, float scale, int chunk, int splits, float* part_o, float* part_ml,
                    int* status, int cluster_merge, int table_rows, int* fault, const RopeFold& R, cudaStream_t stream) {
#if HEAD_DIM % 64 == 0
    if (B <= 0) return 0;
    if (R.inv_freq && ((q_stride & 7) || ((uintptr_t)q & 15) || (R.bias && ((uintptr_t)R.bias & 15)))) return 2;
    if (page_size < 8 || page_size > 64 || (page_size & (page_size - 1))) return 2;
    // cluster_merge: the key ranges of a (request, KV head) merge inside a thread-block cluster, no partials needed
    if (cluster_merge && (splits < 2 || splits > TMA_MAX_RANGES || nq / (nkv > 0 ? nkv : 1) > 16)) return 1;
    if (nq % nkv || chunk % BN || splits < 1 || (splits > 1 && !cluster_merge && (!part_o || !part_ml))) return 1;
    if (((uintptr_t)k_pages & 127) || ((uintptr_t)v_pages & 127)) return 2;
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn ||
            qres != cudaDriverEntryPointSuccess) return 100;
        g_encode = (EncodeTiledFn)fn;
    }
    const int tab_entries = chunk / page_size;
    if (tab_entries > DECODE_MAX_TAB) return 1;
    const int smem = tma_tab_offset(cluster_merge ? splits : 0) + tab_entries * 4 + 1024;
    const int dev_index = tl_device_index();
    if (dev_index < 0) return 1;
    if (!g_tma_attr_done[dev_index]) {
        cudaError_t ce = cudaFuncSetAttribute(attn_decode_tma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              tma_tab_offset(TMA_MAX_RANGES) + DECODE_MAX_TAB * 4 + 1024);
        if (ce == cudaSuccess)
            ce = cudaFuncSetAttribute(attn_decode_tma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      tma_tab_offset(TMA_MAX_RANGES) + DECODE_MAX_TAB * 4 + 1024);
        if (ce == cudaSuccess)                             // clusters of 9 to 16 blocks
            ce = cudaFuncSetAttribute(attn_decode_tma_kernel<true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (ce != cudaSuccess) return (int)ce;
        g_tma_attr_done[dev_index] = true;
    }
    int e = set_attrs();                                   // the combine kernel's library state
    if (e) return e;
    CUtensorMap mk, mv;
    const long long rows = total_pages * nkv * page_size;
    if ((e = make_pages_map(&mk, k_pages, rows, page_size))) return e;
    if ((e = make_pages_map(&mv, v_pages, rows, page_size))) return e;
    AttnArgs A{};
    A.q = (const bf16*)q; A.q_stride = q_stride; A.out = (bf16*)out;
    A.k_pages = (const bf16*)k_pages; A.v_pages = (const bf16*)v_pages;
    A.table = table; A.max_pages = max_pages; A.page_size = page_size;
    A.q_start = q_start; A.start_pos = start_pos; A.slots = slots;
    A.B = B; A.nq = nq; A.nkv = nkv; A.window = window; A.scale_log2 = scale * LOG2E;
    A.chunk = chunk; A.splits = splits; A.part_o = part_o; A.part_ml = part_ml;
    A.lim = TlLimits{table_rows, (int)total_pages, fault};
    A.rope_inv_freq = R.inv_freq; A.rope_bias = R.bias; A.rope_bias_f32 = R.bias_f32; A.rope_write = R.write_kv;
    A.trace = g_trace.take((unsigned)(splits * ((nq / nkv + 15) / 16) * nkv * B));
    A.k_pages_w = (bf16*)const_cast<void*>(k_pages); A.v_pages_w = (bf16*)const_cast<void*>(v_pages);
    const int g = nq / nkv, m_tiles = (g + 15) / 16;
    dim3 grid(splits * m_tiles, nkv, B);
    if (grid.z > 65535) return 1;
    if (cluster_merge) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid; cfg.blockDim = dim3(TMA_DEC_THREADS); cfg.dynamicSmemBytes = (size_t)smem; cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = tl_dependent_launch_enabled() ? 2 : 1;
        const cudaError_t ce = cudaLaunchKernelEx(&cfg, attn_decode_tma_kernel<true>, mk, mv, A, status);
        return ce != cudaSuccess ? (int)ce : tl_launch_status();
    }
    e = launch_after_wait(attn_decode_tma_kernel<false>, grid, dim3(TMA_DEC_THREADS), (size_t)smem, stream, mk, mv, A, status);
    if (e || splits == 1) return e;
    dim3 cgrid(nq, B);
    return launch_after_wait(attn_combine_kernel, cgrid, dim3(D < 128 ? ((D + 31) / 32) * 32 : 128), 0, stream, A);
#else
    return 2;
#endif
}
}  // namespace

// Tracing build: the TMA decode launches from now on leave their stamps in buf [slots][512][8] (device, zeroed by the
// caller), one slot a launch from `first` on; null: no more stamps.  Accepted and without effect in the ordinary build.
TL_EXPORT int tl_trace_set(long long* buf, int slots, int first) {
    g_trace.buf = buf; g_trace.slots = slots; g_trace.next = first;
    return g_trace.next;
}
TL_EXPORT int tl_trace_next() { return g_trace.next; }
TL_EXPORT int tl_trace_build() { return TL_TRACING; }

// Dynamic shared memory of a TMA decode block that merges `cluster_ranges` key ranges inside a cluster (0: no cluster) and
// copies `table_entries` block-table entries; -1 where this head size has no TMA kernel.  Two blocks share an SM (the plan
// of the key ranges counts on it) while twice this plus 2 KB stays within the SM's 228 KB.
TL_EXPORT int tl_attn_decode_tma_smem(int cluster_ranges, int table_entries) {
#if HEAD_DIM % 64 == 0
    return tma_tab_offset(cluster_ranges) + table_entries * 4 + 1024;
#else
    return -1;
#endif
}

TL_EXPORT int tl_attn_decode_tma(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                 long long total_pages, const int* table, int max_pages, int page_size,
                                 const int* q_start, const int* start_pos, const int* slots, int B, int nq, int nkv,
                                 int window, float scale, int chunk, int splits, float* part_o, float* part_ml,
                                 int* status, int cluster_merge, int table_rows, int* fault, cudaStream_t stream) {
    return decode_tma_impl(q, q_stride, out, k_pages, v_pages, total_pages, table, max_pages, page_size, q_start, start_pos, slots,
                           B, nq, nkv, window, scale, chunk, splits, part_o, part_ml, status, cluster_merge, table_rows, fault,
                           RopeFold{nullptr, nullptr, 0, 0}, stream);
}

// The same with the rotary step folded in (full rotation over rotate-half pairs, no q/k norm): `q` points at the step's q|k|v
// rows as the projection left them, [T, (nq + 2 nkv) * D] with row stride q_stride; bias (float or bfloat16, may be null)
// and inv_freq [D / 2] as tl_rope_kv_write takes them; write_kv: the token's key and value are written to their page.
// Returns 2 (nothing launched) for what it does not take; the caller then runs the rotary kernel and the decode kernel apart.
TL_EXPORT int tl_attn_decode_tma_rope(const void* qkv, int q_stride, void* out, void* k_pages, void* v_pages,
                                      long long total_pages, const int* table, int max_pages, int page_size,
                                      const int* q_start, const int* start_pos, const int* slots, int B, int nq, int nkv,
                                      int window, float scale, int chunk, int splits, float* part_o, float* part_ml,
                                      int* status, int cluster_merge, int table_rows, int* fault,
                                      const float* inv_freq, const void* bias, int bias_f32, int write_kv, cudaStream_t stream) {
    if (inv_freq == nullptr) return 1;
    return decode_tma_impl(qkv, q_stride, out, k_pages, v_pages, total_pages, table, max_pages, page_size, q_start, start_pos, slots,
                           B, nq, nkv, window, scale, chunk, splits, part_o, part_ml, status, cluster_merge, table_rows, fault,
                           RopeFold{inv_freq, bias, bias_f32, write_kv}, stream);
}

// ------------------------------------------------------------------------------------ no allocation
// tl_attn_decode_static: the split-KV decode attention for callers that cannot allocate device
// memory (declared in attn_static.h, which says who they are).  Same kernels as tl_attn_decode; the
// float partials of the key ranges live in the file-scope array below instead of caller-provided
// buffers.  This file has no counterpart for it in tzar-beep/Tensorline.
#include "attn_static.h"
#include <stdio.h>

static __device__ __align__(256) float g_static_partials[TL_ATTN_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = TL_MAX_DEVICES;
float* g_static_ptr[MAX_DEVICES] = {};      // device address of the array, per device, set at the first call

int fail(char* err, int err_len, int code, const char* msg) {
    if (err && err_len > 0) snprintf(err, (size_t)err_len, "%s", msg);
    return code;
}
}  // namespace

TL_EXPORT int tl_attn_decode_static(const void* q, int q_stride, void* out, const void* k_pages,
                                    const void* v_pages, const int* table, int max_pages, int page_size,
                                    const int* q_start, const int* start_pos, const int* slots, int B, int nq,
                                    int nkv, int window, float scale, int chunk, int splits,
                                    cudaStream_t stream, char* err, int err_len) {
    if (err && err_len > 0) err[0] = 0;
    if (B <= 0) return 0;
    if (nkv <= 0 || nq % nkv || page_size <= 0 || BN % page_size || chunk <= 0 || chunk % BN || splits < 1)
        return fail(err, err_len, 1, "tl_attn_decode_static: heads must group evenly, the page size must divide 64, "
                                     "chunk must be a positive multiple of 64 and splits at least 1");
    const size_t need = (size_t)B * nq * splits * (D + 2);         // partial outputs, then (max, sum) pairs
    if (splits > 1 && need > (size_t)TL_ATTN_STATIC_SCRATCH_FLOATS) {
        char msg[256];
        snprintf(msg, sizeof msg, "tl_attn_decode_static: B*nq*splits*(head_dim+2) = %zu floats of partials exceed "
                 "the static scratch of %d floats; use fewer splits or a smaller batch", need,
                 (int)TL_ATTN_STATIC_SCRATCH_FLOATS);
        return fail(err, err_len, 2, msg);
    }
    int dev = -1;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
        return fail(err, err_len, 3, "tl_attn_decode_static: no current CUDA device (or its index is 64 or more)");
    if (g_static_ptr[dev] == nullptr) {
        // Set-up, once per device, with that device current: in host code the array's name is only a
        // handle; the address the kernels need comes from the runtime.
        void* p = nullptr;
        ce = cudaGetSymbolAddress(&p, g_static_partials);
        if (ce != cudaSuccess || p == nullptr) {
            char msg[256];
            snprintf(msg, sizeof msg, "tl_attn_decode_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(ce));
            return fail(err, err_len, 4, msg);
        }
        g_static_ptr[dev] = static_cast<float*>(p);
    }
    int e = set_attrs();
    if (e) return fail(err, err_len, 5, "tl_attn_decode_static: cannot raise the kernels' shared-memory limit");
    const int tab_entries = chunk / page_size;
    if (tab_entries > DECODE_MAX_TAB)
        return fail(err, err_len, 6, "tl_attn_decode_static: chunk / page_size exceeds the block-table copy of a block");
    AttnArgs A{};
    A.q = (const bf16*)q; A.q_stride = q_stride; A.out = (bf16*)out;
    A.k_pages = (const bf16*)k_pages; A.v_pages = (const bf16*)v_pages;
    A.table = table; A.max_pages = max_pages; A.page_size = page_size;
    A.q_start = q_start; A.start_pos = start_pos; A.slots = slots;
    A.B = B; A.nq = nq; A.nkv = nkv; A.window = window; A.scale_log2 = scale * LOG2E;
    A.chunk = chunk; A.splits = splits;
    A.part_o = g_static_ptr[dev];
    A.part_ml = g_static_ptr[dev] + (size_t)B * nq * splits * D;
    const int g = nq / nkv, m_tiles = (g + 15) / 16;
    dim3 grid(splits * m_tiles, nkv, B);
    if (grid.z > 65535) return fail(err, err_len, 7, "tl_attn_decode_static: more than 65535 requests in one call");
    attn_decode_kernel<<<grid, 128, DECODE_TAB_OFFSET + tab_entries * 4, stream>>>(A);
    ce = cudaGetLastError();
    if (ce == cudaSuccess && splits > 1) {
        dim3 cgrid(nq, B);
        attn_combine_kernel<<<cgrid, D < 128 ? ((D + 31) / 32) * 32 : 128, 0, stream>>>(A);
        ce = cudaGetLastError();
    }
    if (ce != cudaSuccess) {
        char msg[256];
        snprintf(msg, sizeof msg, "tl_attn_decode_static: launch failed: %s", cudaGetErrorString(ce));
        return fail(err, err_len, 8, msg);
    }
    return 0;
}
