// Paged causal grouped-query flash attention for prompt portions on the 5th-generation tensor cores
// (sm_100a), compiled for one head size (-DHEAD_DIM=d, d a multiple of 64 up to 256).
//
// One block = one (request, KV head, tile of 128 query rows); a row is a (token, query head of the
// group) pair, so the g heads that share a KV head share every K/V load (tensorline/paged_attn.py:33-35).
// Per tile of 64 keys:
//     S = Q K^T          tcgen05.mma, Q and K in shared memory (K-major, 128-byte swizzle), S in tensor memory
//     P = exp2(S - m)    128 threads, one row each: tcgen05.ld, mask (key <= position, window), running
//                        max and sum in float, P rounded to bfloat16 into shared memory (the same swizzle)
//     O += P V           tcgen05.mma, V as the MN-major operand, O in tensor memory
// K and V come straight from the cache pages (cp.async, 16 bytes, swizzled on the way in): this step's own
// tokens were written there first (tensorline/paged.py:252-253), so fresh prompts, resumed portions and
// decoded tokens riding along are one case.  The running maximum is only raised when a tile exceeds it by
// more than 2^8, so the correction of O (a round trip through registers) is rare.  Formulas as in
// tensorline/paged_attn.py:46-57: scores, max, sum and the accumulator in float, P in bfloat16 for P V.
// Every mbarrier wait is bounded; on a time-out the block records a code in `status` and leaves.
#include "common.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size>"
#endif
#if HEAD_DIM % 64 != 0 || HEAD_DIM < 64 || HEAD_DIM > 256
#error "the tcgen05 attention kernel takes head sizes 64, 128, 192, 256"
#endif

namespace {

constexpr int D = HEAD_DIM;
constexpr int BM = 128;                 // query rows per block = MMA M = tensor-memory lanes
constexpr int BN = 64;                  // keys per tile
constexpr int THREADS = 160;            // warps 0..3: loads, softmax, epilogue (one row each); warp 4: MMA issue
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;
constexpr long long WAIT_CYCLES = 4000000000LL;

constexpr int Q_BYTES = BM * D * 2, K_BYTES = BN * D * 2, V_BYTES = BN * D * 2, P_BYTES = BM * BN * 2;
constexpr int SMEM_TILES = Q_BYTES + K_BYTES + 2 * V_BYTES + P_BYTES;
constexpr int SMEM_BYTES = SMEM_TILES + 1024 + 64;
constexpr uint32_t TMEM_COLS = (BN + D) <= 256 ? 256 : 512;
constexpr uint32_t S_COL = 0, O_COL = BN;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_CYCLES) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Offset of 16-byte chunk `c` (0..D/8-1) of row `r` in a [rows][D] tile stored as D/64 blocks of
// [rows][64 elements] with the 128-byte swizzle (chunk index xor row mod 8), the layout the MMA's
// shared-memory descriptors with SWIZZLE_128B describe.
__device__ __forceinline__ uint32_t swz(int rows, int r, int c) {
    return (uint32_t)((c >> 3) * rows * 128 + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

// K-major operand: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand (V: the head dimension is contiguous): 64-element blocks of the MN dimension
// `lbo` bytes apart, 8-key groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t lbo) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&r)[32]) {
    uint32_t* u = reinterpret_cast<uint32_t*>(r);
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]),
                   "=r"(u[8]), "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]),
                   "=r"(u[16]), "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]),
                   "=r"(u[24]), "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&r)[32]) {
    const uint32_t* u = reinterpret_cast<const uint32_t*>(r);
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]),
                   "r"(u[8]), "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]),
                   "r"(u[16]), "r"(u[17]), "r"(u[18]), "r"(u[19]), "r"(u[20]), "r"(u[21]), "r"(u[22]), "r"(u[23]),
                   "r"(u[24]), "r"(u[25]), "r"(u[26]), "r"(u[27]), "r"(u[28]), "r"(u[29]), "r"(u[30]), "r"(u[31])
                 : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct TcAttnArgs {
    const bf16* q; int q_stride;
    bf16* out;
    const bf16* k_pages; const bf16* v_pages;
    const int* table; int max_pages; int page_size;
    const int* q_start; const int* start_pos; const int* slots;
    int B, nq, nkv, window;
    float scale_log2;
    int* status;
};

// Keys [key0, key0 + BN) of one KV head into a swizzled [BN][D] tile; keys past last_key are zeros.
__device__ __forceinline__ void load_kv(uint32_t dst, const bf16* pages, const int* tab, int page_size, size_t page_stride,
                                        int key0, int last_key, int tid) {
    constexpr int CH = D / 8;
    for (int idx = tid; idx < BN * CH; idx += 128) {
        const int key = idx / CH, c = idx - key * CH;
        const int j = key0 + key;
        const bool valid = j <= last_key;
        const bf16* src = pages;
        if (valid) src = pages + (size_t)tab[j / page_size] * page_stride + (size_t)(j % page_size) * D + c * 8;
        cp_async16(dst + swz(BN, key, c), src, valid);
    }
}

__global__ void __launch_bounds__(THREADS, 1) attn_tc_prefill_kernel(const TcAttnArgs A) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sQ = smem_addr(base), sK = sQ + Q_BYTES, sV = sK + K_BYTES, sP = sV + 2 * V_BYTES;
    uint64_t* bar_s = reinterpret_cast<uint64_t*>(base + SMEM_TILES);      // an MMA batch finished (commit)
    uint64_t* bar_p = bar_s + 1;                                           // 128 rows handed P / the next K, V over
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_p + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int kh = blockIdx.y, g = A.nq / A.nkv;

    int tile = gridDim.x - 1 - blockIdx.x, b = 0;          // longest tiles (late rows of a request) first
    for (; b < A.B; ++b) {
        const int nt = ((A.q_start[b + 1] - A.q_start[b]) * g + BM - 1) / BM;
        if (tile < nt) break;
        tile -= nt;
    }
    if (b >= A.B) return;
    const int qs = A.q_start[b], qlen = A.q_start[b + 1] - qs, sp = A.start_pos[b];
    const int rows_total = qlen * g, row0 = tile * BM;
    const int row_end = min(row0 + BM, rows_total);
    const int* tab = A.table + (size_t)A.slots[b] * A.max_pages;
    const int pos_hi = sp + (row_end - 1) / g, pos_first = sp + row0 / g;
    const int key_lo = A.window > 0 ? max(0, pos_first - A.window + 1) : 0;
    const int kt_lo = key_lo / BN, kt_hi = pos_hi / BN, n_kt = kt_hi - kt_lo + 1;

    if (tid == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_p, 128);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const size_t page_stride = (size_t)A.nkv * A.page_size * D;
    const bf16* kbase = A.k_pages + (size_t)kh * A.page_size * D;
    const bf16* vbase = A.v_pages + (size_t)kh * A.page_size * D;

    if (warp < 4) {
        // ------------------------------------------------------------ loads, softmax, epilogue: thread = row
        constexpr int CH = D / 8;
        for (int idx = tid; idx < BM * CH; idx += 128) {    // Q tile: row = (token, head of the group)
            const int r = idx / CH, c = idx - r * CH;
            const int R = row0 + r;
            const bool valid = R < rows_total;
            const bf16* src = A.q;
            if (valid) src = A.q + (size_t)(qs + R / g) * A.q_stride + (size_t)(kh * g + R % g) * D + c * 8;
            cp_async16(sQ + swz(BM, r, c), src, valid);
        }
        load_kv(sK, kbase, tab, A.page_size, page_stride, kt_lo * BN, pos_hi, tid);
        load_kv(sV, vbase, tab, A.page_size, page_stride, kt_lo * BN, pos_hi, tid);
        cp_async_wait_all();
        fence_async_proxy();
        mbar_arrive(bar_p);                                 // phase 0: Q, K(0), V(0) are in shared memory

        const int R = row0 + tid;
        const int pos_r = R < rows_total ? sp + R / g : -1; // -1: no key is visible
        const int lo_r = A.window > 0 ? max(0, pos_r - A.window + 1) : 0;
        const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;

        for (int i = 0; i < n_kt && ok; ++i) {
            const int kt = kt_lo + i;
            ok = mbar_wait(bar_s, i & 1, abort_flag, A.status, 1);          // S(kt) ready; K, P and the other V buffer are free
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (i + 1 < n_kt) {
                load_kv(sK, kbase, tab, A.page_size, page_stride, (kt + 1) * BN, pos_hi, tid);
                load_kv(sV + ((i + 1) & 1) * V_BYTES, vbase, tab, A.page_size, page_stride, (kt + 1) * BN, pos_hi, tid);
            }
            float s[BN];
            tmem_ld32(lane_addr + S_COL, reinterpret_cast<float(&)[32]>(s[0]));
            tmem_ld32(lane_addr + S_COL + 32, reinterpret_cast<float(&)[32]>(s[32]));
            const int key0 = kt * BN;
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < BN; ++c) {
                const int j = key0 + c;
                if (!(j <= pos_r && j >= lo_r)) s[c] = -INFINITY;
                mx = fmaxf(mx, s[c]);
            }
            mx *= A.scale_log2;
            // Raise the reference maximum only when a tile exceeds it by more than the threshold.  The
            // tensor-memory loads and stores are warp-wide instructions, so the warp corrects O together
            // (factor 1 for rows that do not move) if any of its rows has to.
            const bool raise = mx > m_ref + RESCALE_THRESHOLD || (m_ref == -INFINITY && mx != -INFINITY);
            const float m_new = raise ? fmaxf(mx, m_ref) : m_ref;
            const bool fix_o = raise && i > 0 && m_ref != -INFINITY;        // O holds earlier tiles of this row
            if (__any_sync(0xffffffffu, fix_o)) {
                const float alpha = fix_o ? fast_exp2(m_ref - m_new) : 1.0f;
                l *= alpha;
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    float o[32];
                    tmem_ld32(lane_addr + O_COL + c0, o);
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c] *= alpha;
                    tmem_st32(lane_addr + O_COL + c0, o);
                }
            }
            m_ref = m_new;
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            // P = exp2(S * scale - m), rounded to bfloat16, into the swizzled A-operand tile (row = tid)
#pragma unroll
            for (int j8 = 0; j8 < BN / 8; ++j8) {
                float p[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    p[e] = fast_exp2(fmaf(s[j8 * 8 + e], A.scale_log2, -m_use));
                    l += p[e];
                }
                const uint32_t dst = sP + swz(BM, tid, j8);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pack_bf16(p[0], p[1])),
                             "r"(pack_bf16(p[2], p[3])), "r"(pack_bf16(p[4], p[5])), "r"(pack_bf16(p[6], p[7])) : "memory");
            }
            cp_async_wait_all();                            // this thread's share of K(kt+1), V(kt+1) has landed
            fence_async_proxy();                            // generic-proxy writes (P, cp.async) before the MMA reads
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(bar_p);
        }
        // ------------------------------------------------------------ epilogue
        if (ok && mbar_wait(bar_s, n_kt & 1, abort_flag, A.status, 2)) {   // the last P V has finished
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* dst = nullptr;
            if (R < rows_total) dst = A.out + ((size_t)(qs + R / g) * A.nq + (kh * g + R % g)) * D;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                float o[32];
                tmem_ld32(lane_addr + O_COL + c0, o);
                if (dst) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 v;
                        v.x = pack_bf16(o[c] * inv, o[c + 1] * inv); v.y = pack_bf16(o[c + 2] * inv, o[c + 3] * inv);
                        v.z = pack_bf16(o[c + 4] * inv, o[c + 5] * inv); v.w = pack_bf16(o[c + 6] * inv, o[c + 7] * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + c) = v;
                    }
                }
            }
        }
    } else if (tid == 128) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
        constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
        bool ok = mbar_wait(bar_p, 0, abort_flag, A.status, 3);
        for (int i = 0; i < n_kt && ok; ++i) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (i > 0) {                                    // O += P(i-1) V(i-1)
                const uint32_t v_addr = sV + ((i - 1) & 1) * V_BYTES;
#pragma unroll
                for (int k = 0; k < BN / 16; ++k)
                    umma(tmem + O_COL, desc_kmajor(sP + k * 32), desc_mnmajor(v_addr + k * 16 * 128, BN * 128), idesc_o,
                         (i > 1 || k > 0) ? 1u : 0u);
            }
#pragma unroll
            for (int k = 0; k < D / 16; ++k)                // S = Q K(i)^T
                umma(tmem + S_COL, desc_kmajor(sQ + (k >> 2) * BM * 128 + (k & 3) * 32),
                     desc_kmajor(sK + (k >> 2) * BN * 128 + (k & 3) * 32), idesc_s, k > 0 ? 1u : 0u);
            umma_commit(bar_s);
            ok = mbar_wait(bar_p, (i + 1) & 1, abort_flag, A.status, 4);    // P(i) and the next K, V are ready
        }
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t v_addr = sV + ((n_kt - 1) & 1) * V_BYTES;
#pragma unroll
            for (int k = 0; k < BN / 16; ++k)
                umma(tmem + O_COL, desc_kmajor(sP + k * 32), desc_mnmajor(v_addr + k * 16 * 128, BN * 128), idesc_o,
                     (n_kt > 1 || k > 0) ? 1u : 0u);
            umma_commit(bar_s);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
    }
    if (warp == 4) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

bool g_attr_done = false;

}  // namespace

TL_EXPORT int tl_attn_tc_head_dim() { return D; }

// total_tiles = sum over requests of ceil(q_len * g / 128).  `status`: device int, zero before the call.
TL_EXPORT int tl_attn_tc_prefill(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                 const int* table, int max_pages, int page_size, const int* q_start,
                                 const int* start_pos, const int* slots, int B, int nq, int nkv, int window,
                                 float scale, int total_tiles, int* status, cudaStream_t stream) {
    if (total_tiles <= 0 || B <= 0) return 0;
    if (nq % nkv || page_size <= 0 || (q_stride & 7) || ((uintptr_t)q & 15)) return 1;
    if (!g_attr_done) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        g_attr_done = true;
    }
    TcAttnArgs A{};
    A.q = (const bf16*)q; A.q_stride = q_stride; A.out = (bf16*)out;
    A.k_pages = (const bf16*)k_pages; A.v_pages = (const bf16*)v_pages;
    A.table = table; A.max_pages = max_pages; A.page_size = page_size;
    A.q_start = q_start; A.start_pos = start_pos; A.slots = slots;
    A.B = B; A.nq = nq; A.nkv = nkv; A.window = window; A.scale_log2 = scale * LOG2E; A.status = status;
    dim3 grid(total_tiles, nkv);
    attn_tc_prefill_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(A);
    return tl_launch_status();
}
