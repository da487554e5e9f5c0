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
// Three roles run concurrently.  Warps 0..3 do the softmax, one row per thread.  One thread of warp 4
// issues the MMAs.  Warps 5 and 6 copy K and V from the cache pages (cp.async, 16 bytes, swizzled on the way in):
// this step's own tokens were written there first (tensorline/paged.py:252-253), so fresh prompts, resumed
// portions and decoded tokens riding along are one case.  S, P, K and V are double-buffered, so the
// tensor cores compute S of tile i+1 and O of tile i-1 while the softmax threads work on tile i, and the
// copies run two tiles ahead; the softmax, not the hand-over between roles, sets the pace.  The running
// maximum is only raised when a tile exceeds it by more than 2^8, so the correction of O (a round trip
// through registers) is rare.  Formulas as in tensorline/paged_attn.py:46-57: scores, max, sum and the
// accumulator in float, P in bfloat16 for P V.  Every mbarrier wait is bounded; on a time-out the block
// records a code in `status` and leaves.
#include "common.cuh"
#include <cuda.h>

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size>"
#endif
#if HEAD_DIM % 64 != 0 || HEAD_DIM < 64 || HEAD_DIM > 256
#error "the tcgen05 attention kernel takes head sizes 64, 128, 192, 256"
#endif

namespace {

constexpr int D = HEAD_DIM;
constexpr int BM = 128;                 // query rows per block = MMA M = tensor-memory lanes
#ifndef TL_TC_KEYS
#define TL_TC_KEYS 64
#endif
constexpr int BN = TL_TC_KEYS;          // keys per tile (128 was measured slower than 64)
constexpr int THREADS = 224;            // warps 0..3: softmax and epilogue (one row each); warp 4: MMA issue; warps 5, 6: copies of K, of V
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;
constexpr long long WAIT_CYCLES = 4000000000LL;

constexpr int Q_BYTES = BM * D * 2, K_BYTES = BN * D * 2, V_BYTES = BN * D * 2, P_BYTES = BM * BN * 2;
constexpr int SMEM_TILES = Q_BYTES + 2 * K_BYTES + 2 * V_BYTES + 2 * P_BYTES;
constexpr int SMEM_BYTES = SMEM_TILES + 1024 + 128;
constexpr uint32_t TMEM_COLS = (2 * BN + D) <= 256 ? 256 : 512;
constexpr uint32_t S_COL = 0, O_COL = 2 * BN;             // S[0], S[1], then O

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
// `backoff`: the waiting warp sleeps between polls, so that its spinning does not take issue slots from
// the softmax warp that shares its scheduler (used by the MMA and copy warps, whose hand-overs have slack).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                          bool backoff = false) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (backoff) __nanosleep(40);
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
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
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
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// the largest of a row's scores: two chains of three-input maxima (half the instructions of two-input ones)
template <int N>
__device__ __forceinline__ float row_max(const float (&s)[N]) {
    static_assert(N % 4 == 0 && N >= 8, "row_max");
    float a = max3(s[0], s[1], s[2]), b = max3(s[3], s[4], s[5]);
#pragma unroll
    for (int c = 6; c + 3 < N; c += 4) { a = max3(a, s[c], s[c + 1]); b = max3(b, s[c + 2], s[c + 3]); }
    return max3(a, b, fmaxf(s[N - 2], s[N - 1]));
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
    // the tiles in the order in which blocks take them, (request << 16 | tile), longest first over all requests;
    // null: one request after the other from the end
    const int* order;
    TlLimits lim;                      // for the checking build; zeros: nothing known, nothing checked
    // The pair kernel only.  ksplit > 1: the key tiles of every block are dealt out to ksplit blocks in equal runs; each
    // leaves its unnormalised O rows in part_o [ksplit][tokens][nq][D] and (m, l) in part_ml [ksplit][tokens][nq][2]
    // (m = -inf: that run held no key for the row) and a second kernel merges them.  For portions on long contexts whose
    // query tiles alone would leave most of the GPU idle.
    int ksplit, tokens;
    float* part_o; float* part_ml;
};

// One thread's share of a 128-row Q tile, 16-byte chunks r, r + 128, ... of its BM x D / 8 chunks; row = (token, head of
// the group).  Where 128 is a multiple of the chunks a row has (head sizes 64, 128, 256) a thread keeps its chunk
// column and its rows are 128 / CH apart: token and head then advance by additions from one division.
__device__ __forceinline__ void load_q_rows(uint32_t dst_tile, const bf16* q, int q_stride, int qs, int head0, int g,
                                            int row0, int rows_total, int r) {
    constexpr int CH = D / 8;
    if constexpr (BM % CH == 0) {
        constexpr int ROW_STEP = BM / CH;
        const int c = r % CH;
        int qr = r / CH;
        int tok = (row0 + qr) / g, rem = (row0 + qr) - tok * g;
        const int d_tok = ROW_STEP / g, d_rem = ROW_STEP - d_tok * g;
#pragma unroll 4
        for (int k = 0; k < CH; ++k, qr += ROW_STEP) {
            const bool valid = row0 + qr < rows_total;
            const bf16* src = valid ? q + (size_t)(qs + tok) * q_stride + (size_t)(head0 + rem) * D + c * 8 : q;
            cp_async16(dst_tile + swz(BM, qr, c), src, valid);
            tok += d_tok; rem += d_rem;
            if (rem >= g) { rem -= g; ++tok; }
        }
    } else {
        for (int idx = r; idx < BM * CH; idx += BM) {
            const int qr = idx / CH, c = idx - qr * CH;
            const int QR = row0 + qr;
            const bool valid = QR < rows_total;
            const bf16* src = valid ? q + (size_t)(qs + QR / g) * q_stride + (size_t)(head0 + QR % g) * D + c * 8 : q;
            cp_async16(dst_tile + swz(BM, qr, c), src, valid);
        }
    }
}

// Keys [key0, key0 + BN) of one KV head into a swizzled [BN][D] tile, by one warp; keys past
// last_key are zeros.  The page size is a power of two, at least BN / 32 (shift, mask).  The tile's
// page numbers are read once (one per lane) and handed around with shuffles, so no copy waits on a
// table read of its own.
__device__ __forceinline__ void load_kv(uint32_t dst, const bf16* pages, const int* tab, int ps_shift, size_t page_stride,
                                        int key0, int last_key, int lane, const TlLimits& L) {
    constexpr int CH = D / 8;
    const int ps_mask = (1 << ps_shift) - 1;
    int my_page = 0;
    if (lane < (BN >> ps_shift) && key0 + (lane << ps_shift) <= last_key)
        my_page = tl_checked(tab[(key0 >> ps_shift) + lane], L.total_pages, L, TL_K_TC_PREFILL);
#pragma unroll
    for (int i = 0; i < BN * CH / 32; ++i) {
        const int idx = lane + 32 * i;
        const int key = idx / CH, c = idx - key * CH;
        const int page = __shfl_sync(0xffffffffu, my_page, key >> ps_shift);
        const bool valid = key0 + key <= last_key;
        const bf16* src = pages + (size_t)page * page_stride + (size_t)((key & ps_mask) * D + c * 8);
        cp_async16(dst + swz(BN, key, c), src, valid);
    }
}

__global__ void __launch_bounds__(THREADS, 1) attn_tc_prefill_kernel(const TcAttnArgs A) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sQ = smem_addr(base), sK = sQ + Q_BYTES, sV = sK + 2 * K_BYTES, sP = sV + 2 * V_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + SMEM_TILES);
    uint64_t* bar_s = bars;         // [2] S(i) is complete (commit)
    uint64_t* bar_o = bars + 2;     // [2] O += P(i) V(i) is complete (commit): P and V of that slot are free
    uint64_t* bar_p = bars + 4;     // [2] the 128 rows have written P(i)
    uint64_t* bar_k = bars + 6;     // [2] K(i) is in shared memory
    uint64_t* bar_v = bars + 8;     // [2] V(i) is in shared memory
    uint64_t* bar_q = bars + 10;    // the Q tile is in shared memory (brought by the 128 softmax threads)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kh = blockIdx.x % A.nkv, g = A.nq / A.nkv;   // blocks in order of falling length over all KV heads

    int tile = (int)(gridDim.x / A.nkv) - 1 - (int)(blockIdx.x / A.nkv), b = 0;          // longest tiles (late rows of a request) first
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
    const int* tab = A.table + (size_t)tl_checked(A.slots[b], A.lim.table_rows, A.lim, TL_K_TC_PREFILL) * A.max_pages;
    const int pos_hi = sp + (row_end - 1) / g, pos_first = sp + row0 / g;
    tl_checked(pos_hi / A.page_size, A.max_pages, A.lim, TL_K_TC_PREFILL);  // the last table entry this tile reads
    const int key_lo = A.window > 0 ? max(0, pos_first - A.window + 1) : 0;
    const int kt_lo = key_lo / BN, kt_hi = pos_hi / BN, n_kt = kt_hi - kt_lo + 1;

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_s + i, 1); mbar_init(bar_o + i, 1); mbar_init(bar_p + i, 128);
            mbar_init(bar_k + i, 32); mbar_init(bar_v + i, 32);
        }
        mbar_init(bar_q, BM);
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

    if (warp < 4) {
        // ------------------------------------------------------------ softmax and epilogue: thread = row
        const int R = row0 + tid;
        const int pos_r = R < rows_total ? sp + R / g : -1; // -1: no key is visible
        const int lo_r = A.window > 0 ? max(0, pos_r - A.window + 1) : 0;
        const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        {   // the Q tile, row = (token, head of the group), while the first K and V tiles are on their way
            load_q_rows(sQ, A.q, A.q_stride, qs, kh * g, g, row0, rows_total, tid);
            cp_async_wait_all();
            fence_async_proxy();
            mbar_arrive(bar_q);
        }

        for (int i = 0; i < n_kt && ok; ++i) {
            const int sl = i & 1, kt = kt_lo + i;
            ok = mbar_wait(bar_s + sl, (i >> 1) & 1, abort_flag, A.status, 1);          // S(i) is ready
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float s[BN];
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 32)
                tmem_ld32(lane_addr + S_COL + sl * BN + c0, reinterpret_cast<float(&)[32]>(s[c0]));
            tmem_ld_wait();                                 // all parts in flight, one wait
            const int key0 = kt * BN;
            if (!(key0 + BN - 1 <= pos_r && key0 >= lo_r)) {   // not every key of the tile is visible to this row
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    const int j = key0 + c;
                    if (!(j <= pos_r && j >= lo_r)) s[c] = -INFINITY;
                }
            }
            const float mx = row_max(s) * A.scale_log2;
            // Raise the reference maximum only when a tile exceeds it by more than the threshold.  The
            // tensor-memory loads and stores are warp-wide instructions, so the warp corrects O together
            // (factor 1 for rows that do not move) if any of its rows has to.
            const bool raise = mx > m_ref + RESCALE_THRESHOLD || (m_ref == -INFINITY && mx != -INFINITY);
            const float m_new = raise ? fmaxf(mx, m_ref) : m_ref;
            const bool fix_o = raise && i > 0 && m_ref != -INFINITY;        // O holds earlier tiles of this row
            if (__any_sync(0xffffffffu, fix_o)) {
                // O must be at rest: P(i-1) V(i-1), the last product issued so far, has to be complete
                ok = mbar_wait(bar_o + ((i - 1) & 1), ((i - 1) >> 1) & 1, abort_flag, A.status, 2);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float alpha = fix_o ? fast_exp2(m_ref - m_new) : 1.0f;
                l *= alpha;
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    float o[32];
                    tmem_ld32(lane_addr + O_COL + c0, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c] *= alpha;
                    tmem_st32(lane_addr + O_COL + c0, o);
                }
            }
            m_ref = m_new;
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            if (i >= 2) {                                   // the P slot is free once P(i-2) V(i-2) is complete
                ok = mbar_wait(bar_o + sl, ((i - 2) >> 1) & 1, abort_flag, A.status, 3);
                if (!ok) break;
            }
            // P = exp2(S * scale - m), rounded to bfloat16, into the swizzled A-operand tile (row = tid)
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j8 = 0; j8 < BN / 8; ++j8) {
                float p[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    p[e] = fast_exp2(fmaf(s[j8 * 8 + e], A.scale_log2, -m_use));
                    l4[e & 3] += p[e];
                }
                const uint32_t dst = sP + sl * P_BYTES + swz(BM, tid, j8);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pack_bf16(p[0], p[1])),
                             "r"(pack_bf16(p[2], p[3])), "r"(pack_bf16(p[4], p[5])), "r"(pack_bf16(p[6], p[7])) : "memory");
            }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            fence_async_proxy();                            // generic-proxy writes of P before the MMA reads them
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(bar_p + sl);
        }
        // ------------------------------------------------------------ epilogue: the last P V has finished
        if (ok && mbar_wait(bar_o + ((n_kt - 1) & 1), ((n_kt - 1) >> 1) & 1, abort_flag, A.status, 4)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* dst = nullptr;
            if (R < rows_total) dst = A.out + ((size_t)(qs + R / g) * A.nq + (kh * g + R % g)) * D;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                float o[32];
                tmem_ld32(lane_addr + O_COL + c0, o);
                tmem_ld_wait();
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
    } else if (warp == 4) {
        // ------------------------------------------------------------ MMA issuer (one thread)
        if (lane == 0) {
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            auto issue_qk = [&](int j) {                    // S[j & 1] = Q K(j)^T
                const uint32_t k_addr = sK + (j & 1) * K_BYTES;
#pragma unroll
                for (int k = 0; k < D / 16; ++k)
                    umma(tmem + S_COL + (j & 1) * BN, desc_kmajor(sQ + (k >> 2) * BM * 128 + (k & 3) * 32),
                         desc_kmajor(k_addr + (k >> 2) * BN * 128 + (k & 3) * 32), idesc_s, k > 0 ? 1u : 0u);
                umma_commit(bar_s + (j & 1));
            };
            bool ok = mbar_wait(bar_q, 0, abort_flag, A.status, 11, true);
            for (int j = 0; j < 2 && j < n_kt && ok; ++j) {
                ok = mbar_wait(bar_k + j, 0, abort_flag, A.status, 5, true);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_qk(j);
            }
            for (int i = 0; i < n_kt && ok; ++i) {
                const int sl = i & 1, ph = (i >> 1) & 1;
                ok = mbar_wait(bar_p + sl, ph, abort_flag, A.status, 6, true) &&          // P(i) is written, S[sl] is free
                     mbar_wait(bar_v + sl, ph, abort_flag, A.status, 7, true);            // V(i) is in shared memory
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t v_addr = sV + sl * V_BYTES, p_addr = sP + sl * P_BYTES;
#pragma unroll
                for (int k = 0; k < BN / 16; ++k)           // O += P(i) V(i)
                    umma(tmem + O_COL, desc_kmajor(p_addr + (k >> 2) * BM * 128 + (k & 3) * 32),
                         desc_mnmajor(v_addr + k * 16 * 128, BN * 128), idesc_o,
                         (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(bar_o + sl);
                if (i + 2 < n_kt) {
                    ok = mbar_wait(bar_k + sl, ((i + 2) >> 1) & 1, abort_flag, A.status, 8, true);   // K(i+2) is in
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    issue_qk(i + 2);
                }
            }
        }
    } else {
        // ------------------------------------------------------------ copies: warp 5 brings K, warp 6 brings V,
        // each up to two tiles ahead of the softmax
        int ps_shift = 0;
        while ((1 << ps_shift) < A.page_size) ++ps_shift;
        const size_t page_stride = (size_t)A.nkv * A.page_size * D;
        const bool is_k = warp == 5;
        const bf16* pages = (is_k ? A.k_pages : A.v_pages) + (size_t)kh * A.page_size * D;
        uint64_t* bar_free = is_k ? bar_s : bar_o;           // K slot: free once S(j-2) is complete; V slot: once P V(j-2) is
        uint64_t* bar_full = is_k ? bar_k : bar_v;
        const uint32_t tiles = is_k ? sK : sV;
        bool ok = true;
        for (int j = 0; j < n_kt && ok; ++j) {
            const int sl = j & 1;
            if (j >= 2) {
                ok = mbar_wait(bar_free + sl, ((j - 2) >> 1) & 1, abort_flag, A.status, is_k ? 9 : 10, true);
                if (!ok) break;
            }
            load_kv(tiles + sl * K_BYTES, pages, tab, ps_shift, page_stride, (kt_lo + j) * BN, pos_hi, lane, A.lim);
            cp_async_wait_all();
            fence_async_proxy();
            mbar_arrive(bar_full + sl);
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

#if HEAD_DIM <= 128
// ------------------------------------------------------------------------------------------------
// Two query tiles per block (head sizes 64 and 128, pages of 8 to 64 tokens).
//
// Time stamps per role in the kernel above showed every role at about 1,700 cycles a key tile: the softmax
// warps alone on their schedulers (64 exponentials a row on the special-function unit, then packing and
// stores), the copy warps issuing a thousand cp.async each, and the one MMA thread, which needs about 90
// cycles to issue a tcgen05.mma whatever its size - more than these small products take to run (47 cycles for
// S with 64 keys, 63 for P V; two issuing threads reach the tensor core's rate).  Here a block takes 256
// query rows as two tiles that share every K and V tile: eight softmax warps, two per scheduler; four MMA
// issuers (S and P V of each tile); K and V as TMA boxes (one page of one KV head, 64 elements wide, 128-byte
// swizzle) issued by one thread each, from the block's first cycle on, while the softmax warps fetch their Q tile
// (a copy warp fetching Q first cost every block 7 to 10 us before its first product).  Measured: about 2,000 cycles
// a key tile for both query tiles.  The exponentials of 2 x 128 x 64 scores are 1,024 of them on the special-function
// unit, and the softmax body of two warps on one scheduler, run alone, takes 1,320; what the step cannot go below
// here is shared memory: the products read Q and K (6 KB an instruction for S), P and V (8 KB for P V), the softmax
// writes P and the copies write K and V, 224 KB a key tile at 128 bytes a cycle = 1,750 cycles.  (P as a tensor-memory
// operand would take 64 KB of that away; tensor memory is full with two S slots a tile.)  Tensor memory: S[tile][2]
// at columns 0..255, O[tile] behind them.
constexpr int QT = 2;
constexpr int TURN_AT = 6;               // the turn at the exponentials passes on after this 8-score group of 0..7 (measured best)
constexpr int THREADS2 = 448;           // warps 0..7: softmax (tile = warp / 4); 8..11: MMA issue; 12: K copies; 13: V copies
constexpr int SMEM2_TILES = QT * Q_BYTES + 2 * K_BYTES + 2 * V_BYTES + QT * 2 * P_BYTES;
constexpr int SMEM2_BYTES = SMEM2_TILES + 1024 + 256;
constexpr uint32_t TMEM2_COLS = 512;
constexpr uint32_t S2_COL = 0, O2_COL = QT * 2 * BN;
static_assert(O2_COL + QT * D <= 512, "S and O of both tiles must fit the tensor memory");
static_assert(SMEM2_BYTES <= 227 * 1024, "shared memory");

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_box(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y) : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (P: one row a lane, two bfloat16 a column) comes from tensor memory.
__device__ __forceinline__ void umma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_st32_nowait(uint32_t taddr, const uint32_t (&u)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]),
                   "r"(u[8]), "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]),
                   "r"(u[16]), "r"(u[17]), "r"(u[18]), "r"(u[19]), "r"(u[20]), "r"(u[21]), "r"(u[22]), "r"(u[23]),
                   "r"(u[24]), "r"(u[25]), "r"(u[26]), "r"(u[27]), "r"(u[28]), "r"(u[29]), "r"(u[30]), "r"(u[31])
                 : "memory");
}

// P_TMEM: the softmax does not write P to shared memory but back into the S slot it has just read, as packed bfloat16
// (32 of the slot's 64 columns), and O += P V takes P as its tensor-memory operand.  A key-tile step then moves 160 KB
// through shared memory instead of 224 KB (the bound of this kernel: see the notes above).  The S slot of product i is
// free again when P(i) V is complete, not when the softmax has read S(i): that is what the S issuer then waits for.
template <bool P_TMEM>
__global__ void __launch_bounds__(THREADS2, 1)
attn_tc2_prefill_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const TcAttnArgs A) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sQ = smem_addr(base), sK = sQ + QT * Q_BYTES, sV = sK + 2 * K_BYTES, sP = sV + 2 * V_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + SMEM2_TILES);
    uint64_t* bar_s = bars;          // [tile * 2 + slot] S is complete (commit)
    uint64_t* bar_p = bars + 4;      // [tile * 2 + slot] the tile's 128 rows have written P
    uint64_t* bar_o = bars + 8;      // [tile * 2 + slot] O += P V is complete (commit): that P slot is free, O is at rest
    uint64_t* bar_k = bars + 12;     // [slot] K has landed (TMA bytes)
    uint64_t* bar_v = bars + 14;     // [slot] V has landed
    uint64_t* bar_kfree = bars + 16; // [slot] both S issuers are done with this K slot (a commit, or a plain arrival)
    uint64_t* bar_vfree = bars + 18; // [slot] both P V issuers are done with this V slot
    uint64_t* bar_q = bars + 20;     // both Q tiles are in shared memory
    uint64_t* bar_x = bars + 21;     // [tile * 4 + warp of the tile] that warp's exponentials of a key tile are issued
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 29);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ksplit = A.ksplit > 1 ? A.ksplit : 1, run = (int)(blockIdx.x % (unsigned)ksplit);
    const int bx = (int)(blockIdx.x / (unsigned)ksplit), nbx = (int)(gridDim.x / (unsigned)ksplit);
    const int kh = bx % A.nkv, g = A.nq / A.nkv;           // blocks in order of falling length over all KV heads

    int tile = nbx / A.nkv - 1 - bx / A.nkv, b = 0;        // longest tiles (late rows of a request) first
    if (A.order != nullptr) {
        const int packed = A.order[bx / A.nkv];
        b = packed >> 16; tile = packed & 0xFFFF;
    } else {
        for (; b < A.B; ++b) {
            const int nt = ((A.q_start[b + 1] - A.q_start[b]) * g + QT * BM - 1) / (QT * BM);
            if (tile < nt) break;
            tile -= nt;
        }
    }
    if (b >= A.B) return;
    const int qs = A.q_start[b], qlen = A.q_start[b + 1] - qs, sp = A.start_pos[b];
    const int rows_total = qlen * g;
    const int* tab = A.table + (size_t)tl_checked(A.slots[b], A.lim.table_rows, A.lim, TL_K_TC2_PREFILL) * A.max_pages;
    // the two tiles: rows, and the range of key tiles each of them reads
    int row0[QT], kt_first[QT], kt_last[QT];
#pragma unroll
    for (int t = 0; t < QT; ++t) {
        row0[t] = (tile * QT + t) * BM;
        if (row0[t] < rows_total) {
            const int row_end = min(row0[t] + BM, rows_total);
            const int pos_first = sp + row0[t] / g, pos_last = sp + (row_end - 1) / g;
            const int key_lo = A.window > 0 ? max(0, pos_first - A.window + 1) : 0;
            kt_first[t] = key_lo / BN; kt_last[t] = pos_last / BN;
        } else {                                           // no rows: reads nothing
            kt_first[t] = 1; kt_last[t] = 0;
        }
    }
    // tile 1 holds the later rows: its range starts and ends no earlier than tile 0's
    int kt_lo = kt_first[0], kt_hi = max(kt_last[0], kt_last[1]), n_kt = kt_hi - kt_lo + 1;
    if (ksplit > 1) {                                      // this block's run of the key tiles; a query tile may have none in it
        const int per = (n_kt + ksplit - 1) / ksplit;
        kt_lo += run * per;
        kt_hi = min(kt_hi, kt_lo + per - 1);
        n_kt = kt_hi - kt_lo + 1;                          // <= 0: nothing to read, the rows' parts say so
#pragma unroll
        for (int t = 0; t < QT; ++t) { kt_first[t] = max(kt_first[t], kt_lo); kt_last[t] = min(kt_last[t], kt_hi); }
    }
    auto reads = [&](int t, int j) { return kt_lo + j >= kt_first[t] && kt_lo + j <= kt_last[t]; };

    if (tid == 0) {
        for (int i = 0; i < 4; ++i) { mbar_init(bar_s + i, 1); mbar_init(bar_p + i, 128); mbar_init(bar_o + i, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(bar_k + i, 1); mbar_init(bar_v + i, 1); mbar_init(bar_kfree + i, 2); mbar_init(bar_vfree + i, 2); }
        mbar_init(bar_q, QT * BM);
        for (int i = 0; i < 8; ++i) mbar_init(bar_x + i, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(TMEM2_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp < 8) {
        // ------------------------------------------------------------ softmax and epilogue: thread = row of tile t
        const int t = warp >> 2, r = tid & 127;
        const int R = row0[t] + r;
        const int pos_r = R < rows_total ? sp + R / g : -1; // -1: no key is visible
        const int lo_r = A.window > 0 ? max(0, pos_r - A.window + 1) : 0;
        const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const int n_mine = kt_last[t] - kt_first[t] + 1;   // <= 0: this tile has no rows
        // The two warps of a scheduler (one of each query tile) take turns at the exponentials.  Left alone they run
        // in step: both load and reduce (the special-function unit idle), then both want that unit at once, 2,060
        // cycles a key tile where the two phases side by side need 1,300.  Over the key tiles that both query tiles
        // read, tile 1's warp starts its exponentials of key tile j when tile 0's warp is through its own of j, and
        // tile 0's of j + 1 when tile 1's of j are through; the order follows the key tiles, so neither waits for
        // anything the other can only reach later.
        const int x_lo = max(kt_first[0], kt_first[1]), x_hi = min(kt_last[0], kt_last[1]);   // empty if tile 1 has no rows
        uint64_t* const x_mine = bar_x + t * 4 + (warp & 3);
        uint64_t* const x_other = bar_x + (1 - t) * 4 + (warp & 3);
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        {   // the tile's Q rows, row = (token, head of the group), while the first K and V tiles are on their way
            load_q_rows(sQ + t * Q_BYTES, A.q, A.q_stride, qs, kh * g, g, row0[t], rows_total, r);
            cp_async_wait_all();
            fence_async_proxy();
            mbar_arrive(bar_q);
        }

        for (int i = 0; i < n_mine && ok; ++i) {
            const int sl = i & 1, kt = kt_first[t] + i, bi = t * 2 + sl;
            ok = mbar_wait(bar_s + bi, (i >> 1) & 1, abort_flag, A.status, 1);           // S(i) is ready
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t s_addr = lane_addr + S2_COL + bi * BN;
            const int key0 = kt * BN;
            float s[BN];
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 32)
                tmem_ld32(s_addr + c0, reinterpret_cast<float(&)[32]>(s[c0]));
            tmem_ld_wait();                                 // all parts in flight, one wait
            if (!(key0 + BN - 1 <= pos_r && key0 >= lo_r)) {   // not every key of the tile is visible to this row
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    const int j = key0 + c;
                    if (!(j <= pos_r && j >= lo_r)) s[c] = -INFINITY;
                }
            }
            const float mx = row_max(s) * A.scale_log2;
            const bool raise = mx > m_ref + RESCALE_THRESHOLD || (m_ref == -INFINITY && mx != -INFINITY);
            const float m_new = raise ? fmaxf(mx, m_ref) : m_ref;
            const bool fix_o = raise && i > 0 && m_ref != -INFINITY;        // O holds earlier tiles of this row
            if (__any_sync(0xffffffffu, fix_o)) {
                ok = mbar_wait(bar_o + t * 2 + ((i - 1) & 1), ((i - 1) >> 1) & 1, abort_flag, A.status, 2);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float alpha = fix_o ? fast_exp2(m_ref - m_new) : 1.0f;
                l *= alpha;
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    float o[32];
                    tmem_ld32(lane_addr + O2_COL + t * D + c0, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c] *= alpha;
                    tmem_st32(lane_addr + O2_COL + t * D + c0, o);
                }
            }
            m_ref = m_new;
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            if (!P_TMEM && i >= 2) {                        // the P slot is free once P(i-2) V(i-2) is complete
                ok = mbar_wait(bar_o + bi, ((i - 2) >> 1) & 1, abort_flag, A.status, 3);
                if (!ok) break;
            }
            const bool in_turns = kt >= x_lo && kt <= x_hi;
            if (in_turns && (t == 1 || kt > x_lo)) {
                ok = mbar_wait(x_other, (kt - x_lo - (t == 0 ? 1 : 0)) & 1, abort_flag, A.status, 12);
                if (!ok) break;
            }
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[P_TMEM ? BN / 2 : 1];                // P_TMEM: the row's P, two bfloat16 a column
#pragma unroll
            for (int j8 = 0; j8 < BN / 8; ++j8) {
                float p[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    p[e] = fast_exp2(fmaf(s[j8 * 8 + e], A.scale_log2, -m_use));
                    l4[e & 3] += p[e];
                }
                if constexpr (P_TMEM) {
                    pk[j8 * 4] = pack_bf16(p[0], p[1]); pk[j8 * 4 + 1] = pack_bf16(p[2], p[3]);
                    pk[j8 * 4 + 2] = pack_bf16(p[4], p[5]); pk[j8 * 4 + 3] = pack_bf16(p[6], p[7]);
                } else {
                    const uint32_t dst = sP + bi * P_BYTES + swz(BM, r, j8);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pack_bf16(p[0], p[1])),
                                 "r"(pack_bf16(p[2], p[3])), "r"(pack_bf16(p[4], p[5])), "r"(pack_bf16(p[6], p[7])) : "memory");
                }
                if (j8 == TURN_AT && in_turns) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(x_mine);
                }
            }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            if constexpr (P_TMEM) {
                static_assert(BN == 64, "one 32-column store holds the row's P");
                tmem_st32_nowait(s_addr, reinterpret_cast<const uint32_t(&)[32]>(pk));
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            } else {
                fence_async_proxy();                        // generic-proxy writes of P before the MMA reads them
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(bar_p + bi);
        }
        // ------------------------------------------------------------ epilogue: the tile's last P V has finished
        if (ksplit > 1) {                                   // this run's part of the row: (m, l) and the unnormalised O
            const bool any = n_mine > 0;                   // the same for all rows of the tile
            if (any && ok) ok = mbar_wait(bar_o + t * 2 + ((n_mine - 1) & 1), ((n_mine - 1) >> 1) & 1, abort_flag, A.status, 4);
            const bool row = R < rows_total, live = any && ok && m_ref != -INFINITY;
            const size_t slot = row ? ((size_t)run * A.tokens + (qs + R / g)) * A.nq + (kh * g + R % g) : 0;
            if (row) *reinterpret_cast<float2*>(A.part_ml + slot * 2) = make_float2(live ? m_ref : -INFINITY, live ? l : 0.f);
            if (any && ok) {                                // every lane of the warp takes part in the loads
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                float* dst = A.part_o + slot * D;
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    float o[32];
                    tmem_ld32(lane_addr + O2_COL + t * D + c0, o);
                    tmem_ld_wait();
                    if (row && live) {
#pragma unroll
                        for (int c = 0; c < 32; c += 4)
                            *reinterpret_cast<float4*>(dst + c0 + c) = make_float4(o[c], o[c + 1], o[c + 2], o[c + 3]);
                    }
                }
            }
        } else if (ok && n_mine > 0 &&
            mbar_wait(bar_o + t * 2 + ((n_mine - 1) & 1), ((n_mine - 1) >> 1) & 1, abort_flag, A.status, 4)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* dst = nullptr;
            if (R < rows_total) dst = A.out + ((size_t)(qs + R / g) * A.nq + (kh * g + R % g)) * D;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                float o[32];
                tmem_ld32(lane_addr + O2_COL + t * D + c0, o);
                tmem_ld_wait();
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
    } else if (warp < 12) {
        // ------------------------------------------------------------ MMA issuers: one thread each in warps 8..11.
        // A thread needs about 90 cycles to issue one tcgen05.mma whatever its size, more than these products take
        // to run (47 cycles for S with 64 keys, 63 for P V), so one issuer would be the bottleneck (measured: two
        // issuers run at the tensor core's rate).  Warps 8, 9 issue S = Q_t K^T for tile t = 0, 1; warps 10, 11
        // issue O_t += P V.  Every issuer walks all key tiles, also those its query tile does not read, and
        // hands each K (V) slot back with one of the two arrivals its barrier counts.
        if (lane == 0) {
            const int t = warp & 1;
            bool ok = true;
            if (warp < 10) {
                constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
                ok = mbar_wait(bar_q, 0, abort_flag, A.status, 11, true);
                int i = 0;                                  // products issued for this tile
                for (int j = 0; j < n_kt && ok; ++j) {
                    const int sl = j & 1;
                    ok = mbar_wait(bar_k + sl, (j >> 1) & 1, abort_flag, A.status, 5, true);        // K(j) is in
                    if (!ok) break;
                    if (!reads(t, j)) { mbar_arrive(bar_kfree + sl); continue; }
                    const int bi = t * 2 + (i & 1);
                    if (i >= 2) {                           // that S slot is free once the softmax of product i-2 has written its P
                        ok = P_TMEM ? mbar_wait(bar_o + bi, ((i - 2) >> 1) & 1, abort_flag, A.status, 6, true)   // ... and P(i-2) V has read it there
                                    : mbar_wait(bar_p + bi, ((i - 2) >> 1) & 1, abort_flag, A.status, 6, true);
                        if (!ok) break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t k_addr = sK + sl * K_BYTES;
#pragma unroll
                    for (int k = 0; k < D / 16; ++k)
                        umma(tmem + S2_COL + bi * BN, desc_kmajor(sQ + t * Q_BYTES + (k >> 2) * BM * 128 + (k & 3) * 32),
                             desc_kmajor(k_addr + (k >> 2) * BN * 128 + (k & 3) * 32), idesc_s, k > 0 ? 1u : 0u);
                    umma_commit(bar_s + bi);
                    umma_commit(bar_kfree + sl);
                    ++i;
                }
            } else {
                constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
                int i = 0;
                for (int j = 0; j < n_kt && ok; ++j) {
                    const int sl = j & 1;
                    ok = mbar_wait(bar_v + sl, (j >> 1) & 1, abort_flag, A.status, 7, true);        // V(j) is in
                    if (!ok) break;
                    if (!reads(t, j)) { mbar_arrive(bar_vfree + sl); continue; }
                    const int bi = t * 2 + (i & 1);
                    ok = mbar_wait(bar_p + bi, (i >> 1) & 1, abort_flag, A.status, 8, true);        // P is written
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t v_addr = sV + sl * V_BYTES, p_addr = sP + bi * P_BYTES;
#pragma unroll
                    for (int k = 0; k < BN / 16; ++k) {     // O_t += P V(j)
                        if constexpr (P_TMEM)
                            umma_a_tmem(tmem + O2_COL + t * D, tmem + S2_COL + bi * BN + k * 8,
                                        desc_mnmajor(v_addr + k * 16 * 128, BN * 128), idesc_o, (i > 0 || k > 0) ? 1u : 0u);
                        else
                            umma(tmem + O2_COL + t * D, desc_kmajor(p_addr + (k >> 2) * BM * 128 + (k & 3) * 32),
                                 desc_mnmajor(v_addr + k * 16 * 128, BN * 128), idesc_o, (i > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(bar_o + bi);
                    umma_commit(bar_vfree + sl);
                    ++i;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ copies: one thread of warp 12 issues the TMA
        // boxes of K, one of warp 13 those of V, up to two tiles ahead (the softmax warps bring their own Q tile)
        if (lane == 0) {
            const bool is_k = warp == 12;
            const CUtensorMap* map = is_k ? &map_k : &map_v;
            asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
            uint64_t* bar_free = is_k ? bar_kfree : bar_vfree;
            uint64_t* bar_full = is_k ? bar_k : bar_v;
            const uint32_t tiles = is_k ? sK : sV;
            int ps_shift = 0;
            while ((1 << ps_shift) < A.page_size) ++ps_shift;
            const int ppt = BN >> ps_shift;                 // pages per key tile: 1 to 8
            bool ok = true;
            for (int j = 0; j < n_kt && ok; ++j) {
                const int sl = j & 1;
                int page[8];
#pragma unroll
                for (int pg = 0; pg < 8; ++pg)              // the tile's page numbers, all requested before the wait
                    if (pg < ppt) page[pg] = tl_checked(tab[min((((kt_lo + j) * BN) >> ps_shift) + pg, A.max_pages - 1)],
                                                        A.lim.total_pages, A.lim, TL_K_TC2_PREFILL);
                if (j >= 2) {
                    ok = mbar_wait(bar_free + sl, ((j - 2) >> 1) & 1, abort_flag, A.status, is_k ? 9 : 10, true);
                    if (!ok) break;
                }
                mbar_expect_tx(bar_full + sl, K_BYTES);
#pragma unroll
                for (int pg = 0; pg < 8; ++pg) {
                    if (pg >= ppt) break;
                    const int row = (page[pg] * A.nkv + kh) << ps_shift;
#pragma unroll
                    for (int db = 0; db < D / 64; ++db)
                        tma_box(tiles + sl * K_BYTES + db * (BN * 128) + ((pg << ps_shift) * 128), map, bar_full + sl, db * 64, row);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
    }
    if (warp == 8) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM2_COLS) : "memory");
    }
}


// ------------------------------------------------------------------------------------------------
// Key tiles of 128 with P kept in tensor memory (head sizes 64 and 128, pages of 8 to 64 tokens).
//
// The kernel above is bound by shared memory: every key-tile step the softmax writes P there and P V reads it
// back, and tiles of 64 keys read Q twice as often as tiles of 128 would.  Here a tile's S (128 rows x 128 keys,
// float) is one slot of tensor memory, and the softmax writes P back INTO that slot as packed bfloat16 (64 of
// its 128 columns); O += P V then takes P as its tensor-memory operand.  P never touches shared memory, which
// holds only Q (2 tiles), K and V (2 stages of 128 keys each).  Tensor memory: S/P of the two query tiles at
// columns 0 and 128, their O behind them: all 512 columns.  With one S slot a tile, S(i + 1) of a tile can only
// be issued once P(i) V has read P(i): a tile's products and softmax alternate, and the block's two query tiles
// keep the tensor core busy in turns.  A row's 128 scores are read from tensor memory twice (once for the
// maximum, once for the exponentials) in parts of 32, so a softmax thread needs no more registers than before.
constexpr int BN3 = 128;
constexpr int KV3_BYTES = BN3 * D * 2;
constexpr int SMEM3_TILES = QT * Q_BYTES + 2 * KV3_BYTES + 2 * KV3_BYTES;
constexpr int SMEM3_BYTES = SMEM3_TILES + 1024 + 256;
constexpr uint32_t TMEM3_COLS = 512;
constexpr uint32_t S3_COL = 0, O3_COL = QT * BN3;
static_assert(O3_COL + QT * D <= 512, "S and O of both tiles must fit the tensor memory");
static_assert(SMEM3_BYTES <= 227 * 1024, "shared memory");

__global__ void __launch_bounds__(THREADS2, 1)
attn_tc3_prefill_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const TcAttnArgs A) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sQ = smem_addr(base), sK = sQ + QT * Q_BYTES, sV = sK + 2 * KV3_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + SMEM3_TILES);
    uint64_t* bar_s = bars;          // [tile] S is complete (commit)
    uint64_t* bar_p = bars + 2;      // [tile] the tile's 128 rows have written P over S
    uint64_t* bar_o = bars + 4;      // [tile] O += P V is complete (commit): the S/P slot is free, O is at rest
    uint64_t* bar_k = bars + 6;      // [slot] K has landed (TMA bytes)
    uint64_t* bar_v = bars + 8;      // [slot] V has landed
    uint64_t* bar_kfree = bars + 10; // [slot] both S issuers are done with this K slot
    uint64_t* bar_vfree = bars + 12; // [slot] both P V issuers are done with this V slot
    uint64_t* bar_q = bars + 14;     // both Q tiles are in shared memory
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kh = blockIdx.x % A.nkv, g = A.nq / A.nkv;   // blocks in order of falling length over all KV heads

    int tile = (int)(gridDim.x / A.nkv) - 1 - (int)(blockIdx.x / A.nkv), b = 0;          // longest tiles (late rows of a request) first
    if (A.order != nullptr) {
        const int packed = A.order[blockIdx.x / A.nkv];
        b = packed >> 16; tile = packed & 0xFFFF;
    } else {
        for (; b < A.B; ++b) {
            const int nt = ((A.q_start[b + 1] - A.q_start[b]) * g + QT * BM - 1) / (QT * BM);
            if (tile < nt) break;
            tile -= nt;
        }
    }
    if (b >= A.B) return;
    const int qs = A.q_start[b], qlen = A.q_start[b + 1] - qs, sp = A.start_pos[b];
    const int rows_total = qlen * g;
    const int* tab = A.table + (size_t)tl_checked(A.slots[b], A.lim.table_rows, A.lim, TL_K_TC2_PREFILL) * A.max_pages;
    int row0[QT], kt_first[QT], kt_last[QT];
#pragma unroll
    for (int t = 0; t < QT; ++t) {
        row0[t] = (tile * QT + t) * BM;
        if (row0[t] < rows_total) {
            const int row_end = min(row0[t] + BM, rows_total);
            const int pos_first = sp + row0[t] / g, pos_last = sp + (row_end - 1) / g;
            const int key_lo = A.window > 0 ? max(0, pos_first - A.window + 1) : 0;
            kt_first[t] = key_lo / BN3; kt_last[t] = pos_last / BN3;
        } else {                                           // no rows: reads nothing
            kt_first[t] = 1; kt_last[t] = 0;
        }
    }
    const int kt_lo = kt_first[0], kt_hi = max(kt_last[0], kt_last[1]), n_kt = kt_hi - kt_lo + 1;
    auto reads = [&](int t, int j) { return kt_lo + j >= kt_first[t] && kt_lo + j <= kt_last[t]; };

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_s + i, 1); mbar_init(bar_p + i, 128); mbar_init(bar_o + i, 1);
            mbar_init(bar_k + i, 1); mbar_init(bar_v + i, 1); mbar_init(bar_kfree + i, 2); mbar_init(bar_vfree + i, 2);
        }
        mbar_init(bar_q, QT * BM);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(TMEM3_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp < 8) {
        // ------------------------------------------------------------ softmax and epilogue: thread = row of tile t
        const int t = warp >> 2, r = tid & 127;
        const int R = row0[t] + r;
        const int pos_r = R < rows_total ? sp + R / g : -1; // -1: no key is visible
        const int lo_r = A.window > 0 ? max(0, pos_r - A.window + 1) : 0;
        const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_addr = lane_addr + S3_COL + t * BN3, o_addr = lane_addr + O3_COL + t * D;
        const int n_mine = kt_last[t] - kt_first[t] + 1;   // <= 0: this tile has no rows
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        load_q_rows(sQ + t * Q_BYTES, A.q, A.q_stride, qs, kh * g, g, row0[t], rows_total, r);
        cp_async_wait_all();
        fence_async_proxy();
        mbar_arrive(bar_q);

        for (int i = 0; i < n_mine && ok; ++i) {
            const int key0 = (kt_first[t] + i) * BN3;
            ok = mbar_wait(bar_s + t, i & 1, abort_flag, A.status, 1);                   // S(i) is ready; P(i-1) V is complete
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool all_visible = key0 + BN3 - 1 <= pos_r && key0 >= lo_r;
            // first reading: the row's largest score
            float mx = -INFINITY;
#pragma unroll
            for (int c0 = 0; c0 < BN3; c0 += 64) {
                float s[64];
                tmem_ld32(s_addr + c0, reinterpret_cast<float(&)[32]>(s[0]));
                tmem_ld32(s_addr + c0 + 32, reinterpret_cast<float(&)[32]>(s[32]));
                tmem_ld_wait();
                if (!all_visible) {
#pragma unroll
                    for (int c = 0; c < 64; ++c) {
                        const int j = key0 + c0 + c;
                        if (!(j <= pos_r && j >= lo_r)) s[c] = -INFINITY;
                    }
                }
                mx = fmaxf(mx, row_max(s));
            }
            mx *= A.scale_log2;
            const bool raise = mx > m_ref + RESCALE_THRESHOLD || (m_ref == -INFINITY && mx != -INFINITY);
            const float m_new = raise ? fmaxf(mx, m_ref) : m_ref;
            const bool fix_o = raise && i > 0 && m_ref != -INFINITY;        // O holds earlier tiles of this row, at rest
            if (__any_sync(0xffffffffu, fix_o)) {
                const float alpha = fix_o ? fast_exp2(m_ref - m_new) : 1.0f;
                l *= alpha;
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    float o[32];
                    tmem_ld32(o_addr + c0, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c] *= alpha;
                    tmem_st32(o_addr + c0, o);
                }
            }
            m_ref = m_new;
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            // second reading: exponentials, packed two a column over the first half of the slot.  Keys 0..63 go to
            // columns 0..31 after columns 0..63 were read; keys 64..127 to columns 32..63, which were read before.
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c0 = 0; c0 < BN3; c0 += 64) {
                float s[64];
                tmem_ld32(s_addr + c0, reinterpret_cast<float(&)[32]>(s[0]));
                tmem_ld32(s_addr + c0 + 32, reinterpret_cast<float(&)[32]>(s[32]));
                tmem_ld_wait();
                uint32_t packed[32];
#pragma unroll
                for (int c = 0; c < 64; c += 2) {
                    float p0 = fast_exp2(fmaf(s[c], A.scale_log2, -m_use)), p1 = fast_exp2(fmaf(s[c + 1], A.scale_log2, -m_use));
                    if (!all_visible) {
                        const int j = key0 + c0 + c;
                        if (!(j <= pos_r && j >= lo_r)) p0 = 0.f;
                        if (!(j + 1 <= pos_r && j + 1 >= lo_r)) p1 = 0.f;
                    }
                    l4[(c >> 1) & 3] += p0 + p1;
                    packed[c >> 1] = pack_bf16(p0, p1);
                }
                tmem_st32_nowait(s_addr + (c0 >> 1), packed);
            }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(bar_p + t);
        }
        // ------------------------------------------------------------ epilogue: the tile's last P V has finished
        if (ok && n_mine > 0 && mbar_wait(bar_o + t, (n_mine - 1) & 1, abort_flag, A.status, 4)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* dst = nullptr;
            if (R < rows_total) dst = A.out + ((size_t)(qs + R / g) * A.nq + (kh * g + R % g)) * D;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                float o[32];
                tmem_ld32(o_addr + c0, o);
                tmem_ld_wait();
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
    } else if (warp < 12) {
        // ------------------------------------------------------------ MMA issuers: one thread each in warps 8..11
        // (S of tile 0, S of tile 1, P V of tile 0, P V of tile 1).  Every issuer walks all key tiles, also those
        // its query tile does not read, and hands each K (V) slot back with one of the two arrivals its barrier counts.
        if (lane == 0) {
            const int t = warp & 1;
            bool ok = true;
            if (warp < 10) {
                constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN3 >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
                ok = mbar_wait(bar_q, 0, abort_flag, A.status, 11, true);
                int i = 0;                                  // products issued for this tile
                for (int j = 0; j < n_kt && ok; ++j) {
                    const int sl = j & 1;
                    ok = mbar_wait(bar_k + sl, (j >> 1) & 1, abort_flag, A.status, 5, true);        // K(j) is in
                    if (!ok) break;
                    if (!reads(t, j)) { mbar_arrive(bar_kfree + sl); continue; }
                    if (i >= 1) {                           // the slot is free once P(i-1) V has read P(i-1)
                        ok = mbar_wait(bar_o + t, (i - 1) & 1, abort_flag, A.status, 6, true);
                        if (!ok) break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t k_addr = sK + sl * KV3_BYTES;
#pragma unroll
                    for (int k = 0; k < D / 16; ++k)
                        umma(tmem + S3_COL + t * BN3, desc_kmajor(sQ + t * Q_BYTES + (k >> 2) * BM * 128 + (k & 3) * 32),
                             desc_kmajor(k_addr + (k >> 2) * BN3 * 128 + (k & 3) * 32), idesc_s, k > 0 ? 1u : 0u);
                    umma_commit(bar_s + t);
                    umma_commit(bar_kfree + sl);
                    ++i;
                }
            } else {
                constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
                int i = 0;
                for (int j = 0; j < n_kt && ok; ++j) {
                    const int sl = j & 1;
                    ok = mbar_wait(bar_v + sl, (j >> 1) & 1, abort_flag, A.status, 7, true);        // V(j) is in
                    if (!ok) break;
                    if (!reads(t, j)) { mbar_arrive(bar_vfree + sl); continue; }
                    ok = mbar_wait(bar_p + t, i & 1, abort_flag, A.status, 8, true);                // P is written
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t v_addr = sV + sl * KV3_BYTES;
#pragma unroll
                    for (int k = 0; k < BN3 / 16; ++k)      // O_t += P V(j): 16 keys = 8 columns of P a product
                        umma_a_tmem(tmem + O3_COL + t * D, tmem + S3_COL + t * BN3 + k * 8,
                                    desc_mnmajor(v_addr + k * 16 * 128, BN3 * 128), idesc_o, (i > 0 || k > 0) ? 1u : 0u);
                    umma_commit(bar_o + t);
                    umma_commit(bar_vfree + sl);
                    ++i;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ copies: one thread of warp 12 issues the TMA
        // boxes of K, one of warp 13 those of V, up to two tiles ahead
        if (lane == 0) {
            const bool is_k = warp == 12;
            const CUtensorMap* map = is_k ? &map_k : &map_v;
            asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
            uint64_t* bar_free = is_k ? bar_kfree : bar_vfree;
            uint64_t* bar_full = is_k ? bar_k : bar_v;
            const uint32_t tiles = is_k ? sK : sV;
            int ps_shift = 0;
            while ((1 << ps_shift) < A.page_size) ++ps_shift;
            const int ppt = BN3 >> ps_shift;                // pages per key tile: 2 to 16
            bool ok = true;
            for (int j = 0; j < n_kt && ok; ++j) {
                const int sl = j & 1;
                int page[16];
#pragma unroll
                for (int pg = 0; pg < 16; ++pg)             // the tile's page numbers, all requested before the wait
                    if (pg < ppt) page[pg] = tl_checked(tab[min((((kt_lo + j) * BN3) >> ps_shift) + pg, A.max_pages - 1)],
                                                        A.lim.total_pages, A.lim, TL_K_TC2_PREFILL);
                if (j >= 2) {
                    ok = mbar_wait(bar_free + sl, ((j - 2) >> 1) & 1, abort_flag, A.status, is_k ? 9 : 10, true);
                    if (!ok) break;
                }
                mbar_expect_tx(bar_full + sl, KV3_BYTES);
#pragma unroll
                for (int pg = 0; pg < 16; ++pg) {
                    if (pg >= ppt) break;
                    const int row = (page[pg] * A.nkv + kh) << ps_shift;
#pragma unroll
                    for (int db = 0; db < D / 64; ++db)
                        tma_box(tiles + sl * KV3_BYTES + db * (BN3 * 128) + ((pg << ps_shift) * 128), map, bar_full + sl, db * 64, row);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
    }
    if (warp == 8) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM3_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
bool g_attr2_done[TL_MAX_DEVICES] = {};
bool g_attr3_done[TL_MAX_DEVICES] = {};

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
#endif  // HEAD_DIM <= 128

bool g_attr_done[TL_MAX_DEVICES] = {};

}  // namespace

TL_EXPORT int tl_attn_tc_head_dim() { return D; }
// 1 if this library was compiled as the checking build (-DTL_CHECK=1).
TL_EXPORT int tl_check_build() { return TL_CHECKING; }

// total_tiles = sum over requests of ceil(q_len * g / 128).  `status`: device int, zero before the call.
TL_EXPORT int tl_attn_tc_prefill(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                 const int* table, int max_pages, int page_size, const int* q_start,
                                 const int* start_pos, const int* slots, int B, int nq, int nkv, int window,
                                 float scale, int total_tiles, int* status, const int* order, int table_rows, int total_pages,
                                 int* fault, cudaStream_t stream) {
    if (total_tiles <= 0 || B <= 0) return 0;
    if (nq % nkv || page_size <= 0 || (page_size & (page_size - 1)) || page_size * 32 < BN || page_size > 64 || (q_stride & 7) || ((uintptr_t)q & 15)) return 1;
    const int dev = tl_device_index();
    if (dev < 0) return 1;
    if (!g_attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        g_attr_done[dev] = true;
    }
    TcAttnArgs A{};
    A.q = (const bf16*)q; A.q_stride = q_stride; A.out = (bf16*)out;
    A.k_pages = (const bf16*)k_pages; A.v_pages = (const bf16*)v_pages;
    A.table = table; A.max_pages = max_pages; A.page_size = page_size;
    A.q_start = q_start; A.start_pos = start_pos; A.slots = slots;
    A.B = B; A.nq = nq; A.nkv = nkv; A.window = window; A.scale_log2 = scale * LOG2E; A.status = status; A.order = order;
    A.lim = TlLimits{table_rows, total_pages, fault};
    dim3 grid((unsigned)total_tiles * (unsigned)nkv);
    attn_tc_prefill_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(A);
    return tl_launch_status();
}

// The same attention with two query tiles (256 rows) per block and K, V loaded by TMA.  total_tiles = sum over
// requests of ceil(q_len * g / 256); `total_pages`: first dimension of the cache tensors.  Returns 2 if this build
// or these sizes do not take this kernel (head size above 128, pages of fewer than 8 tokens, unaligned pages).
// The parts that the runs of a split launch have left, merged: one (token, head) a group of D / 4 threads.  rows: the
// tokens to merge (the step may hold tokens that another kernel serves).
__global__ void attn_tc_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                                     const int* __restrict__ rows, int n_rows, int tokens, int nq, int ksplit) {
    constexpr int PER = D / 4;                             // threads a (token, head)
    const size_t item = (size_t)blockIdx.x * (blockDim.x / PER) + threadIdx.x / PER;
    if (item >= (size_t)n_rows * nq) return;
    const int token = rows[item / nq], head = (int)(item % nq), c = (threadIdx.x % PER) * 4;
    float m = -INFINITY;
    for (int r = 0; r < ksplit; ++r) m = fmaxf(m, part_ml[(((size_t)r * tokens + token) * nq + head) * 2]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float l = 0.f;
    for (int r = 0; r < ksplit; ++r) {                     // in run order: the sum does not depend on who finished first
        const size_t slot = ((size_t)r * tokens + token) * nq + head;
        const float mr = part_ml[slot * 2];
        if (mr == -INFINITY) continue;                     // that run held no key for this row: its O was never written
        const float f = exp2f(mr - m);
        const float4 o = *reinterpret_cast<const float4*>(part_o + slot * D + c);
        acc.x += f * o.x; acc.y += f * o.y; acc.z += f * o.z; acc.w += f * o.w;
        l += f * part_ml[slot * 2 + 1];
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    uint2 v;
    v.x = pack_bf16(acc.x * inv, acc.y * inv); v.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(out + ((size_t)token * nq + head) * D + c) = v;
}

static int tc2_prefill_impl(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                            long long total_pages, const int* table, int max_pages, int page_size,
                            const int* q_start, const int* start_pos, const int* slots, int B, int nq, int nkv,
                            int window, float scale, int total_tiles, int* status, const int* order, int table_rows,
                            int* fault, bool p_tmem, int ksplit, int tokens, float* part_o, float* part_ml,
                            const int* merge_rows, int n_merge_rows, cudaStream_t stream) {
#if HEAD_DIM <= 128
    if (total_tiles <= 0 || B <= 0) return 0;
    if (page_size < 8 || page_size > 64 || (page_size & (page_size - 1))) return 2;
    if (((uintptr_t)k_pages & 127) || ((uintptr_t)v_pages & 127)) return 2;
    if (nq % nkv || (q_stride & 7) || ((uintptr_t)q & 15)) return 1;
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn ||
            qres != cudaDriverEntryPointSuccess) return 100;
        g_encode = (EncodeTiledFn)fn;
    }
    const int dev = tl_device_index();
    if (dev < 0) return 1;
    if (!g_attr2_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc2_prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_BYTES);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_tc2_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_BYTES);
        if (e != cudaSuccess) return (int)e;
        g_attr2_done[dev] = true;
    }
    CUtensorMap mk, mv;
    const long long rows = total_pages * nkv * page_size;
    int e;
    if ((e = make_pages_map(&mk, k_pages, rows, page_size))) return e;
    if ((e = make_pages_map(&mv, v_pages, rows, page_size))) return e;
    TcAttnArgs A{};
    A.q = (const bf16*)q; A.q_stride = q_stride; A.out = (bf16*)out;
    A.k_pages = (const bf16*)k_pages; A.v_pages = (const bf16*)v_pages;
    A.table = table; A.max_pages = max_pages; A.page_size = page_size;
    A.q_start = q_start; A.start_pos = start_pos; A.slots = slots;
    A.B = B; A.nq = nq; A.nkv = nkv; A.window = window; A.scale_log2 = scale * LOG2E; A.status = status; A.order = order;
    A.lim = TlLimits{table_rows, (int)total_pages, fault};
    if (ksplit > 1 && (ksplit > 8 || !part_o || !part_ml || !merge_rows || tokens <= 0 || ((uintptr_t)part_o & 15) || ((uintptr_t)part_ml & 7))) return 1;
    A.ksplit = ksplit > 1 ? ksplit : 1; A.tokens = tokens; A.part_o = part_o; A.part_ml = part_ml;
    dim3 grid((unsigned)total_tiles * (unsigned)nkv * (unsigned)A.ksplit);
    if (p_tmem) attn_tc2_prefill_kernel<true><<<grid, THREADS2, SMEM2_BYTES, stream>>>(mk, mv, A);
    else        attn_tc2_prefill_kernel<false><<<grid, THREADS2, SMEM2_BYTES, stream>>>(mk, mv, A);
    int rc = tl_launch_status();
    if (rc || A.ksplit == 1 || n_merge_rows <= 0) return rc;
    constexpr int GROUPS = 256 / (D / 4);                  // (token, head) pairs a block of 256 threads
    const long long items = (long long)n_merge_rows * nq;
    attn_tc_merge_kernel<<<(unsigned)((items + GROUPS - 1) / GROUPS), 256, 0, stream>>>(part_o, part_ml, (bf16*)out, merge_rows, n_merge_rows,
                                                                                       tokens, nq, A.ksplit);
    return tl_launch_status();
#else
    return 2;
#endif
}

TL_EXPORT int tl_attn_tc2_prefill(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                  long long total_pages, const int* table, int max_pages, int page_size,
                                  const int* q_start, const int* start_pos, const int* slots, int B, int nq, int nkv,
                                  int window, float scale, int total_tiles, int* status, const int* order, int table_rows,
                                  int* fault, cudaStream_t stream) {
    return tc2_prefill_impl(q, q_stride, out, k_pages, v_pages, total_pages, table, max_pages, page_size, q_start, start_pos, slots,
                            B, nq, nkv, window, scale, total_tiles, status, order, table_rows, fault, false, 1, 0, nullptr, nullptr, nullptr, 0, stream);
}

// The same kernel with P kept in tensor memory (key tiles of 64 still, two S slots a query tile).
TL_EXPORT int tl_attn_tc2p_prefill(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                   long long total_pages, const int* table, int max_pages, int page_size,
                                   const int* q_start, const int* start_pos, const int* slots, int B, int nq, int nkv,
                                   int window, float scale, int total_tiles, int* status, const int* order, int table_rows,
                                   int* fault, cudaStream_t stream) {
    return tc2_prefill_impl(q, q_stride, out, k_pages, v_pages, total_pages, table, max_pages, page_size, q_start, start_pos, slots,
                            B, nq, nkv, window, scale, total_tiles, status, order, table_rows, fault, true, 1, 0, nullptr, nullptr, nullptr, 0, stream);
}

// The pair kernel with every block's key tiles dealt out to `ksplit` blocks (2..8) and a merge kernel behind them: for
// portions on long contexts whose query tiles alone leave most of the GPU idle.  part_o: float [ksplit, tokens, nq, D],
// part_ml: float [ksplit, tokens, nq, 2] (scratch); merge_rows: the n_merge_rows tokens this launch serves; tokens: rows of out.
TL_EXPORT int tl_attn_tc2_prefill_split(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                        long long total_pages, const int* table, int max_pages, int page_size,
                                        const int* q_start, const int* start_pos, const int* slots, int B, int nq, int nkv,
                                        int window, float scale, int total_tiles, int* status, const int* order, int table_rows,
                                        int* fault, int p_tmem, int ksplit, int tokens, float* part_o, float* part_ml,
                                        const int* merge_rows, int n_merge_rows, cudaStream_t stream) {
    return tc2_prefill_impl(q, q_stride, out, k_pages, v_pages, total_pages, table, max_pages, page_size, q_start, start_pos, slots,
                            B, nq, nkv, window, scale, total_tiles, status, order, table_rows, fault, p_tmem != 0, ksplit, tokens,
                            part_o, part_ml, merge_rows, n_merge_rows, stream);
}

// Two query tiles (256 rows) per block, key tiles of 128, P kept in tensor memory; K, V loaded by TMA.  total_tiles = sum over
// requests of ceil(q_len * g / 256); `total_pages`: first dimension of the cache tensors.  Returns 2 if this build
// or these sizes do not take this kernel (head size above 128, pages of fewer than 8 tokens, unaligned pages).
TL_EXPORT int tl_attn_tc3_prefill(const void* q, int q_stride, void* out, const void* k_pages, const void* v_pages,
                                  long long total_pages, const int* table, int max_pages, int page_size,
                                  const int* q_start, const int* start_pos, const int* slots, int B, int nq, int nkv,
                                  int window, float scale, int total_tiles, int* status, const int* order, int table_rows,
                                  int* fault, cudaStream_t stream) {
#if HEAD_DIM <= 128
    if (total_tiles <= 0 || B <= 0) return 0;
    if (page_size < 8 || page_size > 64 || (page_size & (page_size - 1))) return 2;
    if (((uintptr_t)k_pages & 127) || ((uintptr_t)v_pages & 127)) return 2;
    if (nq % nkv || (q_stride & 7) || ((uintptr_t)q & 15)) return 1;
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn ||
            qres != cudaDriverEntryPointSuccess) return 100;
        g_encode = (EncodeTiledFn)fn;
    }
    const int dev = tl_device_index();
    if (dev < 0) return 1;
    if (!g_attr3_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc3_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM3_BYTES);
        if (e != cudaSuccess) return (int)e;
        g_attr3_done[dev] = true;
    }
    CUtensorMap mk, mv;
    const long long rows = total_pages * nkv * page_size;
    int e;
    if ((e = make_pages_map(&mk, k_pages, rows, page_size))) return e;
    if ((e = make_pages_map(&mv, v_pages, rows, page_size))) return e;
    TcAttnArgs A{};
    A.q = (const bf16*)q; A.q_stride = q_stride; A.out = (bf16*)out;
    A.k_pages = (const bf16*)k_pages; A.v_pages = (const bf16*)v_pages;
    A.table = table; A.max_pages = max_pages; A.page_size = page_size;
    A.q_start = q_start; A.start_pos = start_pos; A.slots = slots;
    A.B = B; A.nq = nq; A.nkv = nkv; A.window = window; A.scale_log2 = scale * LOG2E; A.status = status; A.order = order;
    A.lim = TlLimits{table_rows, (int)total_pages, fault};
    dim3 grid((unsigned)total_tiles * (unsigned)nkv);
    attn_tc3_prefill_kernel<<<grid, THREADS2, SMEM3_BYTES, stream>>>(mk, mv, A);
    return tl_launch_status();
#else
    return 2;
#endif
}
