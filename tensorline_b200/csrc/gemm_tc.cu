// bfloat16 matrix product on the 5th-generation tensor cores (sm_100a): tcgen05.mma with the
// accumulator in tensor memory, operands brought to shared memory by TMA.
//
//     D[a, b] = sum_k  A[a, k] * B[b, k]        A: [RA, K],  B: [RB, K],  both row-major (K-major)
//
// A is the operand that fills the 128 rows of the MMA tile, B the N side (BN = 16..256 columns).
// The launcher maps a linear layer y = x W^T onto it in one of two ways:
//   * many tokens (prefill):  A = x [T, K],  B = W [N, K];   y[a, b] = D[a, b]
//   * few tokens (decode):    A = W [N, K],  B = x [T, K];   y[b, a] = D[a, b]   ("swap": the weight
//     matrix takes the 128-row side, so a batch of 1..64 tokens wastes no tensor-core rows and every
//     weight byte is streamed exactly once by large TMA copies).  With few 128-row tiles the K range is
//     split over blockIdx.z and the float partials are summed by a second small kernel.
//
// One block = 6 warps: warp 0 issues the TMA loads (one thread), warp 1 allocates tensor memory and
// issues the MMAs (one thread), warps 2..5 read the accumulator back (tcgen05.ld, one quarter of the
// 128 lanes each) and store it.  A ring of STAGES shared-memory tiles (128-byte swizzle, as TMA writes
// them and the MMA's shared-memory descriptors read them) is handed back and forth with mbarriers.
// Every wait on an mbarrier is bounded: if it does not complete in about two seconds the block
// records an error code in `status`, stops issuing work, frees its tensor memory and returns.
#include "common.cuh"
#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace {

constexpr int BM = 128;                // rows of A per tile = MMA M
constexpr int BK = 64;                 // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr long long WAIT_CYCLES = 4000000000LL;     // ~2 s at 2 GHz; tl_gemm_tc_test_hooks can shorten it

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and records `code`) if the barrier did not flip in time or another
// role of the block already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                          long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(c0), "r"(c1) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes, groups
// of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);             // start address, 16-byte units
    d |= (uint64_t)1 << 16;                             // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset
    d |= (uint64_t)1 << 46;                             // version
    d |= (uint64_t)2 << 61;                             // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");   // not .aligned: lanes of a warp may arrive apart
}
// The same shared-memory location in block `rank` of this cluster.
__device__ __forceinline__ const float* cluster_peer(const float* p, int rank) {
    uint64_t out;
    asm volatile("mapa.u64 %0, %1, %2;" : "=l"(out) : "l"(reinterpret_cast<uint64_t>(p)), "r"(rank));
    return reinterpret_cast<const float*>(out);
}

// silu(gate) * up of two accumulator values, each rounded to bfloat16 first (as a stored gate|up product would have been).
__device__ __forceinline__ float silu_mul_rounded(float gate, float up) {
    return tl_silu_mul(__bfloat162float(__float2bfloat16_rn(gate)), __bfloat162float(__float2bfloat16_rn(up)));
}

struct GemmArgs {
    void* out;            // bf16 or float [rows, ldo]
    float* partial;       // [splits, RB or RA rows..] float, when splits > 1
    int ldo;
    int RA, RB, K;        // rows of A, rows of B, reduction length
    int k_tiles_per_split;
    int swap;             // 1: out[b, a] = D[a, b];  0: out[a, b] = D[a, b]
    int out_f32;
    int* status;
    int* counters;        // one per output tile, zero between calls: the last block of a tile to finish sums the partials
    int cluster_reduce;   // the K ranges of a tile are a thread-block cluster (grid z) and sum their tiles through
                          // distributed shared memory: no pieces in global memory (swap = 1, 2..8 ranges)
    int gated;            // swap, one split: rows 0..63 of every 128-row tile of A are gate features, rows 64..127 the
                          // up features of the same 64 columns; out[b, 64 tile + j] = silu(gate) * up, [RB, RA / 2]
    long long wait_cycles;   // how long a wait on a barrier may take before the block gives up
    int drop_last_load;      // tests only: the copy thread leaves out its last stage, so the MMA thread's wait runs out
    // The residual add folded into the product that makes the addend (swap, cluster_reduce): the block that finishes a
    // share of the tile adds the bfloat16-rounded sums into the float residual stream res_x [RB, res_ld] in place and
    // leaves the sum of squares of the new values of every (token, 128-row tile) in ssq_out [RB, tiles of RA].
    float* res_x; int res_ld; float* ssq_out;
    // The norm folded into the product that reads its result (swap): the B operand is not loaded by TMA but made by the
    // epilogue warps from the float residual stream nx [rows, K]: h = cast(cast(x * rstd) * w), rstd of a row from the
    // nparts partial sums of squares nssq [rows, nparts] (summed in a fixed order), K and eps.
    const float* nx; const float* nssq; int nparts; const void* nw; int nw_f32; float neps;
    // tracing build: stamps 0 block start, 1 dependency wait returned, 2 first stage ready for the MMA, 3 last stage
    // ready, 4 block end; with a made B operand 5 rstd known, 6 first raw tile landed, 7 first operand tile made
    TlTrace trace;
};

// The B operand (activations, BN tokens x 64 k a stage) made from the residual stream instead of loaded.  The copy thread
// brings the raw material of a stage to shared memory by TMA beside the weight tile (a [BN, 64] box of the float stream and
// the 64 norm weights of the k range, onto a barrier of their own); the four epilogue warps, idle while the products run,
// normalise it with the row's rstd (cast to bfloat16 before the weight multiply and after it, as the norm kernel does) and
// write the tile in the layout TMA would have left for a bfloat16 matrix (rows of 128 bytes, 16-byte chunks swizzled by
// the row within its group of 8), then hand the stage to the MMA thread.  Only shared memory is read here: loading the
// stream with ordinary loads made every block wait on the same few cache lines (1,000 to 2,800 cycles a tile, measured).
constexpr int RAW_W_BYTES = 256;                                         // 64 norm weights of a stage, float at most
template <int BN> __host__ __device__ constexpr int raw_stage_bytes() { return BN * BK * 4 + RAW_W_BYTES; }

// Whether the partial sums of squares of this block's tokens go to shared memory by one bulk copy (16-byte rules, and room
// in one operand tile of BN x 64 bfloat16).
template <int BN>
__device__ __forceinline__ bool ssq_in_smem(const GemmArgs& G, int b0) {
    const int n = min(BN, G.RB - b0) * G.nparts;
    return (n & 3) == 0 && n * 4 <= BN * BK * 2 && ((reinterpret_cast<uintptr_t>(G.nssq + (size_t)b0 * G.nparts)) & 15) == 0;
}

template <int BN, int STAGES>
__device__ __forceinline__ void make_b_tiles(const GemmArgs& G, unsigned char* tiles, unsigned char* raw, uint64_t* full_bar,
                                             uint64_t* raw_bar, uint64_t* ssq_bar, float* rstd_s, volatile int* abort_flag, int b0, int kt_begin, int n_kt) {
    constexpr int A_BYTES = BM * BK * 2, STAGE_BYTES = A_BYTES + BN * BK * 2, RAW_BYTES = raw_stage_bytes<BN>();
    constexpr int CHUNKS = BN * 8 / 128 > 0 ? BN * 8 / 128 : 1;          // 16-byte chunks of the tile a thread writes
    const int e = (int)threadIdx.x - 64;                                 // 0..127
    // The partial sums of squares: every block of the launch wants the same few hundred bytes at the same moment, and
    // ordinary loads of such lines take two microseconds where a bulk copy takes one (measured with time stamps).  Where
    // they fit, the copy thread has brought them into the operand tile of the last stage, which nothing writes before here.
    const float* ssq_s = nullptr;
    if (ssq_in_smem<BN>(G, b0)) {
        if (!mbar_wait(ssq_bar, 0, abort_flag, G.status, 4, G.wait_cycles)) return;
        ssq_s = reinterpret_cast<const float*>(tiles + (STAGES - 1) * STAGE_BYTES + A_BYTES);
    }
    // rstd of every token: eight lanes a token, each sums the partial sums p = lane, lane + 8, ... (loads independent of one
    // another), then the eight are added in a fixed order
    for (int t0 = 0; t0 < BN; t0 += 16) {
        const int tl = t0 + (e >> 3), b = b0 + tl, l8 = e & 7;
        float ss = 0.f;
        const bool live = tl < BN && b < G.RB;
        if (live) {
            const float* src = ssq_s ? ssq_s + (size_t)tl * G.nparts : G.nssq + (size_t)b * G.nparts;
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
            int p = l8;
            for (; p + 24 < G.nparts; p += 32) { s0 += src[p]; s1 += src[p + 8]; s2 += src[p + 16]; s3 += src[p + 24]; }
            for (; p < G.nparts; p += 8) s0 += src[p];
            ss = (s0 + s1) + (s2 + s3);
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
        if (l8 == 0 && tl < BN) rstd_s[tl] = live ? 1.0f / sqrtf(ss / (float)G.K + G.neps) : 0.f;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (e == 0) tl_stamp(G.trace, 5);
    for (int i = 0; i < n_kt; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(raw_bar + s, (i / STAGES) & 1, abort_flag, G.status, 4, G.wait_cycles)) return;   // the stage's raw material is in
        if (i == 0 && e == 0) tl_stamp(G.trace, 6);
        const unsigned char* rx = raw + s * RAW_BYTES;
        const unsigned char* rw = rx + BN * BK * 4;
        unsigned char* bt = tiles + s * STAGE_BYTES + A_BYTES;
        const int k0 = (kt_begin + i) * BK;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int item = e + 128 * c, b = item >> 3, ch = item & 7;
            if (b >= BN) continue;
            uint32_t packed[4] = {0u, 0u, 0u, 0u};
            if (k0 + ch * 8 < G.K) {                                     // K % 8 == 0: a chunk is whole or absent (absent: zeros)
                const float rs = rstd_s[b];
                const float4 x0 = *reinterpret_cast<const float4*>(rx + b * (BK * 4) + ch * 32);
                const float4 x1 = *reinterpret_cast<const float4*>(rx + b * (BK * 4) + ch * 32 + 16);
                const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                float ws[8];
                if (G.nw_f32) {
                    const float4 w0 = *reinterpret_cast<const float4*>(rw + ch * 32), w1 = *reinterpret_cast<const float4*>(rw + ch * 32 + 16);
                    ws[0] = w0.x; ws[1] = w0.y; ws[2] = w0.z; ws[3] = w0.w; ws[4] = w1.x; ws[5] = w1.y; ws[6] = w1.z; ws[7] = w1.w;
                } else {
                    const uint4 wq = *reinterpret_cast<const uint4*>(rw + ch * 16);
                    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wq);
#pragma unroll
                    for (int j = 0; j < 4; ++j) { ws[2 * j] = __low2float(w2[j]); ws[2 * j + 1] = __high2float(w2[j]); }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float n0 = __bfloat162float(__float2bfloat16_rn(xs[2 * j] * rs)), n1 = __bfloat162float(__float2bfloat16_rn(xs[2 * j + 1] * rs));
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(n0 * ws[2 * j], n1 * ws[2 * j + 1]);
                    packed[j] = *reinterpret_cast<uint32_t*>(&h2);
                }
            }
            const uint32_t dst = smem_addr(bt + (b >> 3) * 1024 + (b & 7) * 128 + ((ch ^ (b & 7)) << 4));
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[0]), "r"(packed[1]), "r"(packed[2]), "r"(packed[3]) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy writes before the MMA reads them
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (e == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(full_bar + s)) : "memory");
        if (i == 0 && e == 0) tl_stamp(G.trace, 7);
    }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmArgs G) {
    // (with a made B operand, map_b describes the float residual stream: boxes of [BN rows, 64 floats], no swizzle)
    extern __shared__ unsigned char smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int RAW_BYTES = BN <= 64 ? raw_stage_bytes<BN>() : 0;
    const bool made_b = BN <= 64 && G.nx != nullptr;     // the raw material of the B tiles has a ring of its own behind the stages
    unsigned char* raw = tiles + STAGES * STAGE_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(raw + (made_b ? STAGES * RAW_BYTES : 0));
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* done_bar = empty_bar + STAGES;
    uint64_t* raw_bar = done_bar + 1;                    // [STAGES] the stage's raw material has landed
    uint64_t* ssq_bar = raw_bar + STAGES;                // the partial sums of squares have landed (made B operand)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ssq_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* last_flag = abort_flag + 1;
    float* rstd_s = reinterpret_cast<float*>(const_cast<int*>(last_flag) + 1);      // [BN] with a made B operand

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a0 = blockIdx.x * BM, b0 = blockIdx.y * BN, split = blockIdx.z;
    const int k_tiles_total = (G.K + BK - 1) / BK;
    const int kt_begin = split * G.k_tiles_per_split;
    const int kt_end = min(k_tiles_total, kt_begin + G.k_tiles_per_split);
    const int n_kt = kt_end - kt_begin;                  // > 0 by construction of the grid
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;

    if (threadIdx.x == 0) {
        tl_stamp(G.trace, 0);
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar + s, made_b ? 2 : 1); mbar_init(empty_bar + s, 1); mbar_init(raw_bar + s, 1); }
        mbar_init(done_bar, 1);
        mbar_init(ssq_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                                     // one warp allocates the accumulator columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // With the residual add folded in, a thread's first four values of the stream are fetched as soon as the kernel in front
    // has finished, long before the accumulators are summed: the add then costs no round trip of its own.
    float4 x_first = make_float4(0.f, 0.f, 0.f, 0.f);
    int x_first_idx = -1;

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------------- TMA producer
        // The weights are nobody's output: the first ring of weight tiles is requested before the wait for the
        // kernel that writes the activations, so the stream from memory is already running when that kernel ends.
        // the activations' descriptor is first used after the wait: fetched now, that round trip is off the critical path
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
        const int ahead = (n_kt < STAGES ? n_kt : STAGES) - ((G.drop_last_load && n_kt <= STAGES) ? 1 : 0);
        const uint32_t tx_bytes = made_b ? A_BYTES : STAGE_BYTES;      // made: the epilogue warps write the B tiles
        const int w_elem = G.nw_f32 ? 4 : 2;
        auto load_raw = [&](int s, int kt) {             // the float stream's [BN, 64] box and the k range's norm weights
            const int k0 = kt * BK, wn = min(BK, G.K - k0) * w_elem;
            unsigned char* rx = raw + s * RAW_BYTES;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(raw_bar + s)), "r"((uint32_t)(BN * BK * 4 + wn)) : "memory");
            tma_load_2d(rx, &map_b, raw_bar + s, k0, b0);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_addr(rx + BN * BK * 4)), "l"((const unsigned char*)G.nw + (size_t)k0 * w_elem), "r"((uint32_t)wn),
                           "r"(smem_addr(raw_bar + s)) : "memory");
        };
        for (int i = 0; i < ahead; ++i) {
            mbar_expect_tx(full_bar + i, tx_bytes);
            unsigned char* st = tiles + i * STAGE_BYTES;
            if (G.swap) tma_load_2d(st, &map_a, full_bar + i, (kt_begin + i) * BK, a0);
            else        tma_load_2d(st + A_BYTES, &map_b, full_bar + i, (kt_begin + i) * BK, b0);
        }
        grid_dependency_wait();
        tl_stamp(G.trace, 1);
        grid_dependency_trigger();
        if constexpr (BN <= 64) {
            if (made_b && ssq_in_smem<BN>(G, b0)) {
                const uint32_t bytes = (uint32_t)(min(BN, G.RB - b0) * G.nparts * 4);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(ssq_bar)), "r"(bytes) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smem_addr(tiles + (STAGES - 1) * STAGE_BYTES + A_BYTES)), "l"(G.nssq + (size_t)b0 * G.nparts), "r"(bytes),
                               "r"(smem_addr(ssq_bar)) : "memory");
            }
        }
        for (int i = 0; i < ahead; ++i) {
            unsigned char* st = tiles + i * STAGE_BYTES;
            if (made_b)      load_raw(i, kt_begin + i);
            else if (G.swap) tma_load_2d(st + A_BYTES, &map_b, full_bar + i, (kt_begin + i) * BK, b0);
            else             tma_load_2d(st, &map_a, full_bar + i, (kt_begin + i) * BK, a0);
        }
        for (int i = ahead; i < n_kt - G.drop_last_load; ++i) {
            const int s = i % STAGES;
            if (!mbar_wait(empty_bar + s, ((i / STAGES) - 1) & 1, abort_flag, G.status, 1, G.wait_cycles)) break;
            mbar_expect_tx(full_bar + s, tx_bytes);
            unsigned char* st = tiles + s * STAGE_BYTES;
            tma_load_2d(st, &map_a, full_bar + s, (kt_begin + i) * BK, a0);
            if (made_b) load_raw(s, kt_begin + i);
            else        tma_load_2d(st + A_BYTES, &map_b, full_bar + s, (kt_begin + i) * BK, b0);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------------------------------------------------------- MMA issuer
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
        bool ok = true;
        grid_dependency_wait();                          // the bounded waits below start counting once the copies can land
        for (int i = 0; i < n_kt && ok; ++i) {
            const int s = i % STAGES;
            ok = mbar_wait(full_bar + s, (i / STAGES) & 1, abort_flag, G.status, 2, G.wait_cycles);
            if (!ok) break;
            if (i == 0) tl_stamp(G.trace, 2);
            if (i == n_kt - 1) tl_stamp(G.trace, 3);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_addr = smem_addr(tiles + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
                umma_bf16(tmem_base, smem_desc(a_addr + k * UMMA_K * 2), smem_desc(b_addr + k * UMMA_K * 2), idesc,
                          (i > 0 || k > 0) ? 1u : 0u);
            umma_commit(empty_bar + s);                  // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(done_bar);                   // the accumulator is complete
    } else if (warp >= 2) {
        // ---------------------------------------------------------------- epilogue: 4 warps, 32 lanes of TMEM each
        grid_dependency_wait();                          // the output may still be read by the kernel before
        if (G.res_x != nullptr && G.cluster_reduce) {
            const int nz = (int)gridDim.z, ntok = min(BN, G.RB - b0);
            const int share = ((ntok + nz - 1) / nz) * BM, lo = split * share, hi = min(ntok * BM, lo + share);
            const int idx = lo + 4 * ((int)threadIdx.x - 64);
            if (idx < hi) {
                const int tok = idx / BM, a = a0 + (idx - tok * BM);
                if (a + 3 < G.RA) { x_first = *reinterpret_cast<const float4*>(G.res_x + (size_t)(b0 + tok) * G.res_ld + a); x_first_idx = idx; }
            }
        }
        if constexpr (BN <= 64) {                        // the few-token order only
            if (made_b) make_b_tiles<BN, STAGES>(G, tiles, raw, full_bar, raw_bar, ssq_bar, rstd_s, abort_flag, b0, kt_begin, n_kt);
        }
        if (mbar_wait(done_bar, 0, abort_flag, G.status, 3, G.wait_cycles)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int quarter = warp & 3;                // the TMEM lanes a warp may read: 32 * (warp % 4)
            const int a = a0 + quarter * 32 + lane;      // row of A = TMEM lane
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(taddr + c0, r);
                if (a >= G.RA && !G.gated && !G.cluster_reduce) continue;
                if (G.gated) {
                    // A feature's gate value sits in TMEM lane f, its up value in lane 64 + f: two threads.  They share the
                    // step's tokens: the up thread hands its values of the first half over through shared memory (the tile
                    // ring is idle by now), the gate thread its values of the second half; each rounds both to bfloat16 as
                    // a stored gate|up product would have been and writes silu(gate) * up for its half of the tokens.
                    float* hand = reinterpret_cast<float*>(tiles) + ((c0 >> 4) & 1) * (16 * 64);   // [16 tokens][64 features], two in turn
                    const int f = (quarter & 1) * 32 + lane;
                    const bool up_side = quarter >= 2;
#pragma unroll
                    for (int j = 0; j < 8; ++j) hand[(up_side ? j : 8 + j) * 64 + f] = __uint_as_float(up_side ? r[j] : r[8 + j]);
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    const int col = blockIdx.x * 64 + f;                           // feature of the output
                    float res[8];                        // no branch in here: the eight tokens' chains overlap
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int t = up_side ? 8 + j : j;
                        const float mine = __uint_as_float(up_side ? r[8 + j] : r[j]), other = hand[t * 64 + f];
                        res[j] = silu_mul_rounded(up_side ? other : mine, up_side ? mine : other);
                    }
                    if (col < (G.RA >> 1)) {
                        bf16* dst = (bf16*)G.out + (size_t)(b0 + c0 + (up_side ? 8 : 0)) * G.ldo + col;
                        const int left = G.RB - (b0 + c0 + (up_side ? 8 : 0));
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (j < left) dst[(size_t)j * G.ldo] = __float2bfloat16_rn(res[j]);
                    }
                    continue;                            // the next 16 tokens use the other buffer: no second barrier
                }
                if (G.cluster_reduce) {                  // [token][128 rows of A] floats in the idle tile ring
                    float* red = reinterpret_cast<float*>(tiles);
#pragma unroll
                    for (int j = 0; j < 16; ++j) red[(c0 + j) * BM + quarter * 32 + lane] = __uint_as_float(r[j]);
                    continue;
                }
                if (gridDim.z > 1) {                     // float partial, laid out like the output
                    float* part = G.partial + (size_t)split * (size_t)G.RA * G.RB;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int b = b0 + c0 + j;
                        if (b < G.RB) part[G.swap ? (size_t)b * G.RA + a : (size_t)a * G.RB + b] = __uint_as_float(r[j]);
                    }
                } else if (G.swap) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int b = b0 + c0 + j;
                        if (b < G.RB) {
                            if (G.out_f32) ((float*)G.out)[(size_t)b * G.ldo + a] = __uint_as_float(r[j]);
                            else ((bf16*)G.out)[(size_t)b * G.ldo + a] = __float2bfloat16_rn(__uint_as_float(r[j]));
                        }
                    }
                } else {
                    const int b = b0 + c0;
                    if (G.out_f32) {
                        float* dst = (float*)G.out + (size_t)a * G.ldo + b;
#pragma unroll
                        for (int j = 0; j < 16; ++j) if (b + j < G.RB) dst[j] = __uint_as_float(r[j]);
                    } else {
                        bf16* dst = (bf16*)G.out + (size_t)a * G.ldo + b;
                        if (b + 16 <= G.RB && ((((uintptr_t)dst) & 15) == 0)) {
                            uint4 v0, v1;
                            uint32_t* p0 = reinterpret_cast<uint32_t*>(&v0);
                            uint32_t* p1 = reinterpret_cast<uint32_t*>(&v1);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                __nv_bfloat162 lo = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                                __nv_bfloat162 hi = __floats2bfloat162_rn(__uint_as_float(r[8 + 2 * j]), __uint_as_float(r[8 + 2 * j + 1]));
                                p0[j] = *reinterpret_cast<uint32_t*>(&lo);
                                p1[j] = *reinterpret_cast<uint32_t*>(&hi);
                            }
                            reinterpret_cast<uint4*>(dst)[0] = v0;
                            reinterpret_cast<uint4*>(dst)[1] = v1;
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j) if (b + j < G.RB) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
                        }
                    }
                }
            }
            if (gridDim.z > 1 && G.counters != nullptr) {
                // Split K inside one launch: every block of a tile publishes its partial, the block that
                // arrives last adds them up in split order (so the sum does not depend on who was last).
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");            // the four epilogue warps
                const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
                if (threadIdx.x == 64) *last_flag = atomicAdd(G.counters + tile_id, 1) == (int)gridDim.z - 1;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (*last_flag) {
                    __threadfence();
                    if (a < G.RA) {
                        const size_t plane = (size_t)G.RA * G.RB;
                        for (int c = 0; c < BN; ++c) {
                            const int b = b0 + c;
                            if (b >= G.RB) break;
                            const size_t idx = G.swap ? (size_t)b * G.RA + a : (size_t)a * G.RB + b;
                            float acc = 0.f;
                            for (int sp = 0; sp < (int)gridDim.z; ++sp) acc += __ldcg(G.partial + sp * plane + idx);
                            const size_t o = G.swap ? (size_t)b * G.ldo + a : (size_t)a * G.ldo + b;
                            if (G.out_f32) ((float*)G.out)[o] = acc;
                            else ((bf16*)G.out)[o] = __float2bfloat16_rn(acc);
                        }
                    }
                    if (threadIdx.x == 64) G.counters[tile_id] = 0;       // ready for the next call
                }
            }
        }
    }
    if (G.cluster_reduce) {
        // Every block of the cluster (one per K range of this tile) has laid its accumulator out in its shared
        // memory; block z now sums a z-th share of the tile over all blocks, in range order, and stores it.
        cluster_barrier();
        if (warp >= 2 && !*abort_flag) {
            const float* red = reinterpret_cast<const float*>(tiles);
            const int nz = (int)gridDim.z, ntok = min(BN, G.RB - b0);
            // with the residual add folded in, a block's share is whole tokens: a warp then holds all 128 rows of one
            const int total = ntok * BM, share = G.res_x ? ((ntok + nz - 1) / nz) * BM : (((total + nz - 1) / nz) + 3) & ~3;
            const int lo = split * share, hi = min(total, lo + share);
            // four rows of A a thread and step (shares and BM are multiples of 4): one 16-byte load a peer
            const bool wide = (G.ldo & 3) == 0 && (((uintptr_t)G.out) & 15) == 0;
            const float* peer[8];                        // the tile of every block of the cluster
#pragma unroll
            for (int z = 0; z < 8; ++z) peer[z] = cluster_peer(red, z < nz ? z : 0);
            for (int idx = lo + 4 * ((int)threadIdx.x - 64); idx < hi; idx += 4 * 128) {
                float4 v[8];                             // all loads are on their way before the first addition
#pragma unroll
                for (int z = 0; z < 8; ++z)
                    if (z < nz) v[z] = *reinterpret_cast<const float4*>(peer[z] + idx);
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int z = 0; z < 8; ++z)
                    if (z < nz) { acc.x += v[z].x; acc.y += v[z].y; acc.z += v[z].z; acc.w += v[z].w; }
                const int tok = idx / BM, a = a0 + (idx - tok * BM);
                if (G.res_x) {
                    // x += the sums rounded to bfloat16 (what the addend would have been stored as); the sum of squares of the
                    // new values of this token's 128 rows goes to its place, in the fixed order of the warp's butterfly
                    float sq = 0.f;
                    if (a + 3 < G.RA) {
                        float* xp = G.res_x + (size_t)(b0 + tok) * G.res_ld + a;
                        float4 xv = idx == x_first_idx ? x_first : *reinterpret_cast<float4*>(xp);
                        xv.x += __bfloat162float(__float2bfloat16_rn(acc.x)); xv.y += __bfloat162float(__float2bfloat16_rn(acc.y));
                        xv.z += __bfloat162float(__float2bfloat16_rn(acc.z)); xv.w += __bfloat162float(__float2bfloat16_rn(acc.w));
                        *reinterpret_cast<float4*>(xp) = xv;
                        sq = fmaf(xv.x, xv.x, fmaf(xv.y, xv.y, fmaf(xv.z, xv.z, xv.w * xv.w)));
                    }
                    sq = warp_sum(sq);
                    if (lane == 0) G.ssq_out[(size_t)(b0 + tok) * gridDim.x + blockIdx.x] = sq;
                    continue;
                }
                const size_t o = (size_t)(b0 + tok) * G.ldo + a;
                if (wide && a + 3 < G.RA) {
                    if (G.out_f32) {
                        *reinterpret_cast<float4*>((float*)G.out + o) = acc;
                    } else {
                        __nv_bfloat162 lo2 = __floats2bfloat162_rn(acc.x, acc.y), hi2 = __floats2bfloat162_rn(acc.z, acc.w);
                        uint2 packed;
                        packed.x = *reinterpret_cast<uint32_t*>(&lo2); packed.y = *reinterpret_cast<uint32_t*>(&hi2);
                        *reinterpret_cast<uint2*>((bf16*)G.out + o) = packed;
                    }
                } else {
                    const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
                    for (int j = 0; j < 4; ++j) {
                        if (a + j < G.RA) {
                            if (G.out_f32) ((float*)G.out)[o + j] = vals[j];
                            else ((bf16*)G.out)[o + j] = __float2bfloat16_rn(vals[j]);
                        }
                    }
                }
            }
        }
        cluster_barrier();                               // nobody leaves while its shared memory is still read
    }
    // ---------------------------------------------------------------- teardown
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) tl_stamp(G.trace, 4);
    if (*abort_flag) {                                   // give copies in flight time to land before the block's
        const long long t0 = clock64();                  // shared memory is handed to another block
        while (clock64() - t0 < 2000000LL) { }
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// out = sum over splits of partial[s], converted; partial is [S, R, C] float, out [R, ldo].
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, void* __restrict__ out, int out_f32,
                                     int S, int R, int C, int ldo) {
    const size_t total = (size_t)R * C;
    grid_dependency_wait();
    grid_dependency_trigger();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < S; ++s) acc += partial[(size_t)s * total + idx];
        const size_t r = idx / C, c = idx - r * C;
        if (out_f32) ((float*)out)[r * ldo + c] = acc;
        else ((bf16*)out)[r * ldo + c] = __float2bfloat16_rn(acc);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int get_encode() {
    if (g_encode) return 0;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || fn == nullptr || q != cudaDriverEntryPointSuccess) return 100;
    g_encode = (EncodeTiledFn)fn;
    return 0;
}

// A [rows, K] bfloat16 row-major matrix as a 2-D tensor map with boxes of [box_rows, 64] and 128-byte swizzle.
// box_rows < 0: a [rows, K] float matrix with boxes of [-box_rows, 64] and no swizzle (the residual stream as raw material).
int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    const bool f32 = box_rows < 0;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * (f32 ? 4 : 2)};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)(f32 ? -box_rows : box_rows)};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = g_encode(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                          dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          f32 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 101;
}

// Encoding a tensor map costs the host a microsecond or two; the same (matrix, box) pairs come back with every
// step (weights always, activations whenever the allocator hands out the same block), so maps are kept by key.
struct MapKey {
    const void* base; int rows, K, box_rows;
    bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && K == o.K && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.base) * 0x9E3779B97F4A7C15ull;
        h ^= ((size_t)(unsigned)k.rows << 32 | (unsigned)k.K) + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
        return h ^ ((size_t)k.box_rows * 0xC2B2AE3D27D4EB4Full);
    }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
std::mutex g_maps_lock;
constexpr size_t MAP_CACHE_ENTRIES = 8192;

int cached_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    const MapKey key{base, rows, K, box_rows};
    std::lock_guard<std::mutex> hold(g_maps_lock);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *map = it->second; return 0; }
    const int e = make_map(map, base, rows, K, box_rows);
    if (e) return e;
    if (g_maps.size() >= MAP_CACHE_ENTRIES) g_maps.clear();
    g_maps.emplace(key, *map);
    return 0;
}

long long g_wait_cycles = WAIT_CYCLES;
TlTraceHost g_trace;
int g_drop_last_load = 0;

template <int BN, int STAGES>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& G, dim3 grid, cudaStream_t stream) {
    constexpr int RAW = BN <= 64 ? STAGES * raw_stage_bytes<BN>() : 0;
    constexpr int SMEM_PLAIN = STAGES * (BM + BN) * BK * 2 + 1024 + (3 * STAGES + 2) * 8 + 32 + BN * 4;
    constexpr int SMEM_MAX = SMEM_PLAIN + RAW;
    const int SMEM = SMEM_PLAIN + (G.nx != nullptr ? RAW : 0);
    // two blocks of the few-token tiles share an SM (the plan of the K ranges and the ring depth count on it)
    static_assert(BN > 64 || 2 * ((BN == 16 ? SMEM_MAX : SMEM_PLAIN) + 1024) <= 228 * 1024,
                  "two blocks of this tile no longer fit an SM's shared memory");     // 16 tokens: with the norm fold too
    static bool attr_set[TL_MAX_DEVICES] = {};
    const int dev = tl_device_index();
    if (dev < 0) return 1;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_MAX);
        if (e != cudaSuccess) return (int)e;
        attr_set[dev] = true;
    }
    if (G.cluster_reduce) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid; cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = SMEM; cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = grid.z;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = tl_dependent_launch_enabled() ? 2 : 1;
        const cudaError_t ce = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, STAGES>, ma, mb, G);
        return ce != cudaSuccess ? (int)ce : tl_launch_status();
    }
    return launch_after_wait(gemm_tc_kernel<BN, STAGES>, grid, dim3(THREADS), SMEM, stream, ma, mb, G);
}

}  // namespace

// y[T, N] = x[T, K] w[N, K]^T.  swap = 1 puts w on the 128-row side (few tokens), swap = 0 puts x there.
// bn: columns of the other side per tile (16, 32, 64, 128 or 256).  splits > 1 needs `partial`
// (splits * T * N floats); with `counters` (n_counters zeroed ints, at least one per tile, left zeroed) the
// last block of a tile sums the partials inside the same launch, else a second kernel does.  `status` (device int, zero before
// the call) receives a non-zero code if a wait inside the kernel ran out.  `gated` (swap = 1, one split, N % 128 == 0, bfloat16 out):
// w holds gate and up rows interleaved in blocks of 64 and y [T, N / 2] receives silu(gate) * up.  `cluster_reduce` (swap = 1,
// 2..8 ranges): the ranges of a tile are a thread-block cluster and sum their tiles through distributed shared memory.
namespace {
// The two fusions with the layer's norms (see GemmArgs).  All null / zero: the plain product.
struct NormFusion {
    float* res_x; int res_ld; float* ssq_out;                                      // the residual add, in the epilogue
    const float* nx; const float* nssq; int nparts; const void* nw; int nw_f32; float neps;   // the norm, in the B operand
};

int gemm_impl(const void* x, const void* w, void* y, int out_f32, int ldo, int T, int N, int K, int swap,
              int bn, int splits, float* partial, int* status, int* counters, int n_counters,
              int gated, int cluster_reduce, const NormFusion& F, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    const bool made_b = F.nx != nullptr, adds = F.res_x != nullptr;
    if (made_b && (!swap || bn > 64 || F.nssq == nullptr || F.nw == nullptr || F.nparts < 1 || ((uintptr_t)F.nx & 15) || ((uintptr_t)F.nw & 15))) return 1;
    if (adds && (!swap || !cluster_reduce || F.ssq_out == nullptr || (N & 3) || (F.res_ld & 3) || ((uintptr_t)F.res_x & 15))) return 1;
    if (K <= 0 || (K & 7) || (!made_b && ((uintptr_t)x & 15)) || ((uintptr_t)w & 15)) return 1;      // TMA: 16-byte rows and bases
    if (splits < 1 || (splits > 1 && partial == nullptr && !cluster_reduce)) return 1;
    int e = get_encode();
    if (e) return e;
    const void* a = swap ? w : x;
    const void* b = swap ? x : w;
    const int RA = swap ? N : T, RB = swap ? T : N;
    CUtensorMap ma, mb;
    if ((e = cached_map(&ma, a, RA, K, BM))) return e;
    if (made_b) {                                                                        // the float stream: boxes of [bn rows, 64 floats]
        if ((e = cached_map(&mb, F.nx, RB, K, -bn))) return e;
    } else if ((e = cached_map(&mb, b, RB, K, bn))) return e;
    const int k_tiles = (K + BK - 1) / BK;
    if (splits > k_tiles) splits = k_tiles;
    const int per = (k_tiles + splits - 1) / splits;
    splits = (k_tiles + per - 1) / per;                                                  // no empty split
    if (y == nullptr && splits < 2) return 1;
    if (gated && (!swap || splits != 1 || out_f32 || (N & 127) || y == nullptr)) return 1;   // whole 64 + 64 tiles, one split
    GemmArgs G{};
    G.gated = gated;
    G.cluster_reduce = (cluster_reduce && splits >= 2) ? 1 : 0;
    if (cluster_reduce && (!swap || splits > 8 || (y == nullptr && !adds))) return 1;
    if (adds && !G.cluster_reduce) return 1;                                             // the caller's plan must give 2..8 ranges
    G.res_x = F.res_x; G.res_ld = F.res_ld; G.ssq_out = F.ssq_out;
    G.nx = F.nx; G.nssq = F.nssq; G.nparts = F.nparts; G.nw = F.nw; G.nw_f32 = F.nw_f32; G.neps = F.neps;
    G.out = y; G.partial = partial; G.ldo = ldo; G.RA = RA; G.RB = RB; G.K = K;
    G.k_tiles_per_split = per; G.swap = swap; G.out_f32 = out_f32; G.status = status;
    G.wait_cycles = g_wait_cycles; G.drop_last_load = g_drop_last_load;
    dim3 grid((RA + BM - 1) / BM, (RB + bn - 1) / bn, splits);
    if (grid.y > 65535 || grid.z > 65535) return 1;
    G.trace = g_trace.take(grid.x * grid.y * grid.z);
    G.counters = (splits > 1 && counters != nullptr && (long long)grid.x * grid.y <= n_counters) ? counters : nullptr;
    switch (bn) {
        case 16:  e = launch<16, 5>(ma, mb, G, grid, stream); break;
        case 32:  e = launch<32, 5>(ma, mb, G, grid, stream); break;
        case 64:  e = launch<64, 4>(ma, mb, G, grid, stream); break;
        case 128: e = launch<128, 6>(ma, mb, G, grid, stream); break;
        case 256: e = launch<256, 4>(ma, mb, G, grid, stream); break;
        default: return 1;
    }
    if (e || splits == 1 || G.counters != nullptr || y == nullptr || G.cluster_reduce) return e;      // y null: the caller sums the pieces
    const size_t total = (size_t)T * N;
    const size_t cap = (size_t)tl_num_sms() * 8;
    const int blocks = (int)((total + 255) / 256 < cap ? (total + 255) / 256 : cap);
    return launch_after_wait(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream, (const float*)partial, (void*)y, out_f32, splits, T, N, ldo);
}
}  // namespace

TL_EXPORT int tl_gemm_tc(const void* x, const void* w, void* y, int out_f32, int ldo, int T, int N, int K, int swap,
                         int bn, int splits, float* partial, int* status, int* counters, int n_counters,
                         int gated, int cluster_reduce, cudaStream_t stream) {
    return gemm_impl(x, w, y, out_f32, ldo, T, N, K, swap, bn, splits, partial, status, counters, n_counters, gated, cluster_reduce,
                     NormFusion{}, stream);
}

// The product with the layer's norms folded in (few-token order only).
//   res_x, res_ld, ssq_out: y is not stored; its values, rounded to bfloat16, are added into the float residual stream res_x
//     [T, res_ld] in place, and ssq_out [T, ceil(N / 128)] receives the sums of squares of the new values per (token, tile of
//     128 features).  Needs 2..8 K ranges summed inside a cluster (`cluster_reduce`), N % 4 == 0.
//   nx, nssq, nparts, nw, nw_f32, neps: x is not read; the activations are rms_norm(nx[row]) * nw, made on the fly from the
//     float residual stream nx [T, K], with the row's sum of squares taken from its nparts partial sums nssq [T, nparts].
TL_EXPORT int tl_gemm_tc_normed(const void* x, const void* w, void* y, int out_f32, int ldo, int T, int N, int K, int swap,
                                int bn, int splits, float* partial, int* status, int* counters, int n_counters,
                                int gated, int cluster_reduce, float* res_x, int res_ld, float* ssq_out,
                                const float* nx, const float* nssq, int nparts, const void* nw, int nw_f32, float neps,
                                cudaStream_t stream) {
    NormFusion F{res_x, res_ld, ssq_out, nx, nssq, nparts, nw, nw_f32, neps};
    return gemm_impl(x, w, y, out_f32, ldo, T, N, K, swap, bn, splits, partial, status, counters, n_counters, gated, cluster_reduce,
                     F, stream);
}

// Tracing build: the products launched from now on leave their stamps in buf [slots][512][8] (device, zeroed by the caller),
// one slot a launch, starting at slot `first`; null: no more stamps.  Returns the next free slot.  In the ordinary build
// the call is accepted and nothing is recorded.
TL_EXPORT int tl_trace_set(long long* buf, int slots, int first) {
    g_trace.buf = buf; g_trace.slots = slots; g_trace.next = first;
    return g_trace.next;
}
TL_EXPORT int tl_trace_next() { return g_trace.next; }
TL_EXPORT int tl_trace_build() { return TL_TRACING; }

// For tests of the failure path only.  `wait_cycles` > 0: how many clock cycles a wait on a barrier may take from
// now on (0: back to the default of about two seconds).  `drop_last_load` = 1: the copy thread of every block leaves
// out its last stage of operands, so the MMA thread's bounded wait for it runs out, the block records status 2,
// frees its tensor memory and returns with invalid output; nothing is left in flight.  Never set in serving.
TL_EXPORT void tl_gemm_tc_test_hooks(long long wait_cycles, int drop_last_load) {
    g_wait_cycles = wait_cycles > 0 ? wait_cycles : WAIT_CYCLES;
    g_drop_last_load = drop_last_load ? 1 : 0;
}

// out[T, ldo] = the sum of the S pieces partial[S][T][N] in split order, converted.
TL_EXPORT int tl_splitk_reduce(const float* partial, void* y, int out_f32, int splits, int T, int N, int ldo,
                               cudaStream_t stream) {
    const size_t total = (size_t)T * N;
    if (total == 0) return 0;
    const size_t cap = (size_t)tl_num_sms() * 8;
    const int blocks = (int)((total + 255) / 256 < cap ? (total + 255) / 256 : cap);
    return launch_after_wait(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream, partial, y, out_f32, splits, T, N, ldo);
}
