// bfloat16 matrix product for steps of many tokens: tcgen05.mma with cta_group::2, persistent blocks.
//
//     y[t, n] = sum_k x[t, k] * w[n, k]          x: [T, K], w: [N, K], both row-major (K-major), bfloat16
//
// Two thread blocks on neighbouring SMs (a cluster of two) work on one 256 x 256 output tile.  Each block
// brings its own 128 rows of x and its own 128 rows of w to its shared memory by TMA (plain loads, no
// multicast; the `cta_group::2` form lets their bytes count on the leader block's barrier); one thread of the
// leader block issues `tcgen05.mma.cta_group::2` instructions of 256 x 256 x 16, which read both blocks'
// shared memory and leave 128 x 256 float accumulators in each block's tensor memory.  A block's 128 x 64
// tile of x and of w is read from shared memory once for 256 output columns and rows: half the shared-memory
// traffic per flop of the one-block kernel in gemm_tc.cu, which that kernel is bound by at these shapes.
//
// The pairs are persistent: a pair takes tiles pair, pair + pairs, ... in an order that keeps the x rows and
// the w rows of the tiles in flight inside the L2.  The accumulator is double-buffered in tensor memory
// (2 x 256 of the 512 columns), so the four epilogue warps of each block read, convert and store tile i while
// the MMA thread already runs tile i + 1.  Two epilogues:
//   * plain: y[t, n] in bfloat16 or float;
//   * gated: w holds gate and up rows interleaved in blocks of 64 (rows 128 j .. 128 j + 63 the gate features
//     64 j .., rows 128 j + 64 .. the up features of the same columns); y[t, 64 j + c] = silu(gate) * up, both
//     rounded to bfloat16 first (what a stored gate|up product would hold), y is [T, N / 2] bfloat16.
// Every wait on a barrier is bounded; a block whose wait runs out records a code in `status`, stops, and meets
// its peer at the cluster barrier before the tensor memory is freed.
#include "common.cuh"
#include <cuda.h>
#include <mutex>
#include <unordered_map>

namespace {

constexpr int BM = 128;                // rows of x per block (a pair: 256)
constexpr int BN = 256;                // rows of w per pair (a block loads 128 of them)
constexpr int BK = 64;                 // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int THREADS = 192;           // warp 0: TMA, warp 1: tensor memory + MMA, warps 2..5: epilogue
constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr uint32_t TMEM_COLS = 512;    // two accumulators of 256 columns
constexpr long long WAIT_CYCLES = 4000000000LL;     // ~2 s

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
// The shared::cluster address of the same shared-memory location in block `rank` of this cluster.
__device__ __forceinline__ uint32_t peer_addr(uint32_t local, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(local), "r"(rank));
    return out;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_address) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_address) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false (and `code` recorded) if the barrier did not flip in time or another role of the block gave up.
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
// A 2-D tile by TMA into this block's shared memory; its bytes count on `bar`, which may be the peer's barrier.
__device__ __forceinline__ void tma_load_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_address, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar_cluster_address), "r"(c0), "r"(c1) : "memory");
}
// K-major tile, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// When the MMAs issued so far are done, arrive on the barrier at this address in both blocks of the pair.
__device__ __forceinline__ void umma_commit_both(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_addr(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}

struct Gemm2Args {
    void* out;             // [T, ldo] bf16 or float; gated: [T, N / 2] bf16
    int ldo;
    int T, N, K;
    int m_tiles, n_tiles;  // tiles of 256 rows and 256 columns
    int out_f32, gated;
    int* status;
};

__device__ __forceinline__ void store16_bf16(bf16* dst, const float (&v)[16], int valid) {
    if (valid >= 16 && ((((uintptr_t)dst) & 15) == 0)) {
        uint4 a, b;
        uint32_t* pa = reinterpret_cast<uint32_t*>(&a);
        uint32_t* pb = reinterpret_cast<uint32_t*>(&b);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
            __nv_bfloat162 hi = __floats2bfloat162_rn(v[8 + 2 * j], v[8 + 2 * j + 1]);
            pa[j] = *reinterpret_cast<uint32_t*>(&lo);
            pb[j] = *reinterpret_cast<uint32_t*>(&hi);
        }
        reinterpret_cast<uint4*>(dst)[0] = a;
        reinterpret_cast<uint4*>(dst)[1] = b;
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) if (j < valid) dst[j] = __float2bfloat16_rn(v[j]);
    }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const Gemm2Args G) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);   // leader's: both blocks' bytes of a stage
    uint64_t* empty_bar = full_bar + STAGES;          // in each block: the MMAs that read the stage are done
    uint64_t* acc_full = empty_bar + STAGES;          // [2] in each block: the accumulator is complete
    uint64_t* acc_empty = acc_full + 2;               // [2] leader's: the epilogue warps of both blocks have read it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();             // 0: the leader, which issues the MMAs
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int k_tiles = (G.K + BK - 1) / BK;
    const int total_tiles = G.m_tiles * G.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar + s, 1); mbar_init(empty_bar + s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full + b, 1); mbar_init(acc_empty + b, 8); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                                  // one warp of each block allocates the pair's columns
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync();                                   // both blocks' barriers exist before anyone signals them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------------- TMA producer (both blocks)
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        int it = 0;
        bool ok = true;
        for (int tile = pair; tile < total_tiles && ok; tile += pairs) {
            const int tm = tile % G.m_tiles, tn = tile / G.m_tiles;
            const int row_x = tm * 2 * BM + (int)rank * BM, row_w = tn * BN + (int)rank * (BN / 2);
            for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES && !mbar_wait(empty_bar + s, ((it / STAGES) - 1) & 1, abort_flag, G.status, 31)) { ok = false; break; }
                if (rank == 0) mbar_expect_tx(full_bar + s, 2 * STAGE_BYTES);
                const uint32_t bar = peer_addr(smem_addr(full_bar + s), 0);
                const uint32_t st = smem_addr(tiles + s * STAGE_BYTES);
                tma_load_pair(st, &map_x, bar, kt * BK, row_x);
                tma_load_pair(st + A_BYTES, &map_w, bar, kt * BK, row_w);
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---------------------------------------------------------------- MMA issuer (leader block)
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
        int it = 0, ti = 0;
        bool ok = true;
        for (int tile = pair; tile < total_tiles && ok; tile += pairs, ++ti) {
            const int buf = ti & 1;
            if (ti >= 2 && !mbar_wait(acc_empty + buf, ((ti >> 1) - 1) & 1, abort_flag, G.status, 32)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
            for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(full_bar + s, (it / STAGES) & 1, abort_flag, G.status, 33)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_addr(tiles + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    umma_pair(acc, smem_desc(a_addr + k * UMMA_K * 2), smem_desc(b_addr + k * UMMA_K * 2), idesc, (kt > 0 || k > 0) ? 1u : 0u);
                umma_commit_both(empty_bar + s);      // both blocks may refill the stage once these MMAs have read it
            }
            if (ok) umma_commit_both(acc_full + buf);
        }
    } else if (warp >= 2) {
        // ---------------------------------------------------------------- epilogue: 4 warps of each block, 32 lanes of tensor memory each
        const int quarter = warp & 3;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t leader_acc_empty = peer_addr(smem_addr(acc_empty), 0);
        int ti = 0;
        for (int tile = pair; tile < total_tiles; tile += pairs, ++ti) {
            const int buf = ti & 1;
            if (!mbar_wait(acc_full + buf, (ti >> 1) & 1, abort_flag, G.status, 34)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int tm = tile % G.m_tiles, tn = tile / G.m_tiles;
            const int t = tm * 2 * BM + (int)rank * BM + quarter * 32 + lane;      // token = row of x = TMEM lane
            const int n0 = tn * BN;
            const uint32_t taddr = lane_base + (uint32_t)(buf * BN);
            if (G.gated) {
                // columns [128 j, 128 j + 64) of the tile are gate features, the 64 after them the up features
#pragma unroll 1
                for (int half = 0; half < 2; ++half) {
#pragma unroll 1
                    for (int c = 0; c < 64; c += 16) {
                        uint32_t rg[16], ru[16];
                        tmem_ld16(taddr + half * 128 + c, rg);
                        tmem_ld16(taddr + half * 128 + 64 + c, ru);
                        tmem_ld_wait();
                        const int col = (n0 >> 1) + half * 64 + c;                   // feature of the output
                        if (t < G.T && col < (G.N >> 1)) {
                            float v[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(rg[j])));
                                const float u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(ru[j])));
                                v[j] = tl_silu_mul(g, u);
                            }
                            store16_bf16((bf16*)G.out + (size_t)t * G.ldo + col, v, (G.N >> 1) - col);
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r0[16], r1[16];
                    tmem_ld16(taddr + c, r0);
                    tmem_ld16(taddr + c + 16, r1);
                    tmem_ld_wait();
                    if (t < G.T) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int col = n0 + c + 16 * h;
                            if (col >= G.N) break;
                            const uint32_t (&r)[16] = h ? r1 : r0;
                            if (G.out_f32) {
                                float* dst = (float*)G.out + (size_t)t * G.ldo + col;
#pragma unroll
                                for (int j = 0; j < 16; ++j) if (col + j < G.N) dst[j] = __uint_as_float(r[j]);
                            } else {
                                float v[16];
#pragma unroll
                                for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
                                store16_bf16((bf16*)G.out + (size_t)t * G.ldo + col, v, G.N - col);
                            }
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(leader_acc_empty + (uint32_t)(buf * 8));   // this warp is done with the buffer
        }
    }
    // ---------------------------------------------------------------- teardown
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {                                // give copies in flight time to land before the block's
        const long long t0 = clock64();               // shared memory is handed to another block
        while (clock64() - t0 < 2000000LL) { }
    }
    cluster_sync();                                   // the peer has read its accumulators and left its loops
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 101;
}

struct MapKey {
    const void* base; int rows, K;
    bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && K == o.K; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return reinterpret_cast<size_t>(k.base) * 0x9E3779B97F4A7C15ull ^ ((size_t)(unsigned)k.rows << 32 | (unsigned)k.K);
    }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;      // tensor maps by (matrix, shape): encoding one costs the host microseconds
std::mutex g_maps_lock;

int cached_map(CUtensorMap* map, const void* base, int rows, int K) {
    const MapKey key{base, rows, K};
    std::lock_guard<std::mutex> hold(g_maps_lock);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *map = it->second; return 0; }
    const int e = make_map(map, base, rows, K, BM);
    if (e) return e;
    if (g_maps.size() >= 8192) g_maps.clear();
    g_maps.emplace(key, *map);
    return 0;
}

}  // namespace

// y[T, N] = x[T, K] w[N, K]^T (bfloat16 operands; y bfloat16 or float, rows `ldo` elements apart).  `gated`: see the top of
// the file; y is then [T, N / 2] bfloat16 and N a multiple of 128.  `status`: device int, zero before the call; non-zero
// afterwards if a wait inside the kernel ran out.  `max_pairs`: pairs of blocks to launch at most (0: as many as the GPU
// holds).  Returns 0, a CUDA error code, or 1 for arguments it does not take.
TL_EXPORT int tl_gemm_tc2(const void* x, const void* w, void* y, int out_f32, int ldo, int T, int N, int K, int gated,
                          int* status, int max_pairs, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || y == nullptr || status == nullptr) return 1;
    if (gated && (out_f32 || (N & 127))) return 1;
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || fn == nullptr ||
            q != cudaDriverEntryPointSuccess) return 100;
        g_encode = (EncodeTiledFn)fn;
    }
    static bool attr_set[TL_MAX_DEVICES] = {};
    const int dev = tl_device_index();
    if (dev < 0) return 1;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_set[dev] = true;
    }
    CUtensorMap mx, mw;
    int e;
    if ((e = cached_map(&mx, x, T, K))) return e;
    if ((e = cached_map(&mw, w, N, K))) return e;
    Gemm2Args G{};
    G.out = y; G.ldo = ldo; G.T = T; G.N = N; G.K = K;
    G.m_tiles = (T + 2 * BM - 1) / (2 * BM); G.n_tiles = (N + BN - 1) / BN;
    G.out_f32 = out_f32; G.gated = gated; G.status = status;
    long long tiles = (long long)G.m_tiles * G.n_tiles;
    int pairs = tl_num_sms() / 2;
    if (max_pairs > 0 && max_pairs < pairs) pairs = max_pairs;
    if (tiles < pairs) pairs = (int)tiles;
    gemm_tc2_kernel<<<dim3(2 * pairs), dim3(THREADS), SMEM_BYTES, stream>>>(mx, mw, G);
    return tl_launch_status();
}
