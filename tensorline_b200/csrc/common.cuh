// Shared device helpers of the hand-written kernels (sm_100a).
//
// Activation type T is float (the true 32-bit engine) or __nv_bfloat16 (the serving engine);
// the residual stream, every reduction, softmax, norm statistics, rotary angles and silu are
// float in both.  Files are compiled WITHOUT fast-math so that expf, sincosf, division and
// rsqrt/sqrt are the accurate library versions.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

typedef __nv_bfloat16 bf16;

// dtype codes of the C interface
#define TL_F32 0
#define TL_BF16 1

#define TL_EXPORT extern "C" __attribute__((visibility("default")))

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `red` is 33 floats
// of shared memory.  The order of additions depends only on blockDim, so a row's result does
// not depend on how many rows the launch has.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                       // protect `red` from a previous use
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

static inline int tl_launch_status() { return (int)cudaGetLastError(); }

// Host-side state that belongs to a device (kernel attributes that were set, addresses that were looked up) is
// kept per device index, so a process that uses several GPUs sets each of them up.
constexpr int TL_MAX_DEVICES = 64;
static inline int tl_device_index() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= TL_MAX_DEVICES) return -1;
    return dev;
}
// Streaming multiprocessors of the current device, asked once per device.
static inline int tl_num_sms() {
    static int count[TL_MAX_DEVICES] = {};
    const int dev = tl_device_index();
    if (dev < 0) return 1;
    if (count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 1;
        count[dev] = n;
    }
    return count[dev];
}

// The checking build (-DTL_CHECK=1) stands in for a memory checker: every kernel that indexes the block tables
// or the pages checks the request slot against the table's rows, the page index against the table's width and
// the page number against the pool, with the limits its launcher was given.  On a violation it records
// (code 100, kernel, value, limit) in the four ints at `fault`, and reads or writes the sink page / the padding
// row instead: nothing outside the tensors is touched, no trap, no assert.  Without the define the checks
// compile to nothing.
struct TlLimits {
    int table_rows;      // rows of the block table (request slots + the padding row); 0: unknown, not checked
    int total_pages;     // first dimension of the page tensors (pool + the sink page); 0: unknown, not checked
    int* fault;          // four device ints; null: not recorded
};
#ifdef TL_CHECK
#define TL_CHECKING 1
#else
#define TL_CHECKING 0
#endif
enum { TL_K_ROPE = 1, TL_K_TOKENWISE = 2, TL_K_PREFILL = 3, TL_K_DECODE = 4, TL_K_DECODE_TMA = 5, TL_K_TC_PREFILL = 6,
       TL_K_TC2_PREFILL = 7 };
// `v` if 0 <= v < limit (or nothing is known or checked), else limit - 1 after recording the violation.
__device__ __forceinline__ int tl_checked(int v, int limit, const TlLimits& L, int kernel) {
#if TL_CHECKING
    if (limit > 0 && (v < 0 || v >= limit)) {
        if (L.fault && atomicCAS(L.fault, 0, 100) == 0) { L.fault[1] = kernel; L.fault[2] = v; L.fault[3] = limit; }
        return limit - 1;
    }
#endif
    return v;
}
TL_EXPORT int tl_check_build();

// The tracing build (-DTL_TRACE=1): the kernels that wait on the kernel in front of them (the few-token product, the TMA
// decode attention) leave global-timer stamps, eight a block, in a buffer the host names: when the block started, when
// its dependency wait returned, when its first and its last operand tile had landed, when it ended, and three places of
// its own.  From them the host draws the time line of a captured step: how long each kernel's stream of operands lasts
// and how long nothing streams between two kernels.  Without the define a stamp compiles to nothing; the record travels
// in the kernels' arguments either way, so both builds have the same interface.
struct TlTrace {
    long long* buf;      // [slots][TL_TRACE_BLOCKS][8] nanoseconds; null: not recorded
    int slot;            // this launch's slot
};
constexpr int TL_TRACE_BLOCKS = 512;                       // launches of more blocks are not recorded
#ifdef TL_TRACE
#define TL_TRACING 1
#else
#define TL_TRACING 0
#endif
__device__ __forceinline__ void tl_stamp(const TlTrace& T, int i) {
#if TL_TRACING
    if (T.buf) {
        const unsigned block = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        T.buf[((size_t)T.slot * TL_TRACE_BLOCKS + block) * 8 + i] = (long long)t;
    }
#endif
}
// Host side of a library that traces: where the stamps go and which slot the next launch takes.
struct TlTraceHost {
    long long* buf = nullptr; int next = 0, slots = 0;
    TlTrace take(unsigned blocks) {
        TlTrace t{nullptr, 0};
        if (TL_TRACING && buf && next < slots && blocks <= (unsigned)TL_TRACE_BLOCKS) { t.buf = buf; t.slot = next++; }
        return t;
    }
};

// silu(g) * u in the bfloat16 engine (g and u hold bfloat16 values): float32 arithmetic with the division that has no
// special-case branch, so the chains of neighbouring elements overlap (an epilogue of 16 tokens took 2,600 cycles with
// the exact division, 1,500 with this one).  Every bfloat16 path of the activation calls this function and so gives the
// same bits; the 32-bit engine divides exactly.
__device__ __forceinline__ float tl_silu_mul(float g, float u) { return __fdividef(g, 1.0f + expf(-g)) * u; }

// Programmatic dependent launch.  A kernel launched with launch_after_wait() may be placed on the SMs while
// the kernel before it in the stream is still running; its blocks run their set-up and then stop in
// grid_dependency_wait() until that kernel has finished and its writes are visible.  Every kernel launched
// this way calls grid_dependency_wait() before its first access to global memory that another kernel writes
// or reads, and grid_dependency_trigger() right after, which lets the kernel after it be placed in turn (one
// kernel ahead at most).  After a kernel that never triggers (a library's), the wait is an ordinary stream
// dependency.  TENSORLINE_B200_PDL=0 launches everything the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool tl_dependent_launch_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("TENSORLINE_B200_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
static inline int launch_after_wait(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tl_dependent_launch_enabled() ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
