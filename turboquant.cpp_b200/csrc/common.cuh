// Shared helpers of the sm_100a kernels: element types, reductions, error reporting.
//
// Every kernel file exports plain C launchers (extern "C", called through ctypes with raw
// device pointers and the caller's stream).  A launcher returns 0, or a negative code after
// storing a message that tq_last_error() of the same library returns; it never falls back to
// another implementation and never returns a result for sizes it cannot handle.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#define TQ_EXPORT extern "C" __attribute__((visibility("default")))

// element type codes shared with the Python side
#define TQ_F32 0
#define TQ_BF16 1

static thread_local char tq_error_message[512] = "";

#define TQ_FAIL(code, ...)                                                   \
    do {                                                                     \
        snprintf(tq_error_message, sizeof(tq_error_message), __VA_ARGS__);   \
        return (code);                                                       \
    } while (0)

#define TQ_REQUIRE(cond, ...)                                                \
    do {                                                                     \
        if (!(cond)) TQ_FAIL(-2, __VA_ARGS__);                               \
    } while (0)

#define TQ_CHECK_LAUNCH(name)                                                \
    do {                                                                     \
        cudaError_t e__ = cudaGetLastError();                                \
        if (e__ != cudaSuccess)                                              \
            TQ_FAIL(-1, "%s: launch failed: %s", name, cudaGetErrorString(e__)); \
    } while (0)

// ---------------------------------------------------------------------------------------
// Index checks of debug builds (-DTQ_DEBUG_INDEX; TQ_DEBUG_INDEX=1 in the environment builds and loads them).
// Kernels index memory with values they are handed: token ids, page ids from the page tables, expert ids, rows of
// the expert-sorted layout.  The host validates what it can before a launch; these checks are the net below that.
// TQ_CHECKED(value, limit, kind) is `value` in a release build.  In a debug build a value outside [0, limit) is
// recorded (the first one wins: kind, value, limit; every one is counted) and replaced by 0, so the access that
// follows goes to valid memory: nothing traps, the kernel runs to its end with a wrong result, and the host, which
// reads the record with tq_index_fault_read() where it reads results anyway, raises.
// ---------------------------------------------------------------------------------------
#define TQ_IDX_TOKEN 1          // a token id outside the vocabulary
#define TQ_IDX_PAGE 2           // a page id outside the cache (a page that was given back reads -1)
#define TQ_IDX_TABLE_COLUMN 3   // a position beyond the page table's width
#define TQ_IDX_SEQUENCE 4       // a token's sequence index outside the step's batch
#define TQ_IDX_EXPERT 5         // an expert id outside the layer's experts
#define TQ_IDX_ROW 6            // a row of the expert-sorted layout, or a gathered row, outside its tensor

#ifdef TQ_DEBUG_INDEX
static __device__ int tq_index_fault[4];      // kind (0: none), value, limit, how many
template <typename I, typename J>
__device__ __forceinline__ I tq_checked_index(I value, J limit, int kind) {
    if ((long long)value >= 0 && (long long)value < (long long)limit) return value;
    if (atomicCAS(&tq_index_fault[0], 0, kind) == 0) {
        tq_index_fault[1] = (int)value;
        tq_index_fault[2] = (int)limit;
    }
    atomicAdd(&tq_index_fault[3], 1);
    return (I)0;
}
#define TQ_CHECKED(value, limit, kind) tq_checked_index((value), (limit), (kind))
#define TQ_DEFINE_INDEX_FAULT_READ                                                                        \
    TQ_EXPORT int tq_index_fault_read(int* out4) {                                                         \
        int zero[4] = {0, 0, 0, 0};                                                                        \
        cudaError_t e = cudaMemcpyFromSymbol(out4, tq_index_fault, sizeof(zero));                          \
        if (e == cudaSuccess && out4[0] != 0) e = cudaMemcpyToSymbol(tq_index_fault, zero, sizeof(zero));  \
        if (e != cudaSuccess) TQ_FAIL(-1, "index fault record: %s", cudaGetErrorString(e));                \
        return 1;                                                                                          \
    }
#else
#define TQ_CHECKED(value, limit, kind) (value)
// a release build keeps no record: 0 tells the caller so
#define TQ_DEFINE_INDEX_FAULT_READ                                                                        \
    TQ_EXPORT int tq_index_fault_read(int* out4) { out4[0] = out4[1] = out4[2] = out4[3] = 0; return 0; }
#endif

#define TQ_DEFINE_LAST_ERROR                                                 \
    TQ_EXPORT const char* tq_last_error() { return tq_error_message; }      \
    TQ_DEFINE_INDEX_FAULT_READ

__device__ __forceinline__ float tq_to_float(float v) { return v; }
__device__ __forceinline__ float tq_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T tq_from_float(float v);
template <> __device__ __forceinline__ float tq_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 tq_from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float tq_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float tq_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float tq_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = tq_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = tq_warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float tq_block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = tq_warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = tq_warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch.  Kernels are launched so that their CTAs may become resident
// while the previous kernel of the stream is still running; every kernel calls tq_grid_wait()
// before it touches global memory (it returns once the previous kernel has completed and its
// writes are visible) and tq_grid_launch_dependents() once it holds the resources it needs, so
// the next kernel's CTAs can move in as SMs free up.  This removes most of the launch gap between
// the many small kernels of a decode step, inside CUDA graphs too.  TQ_NO_PDL=1 switches it off.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tq_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// A pointer for use after a tq_grid_wait() that is not the kernel's first statement.  The compiler takes data behind
// a `const T* __restrict__` parameter to be read-only for the whole kernel and may move loads of it above the wait's
// inline assembly, i.e. before the kernel ahead has written it; the value returned here is opaque to it, and its
// definition (a volatile statement of its own) stays behind the wait, so loads through it do too.
template <typename T> __device__ __forceinline__ T* tq_fresh(T* p) {
    asm volatile("" : "+l"(p) : : "memory");
    return p;
}
__device__ __forceinline__ void tq_grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

struct TqLaunch {
    dim3 grid, block;
    size_t smem;
    cudaStream_t stream;
    unsigned cluster;          // CTAs per cluster along x (1: no clusters)
    void config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr) const {
        static const bool pdl = [] { const char* e = getenv("TQ_NO_PDL"); return !(e && e[0] && e[0] != '0'); }();
        cfg = cudaLaunchConfig_t{};
        cfg.gridDim = grid;
        cfg.blockDim = block;
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        unsigned n = 0;
        if (pdl) {
            attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[n].val.programmaticStreamSerializationAllowed = 1;
            ++n;
        }
        if (cluster > 1) {
            attr[n].id = cudaLaunchAttributeClusterDimension;
            attr[n].val.clusterDim.x = cluster;
            attr[n].val.clusterDim.y = 1;
            attr[n].val.clusterDim.z = 1;
            ++n;
        }
        cfg.attrs = attr;
        cfg.numAttrs = n;
    }
    template <typename... KArgs, typename... Args>
    void operator()(void (*kernel)(KArgs...), Args&&... args) const {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[2];
        config(cfg, attr);
        cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);      // errors surface in TQ_CHECK_LAUNCH
    }
};
inline TqLaunch tq_launch(dim3 grid, dim3 block, size_t smem, cudaStream_t stream, unsigned cluster = 1) {
    return TqLaunch{grid, block, smem, stream, cluster};
}

// Dispatch on an element type code: TQ_F32 -> float, TQ_BF16 -> __nv_bfloat16.
#define TQ_DISPATCH(code, T, ...)                                            \
    do {                                                                     \
        if ((code) == TQ_F32) { using T = float; __VA_ARGS__; }              \
        else if ((code) == TQ_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else TQ_FAIL(-2, "unknown element type code %d", (int)(code));       \
    } while (0)
