// Shared device helpers for the sm_100a kernels of this package.
//
// Conventions used by every kernel file:
//  * the residual stream is float; "activation" tensors are T = float (the true
//    32-bit path) or __nv_bfloat16 (the serving path); all arithmetic that the
//    exactness rules name (softmax, norms, rotation angles, the residual sum)
//    is done in float, with one rounding to T when a value is stored;
//  * small parameter vectors (norm weights, biases, conv taps) are always float;
//  * every exported function is extern "C", takes raw device pointers and a
//    cudaStream_t, validates its sizes on the host, and returns 0 or a negative
//    error code after recording a message that vapi_last_error() returns.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <stdlib.h>

#define VAPI_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side
#define VAPI_F32 0
#define VAPI_BF16 1

namespace vapi {

// ---- error reporting (host) ------------------------------------------------
inline char* error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}
inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}
inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(-100, "%s: launch failed: %s", what, cudaGetErrorString(e));
    return 0;
}

// Multiprocessors of the current device, asked of the device once per device (host).
inline int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
        cached[dev] = n;
    }
    return cached[dev];
}

// ---- programmatic dependent launch --------------------------------------------------
// Kernels of a step are launched so that the next one may begin while the one before it
// drains: a kernel first does what does not depend on its predecessor (index arithmetic,
// streaming in weights), then calls pdl_wait(), which returns once every earlier kernel has
// completed and its writes are visible.  pdl_trigger() lets the following kernel be scheduled
// as soon as all blocks of this one have started.  Both are no-ops for a kernel launched the
// ordinary way.  Set VAPI_PDL=0 to launch everything the ordinary way.
#ifndef VAPI_TRACE
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#else
// A build with -DVAPI_TRACE (a measuring build, never the serving one) stamps the device's clock when
// the first thread of a kernel's first block starts and when its dependency wait returns, into a
// buffer that vapi_trace_set() names: what a step's kernels do inside a captured graph, where no
// profiler looks.  Two words a stamp: nanoseconds, then kind | library << 4 | threads << 8 | blocks << 24.
__device__ unsigned long long* g_trace_buf;
__device__ unsigned* g_trace_count;
__device__ unsigned g_trace_capacity;
__device__ int g_trace_library;
__device__ __forceinline__ void trace_stamp(int kind) {
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && g_trace_buf) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        const unsigned i = atomicAdd(g_trace_count, 1u);
        if (i < g_trace_capacity) {
            g_trace_buf[2 * (size_t)i] = t;
            g_trace_buf[2 * (size_t)i + 1] = (unsigned long long)kind | ((unsigned long long)g_trace_library << 4) |
                                             ((unsigned long long)blockDim.x << 8) |
                                             ((unsigned long long)gridDim.x * gridDim.y * gridDim.z << 24);
        }
    }
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); trace_stamp(1); }
__device__ __forceinline__ void pdl_trigger() { trace_stamp(0); asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("VAPI_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
inline int check_launch(const char* what, cudaError_t e) {
    if (e != cudaSuccess) return fail(-100, "%s: launch failed: %s", what, cudaGetErrorString(e));
    return check_launch(what);
}

// ---- element conversion ------------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}
// round a float to T's precision and come back (what a store followed by a load gives)
template <typename T> __device__ __forceinline__ float round_to(float v) {
    return to_f32(from_f32<T>(v));
}

// ---- warp / block reductions -----------------------------------------------
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
// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` is 33 floats of shared memory.  The order of the additions depends
// only on blockDim, never on the data or on the rest of the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

}  // namespace vapi

#ifdef VAPI_TRACE
// buffer of 2 * capacity 64-bit words and a 32-bit counter, both in device memory; null switches the stamps off
VAPI_EXPORT int vapi_trace_set(unsigned long long* buf, unsigned* count, unsigned capacity, int library) {
    cudaError_t e = cudaMemcpyToSymbol(vapi::g_trace_count, &count, sizeof(count));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(vapi::g_trace_capacity, &capacity, sizeof(capacity));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(vapi::g_trace_library, &library, sizeof(library));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(vapi::g_trace_buf, &buf, sizeof(buf));
    return e == cudaSuccess ? 0 : vapi::fail(-100, "trace_set: %s", cudaGetErrorString(e));
}
#endif
