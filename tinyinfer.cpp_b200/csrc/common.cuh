// Shared helpers of the sm_100a kernels: dtype codes, conversions, reductions and the
// error convention of the C entry points.
//
// Every entry point is `extern "C" int ti_<name>(..., void* stream)`.  It returns 0 on
// success.  A refused argument (a size the kernel does not take) or a CUDA launch error
// returns non-zero and leaves a message that `ti_last_error()` hands out; nothing is
// launched after a refusal, so a wrong size never gives a wrong result.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TI_F32 0
#define TI_BF16 1

typedef __nv_bfloat16 bf16;

extern "C" const char* ti_last_error();
int ti_fail(const char* fmt, ...);                 // records the message, returns 1
int ti_check_launch(const char* what);             // cudaGetLastError -> 0 or ti_fail

// Attributes of a kernel (its dynamic shared memory limit) belong to a device's context, so they
// are set once per device that launches it.  `TiPerDevice seen;` as a function-local static:
// `seen.first_use()` is true when the current device has not passed here before.
struct TiPerDevice {
    bool done[64] = {};
    bool first_use();          // true also when the device cannot be told (then set it again)
    void mark();
};

#define TI_REQUIRE(cond, ...)            \
    do {                                 \
        if (!(cond)) return ti_fail(__VA_ARGS__); \
    } while (0)

// Programmatic dependent launch.  A kernel launched through ti_launch_pdl may start while the
// kernel before it in the stream is still running; it must call pdl_wait() before it reads
// anything that kernel wrote (what it does before that, such as fetching weights, overlaps
// with the predecessor).  pdl_launch() lets the next kernel's blocks be scheduled early.
// What the kernel before produced must not reach this kernel through a `const T* __restrict__`
// parameter: loads from such a parameter count as loads of memory that never changes, and the
// compiler may move them in front of the wait (it did, in the few-rows product, once its loads
// of the activations stood directly behind the wait).  Weights and the step's host-written
// integers may keep the qualifier; activations, partial results and outputs of the chain do not.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::); }

template <typename... KArgs, typename... Args>
cudaError_t ti_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
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
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds
// 32 floats of shared memory and may be reused after the call returns.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();                       // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float r = lane < nwarps ? scratch[lane] : 0.0f;
    return warp_sum(r);
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float r = lane < nwarps ? scratch[lane] : -INFINITY;
    return warp_max(r);
}
