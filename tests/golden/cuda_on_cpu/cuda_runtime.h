// A stand-in for <cuda_runtime.h> that lets CUDA C++ kernels run on the host.
//
// The reference (beyondHJM/tinyinfer.cpp) keeps all of its model arithmetic in CUDA kernels, and
// every weight path goes through cudaMalloc, so its code cannot run without a GPU as it stands.
// This header and simt.cpp give its sources what they ask of CUDA, on the CPU: a kernel launch
// runs the grid's blocks one after the other, the threads of a block as host threads that meet
// at __syncthreads(), exchange registers in warp shuffles and share `__shared__` variables; the
// runtime calls the sources make (cudaMalloc, cudaMemcpy, ...) work on host memory.  Launches
// `kernel<<<grid, block, smem, stream>>>(args)` are rewritten by make_golden.py into
// `CPU_LAUNCH(kernel, grid, block, args)` before compiling, and the body of the reference's one
// inline-PTX function (mma.sync m16n8k16) is replaced by `cpu_mma_m16n8k16_bf16`.
//
// It is test infrastructure: only tests/golden/make_golden.py compiles it.
#pragma once

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <functional>

#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
#define __launch_bounds__(...)
#define __shared__ static
#define __align__(n) __attribute__((aligned(n)))
#define __grid_constant__

struct uint3 { unsigned x, y, z; };
struct dim3 {
    unsigned x, y, z;
    dim3(unsigned x_ = 1, unsigned y_ = 1, unsigned z_ = 1) : x(x_), y(y_), z(z_) {}
};
struct alignas(16) uint4 { unsigned x, y, z, w; };
struct alignas(16) float4 { float x, y, z, w; };
struct alignas(8) float2 { float x, y; };
static inline float4 make_float4(float x, float y, float z, float w) { return float4{x, y, z, w}; }
static inline uint4 make_uint4(unsigned x, unsigned y, unsigned z, unsigned w) { return uint4{x, y, z, w}; }

extern thread_local uint3 threadIdx;
extern thread_local uint3 blockIdx;
extern thread_local dim3 blockDim;
extern thread_local dim3 gridDim;

// ---- what kernels call -------------------------------------------------------------------------
void __syncthreads();
unsigned long long cpu_shfl(unsigned mask, unsigned long long bits, int src_lane);
template <typename T> static inline T cpu_shfl_t(unsigned mask, T v, int src) {
    static_assert(sizeof(T) <= 8, "shuffle of a wide type");
    unsigned long long bits = 0;
    std::memcpy(&bits, &v, sizeof(T));
    bits = cpu_shfl(mask, bits, src);
    T out;
    std::memcpy(&out, &bits, sizeof(T));
    return out;
}
int cpu_lane_id();
// The value of lane `lane + delta` (own value when that lane lies outside the `width`-wide group).
template <typename T> static inline T __shfl_down_sync(unsigned mask, T v, int delta, int width = 32) {
    const int lane = cpu_lane_id();
    const int src = (lane % width) + delta < width ? lane + delta : lane;
    return cpu_shfl_t(mask, v, src);
}
template <typename T> static inline T __shfl_xor_sync(unsigned mask, T v, int lane_mask, int width = 32) {
    const int lane = cpu_lane_id();
    const int src = (lane ^ lane_mask);
    return cpu_shfl_t(mask, v, (src / width == lane / width) ? src : lane);
}
template <typename T> static inline T __shfl_sync(unsigned mask, T v, int src_lane, int width = 32) {
    const int lane = cpu_lane_id();
    return cpu_shfl_t(mask, v, (lane / width) * width + (src_lane % width));
}
// D += A B for the 16 x 8 x 16 bfloat16 fragments of mma.sync.m16n8k16.row.col.
void cpu_mma_m16n8k16_bf16(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1,
                           float& c0, float& c1, float& c2, float& c3);

template <typename T> static inline T __ldg(const T* p) { return *p; }
#define __expf(x) expf(x)              /* the C library has a function of this name */
static inline float rsqrtf(float x) { return 1.0f / sqrtf(x); }
using std::max;
using std::min;

// ---- launches -----------------------------------------------------------------------------------
void cpu_launch(dim3 grid, dim3 block, const std::function<void()>& thread_body);
#define CPU_LAUNCH(kernel, grid, block, ...) cpu_launch(dim3(grid), dim3(block), [=]() { kernel(__VA_ARGS__); })

// ---- the runtime API the sources use ---------------------------------------------------------
typedef int cudaError_t;
enum { cudaSuccess = 0, cudaErrorNotSupported = 801 };
typedef struct CpuStream* cudaStream_t;
typedef struct CpuGraph* cudaGraph_t;
typedef struct CpuGraphExec* cudaGraphExec_t;
enum cudaMemcpyKind { cudaMemcpyHostToHost, cudaMemcpyHostToDevice, cudaMemcpyDeviceToHost, cudaMemcpyDeviceToDevice };
enum cudaStreamCaptureMode { cudaStreamCaptureModeGlobal, cudaStreamCaptureModeThreadLocal, cudaStreamCaptureModeRelaxed };
struct cudaDeviceProp { int major = 0, minor = 0; char name[64] = "host threads"; };
#define CUDART_VERSION 12090

template <typename T> static inline cudaError_t cudaMalloc(T** p, size_t bytes) {
    *p = static_cast<T*>(std::calloc(bytes ? bytes : 1, 1));
    return *p ? cudaSuccess : 2;
}
static inline cudaError_t cudaFree(void* p) { std::free(p); return cudaSuccess; }
static inline cudaError_t cudaMemcpy(void* d, const void* s, size_t n, cudaMemcpyKind) { std::memcpy(d, s, n); return cudaSuccess; }
static inline cudaError_t cudaMemcpyAsync(void* d, const void* s, size_t n, cudaMemcpyKind, cudaStream_t = nullptr) {
    std::memcpy(d, s, n);
    return cudaSuccess;
}
static inline cudaError_t cudaMemset(void* d, int v, size_t n) { std::memset(d, v, n); return cudaSuccess; }
static inline cudaError_t cudaGetLastError() { return cudaSuccess; }
static inline const char* cudaGetErrorString(cudaError_t e) { return e == cudaSuccess ? "no error" : "error on the host stand-in"; }
static inline cudaError_t cudaGetDevice(int* d) { *d = 0; return cudaSuccess; }
static inline cudaError_t cudaGetDeviceProperties(cudaDeviceProp* p, int) { *p = cudaDeviceProp(); return cudaSuccess; }
static inline cudaError_t cudaDeviceSynchronize() { return cudaSuccess; }
static inline cudaError_t cudaStreamCreate(cudaStream_t* s) { *s = nullptr; return cudaSuccess; }
static inline cudaError_t cudaStreamDestroy(cudaStream_t) { return cudaSuccess; }
static inline cudaError_t cudaStreamSynchronize(cudaStream_t) { return cudaSuccess; }
// CUDA graphs are not imitated: the sources use them only when asked to
static inline cudaError_t cudaStreamBeginCapture(cudaStream_t, cudaStreamCaptureMode) { return cudaErrorNotSupported; }
static inline cudaError_t cudaStreamEndCapture(cudaStream_t, cudaGraph_t*) { return cudaErrorNotSupported; }
static inline cudaError_t cudaGraphInstantiate(cudaGraphExec_t*, cudaGraph_t, unsigned long long) { return cudaErrorNotSupported; }
static inline cudaError_t cudaGraphGetNodes(cudaGraph_t, void*, size_t*) { return cudaErrorNotSupported; }
static inline cudaError_t cudaGraphDestroy(cudaGraph_t) { return cudaSuccess; }
static inline cudaError_t cudaGraphExecDestroy(cudaGraphExec_t) { return cudaSuccess; }
static inline cudaError_t cudaGraphLaunch(cudaGraphExec_t, cudaStream_t) { return cudaErrorNotSupported; }
