// Shared device helpers for the sm_100a kernel library.
//
// Every kernel is launched through an extern "C" function that takes raw device
// pointers and a stream, returns 0 or a negative MX_ERR_* / positive cudaError_t
// code, and never allocates. Activations are `float` (the 32-bit path) or
// `__nv_bfloat16` (serving); statistics, softmax, rotation angles and the
// residual stream are float in both.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MX_OK 0
#define MX_ERR_UNSUPPORTED (-1)   // a size this kernel refuses (see mx_last_error_message)
#define MX_ERR_ARGUMENT (-2)

// Bits a kernel may set in the step's device status word; the host reads it after a step.
#define MX_STATUS_BAD_TOKEN_ID 1
#define MX_STATUS_BAD_SLOT 2
#define MX_STATUS_BAD_PAGE 4
#define MX_STATUS_WAIT_TIMEOUT 8

#define MX_DTYPE_F32 0
#define MX_DTYPE_BF16 1

extern "C" const char* mx_last_error_message();
void mx_set_error(const char* fmt, ...);

#define MX_REFUSE(...)              \
    do {                            \
        mx_set_error(__VA_ARGS__);  \
        return MX_ERR_UNSUPPORTED;  \
    } while (0)

static inline int mx_launch_status() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        mx_set_error("CUDA launch failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return MX_OK;
}

// ---- programmatic dependent launch: a kernel launched with mx_launch_chained may start while the
// kernel before it in the stream is still running. It must call pdl_wait() before it reads anything
// an earlier kernel wrote and before it writes global memory at all; what it does before that
// (reading weights, setting up shared memory) overlaps the predecessor's tail. pdl_trigger() lets
// the NEXT kernel in the stream begin its own preamble.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
// A pointer to what the kernel before wrote, as it may be used after pdl_wait(): the compiler is told that it
// no longer knows the pointer, so no load through it can be moved above the wait. Without this a load through
// a `const __restrict__` parameter is fair game for the scheduler (the qualifiers promise that nothing writes
// the data while the kernel runs, which is not true of the time before the wait): LayerNorm read rows that
// the product before it had not finished when other loads were placed ahead of its wait.
template <typename T>
__device__ __forceinline__ T* after_wait(T* p) {
    asm volatile("" : "+l"(p)::"memory");
    return p;
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p));
}

bool mx_chained_launch_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t mx_launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                            cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = mx_chained_launch_enabled() ? 1 : 0;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, KArgs(args)...);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

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

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 32
// floats. The order of additions is fixed by the thread layout alone.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarps; ++w) total += scratch[w];
    return total;
}

// tanh-approximated GELU: 0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3))).
__device__ __forceinline__ float gelu_tanh(float u) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * u * (1.f + tanhf(k0 * (u + k1 * u * u * u)));
}
// The same with the hardware tanh (relative error about 2^-11): for results that are rounded to
// bfloat16 (2^-9) right after; the 32-bit path keeps tanhf.
__device__ __forceinline__ float gelu_tanh_fast(float u) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    float t;
    asm("tanh.approx.f32 %0, %1;\n" : "=f"(t) : "f"(k0 * (u + k1 * u * u * u)));
    return 0.5f * u * (1.f + t);
}
