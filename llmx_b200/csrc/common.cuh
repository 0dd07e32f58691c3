// Shared helpers of the sm_100a kernels: element types, conversions, reductions.
//
// Every exported function is `extern "C"`, takes raw device pointers and a
// stream, launches on that stream and returns the CUDA error code of the launch
// (0 on success).  Nothing here allocates.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

#define LLMX_EXPORT extern "C" __attribute__((visibility("default")))

// Element type codes shared with the Python side.
enum : int { LLMX_F32 = 0, LLMX_BF16 = 1 };

// Error codes above the CUDA range, for argument refusals made on the host.
enum : int { LLMX_ERR_BAD_ARGUMENT = 10001, LLMX_ERR_UNSUPPORTED = 10002 };

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads, in a fixed order (lane tree, then warps in index order),
// so a row's sum does not depend on what else the launch holds.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float total = 0.0f;
    for (int w = 0; w < nwarps; ++w) total += scratch[w];
    return total;
}

static inline int launch_status() { return (int)cudaGetLastError(); }

// ---- programmatic dependent launch --------------------------------------------------------------
// Kernels of a step run one after another on one stream.  Launched with the "programmatic stream
// serialization" attribute, a kernel's blocks may be placed on the SMs and run their prologue (barriers,
// tensor memory, descriptor prefetch) while the kernel before it drains.  The rule every kernel here
// keeps: `pdl_trigger()` first (the next kernel may start arriving), then `pdl_wait()` before the first
// access to global memory another kernel writes or reads.  `pdl_wait()` returns only when the kernel
// before has finished and its writes are visible, so nothing after it can race; without the attribute
// both are no-ops.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

static inline bool llmx_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("LLMX_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
static inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
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
    cfg.numAttrs = llmx_pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
