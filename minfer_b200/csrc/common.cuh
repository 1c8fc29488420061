// Shared helpers of the hand-written kernels: element types, status codes, reductions.
//
// Every launcher is an extern "C" function that takes raw device pointers and a stream,
// launches, and returns cudaGetLastError() (0 = launched).  Sizes that a kernel cannot
// take are refused with MF_ERR_UNSUPPORTED before anything is launched, never computed
// wrongly.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MF_DTYPE_F32 0
#define MF_DTYPE_BF16 1

// Launcher return values beyond cudaError_t (which are < 1000).
#define MF_ERR_UNSUPPORTED 2001   // a size or a dtype this kernel does not take
#define MF_ERR_ARGUMENT 2002      // inconsistent arguments

// Bits a kernel may set in the device status word it is given (never traps).
#define MF_STATUS_BAD_TOKEN 1u        // token id outside the vocabulary
#define MF_STATUS_BAD_POSITION 2u     // position outside the pages of its sequence
#define MF_STATUS_WAIT_TIMEOUT 4u     // a bounded wait on a barrier ran out

#define MF_PAGE 64                    // positions per cache page

template <typename T> struct ElemType;
template <> struct ElemType<float> { static constexpr int code = MF_DTYPE_F32; };
template <> struct ElemType<__nv_bfloat16> { static constexpr int code = MF_DTYPE_BF16; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
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

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds
// 33 floats of shared memory.  The order of the additions depends only on blockDim.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// ---- programmatic dependent launch ---------------------------------------------------------
// Every kernel is launched so that it may start while the kernel before it in the stream is
// still running: the earlier kernel says "dependents may launch" as its first instruction,
// the later one waits for the earlier grid to have completed (and its writes to be visible)
// before it touches any memory that is not constant over the step.  What is hidden is the
// launch latency and a kernel's prologue (and, in the tensor-core GEMM, the first weight
// tiles, which no kernel of the step writes).  EVERY kernel executes the wait, needed or not,
// so that completion stays transitive along the stream.  MINFER_B200_PDL=0 turns the launch
// attribute off; the instructions are then no-ops.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_prologue() {
    pdl_launch_dependents();
    pdl_wait();
}

#ifdef __CUDACC__
#include <cstdlib>
#include <utility>
static inline bool mf_pdl_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* e = getenv("MINFER_B200_PDL");
        enabled = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return enabled == 1;
}

// early = false: an ordinary launch that starts when the kernel before it has completed
template <typename... KArgs, typename... Args>
static inline void mf_launch_ex(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = (early && mf_pdl_enabled()) ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// SMs of the current device (asked once per device); launchers size grids from it
static inline int mf_sm_count() {
    static int sms[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (sms[dev] == 0) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        sms[dev] = n < 2 ? 2 : n;
    }
    return sms[dev];
}

template <typename... KArgs, typename... Args>
static inline void mf_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Args&&... args) {
    mf_launch_ex(true, kernel, grid, block, smem, stream, std::forward<Args>(args)...);
}
#endif

#define MF_LAUNCH_CHECK() ((int)cudaGetLastError())
