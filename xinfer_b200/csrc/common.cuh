// Shared device helpers for the engine's kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Bits of the device-side error word that kernels set instead of faulting.
#define XB_ERR_BAD_TOKEN 1   // a token id outside [0, vocab)
#define XB_ERR_BAD_PAGE 2    // a block-table entry outside [0, num_pages)
#define XB_ERR_WAIT 4        // a bounded wait on an mbarrier gave up
#define XB_ERR_BAD_ROW 8     // a requested row outside [0, tokens)
#define XB_ERR_SCRATCH 16    // scratch memory that a kernel must find zeroed was not
#define XB_ERR_BAD_POSITION 32  // a token position outside the position table

// Element type codes shared with the Python side.
#define XB_F32 0
#define XB_BF16 1

#define XB_EXPORT extern "C" __attribute__((visibility("default")))

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of the
// additions is fixed by the thread layout, so the result does not depend on what else runs.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
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

// silu(g) * u for bfloat16 activations: the exponential and the quotient by the fast intrinsics, whose
// error (a few units in the last place of float32) is far below half a unit of the bfloat16 result.
// Every bfloat16 kernel that forms this product uses this function, so that they agree bit for bit;
// the float32 path divides and exponentiates exactly.
__device__ __forceinline__ float silu_mul_bf16(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

// Last CUDA error of a launch as an int for the caller (0 = ok).
static inline int xb_launch_status() { return (int)cudaGetLastError(); }

// Programmatic dependent launch: a kernel launched through xb_launch may be scheduled while the
// kernel before it in the stream is still running; it calls pdl_wait() before it touches anything
// that kernel may have written (or still reads), and pdl_launch_dependents() as early as it likes
// to let the kernel after it do the same.  Both are no-ops in a kernel launched the plain way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <cstdlib>
static inline bool xb_pdl_enabled() {   // XINFER_B200_PDL=0 switches the overlap off
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("XINFER_B200_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

// `overlap` false: the kernel starts only when the one before it has completed (its pdl_wait() is then a no-op).
template <typename... KArgs, typename... Args>
static inline int xb_launch_opt(bool overlap, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
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
    cfg.numAttrs = overlap && xb_pdl_enabled() ? 1 : 0;
    const cudaError_t rc = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    return rc != cudaSuccess ? (int)rc : xb_launch_status();
}
template <typename... KArgs, typename... Args>
static inline int xb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    return xb_launch_opt(true, kernel, grid, block, smem, stream, args...);
}
