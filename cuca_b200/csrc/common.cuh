// Shared declarations of the kernel library: dtype codes, error reporting and
// scalar load/store helpers. Every exported function returns 0 on success and a
// non-zero code after storing a message that cuca_last_error() returns.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

#define CUCA_F32 0
#define CUCA_BF16 1

#define CUCA_API extern "C" __attribute__((visibility("default")))

// Device-side error word layout: kernels that find a bad index record a code
// and skip the access instead of faulting.
#define CUCA_ERR_TOKEN_RANGE 1
#define CUCA_ERR_BLOCK_RANGE 2
#define CUCA_ERR_WAIT_TIMEOUT 3
#define CUCA_ERR_SMEM_LAYOUT 4

void cuca_set_error(const char* fmt, ...);
extern "C" const char* cuca_last_error();

#define CUCA_CHECK_LAUNCH(name)                                                     \
  do {                                                                              \
    cudaError_t e__ = cudaGetLastError();                                           \
    if (e__ != cudaSuccess) {                                                       \
      cuca_set_error("%s: launch failed: %s", name, cudaGetErrorString(e__));       \
      return 2;                                                                     \
    }                                                                               \
  } while (0)

#define CUCA_REQUIRE(cond, ...)                                                     \
  do {                                                                              \
    if (!(cond)) {                                                                  \
      cuca_set_error(__VA_ARGS__);                                                  \
      return 1;                                                                     \
    }                                                                               \
  } while (0)

// Programmatic dependent launch: a kernel launched with the attribute may start while its predecessor in
// the stream still runs. pdl_trigger() lets the successor's CTAs become resident early; pdl_wait() blocks
// until the predecessor has completed and its writes are visible. Every kernel calls pdl_wait() in every CTA
// before it reads or writes anything an earlier kernel touches (both are no-ops without the attribute).
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

bool cuca_pdl_enabled();

// Launch `kernel`; with `pdl` (and PDL enabled) as a programmatic dependent of the previous kernel in `stream`.
template <typename... KArgs, typename... Args>
cudaError_t cuca_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl,
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
  cfg.numAttrs = (pdl && cuca_pdl_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with thread-block clusters of `cluster_x` CTAs along x (gridDim.x must be a multiple of it).
template <typename... KArgs, typename... Args>
cudaError_t cuca_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                bool pdl, unsigned cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl && cuca_pdl_enabled()) ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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
