// Shared device/host helpers for the sm_100a kernel library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "aoto_sm100.h"

namespace aoto {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}
// low / high bf16 of a packed pair, widened exactly
__device__ __forceinline__ float bf16x2_lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16x2_hi(uint32_t pair) { return __uint_as_float(pair & 0xffff0000u); }

__device__ __forceinline__ uint32_t float_to_bf16_bits(float value) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(value));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  return float_to_bf16_bits(lo) | (float_to_bf16_bits(hi) << 16);
}
// round-trip through bf16: the value a bf16 store followed by a load would give
__device__ __forceinline__ float round_bf16(float value) {
  return __bfloat162float(__float2bfloat16_rn(value));
}

__device__ __forceinline__ uint4 ldg_nc_u4(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr));
  return v;
}

// Read-only loads the compiler must issue where they are written (it is free to sink an
// ordinary load to its first use, which turns a prefetch into an exposed miss).
__device__ __forceinline__ uint32_t ldg_nc_u32(const void* ptr) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(ptr));
  return v;
}
__device__ __forceinline__ uint2 ldg_nc_u2(const void* ptr) {
  uint2 v;
  asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(ptr));
  return v;
}
__device__ __forceinline__ float ldg_nc_bf16(const __nv_bfloat16* ptr) {
  unsigned short raw;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(raw) : "l"(ptr));
  return __uint_as_float(((uint32_t)raw) << 16);
}

// 16-bit load that bypasses L1 (L1 is not coherent across SMs: values another CTA
// wrote during the same kernel must come from L2).
__device__ __forceinline__ float ldcg_bf16(const __nv_bfloat16* ptr) {
  unsigned short raw;
  asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(raw) : "l"(ptr));
  return __uint_as_float(((uint32_t)raw) << 16);
}

// Programmatic dependent launch. Both are no-ops when the kernel was launched
// without the programmatic-serialization attribute.
__device__ __forceinline__ void pdl_wait_for_producers() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_release_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Block-wide sum through shared memory; `scratch` holds >= 32 floats. Every
// thread of the block must call it; every thread receives the total.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < warps; ++w) total += scratch[w];  // fixed order: deterministic
  return total;
}

__device__ __forceinline__ bool aligned_ptr16(const void* ptr) {
  return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0;
}

// Layout shared by every kernel that meets in scratch: arrival counters live in
// the first SCRATCH_HEADER_BYTES (always zero between launches), payload after
// them. A buffer can therefore be reused by different kernels and shapes.
constexpr int SCRATCH_HEADER_BYTES = 4096;
constexpr int SCRATCH_MAX_COUNTERS = SCRATCH_HEADER_BYTES / 4;

inline int launch_status() {
  cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? AOTO_OK : AOTO_ERR_LAUNCH;
}

inline bool aligned_to(const void* ptr, size_t bytes) {
  return (reinterpret_cast<uintptr_t>(ptr) % bytes) == 0;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) belongs to (function, device): a process that
// drives several GPUs must make the call once on each of them. One flag per device ordinal; a
// race between host threads only repeats the idempotent call.
constexpr int MAX_DEVICES = 64;
struct PerDeviceOnce {
  bool done[MAX_DEVICES] = {};
};
template <typename Kernel>
inline int raise_dynamic_smem(Kernel kernel, size_t bytes, PerDeviceOnce& once) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) {
    (void)cudaGetLastError();
    return AOTO_ERR_LAUNCH;
  }
  const bool tracked = device >= 0 && device < MAX_DEVICES;
  if (tracked && once.done[device]) return AOTO_OK;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return AOTO_ERR_LAUNCH;
  }
  if (tracked) once.done[device] = true;
  return AOTO_OK;
}

// Launch with or without the programmatic-dependent-launch attribute.
template <typename Kernel, typename... Args>
inline int launch_kernel(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                         bool pdl, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = pdl ? 1 : 0;
  cudaError_t err = cudaLaunchKernelEx(&config, kernel, args...);
  if (err != cudaSuccess) {
    (void)cudaGetLastError();
    return AOTO_ERR_LAUNCH;
  }
  return AOTO_OK;
}

}  // namespace aoto
