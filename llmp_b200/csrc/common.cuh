// Shared host/device helpers of the llmp_b200 kernels (sm_100a only).
#ifndef LLMP_B200_CSRC_COMMON_CUH_
#define LLMP_B200_CSRC_COMMON_CUH_

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "llmp_b200.h"

namespace llmp_b200 {

// ---- status ---------------------------------------------------------------
// Thread-local message behind llmp_b200_last_error().
char* ErrorBuffer();
int Reject(const char* format, ...);                 // returns LLMP_B200_REJECTED
int Failed(cudaError_t error, const char* what);     // returns a negative status
int DeviceStatus();                                  // 0 or LLMP_B200_NO_DEVICE
int SmCount();
// Device address of the counter of bounded waits that ran out (per device), or null.
unsigned int* FaultCounter();
int ReadFaultCounter();
int ClearFaultCounter();  // the count before, or -1

// After a launch: 0, or a negative status carrying the CUDA error.
inline int Launched(const char* what) {
  const cudaError_t e = cudaPeekAtLastError();
  return e == cudaSuccess ? 0 : Failed(cudaGetLastError(), what);
}

inline bool Aligned(const void* p, std::uintptr_t a) {
  return (reinterpret_cast<std::uintptr_t>(p) % a) == 0;
}

// A launch that may begin while the kernel before it on the stream drains
// (programmatic dependent launch): the kernel orders itself after that
// kernel's writes with GridDependencyWait().
template <typename... KernelArgs, typename... Args>
inline cudaError_t LaunchPdl(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

#ifdef __CUDACC__
// ---- device ---------------------------------------------------------------
__device__ __forceinline__ void GridDependencyWait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void GridLaunchDependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ int Dp4a(int a, int b, int c) { return __dp4a(a, b, c); }

// Streaming loads of weights: read once, kept out of L1.
__device__ __forceinline__ uint4 LoadStream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 LoadStream8(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
               : "=r"(v.x), "=r"(v.y)
               : "l"(p));
  return v;
}
__device__ __forceinline__ std::uint32_t LoadStream4(const void* p) {
  std::uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ float HalfBitsToFloat(std::uint32_t bits16) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
}

__device__ __forceinline__ float Silu(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float GeluTanh(float x) {
  return 0.5f * x * (1.0f + tanhf(0.79788456080286535587989211986876f * x *
                                  (1.0f + 0.044715f * x * x)));
}
// src/kernels/ggml/vecq.cu:184-195.
__device__ __forceinline__ float Glu(int glu, float gate, float up, float limit) {
  if (glu == LLMP_B200_GLU_GEGLU) return GeluTanh(gate) * up;
  if (glu == LLMP_B200_GLU_SWIGLU_CLAMP) {
    gate = fminf(gate, limit);
    up = fmaxf(fminf(up, limit), -limit);
  }
  return Silu(gate) * up;
}
#endif  // __CUDACC__

}  // namespace llmp_b200

#endif  // LLMP_B200_CSRC_COMMON_CUH_
