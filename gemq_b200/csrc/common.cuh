// Shared helpers of the gemq_b200 kernels (sm_100a).
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/gemq_b200.h"

namespace gemq {

__host__ __device__ constexpr int cdiv(int a, int b) { return (a + b - 1) / b; }

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? GEMQ_OK : GEMQ_ERR_LAUNCH;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Streaming 128-bit load: weights are read once per step, so they should not
// displace the activation tables or metadata in L1.
__device__ __forceinline__ uint4 ld_stream_v4(const uint32_t* p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Coherent (L2) loads for data another CTA of the same grid has just written.
__device__ __forceinline__ float ld_cg_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

// tma.cu
bool tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, int inner, long long rows, int box_inner,
                   int box_rows, bool swizzle128);

__device__ __forceinline__ float pow2i(int e) {  // 2^e for e in [-126, 127]
  return __int_as_float((e + 127) << 23);
}

__device__ __forceinline__ float silu_f32(float v) { return v / (1.0f + __expf(-v)); }

}  // namespace gemq
