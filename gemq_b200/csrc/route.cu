// Router: gate GEMV, softmax, top-k and renormalisation in one launch, one CTA per token.
// Results stay on the device (expert ids as int64, like torch.topk returns them).
#include "common.cuh"

namespace gemq {

constexpr int kRouteThreads = 1024;
constexpr int kRouteMaxExperts = 256;
constexpr int kRouteMaxTopK = 16;

template <typename T> struct Act;
template <> struct Act<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Act<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

template <typename T>
__device__ __forceinline__ float dot8(const uint4& a, const uint4& b) {
  const T* pa = reinterpret_cast<const T*>(&a);
  const T* pb = reinterpret_cast<const T*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s = fmaf(Act<T>::to_f(pa[i]), Act<T>::to_f(pb[i]), s);
  return s;
}

// mode 0: logits, probabilities, their sum and the quotient are each rounded to the
//         activation dtype (softmax/topk/renorm of a half tensor);
// mode 1: logits rounded to the activation dtype, softmax and renormalisation in fp32;
// mode 2: fp32 throughout.  The returned weights are cast to the activation dtype.
// PER: experts per lane in the softmax / top-k phase (E <= 32 * PER); the small instances keep the
// serial tail of the kernel (one warp) short.
template <typename T, int PER>
__global__ void __launch_bounds__(kRouteThreads) route_kernel(const T* __restrict__ x, const T* __restrict__ gate,
                                                              int D, int E, int A, int mode, int renorm,
                                                              long long* __restrict__ idx, T* __restrict__ weights,
                                                              float* __restrict__ logits_out) {
  __shared__ float logit[kRouteMaxExperts];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // x may come from the previous kernel of the stream
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const T* xt = x + static_cast<size_t>(t) * D;
  // An expert row is cut into `parts` segments so that all 32 warps pull on the gate matrix at
  // once and every lane has all its 128-bit loads in flight before the first multiply.
  __shared__ float part_sum[kRouteMaxExperts][8];
  constexpr int NW = kRouteThreads / 32;
  int parts = E >= NW ? 1 : NW / E;
  parts = parts > 8 ? 8 : parts;
  while (parts > 1 && (D % (parts * 256)) != 0) parts >>= 1;
  const bool vec = (D % 256 == 0) && ((reinterpret_cast<uintptr_t>(xt) & 15u) == 0) &&
                   ((reinterpret_cast<uintptr_t>(gate) & 15u) == 0);
  if (!vec) parts = 1;
  const int seg = D / parts;
  for (int task = warp; task < E * parts; task += NW) {
    const int e = task / parts, sg = task - e * parts;
    const T* ge = gate + static_cast<size_t>(e) * D + static_cast<size_t>(sg) * seg;
    const T* xs = xt + static_cast<size_t>(sg) * seg;
    float s = 0.f;
    if (vec) {
      for (int k0 = 0; k0 < seg; k0 += 4 * 256) {
        uint4 gq[4], xq[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int k = k0 + (i * 32 + lane) * 8;
          if (k < seg) {
            gq[i] = *reinterpret_cast<const uint4*>(ge + k);
            xq[i] = *reinterpret_cast<const uint4*>(xs + k);
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (k0 + (i * 32 + lane) * 8 < seg) s += dot8<T>(xq[i], gq[i]);
      }
    } else {
      for (int k = lane; k < seg; k += 32) s = fmaf(Act<T>::to_f(xs[k]), Act<T>::to_f(ge[k]), s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) part_sum[e][sg] = s;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kRouteThreads) {
    float s = 0.f;
    for (int q = 0; q < parts; ++q) s += part_sum[e][q];
    if (mode != 2) s = Act<T>::to_f(Act<T>::from_f(s));
    logit[e] = s;
    if (logits_out) logits_out[static_cast<size_t>(t) * E + e] = s;
  }
  __syncthreads();
  if (warp != 0) return;

  float p[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    p[i] = e < E ? logit[e] : -INFINITY;
    mx = fmaxf(mx, p[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    p[i] = (lane + 32 * i) < E ? expf(p[i] - mx) : 0.f;
    sum += p[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    p[i] = p[i] / sum;
    if (mode == 0) p[i] = Act<T>::to_f(Act<T>::from_f(p[i]));
    if ((lane + 32 * i) >= E) p[i] = -1.f;
  }
  // top-k: A rounds of warp arg-max, ties to the lower expert id; lane a keeps the a-th winner
  float my_w = 0.f;
  int my_i = 0;
  for (int a = 0; a < A; ++a) {
    float bv = -2.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (p[i] > bv) { bv = p[i]; bi = lane + 32 * i; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == a) { my_w = bv; my_i = bi; }
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (lane + 32 * i == bi) p[i] = -3.f;
  }
  float tot = 0.f;
  for (int a = 0; a < A; ++a) tot += __shfl_sync(0xffffffffu, my_w, a);  // in selection order, like a sum over the top-k tensor
  if (mode == 0) tot = Act<T>::to_f(Act<T>::from_f(tot));
  if (lane < A) {
    const float w = renorm ? my_w / tot : my_w;
    idx[static_cast<size_t>(t) * A + lane] = my_i;
    weights[static_cast<size_t>(t) * A + lane] = Act<T>::from_f(w);
  }
}

}  // namespace gemq

using namespace gemq;

extern "C" int gemq_moe_route(const void* x, const void* gate, int tokens, int D, int E, int A,
                              int mode, int renorm, int x_is_bf16,
                              int64_t* idx, void* weights, float* logits, gemq_stream_t stream) {
  if (!x || !gate || !idx || !weights || tokens <= 0 || D <= 0 || E <= 0 || A <= 0 || mode < 0 || mode > 2)
    return GEMQ_ERR_BAD_ARG;
  if (E > kRouteMaxExperts || A > kRouteMaxTopK || A > E) return GEMQ_ERR_BAD_SHAPE;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tokens);
  cfg.blockDim = dim3(kRouteThreads);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  auto launch = [&](auto kernel_h, auto kernel_b) {
    return x_is_bf16 ? cudaLaunchKernelEx(&cfg, kernel_b, static_cast<const __nv_bfloat16*>(x),
                                          static_cast<const __nv_bfloat16*>(gate), D, E, A, mode, renorm,
                                          reinterpret_cast<long long*>(idx), static_cast<__nv_bfloat16*>(weights), logits)
                     : cudaLaunchKernelEx(&cfg, kernel_h, static_cast<const __half*>(x), static_cast<const __half*>(gate), D,
                                          E, A, mode, renorm, reinterpret_cast<long long*>(idx),
                                          static_cast<__half*>(weights), logits);
  };
  if (E <= 32) e = launch(route_kernel<__half, 1>, route_kernel<__nv_bfloat16, 1>);
  else if (E <= 64) e = launch(route_kernel<__half, 2>, route_kernel<__nv_bfloat16, 2>);
  else e = launch(route_kernel<__half, kRouteMaxExperts / 32>, route_kernel<__nv_bfloat16, kRouteMaxExperts / 32>);
  if (e != cudaSuccess) return GEMQ_ERR_LAUNCH;
  return launch_status();
}
