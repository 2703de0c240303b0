// Expert-parallel prefill: the device side of the token exchange around the local grouped GEMM.
//
// The reference has no multi-GPU path (its n-token forward loops over the experts of one GPU,
// gemq/inference/moe_block.py:165-198); these kernels are what the all-to-all form of that
// loop needs on each rank:
//   ep_plan_kernel     (token, slot) pairs -> destination rank, position on the destination,
//                      stable order by (destination, expert), rows per destination
//   ep_pack_kernel     gather the rows into the send payload; each row carries its expert
//                      position on the destination and its routing weight in eight extra elements
//   ep_unpack_kernel   received payload -> contiguous rows, expert positions, weights
//   ep_combine_kernel  returned rows -> per token, added in increasing expert id with a rounding
//                      per addition (the index_add_ order of moe_block.py:191-195)
// All of it is integer / byte work bound by launch latency at these sizes (thousands of rows of
// 8 KB): one launch per step instead of the twenty-odd small tensor operations it replaces.
#include "common.cuh"

namespace gemq {
namespace {

constexpr int kPlanThreads = 1024;
constexpr int kPlanWarps = kPlanThreads / 32;
constexpr int kMaxKeys = 2048;  // world * experts
constexpr int kErrBadExpertEp = 31;

// Stable rank of every element among the elements with the same key, for one chunk of up to
// 1024 elements (one per thread): returns base[key] before the chunk + the number of earlier
// threads of the chunk with the same key, and adds the chunk's counts to base[].
__device__ __forceinline__ int chunk_rank(int key, int* base) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned peers = __match_any_sync(0xffffffffu, key);
  const int leader = __ffs(peers) - 1;
  const int before = __popc(peers & ((1u << lane) - 1u));
  int old = 0;
  for (int w = 0; w < kPlanWarps; ++w) {  // warps take their turn in order: that is what makes the rank stable
    if (warp == w && lane == leader && key >= 0) {
      old = base[key];
      base[key] = old + __popc(peers);
    }
    __syncthreads();
  }
  old = __shfl_sync(0xffffffffu, old, leader);
  return old + before;
}

__global__ void __launch_bounds__(kPlanThreads) ep_plan_kernel(const long long* __restrict__ sel, int n, int E, int world,
                                                               int R, const int* __restrict__ rank_tab,
                                                               const int* __restrict__ local_tab,
                                                               const float* __restrict__ upper_tab,
                                                               long long* __restrict__ order, int* __restrict__ loc_sorted,
                                                               long long* __restrict__ where,
                                                               long long* __restrict__ send_counts, int* __restrict__ tmp,
                                                               int* __restrict__ err) {
  __shared__ int base[kMaxKeys];
  __shared__ int count_e[kMaxKeys];
  const int tid = threadIdx.x;
  const int nkeys = world * E;
  for (int k = tid; k < nkeys; k += kPlanThreads) base[k] = 0;
  __syncthreads();
  // pass 1: position of every pair among this rank's pairs of the same expert
  for (int c0 = 0; c0 < n; c0 += kPlanThreads) {
    const int i = c0 + tid;
    int e = -1;
    if (i < n) {
      const long long v = sel[i];
      if (v < 0 || v >= E) {
        atomicExch(err, kErrBadExpertEp);
        e = v < 0 ? 0 : E - 1;
      } else {
        e = static_cast<int>(v);
      }
    }
    const int r = chunk_rank(e, base);
    if (i < n) tmp[i] = r;
  }
  for (int k = tid; k < E; k += kPlanThreads) count_e[k] = base[k];
  __syncthreads();
  for (int k = tid; k < nkeys; k += kPlanThreads) base[k] = 0;
  __syncthreads();
  // pass 2: destination of every pair, stable position among the pairs with the same (destination, expert)
  for (int c0 = 0; c0 < n; c0 += kPlanThreads) {
    const int i = c0 + tid;
    int key = -1;
    if (i < n) {
      const long long v = sel[i];
      const int e = v < 0 ? 0 : (v >= E ? E - 1 : static_cast<int>(v));
      const float frac = (static_cast<float>(tmp[i]) + 0.5f) / static_cast<float>(count_e[e]);
      int rep = 0;
      for (int j = 0; j < R; ++j) rep += frac >= upper_tab[e * R + j] ? 1 : 0;
      rep = min(rep, R - 1);
      key = rank_tab[e * R + rep] * E + e;
      tmp[n + i] = key | (rep << 24);
    }
    const int r = chunk_rank(key, base);
    if (i < n) tmp[i] = r;
  }
  // exclusive prefix over the keys (rank-major, expert-minor), rows per destination
  if (tid < 32) {
    int carry = 0;
    for (int k0 = 0; k0 < nkeys; k0 += 32) {
      const int k = k0 + tid;
      const int v = k < nkeys ? base[k] : 0;
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (tid >= o) incl += t;
      }
      if (k < nkeys) count_e[k] = carry + incl - v;  // count_e is free again: start of the key
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  __syncthreads();
  for (int r = tid; r < world; r += kPlanThreads) {
    const int lo = count_e[r * E];
    const int hi = r + 1 < world ? count_e[(r + 1) * E] : n;
    send_counts[r] = hi - lo;
  }
  for (int i = tid; i < n; i += kPlanThreads) {
    const int packed = tmp[n + i];
    const int key = packed & 0xffffff, rep = packed >> 24;
    const int e = key % E;
    const int p = count_e[key] + tmp[i];
    order[p] = i;
    loc_sorted[p] = local_tab[e * R + rep];
    where[i] = p;
  }
}

// One CTA per payload row: D 16-bit elements of the token's row, then 16 bytes of metadata
// (int32 expert position on the destination, 16-bit routing weight, zero padding).
__global__ void __launch_bounds__(128) ep_pack_kernel(const uint16_t* __restrict__ x, const long long* __restrict__ order,
                                                     const int* __restrict__ loc_sorted, const uint16_t* __restrict__ w,
                                                     int A, int D, uint16_t* __restrict__ out) {
  const int p = blockIdx.x;
  const long long pair = order[p];
  const uint4* src = reinterpret_cast<const uint4*>(x + (pair / A) * D);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(p) * (D + 8));
  for (int i = threadIdx.x; i < D / 8; i += blockDim.x) dst[i] = src[i];
  if (threadIdx.x == 0) {
    uint4 m;
    m.x = static_cast<uint32_t>(loc_sorted[p]);
    m.y = w[pair];
    m.z = 0u;
    m.w = 0u;
    dst[D / 8] = m;
  }
}

__global__ void __launch_bounds__(128) ep_unpack_kernel(const uint16_t* __restrict__ in, int D, uint16_t* __restrict__ rows,
                                                       long long* __restrict__ expert, uint16_t* __restrict__ w) {
  const int p = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(in + static_cast<size_t>(p) * (D + 8));
  uint4* dst = reinterpret_cast<uint4*>(rows + static_cast<size_t>(p) * D);
  for (int i = threadIdx.x; i < D / 8; i += blockDim.x) dst[i] = src[i];
  if (threadIdx.x == 0) {
    const uint4 m = src[D / 8];
    expert[p] = static_cast<int>(m.x);
    w[p] = static_cast<uint16_t>(m.y & 0xffffu);
  }
}

template <typename T>
__device__ __forceinline__ float to_f32(uint16_t v);
template <>
__device__ __forceinline__ float to_f32<__half>(uint16_t v) { return __half2float(__ushort_as_half(v)); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(uint16_t v) { return __uint_as_float(static_cast<uint32_t>(v) << 16); }
template <typename T>
__device__ __forceinline__ uint16_t from_f32(float v);
template <>
__device__ __forceinline__ uint16_t from_f32<__half>(float v) { return __half_as_ushort(__float2half_rn(v)); }
template <>
__device__ __forceinline__ uint16_t from_f32<__nv_bfloat16>(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }

// One CTA per token: its A returned rows, added in increasing expert id (ties by slot), the
// running sum rounded to the activation type after every addition.
template <typename T>
__global__ void __launch_bounds__(128) ep_combine_kernel(const uint16_t* __restrict__ back, const long long* __restrict__ where,
                                                        const long long* __restrict__ sel, int A, int D,
                                                        uint16_t* __restrict__ out) {
  __shared__ long long row_of[16];
  const int t = blockIdx.x;
  if (threadIdx.x == 0) {
    int slot[16];
    for (int a = 0; a < A; ++a) slot[a] = a;
    for (int a = 1; a < A; ++a) {  // insertion sort by expert id, stable
      const int s = slot[a];
      const long long e = sel[static_cast<size_t>(t) * A + s];
      int b = a - 1;
      while (b >= 0 && sel[static_cast<size_t>(t) * A + slot[b]] > e) {
        slot[b + 1] = slot[b];
        --b;
      }
      slot[b + 1] = s;
    }
    for (int a = 0; a < A; ++a) row_of[a] = where[static_cast<size_t>(t) * A + slot[a]];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D / 8; i += blockDim.x) {
    float acc[8];
    {
      const uint4 v = reinterpret_cast<const uint4*>(back + row_of[0] * D)[i];
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        acc[2 * k] = to_f32<T>(static_cast<uint16_t>(u[k] & 0xffffu));
        acc[2 * k + 1] = to_f32<T>(static_cast<uint16_t>(u[k] >> 16));
      }
    }
    for (int a = 1; a < A; ++a) {
      const uint4 v = reinterpret_cast<const uint4*>(back + row_of[a] * D)[i];
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        acc[2 * k] = to_f32<T>(from_f32<T>(acc[2 * k] + to_f32<T>(static_cast<uint16_t>(u[k] & 0xffffu))));
        acc[2 * k + 1] = to_f32<T>(from_f32<T>(acc[2 * k + 1] + to_f32<T>(static_cast<uint16_t>(u[k] >> 16))));
      }
    }
    uint4 o;
    uint32_t* ou = &o.x;
#pragma unroll
    for (int k = 0; k < 4; ++k)
      ou[k] = static_cast<uint32_t>(from_f32<T>(acc[2 * k])) | (static_cast<uint32_t>(from_f32<T>(acc[2 * k + 1])) << 16);
    reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * D)[i] = o;
  }
}

}  // namespace
}  // namespace gemq

extern "C" {

size_t gemq_ep_plan_scratch_bytes(int pairs) { return pairs > 0 ? static_cast<size_t>(pairs) * 2 * sizeof(int) + 16 : 16; }

int gemq_ep_plan(const int64_t* sel, int pairs, int n_experts, int world, int replicas, const int32_t* rank_tab,
                 const int32_t* local_tab, const float* upper_tab, int64_t* order, int32_t* loc_sorted, int64_t* where,
                 int64_t* send_counts, void* scratch, size_t scratch_bytes, gemq_stream_t stream) {
  using namespace gemq;
  if (!sel || !rank_tab || !local_tab || !upper_tab || !order || !loc_sorted || !where || !send_counts || !scratch)
    return GEMQ_ERR_BAD_ARG;
  if (pairs <= 0 || n_experts <= 0 || world <= 0 || replicas <= 0 || replicas > 64) return GEMQ_ERR_BAD_ARG;
  if (static_cast<long long>(world) * n_experts > kMaxKeys || pairs >= (1 << 24) || world * n_experts >= (1 << 24))
    return GEMQ_ERR_BAD_SHAPE;
  if (scratch_bytes < gemq_ep_plan_scratch_bytes(pairs)) return GEMQ_ERR_WORKSPACE;
  int* tmp = static_cast<int*>(scratch) + 4;
  int* err = static_cast<int*>(scratch);
  ep_plan_kernel<<<1, kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const long long*>(sel), pairs, n_experts, world, replicas, rank_tab, local_tab, upper_tab,
      reinterpret_cast<long long*>(order), loc_sorted, reinterpret_cast<long long*>(where),
      reinterpret_cast<long long*>(send_counts), tmp, err);
  return launch_status();
}

int gemq_ep_pack_rows(const void* x, const int64_t* order, const int32_t* loc_sorted, const void* weights, int pairs,
                      int top_k, int D, void* payload, gemq_stream_t stream) {
  using namespace gemq;
  if (!x || !order || !loc_sorted || !weights || !payload) return GEMQ_ERR_BAD_ARG;
  if (pairs <= 0 || top_k <= 0 || D <= 0 || D % 8) return GEMQ_ERR_BAD_SHAPE;
  if (!aligned16(x) || !aligned16(payload)) return GEMQ_ERR_ALIGN;
  ep_pack_kernel<<<pairs, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(x), reinterpret_cast<const long long*>(order), loc_sorted,
      static_cast<const uint16_t*>(weights), top_k, D, static_cast<uint16_t*>(payload));
  return launch_status();
}

int gemq_ep_unpack_rows(const void* payload, int rows, int D, void* x, int64_t* expert, void* weights,
                        gemq_stream_t stream) {
  using namespace gemq;
  if (!payload || !x || !expert || !weights) return GEMQ_ERR_BAD_ARG;
  if (rows <= 0 || D <= 0 || D % 8) return GEMQ_ERR_BAD_SHAPE;
  if (!aligned16(x) || !aligned16(payload)) return GEMQ_ERR_ALIGN;
  ep_unpack_kernel<<<rows, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(payload), D, static_cast<uint16_t*>(x), reinterpret_cast<long long*>(expert),
      static_cast<uint16_t*>(weights));
  return launch_status();
}

int gemq_ep_combine(const void* back, const int64_t* where, const int64_t* sel, int tokens, int top_k, int D,
                    int is_bf16, void* out, gemq_stream_t stream) {
  using namespace gemq;
  if (!back || !where || !sel || !out) return GEMQ_ERR_BAD_ARG;
  if (tokens <= 0 || top_k <= 0 || top_k > 16 || D <= 0 || D % 8) return GEMQ_ERR_BAD_SHAPE;
  if (!aligned16(back) || !aligned16(out)) return GEMQ_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_bf16)
    ep_combine_kernel<__nv_bfloat16><<<tokens, 128, 0, s>>>(static_cast<const uint16_t*>(back),
                                                            reinterpret_cast<const long long*>(where),
                                                            reinterpret_cast<const long long*>(sel), top_k, D,
                                                            static_cast<uint16_t*>(out));
  else
    ep_combine_kernel<__half><<<tokens, 128, 0, s>>>(static_cast<const uint16_t*>(back),
                                                     reinterpret_cast<const long long*>(where),
                                                     reinterpret_cast<const long long*>(sel), top_k, D,
                                                     static_cast<uint16_t*>(out));
  return launch_status();
}

}  // extern "C"
