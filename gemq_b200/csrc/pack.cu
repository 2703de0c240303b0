// Packing format kernels: pack / unpack along columns and the bit-exact de-quantisation.
// Load-time utilities; none of them sits on the per-token path.
#include "common.cuh"

namespace gemq {

// One thread per output word (row, w): OR of up to eps codes, tail lanes zero.
__global__ void pack_over_cols_kernel(const uint8_t* __restrict__ codes, uint32_t* __restrict__ out,
                                      int rows, int cols, int words, int nbits) {
  const size_t id = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (id >= static_cast<size_t>(rows) * words) return;
  const int r = static_cast<int>(id / words), w = static_cast<int>(id % words);
  const int eps = 32 / nbits;
  const uint8_t* src = codes + static_cast<size_t>(r) * cols + static_cast<size_t>(w) * eps;
  const int n = min(eps, cols - w * eps);
  uint32_t v = 0;
  for (int j = 0; j < n; ++j) v |= static_cast<uint32_t>(src[j]) << (j * nbits);
  out[id] = v;
}

// Kernel form: codes [N, K] -> words [Kw, N].  A 32x(32*eps) tile of codes is staged in
// shared memory so both the byte reads (along K) and the word writes (along N) coalesce.
__global__ void pack_kernel_form_kernel(const uint8_t* __restrict__ codes, uint32_t* __restrict__ wq,
                                        int N, int K, int kw, int nbits) {
  extern __shared__ uint8_t tile[];  // [32 columns][32*eps + 1 pad]
  const int eps = 32 / nbits;
  const int span = 32 * eps;
  const int n0 = blockIdx.x * 32, w0 = blockIdx.y * 32;
  const int k0 = w0 * eps;
  for (int i = threadIdx.x; i < 32 * span; i += blockDim.x) {
    const int nn = i / span, kk = i % span;
    uint8_t c = 0;
    if (n0 + nn < N && k0 + kk < K) c = codes[static_cast<size_t>(n0 + nn) * K + k0 + kk];
    tile[nn * (span + 1) + kk] = c;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 32 * 32; i += blockDim.x) {
    const int ww = i / 32, nn = i % 32;
    if (w0 + ww < kw && n0 + nn < N) {
      uint32_t v = 0;
      for (int j = 0; j < eps; ++j) v |= static_cast<uint32_t>(tile[nn * (span + 1) + ww * eps + j]) << (j * nbits);
      wq[static_cast<size_t>(w0 + ww) * N + n0 + nn] = v;
    }
  }
}

__global__ void unpack_over_cols_kernel(const uint32_t* __restrict__ packed, uint8_t* __restrict__ codes,
                                        int rows, int words, int out_cols, int nbits) {
  const size_t id = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (id >= static_cast<size_t>(rows) * out_cols) return;
  const int r = static_cast<int>(id / out_cols), c = static_cast<int>(id % out_cols);
  const int eps = 32 / nbits;
  const uint32_t w = packed[static_cast<size_t>(r) * words + c / eps];
  codes[id] = static_cast<uint8_t>((w >> ((c % eps) * nbits)) & ((1u << nbits) - 1u));
}

// W^T[k, n] = fp16(fma(fp16(q), s, z)): one rounding, as tl.fma on fp16 operands.
__global__ void dequantize_kernel(const uint32_t* __restrict__ wq, const __half* __restrict__ scales,
                                  const __half* __restrict__ zeros, __half* __restrict__ out,
                                  int K, int N, int nbits, int group) {
  const size_t id = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (id >= static_cast<size_t>(K) * N) return;
  const int k = static_cast<int>(id / N), n = static_cast<int>(id % N);
  const int eps = 32 / nbits;
  const uint32_t w = wq[static_cast<size_t>(k / eps) * N + n];
  const int q = static_cast<int>((w >> ((k % eps) * nbits)) & ((1u << nbits) - 1u));
  const size_t m = static_cast<size_t>(k / group) * N + n;
  out[id] = __hfma(__int2half_rn(q), scales[m], zeros[m]);
}

static int grid1d(size_t n, int block, unsigned* g) {
  const size_t blocks = (n + block - 1) / block;
  if (blocks == 0 || blocks > 0x7fffffffu) return GEMQ_ERR_BAD_SHAPE;
  *g = static_cast<unsigned>(blocks);
  return GEMQ_OK;
}

}  // namespace gemq

using namespace gemq;

extern "C" const char* gemq_version(void) { return "gemq_b200 0.1 (sm_100a)"; }

extern "C" int gemq_pack_over_cols(const uint8_t* codes, int32_t* packed, int rows, int cols, int nbits,
                                   gemq_stream_t stream) {
  if (!codes || !packed || rows <= 0 || cols <= 0 || nbits < 1 || nbits > 4) return GEMQ_ERR_BAD_ARG;
  const int words = cdiv(cols, 32 / nbits);
  unsigned g;
  if (int e = grid1d(static_cast<size_t>(rows) * words, 256, &g)) return e;
  pack_over_cols_kernel<<<g, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      codes, reinterpret_cast<uint32_t*>(packed), rows, cols, words, nbits);
  return launch_status();
}

extern "C" int gemq_pack_kernel_form(const uint8_t* codes, int32_t* wq, int N, int K, int nbits,
                                     gemq_stream_t stream) {
  if (!codes || !wq || N <= 0 || K <= 0 || nbits < 1 || nbits > 4) return GEMQ_ERR_BAD_ARG;
  const int eps = 32 / nbits;
  const int kw = cdiv(K, eps);
  const dim3 grid(cdiv(N, 32), cdiv(kw, 32));
  if (grid.y > 65535) return GEMQ_ERR_BAD_SHAPE;
  const size_t smem = static_cast<size_t>(32) * (32 * eps + 1);
  pack_kernel_form_kernel<<<grid, 256, smem, static_cast<cudaStream_t>(stream)>>>(
      codes, reinterpret_cast<uint32_t*>(wq), N, K, kw, nbits);
  return launch_status();
}

extern "C" int gemq_unpack_over_cols(const int32_t* packed, uint8_t* codes, int rows, int words, int out_cols,
                                     int nbits, gemq_stream_t stream) {
  if (!codes || !packed || rows <= 0 || words <= 0 || out_cols <= 0 || nbits < 1 || nbits > 4) return GEMQ_ERR_BAD_ARG;
  if (out_cols > words * (32 / nbits)) return GEMQ_ERR_BAD_SHAPE;
  unsigned g;
  if (int e = grid1d(static_cast<size_t>(rows) * out_cols, 256, &g)) return e;
  unpack_over_cols_kernel<<<g, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(packed), codes, rows, words, out_cols, nbits);
  return launch_status();
}

extern "C" int gemq_dequantize(const int32_t* wq, const void* scales, const void* zeros, void* out_kn,
                               int K, int N, int nbits, int group_size, gemq_stream_t stream) {
  if (!wq || !scales || !zeros || !out_kn || K <= 0 || N <= 0 || group_size <= 0 || nbits < 1 || nbits > 4)
    return GEMQ_ERR_BAD_ARG;
  if (K % group_size != 0) return GEMQ_ERR_BAD_SHAPE;
  unsigned g;
  if (int e = grid1d(static_cast<size_t>(K) * N, 256, &g)) return e;
  dequantize_kernel<<<g, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(wq), static_cast<const __half*>(scales), static_cast<const __half*>(zeros),
      static_cast<__half*>(out_kn), K, N, nbits, group_size);
  return launch_status();
}
