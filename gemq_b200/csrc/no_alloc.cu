// gemq_dequant_gemv_static: the single-matrix decode GEMV for callers that cannot allocate.
//
// Some hosts of this library own no allocator they may call on the hot path: a serving
// process whose memory pool is frozen after start-up, a plugin loaded into a runtime that
// forbids cudaMalloc once the model is resident.  They can still pass inputs and outputs, but
// not the zero-initialised split-K
// workspace the other GEMV entry points ask for.  This variant keeps that workspace in a
// fixed array that is part of the library image, so it exists (2 MiB on every GPU that
// loads the library, until the process exits) without any allocation call.
#include <mutex>

#include "gemv.cuh"

namespace gemq {

constexpr size_t kStaticScratchBytes = 2u << 20;  // 32 KB of arrival counters + fp32 split-K partial slots

// Device-side storage.  In host code the name `g_static_scratch` is only a handle for
// cudaGetSymbolAddress -- it is NOT a device address and must never be handed to a kernel.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of the array on the current device, looked up once per device.  The device
// of the stream a caller passes must be the current one: the lookup resolves against it.
static int static_scratch_ptr(void** out) {
  static std::mutex mu;
  static void* cached[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return GEMQ_ERR_LAUNCH;
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);  // resolves against the current device
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return GEMQ_ERR_LAUNCH;
    }
    cached[dev] = p;
  }
  *out = cached[dev];
  return GEMQ_OK;
}

}  // namespace gemq

using namespace gemq;

extern "C" size_t gemq_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int gemq_dequant_gemv_static(const void* x, const int32_t* wq, const void* scales, const void* zeros,
                                        void* y, int N, int K, int nbits, int group_size, gemq_stream_t stream) {
  if (!x || !wq || !scales || !zeros || !y || N <= 0 || K <= 0 || group_size <= 0 || nbits < 1 || nbits > 4)
    return GEMQ_ERR_BAD_ARG;
  // Same sizing rule as gemq_gemv_workspace_bytes, against the fixed capacity.
  const size_t need = gemv_workspace_bytes(N, K, 1);
  if (need > kStaticScratchBytes) return GEMQ_ERR_WORKSPACE;  // problem too large for the built-in scratch
  void* ws = nullptr;
  if (int rc = static_scratch_ptr(&ws)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left.  Kernels leave counters and partial slots
  // at zero, but a call that was cut short would not have: clear the part this call reads.
  if (cudaMemsetAsync(ws, 0, need, st) != cudaSuccess) return GEMQ_ERR_LAUNCH;
  GemvParams P = {};
  P.n_jobs = 1;
  P.T = 1;
  GemvJob& J = P.jobs[0];
  J.wq = reinterpret_cast<const uint32_t*>(wq);
  J.scales = static_cast<const __half*>(scales);
  J.zeros = static_cast<const __half*>(zeros);
  J.fixed_bits = nbits;
  J.xa = static_cast<const __half*>(x);
  J.y = static_cast<__half*>(y);
  J.N = N; J.K = K; J.ldx = K; J.ldy = N;
  J.wq_rows = cdiv(K, 32 / nbits);
  J.zs_rows = K / group_size;
  return run_gemv_jobs(P, false, group_size, ws, kStaticScratchBytes, st);
}
