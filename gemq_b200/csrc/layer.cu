// One-token forward of a quantised MoE layer: router, fused gate/up projection,
// SiLU*mul + down projection with the top-k combine folded into its epilogue.
// Three launches, no host involvement between them.
#include <cstdlib>

#include "gemv.cuh"

namespace gemq {

struct DecodeScratch {
  void* gemv_ws;
  size_t gemv_ws_bytes;
  float* h;  // [A*F + shared_ffn] fp32 silu(x1) * x3, written by the gate/up epilogue
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static size_t decode_ws_bytes(const gemq_moe_layer_t* L) {
  const int up_cols = 2 * (L->top_k * L->ffn + L->shared_ffn);
  const int down_cols = (L->top_k + (L->shared_ffn > 0 ? 1 : 0)) * L->hidden;
  const int max_k = L->ffn > L->hidden ? L->ffn : L->hidden;
  const int mk = L->shared_ffn > max_k ? L->shared_ffn : max_k;
  // the one-launch layer kernel keeps the partial sums of its two phases in disjoint columns
  return align_up(gemv_workspace_bytes(up_cols + down_cols, mk, 1), 256);
}

static bool carve(const gemq_moe_layer_t* L, void* scratch, size_t bytes, DecodeScratch* S) {
  const size_t ws = decode_ws_bytes(L);
  const size_t act = align_up(static_cast<size_t>(L->top_k * L->ffn + L->shared_ffn) * sizeof(float), 256);
  if (!scratch || bytes < ws + act || !aligned16(scratch)) return false;
  char* p = static_cast<char*>(scratch);
  S->gemv_ws = p;
  S->gemv_ws_bytes = ws;
  S->h = reinterpret_cast<float*>(p + ws);
  return true;
}

static void stacked_job(GemvJob& J, const gemq_stacked_t& W, const int64_t* idx_slot, int N, int K) {
  J.wq = reinterpret_cast<const uint32_t*>(W.wq);
  J.scales = static_cast<const __half*>(W.scales);
  J.zeros = static_cast<const __half*>(W.zeros);
  J.nbits = W.nbits;
  J.wq_strides = W.wq_strides;
  J.zs_strides = W.zs_strides;
  J.idx = reinterpret_cast<const long long*>(idx_slot);
  J.wq_rows = W.wq_rows;
  J.zs_rows = W.zs_rows;
  J.N = N;
  J.K = K;
  J.n_experts = W.n_experts;
}

static void single_job(GemvJob& J, const gemq_single_t& W, int N, int K) {
  J.wq = reinterpret_cast<const uint32_t*>(W.wq);
  J.scales = static_cast<const __half*>(W.scales);
  J.zeros = static_cast<const __half*>(W.zeros);
  J.fixed_bits = W.nbits;
  J.wq_rows = cdiv(K, 32 / (W.nbits >= 1 && W.nbits <= 4 ? W.nbits : 4));
  J.zs_rows = K / kGroup;
  J.N = N;
  J.K = K;
}

// decode_fused.cu
bool decode_fused_ok(const gemq_moe_layer_t* L, size_t partial_floats);
int launch_decode_fused(const gemq_moe_layer_t* L, const __half* x, __half* out, int64_t* idx, __half* w,
                        int route_in_kernel, int route_mode, float* partial, int* counters, float* h,
                        cudaStream_t stream);

// GEMQ_B200_DECODE=stream selects the three-launch path (router, gate/up GEMV, down GEMV) for
// layers the single-launch kernel would take; read once.
static bool fused_enabled() {
  static const bool on = [] {
    const char* v = getenv("GEMQ_B200_DECODE");
    return !(v && v[0] == 's');
  }();
  return on;
}

}  // namespace gemq

using namespace gemq;

extern "C" size_t gemq_moe_decode_scratch_bytes(const gemq_moe_layer_t* L) {
  if (!L || L->hidden <= 0 || L->ffn <= 0 || L->top_k <= 0) return 0;
  const size_t act = align_up(static_cast<size_t>(L->top_k * L->ffn + L->shared_ffn) * sizeof(float), 256);
  return decode_ws_bytes(L) + act;
}

extern "C" int32_t* gemq_workspace_error_word(void* workspace) {
  return workspace ? static_cast<int32_t*>(workspace) + kErrWord : nullptr;
}

extern "C" int32_t* gemq_workspace_wait_limit_word(void* workspace) {
  return workspace ? static_cast<int32_t*>(workspace) + kLimitWord : nullptr;
}

extern "C" int gemq_moe_decode(const gemq_moe_layer_t* L, const void* x, void* out,
                               int64_t* idx, void* w, int tokens, int do_route, int route_mode,
                               void* scratch, size_t scratch_bytes, gemq_stream_t stream) {
  if (!L || !x || !out || !idx || !w || !L->gate || tokens <= 0) return GEMQ_ERR_BAD_ARG;
  const int D = L->hidden, F = L->ffn, A = L->top_k, SF = L->shared_ffn;
  if (D <= 0 || F <= 0 || A <= 0 || A > kMaxSlots || L->n_experts <= 0 || SF < 0) return GEMQ_ERR_BAD_ARG;
  if (L->group_size != kGroup || D % kGroup || F % kGroup || SF % kGroup) return GEMQ_ERR_BAD_SHAPE;
  if (SF > 0 && (L->s1.group_size != kGroup || L->s3.group_size != kGroup || L->s2.group_size != kGroup))
    return GEMQ_ERR_BAD_SHAPE;
  DecodeScratch S;
  if (!carve(L, scratch, scratch_bytes, &S)) return GEMQ_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  // Single-launch path: router, both projections and the combine in one persistent kernel per token.
  {
    int* counters = static_cast<int*>(S.gemv_ws);
    float* partial = reinterpret_cast<float*>(static_cast<char*>(S.gemv_ws) + kMaxCounters * sizeof(int));
    const size_t partial_floats = (S.gemv_ws_bytes - kMaxCounters * sizeof(int)) / sizeof(float);
    if (fused_enabled() && aligned16(x) && aligned16(out) && aligned16(L->gate) && decode_fused_ok(L, partial_floats)) {
      const bool in_kernel = do_route && L->n_experts <= 32 && A <= L->n_experts && D % 256 == 0;
      if (do_route && !in_kernel) {
        const int rc = gemq_moe_route(x, L->gate, tokens, D, L->n_experts, A, route_mode, L->renorm, 0, idx, w, nullptr,
                                      stream);
        if (rc) return rc;
      }
      for (int t = 0; t < tokens; ++t) {
        const int rc = launch_decode_fused(L, static_cast<const __half*>(x) + static_cast<size_t>(t) * D,
                                           static_cast<__half*>(out) + static_cast<size_t>(t) * D,
                                           idx + static_cast<size_t>(t) * A,
                                           static_cast<__half*>(w) + static_cast<size_t>(t) * A, in_kernel ? 1 : 0,
                                           route_mode, partial, counters, S.h, st);
        if (rc) return rc;
      }
      return GEMQ_OK;
    }
  }

  if (do_route) {
    const int rc = gemq_moe_route(x, L->gate, tokens, D, L->n_experts, A, route_mode, L->renorm, 0, idx, w, nullptr,
                                  stream);
    if (rc) return rc;
  }

  for (int t = 0; t < tokens; ++t) {
    const __half* xt = static_cast<const __half*>(x) + static_cast<size_t>(t) * D;
    const int64_t* idx_t = idx + static_cast<size_t>(t) * A;
    // gate / up projections: x1[a*F + f], x3[a*F + f]; shared experts behind the routed slots
    GemvParams P = {};
    P.T = 1;
    int nj = 0;
    for (int a = 0; a < A; ++a) {
      for (int m = 0; m < 2; ++m) {
        GemvJob& J = P.jobs[nj++];
        stacked_job(J, m ? L->w3 : L->w1, idx_t + a, F, D);
        if (m) {  // w1 and w3 share bit-widths and word offsets (fused_dequant_bmm.py:56-57)
          J.nbits = L->w1.nbits;
          J.wq_strides = L->w1.wq_strides;
        }
        J.xa = xt;
        J.ldx = D;
        if (!m) J.h = S.h + static_cast<size_t>(a) * F;
      }
    }
    if (SF > 0) {
      for (int m = 0; m < 2; ++m) {
        GemvJob& J = P.jobs[nj++];
        single_job(J, m ? L->s3 : L->s1, SF, D);
        J.xa = xt;
        J.ldx = D;
        if (!m) J.h = S.h + static_cast<size_t>(A) * F;
      }
    }
    P.n_jobs = nj;
    P.epi = kEpiUpPair;
    int rc = run_gemv_jobs(P, false, kGroup, S.gemv_ws, S.gemv_ws_bytes, st);
    if (rc) return rc;

    // down projection + combine
    GemvParams Q = {};
    Q.T = 1;
    nj = 0;
    for (int a = 0; a < A; ++a) {
      GemvJob& J = Q.jobs[nj++];
      stacked_job(J, L->w2, idx_t + a, D, F);
      J.xa = reinterpret_cast<const __half*>(S.h + static_cast<size_t>(a) * F);
    }
    if (SF > 0) {
      GemvJob& J = Q.jobs[nj++];
      single_job(J, L->s2, D, SF);
      J.xa = reinterpret_cast<const __half*>(S.h + static_cast<size_t>(A) * F);
    }
    Q.n_jobs = nj;
    Q.epi = kEpiCombine;
    Q.x_f32 = 1;
    // The down projection may resolve its experts ahead of its dependency wait only when the ids
    // are older than the whole chain of launches of this call: supplied by the caller, or written
    // by the router two or more launches back (rows after the first).
    Q.plan_early = (!do_route || t > 0) ? 1 : 0;
    Q.comb_out = static_cast<__half*>(out) + static_cast<size_t>(t) * D;
    Q.comb_w = static_cast<const __half*>(w) + static_cast<size_t>(t) * A;
    Q.comb_weighted = A;
    rc = run_gemv_jobs(Q, false, kGroup, S.gemv_ws, S.gemv_ws_bytes, st);
    if (rc) return rc;
  }
  return GEMQ_OK;
}
