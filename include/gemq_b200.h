/*
 * gemq_b200 -- C ABI of the B200 (sm_100a) kernels for GEMQ's real-quantized MoE
 * inference path.
 *
 * Every entry point takes raw device pointers and explicit extents, launches on
 * the given stream, never allocates, never synchronises and returns 0 or a
 * negative GEMQ_ERR_* code.  "Kernel form" tensors are the ones the reference's
 * kernels consume:
 *   wq      int32 [ceil(K/eps), N] contiguous, eps = 32 / nbits, code k of column n
 *           in word (k / eps, n) at bit (k % eps) * nbits
 *           (gemq/triton_kernels/utils.py:47-70, gemq/inference/moe_block.py:111-119)
 *   scales, zeros  fp16 [K/G, N];  W^T[k,n] = fp16(fma(fp16(q), scales, zeros))
 *           (gemq/triton_kernels/utils.py:206-210)
 *   stacked experts: tensors concatenated along dim 0, nbits[E] int32, wq_strides[E] /
 *           zs_strides[E] int32 element offsets (gemq/inference/moe_block.py:122-142)
 * Expert indices are int64 device tensors as produced by torch.topk
 * (gemq/inference/moe_block.py:213).
 */
#ifndef GEMQ_B200_H_
#define GEMQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* gemq_stream_t; /* cudaStream_t */

enum {
  GEMQ_OK = 0,
  GEMQ_ERR_BAD_ARG = -1,     /* null pointer, non-positive extent, unsupported bit-width */
  GEMQ_ERR_BAD_SHAPE = -2,   /* extents the kernels cannot take (see each function) */
  GEMQ_ERR_WORKSPACE = -3,   /* workspace missing or too small */
  GEMQ_ERR_LAUNCH = -4,      /* CUDA reported a launch error */
  GEMQ_ERR_ALIGN = -5        /* a pointer is not 16-byte aligned */
};

/* Library identification; returns a static string. */
const char* gemq_version(void);

/* Bytes of zero-initialised device workspace the GEMV-family calls need for the
 * given problem: fp32 split-K partials plus arrival counters.  The counters are
 * left at zero by every call, so one memset at allocation time is enough.
 * `total_cols` = columns summed over all (slot, matrix) jobs of a launch,
 * `max_k` = largest reduction length, `tokens` = activation rows. */
size_t gemq_gemv_workspace_bytes(int total_cols, int max_k, int tokens);

/* ---- packing format (gemq/triton_kernels/utils.py) ---------------------------- */

/* pack_weights_over_cols_triton, transpose=False form (utils.py:74-113):
 * codes uint8 [rows, cols] -> int32 [rows, ceil(cols/eps)], tail lanes zero. */
int gemq_pack_over_cols(const uint8_t* codes, int32_t* packed, int rows, int cols, int nbits,
                        gemq_stream_t stream);

/* Kernel-form pack: codes uint8 [N, K] -> int32 [ceil(K/eps), N] contiguous, i.e.
 * pack(..., transpose=True).contiguous() (utils.py:110-111, moe_block.py:111-119). */
int gemq_pack_kernel_form(const uint8_t* codes, int32_t* wq, int N, int K, int nbits, gemq_stream_t stream);

/* unpack_over_cols_triton (utils.py:149-189): int32 [rows, words] -> uint8 [rows, out_cols]. */
int gemq_unpack_over_cols(const int32_t* packed, uint8_t* codes, int rows, int words, int out_cols,
                          int nbits, gemq_stream_t stream);

/* dequantize (utils.py:192-212) materialised: kernel-form -> fp16 W^T [K, N], bit-exact
 * single-rounded fp16 fma. */
int gemq_dequantize(const int32_t* wq, const void* scales, const void* zeros, void* out_kn,
                    int K, int N, int nbits, int group_size, gemq_stream_t stream);

/* ---- decode GEMV family ---------------------------------------------------------- */

/* dequant_splitk_gemv_triton (gemq/triton_kernels/dequant_gemv.py:118-156), extended to
 * `tokens` activation rows: y[t, :] = x[t, :] @ deq(wq).  x fp16 [tokens, K] (row stride
 * ldx), y fp16 [tokens, N] (row stride ldy).  Deterministic (fixed-order split-K). */
int gemq_dequant_gemv(const void* x, int ldx, const int32_t* wq, const void* scales, const void* zeros,
                      void* y, int ldy, int tokens, int N, int K, int nbits, int group_size,
                      void* workspace, size_t workspace_bytes, gemq_stream_t stream);

/* Stacked experts of one projection (all pointers device memory): the tensors the reference's
 * blocks build at gemq/inference/moe_block.py:111-142. */
typedef struct {
  const int32_t* wq;
  const void* scales;
  const void* zeros;
  const int32_t* nbits;      /* [E] */
  const int32_t* wq_strides; /* [E] int32 element offsets into wq */
  const int32_t* zs_strides; /* [E] element offsets into scales/zeros, or NULL: expert e starts at row e*(K/G) */
  int64_t wq_rows;           /* rows (dim 0) of the stacked wq tensor */
  int64_t zs_rows;           /* rows (dim 0) of the stacked scales / zeros tensors */
  int32_t n_experts;         /* E, or 0 when unknown: expert ids read on the device are clamped into [0, E) and an
                                id outside it is reported through the workspace's error word */
} gemq_stacked_t;

/* dequant_sel_splitk_gemv_triton (dequant_gemv.py:225-270): expert idx[0] of stacked tensors
 * (scale rows located as in :203, zs_strides is ignored). */
int gemq_dequant_sel_gemv(const void* x, const int64_t* idx, const gemq_stacked_t* w,
                          void* y, int N, int K, int group_size,
                          void* workspace, size_t workspace_bytes, gemq_stream_t stream);

/* fused_dequant_up_proj_triton (gemq/triton_kernels/fused_dequant_bmm.py:122-173):
 * x1[a*N+n], x3[a*N+n] = x @ deq(w1[idx[a]]), x @ deq(w3[idx[a]]); w3 uses w1's nbits and
 * wq_strides (:56-57,80,98) and both use e*(K/G) scale rows (:62). */
int gemq_fused_up_proj(const void* x, const int64_t* idx, int A,
                       const gemq_stacked_t* w1, const gemq_stacked_t* w3,
                       void* x1, void* x3, int N, int K, int group_size,
                       void* workspace, size_t workspace_bytes, gemq_stream_t stream);

/* fused_dequant_down_proj_triton (fused_dequant_bmm.py:264-312):
 * x2[a*N+n] = (silu(x1[a*K+k]) * x3[a*K+k]) @ deq(w2[idx[a]]). */
int gemq_fused_down_proj(const void* x1, const void* x3, const int64_t* idx, int A,
                         const gemq_stacked_t* w2,
                         void* x2, int N, int K, int group_size,
                         void* workspace, size_t workspace_bytes, gemq_stream_t stream);

/* dequant_group_gemm_triton (gemq/triton_kernels/dequant_group_gemm.py:155-202) for a small
 * number of rows: y[g, t, :] = x[t, :] @ deq(W[indices[g]]), x fp16 [tokens, K] (row stride
 * ldx), y fp16 [A, tokens, N] contiguous.  Per-expert scale offsets come from zs_strides
 * (:75,80-81); one group size for all experts. */
int gemq_dequant_group_gemv(const void* x, int ldx, const int64_t* indices, int A,
                            const gemq_stacked_t* w,
                            void* y, int tokens, int N, int K, int group_size,
                            void* workspace, size_t workspace_bytes, gemq_stream_t stream);

/* ---- routing ------------------------------------------------------------------------ */

/* Router: logits = x @ gate^T, softmax, top-k, optional renormalisation.
 * mode 0: everything rounded through fp16 like the Mixtral one-token path
 *         (gemq/inference/moe_block.py:211-214);
 * mode 1: fp16-rounded logits, fp32 softmax (Mixtral n-token, :174-180);
 * mode 2: fp32 logits and softmax (DeepSeek-V2, :457-464, :499-505).
 * x [tokens, D] fp16 or bf16 (x_is_bf16), gate fp16/bf16 [E, D] in the same dtype.
 * Outputs: idx int64 [tokens, A], weights [tokens, A] in the activation dtype,
 * logits fp32 [tokens, E] (may be NULL). */
int gemq_moe_route(const void* x, const void* gate, int tokens, int D, int E, int A,
                   int mode, int renorm, int x_is_bf16,
                   int64_t* idx, void* weights, float* logits, gemq_stream_t stream);

/* Device address of the int32 error word inside a GEMV-family workspace (also the head of the
 * scratch of gemq_moe_decode).  The decode kernels bound every wait on another CTA or warp; when
 * one runs out, or an expert id read on the device lies outside [0, E), the kernel records a
 * non-zero code here and still returns (its output is then undefined).  0 = nothing happened.
 * After a non-zero code zero-fill the workspace before its next use: the counters and partial
 * sums it holds are no longer in their resting state.  The caller reads and clears the word. */
int32_t* gemq_workspace_error_word(void* workspace);

/* Device address of an int32 the one-launch decode layer reads at start: the number of polls a
 * bounded wait may take (0 = the built-in limit, about 2^18).  Exists so that the expiry path can
 * be exercised from the host without a stuck kernel. */
int32_t* gemq_workspace_wait_limit_word(void* workspace);

/* ---- whole decode layer --------------------------------------------------------------- */

/* One single (non-stacked) quantised matrix, e.g. a DeepSeek-V2 shared-expert projection. */
typedef struct {
  const int32_t* wq;
  const void* scales;
  const void* zeros;
  int nbits;
  int group_size;
} gemq_single_t;

typedef struct {
  int hidden;        /* D */
  int ffn;           /* F */
  int n_experts;     /* E */
  int top_k;         /* A */
  int group_size;    /* block_group_size (moe_block.py:130-134) */
  int route_mode;    /* see gemq_moe_route */
  int renorm;        /* norm_topk_prob */
  int shared_ffn;    /* 0, or n_shared * F (moe_block.py:400-412) */
  const void* gate;  /* fp16 [E, D] */
  gemq_stacked_t w1, w3, w2;
  gemq_single_t s1, s3, s2; /* used when shared_ffn > 0 */
} gemq_moe_layer_t;

/* Device scratch of one decode step; sizes from gemq_moe_decode_scratch_bytes. */
size_t gemq_moe_decode_scratch_bytes(const gemq_moe_layer_t* layer);

/* forward_one_token of QuantFusedMixtralMoEBlock / QuantFusedDeepseekV2MoEBlock
 * (gemq/inference/moe_block.py:200-235, :488-531) applied to `tokens` rows one after the
 * other: route (all rows in one launch), then per row the fused gate/up projection and
 * SiLU*mul + down projection whose epilogue does the top-k weighted combine (+ shared
 * experts).  x, out: fp16 [tokens, D].  idx int64 [tokens, A] and w fp16 [tokens, A] hold the
 * routing: written when do_route != 0 (route_mode as in gemq_moe_route, normally
 * layer->route_mode), read when do_route == 0.  `scratch` must have been zero-filled once
 * before its first use; calls sharing it must be ordered on one stream. */
int gemq_moe_decode(const gemq_moe_layer_t* layer, const void* x, void* out,
                    int64_t* idx, void* w, int tokens, int do_route, int route_mode,
                    void* scratch, size_t scratch_bytes, gemq_stream_t stream);

/* ---- prefill: tcgen05 grouped GEMM ----------------------------------------------------------- */

/* dequant_gemm_triton (gemq/triton_kernels/dequant_gemm.py:150-193) and one group of
 * dequant_group_gemm_triton (dequant_group_gemm.py:155-202) on the tcgen05 tensor cores:
 * y[M, N] = x[M, K] @ deq(W[e]), x and y contiguous fp16 (or bf16 when x_is_bf16; the
 * de-quantised fp16 weights are then rounded to bf16).  `expert` = device pointer to the expert
 * id (NULL: expert 0); nbits / wq_strides / zs_strides may be NULL for a single matrix with
 * fixed_bits.  Needs N % 128 == 0, K % 64 == 0, group_size % 64 == 0.  `err` = one device int32
 * that receives a non-zero code if a bounded wait inside the kernel expired. */
int gemq_dequant_gemm_tc(const void* x, const int64_t* expert, const int32_t* wq, const void* scales,
                         const void* zeros, const int32_t* nbits, const int32_t* wq_strides,
                         const int32_t* zs_strides, int fixed_bits, void* y, int M, int N, int K,
                         int group_size, int x_is_bf16, int32_t* err, gemq_stream_t stream);

/* Device scratch of gemq_moe_prefill for `tokens` rows. */
size_t gemq_moe_prefill_scratch_bytes(const gemq_moe_layer_t* layer, int tokens);

/* forward_n_tokens of the quantised blocks (gemq/inference/moe_block.py:165-198, :448-486)
 * without host synchronisation: route (when do_route), count / scan / scatter the (token, expert)
 * pairs into expert-sorted rows, grouped gate/up GEMM with the SiLU*mul epilogue, grouped down
 * GEMM scaled by the routing weight, per-token combine in expert order, shared experts.
 * x, out: [tokens, D] fp16 or bf16; idx int64 [tokens, A]; w [tokens, A] in the activation dtype;
 * logits fp32 [tokens, E] or NULL.  With do_route the gate of `layer` (fp16) is used, so bf16
 * callers route first (gemq_moe_route) and pass do_route = 0. */
int gemq_moe_prefill(const gemq_moe_layer_t* layer, const void* x, void* out, int64_t* idx, void* w,
                     float* logits, int tokens, int do_route, int route_mode, int x_is_bf16,
                     void* scratch, size_t scratch_bytes, gemq_stream_t stream);

/* Device address of the error word gemq_moe_prefill writes in `scratch` (0 = every wait was met). */
const int32_t* gemq_moe_prefill_error_word(const gemq_moe_layer_t* layer, int tokens, void* scratch);

/* ---- expert-parallel prefill: the token exchange around the local grouped GEMM ---------------- */

/* No counterpart in the reference (its n-token forward, gemq/inference/moe_block.py:165-198,
 * loops over the experts of one GPU).  With the experts spread over `world` ranks these four
 * calls are the device side of the all-to-all form of that loop; the collectives themselves are
 * the caller's (NCCL).  A placement table says where expert e lives: replica j (j < replicas) on
 * rank rank_tab[e*replicas + j], at position local_tab[e*replicas + j] among that rank's experts,
 * taking the sender's rows of e whose position, as a fraction of the sender's rows of e, is below
 * upper_tab[e*replicas + j] and not below the previous replica's bound (unused replicas: 2.0).
 *
 * gemq_ep_plan: sel int64 [pairs] (= [tokens, top_k] flattened) ->
 *   order int64 [pairs]       pair indices sorted by (destination rank, expert), ties by pair index
 *   loc_sorted int32 [pairs]  position of the pair's expert on its destination, in that order
 *   where int64 [pairs]       inverse permutation: row of pair i in the sorted order
 *   send_counts int64 [world] pairs per destination
 * One launch, no host read.  scratch: gemq_ep_plan_scratch_bytes(pairs), zero-filled once; its
 * first int32 receives a non-zero code when an id lies outside [0, n_experts) (the id is clamped). */
size_t gemq_ep_plan_scratch_bytes(int pairs);
int gemq_ep_plan(const int64_t* sel, int pairs, int n_experts, int world, int replicas, const int32_t* rank_tab,
                 const int32_t* local_tab, const float* upper_tab, int64_t* order, int32_t* loc_sorted, int64_t* where,
                 int64_t* send_counts, void* scratch, size_t scratch_bytes, gemq_stream_t stream);

/* payload [pairs, D + 8] (16-bit elements): row p = the token row of pair order[p], then the
 * int32 loc_sorted[p], the pair's 16-bit routing weight and zero padding.  D % 8 == 0. */
int gemq_ep_pack_rows(const void* x, const int64_t* order, const int32_t* loc_sorted, const void* weights, int pairs,
                      int top_k, int D, void* payload, gemq_stream_t stream);

/* The inverse on the receiving rank: payload [rows, D + 8] -> x [rows, D], expert int64 [rows],
 * weights 16-bit [rows]. */
int gemq_ep_unpack_rows(const void* payload, int rows, int D, void* x, int64_t* expert, void* weights,
                        gemq_stream_t stream);

/* out [tokens, D] = the token's top_k returned rows back[where[token*top_k + slot]] added in
 * increasing expert id (ties by slot), rounded to the activation type after every addition: the
 * index_add_ order of gemq/inference/moe_block.py:191-195. */
int gemq_ep_combine(const void* back, const int64_t* where, const int64_t* sel, int tokens, int top_k, int D,
                    int is_bf16, void* out, gemq_stream_t stream);

/* ---- for callers that cannot allocate --------------------------------------------------------- */

/* No counterpart in the reference.  y[1, N] = x[1, K] @ deq(wq), the same result as
 * gemq_dequant_gemv with tokens == 1, but without a caller-provided workspace: the split-K
 * scratch lives in a fixed 2 MiB device array inside the library (gemq_static_scratch_bytes),
 * held by every GPU that loads the library until the process exits.  No device memory is
 * allocated or freed, here or in anything it calls.  For hosts that must not allocate device
 * memory on this path: a serving process with a frozen memory pool, a plugin inside a runtime
 * that forbids cudaMalloc after start-up.
 *   - Returns GEMQ_ERR_WORKSPACE when gemq_gemv_workspace_bytes(N, K, 1) exceeds the array
 *     (roughly N * ceil(K / 512) > 490,000; the sizing rule reserves room for an activation
 *     staging area this entry point does not use, so the limit is a little conservative),
 *     GEMQ_ERR_BAD_ARG on null pointers or bad extents.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress), and the first launch of each kernel on a device sets its
 *     shared-memory attribute; the first use of a weight tensor adds an entry to a small
 *     host-side cache of TMA descriptors (host heap only).  Make the first call for a device and
 *     a weight tensor outside any stream capture.
 *   - The device that owns `stream` must be the current device of the calling thread: the
 *     array's address is looked up for the current device.
 *   - All calls on a device share the one array, and the array keeps what the last call left
 *     in it; every call first clears the part it reads.  Two calls that overlap on the GPU
 *     (different streams, no ordering between them) race on it: order them. */
int gemq_dequant_gemv_static(const void* x, const int32_t* wq, const void* scales, const void* zeros,
                             void* y, int N, int K, int nbits, int group_size, gemq_stream_t stream);

/* Capacity in bytes of the built-in scratch used by gemq_dequant_gemv_static. */
size_t gemq_static_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
#endif /* GEMQ_B200_H_ */
