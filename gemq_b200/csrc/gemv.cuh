// Decode GEMV family: job/parameter structures shared by the kernels and the
// host-side launchers.
//
// A launch covers a list of "jobs".  One job is one quantised matrix times one
// activation (vector or a few rows): (expert slot a, projection m) of a fused
// up/down projection, or a single matrix.  Which expert a slot refers to, and
// therefore the bit-width and the weight offset, is read from device memory by
// the kernel (the routing result never visits the host).
#pragma once

#include "common.cuh"

namespace gemq {

constexpr int kCtaWarps = 4;
constexpr int kCtaThreads = 32 * kCtaWarps;
constexpr int kCtaCols = 32 * kCtaWarps;  // output columns per CTA, 32 per warp
constexpr int kMaxSlots = 8;              // top-k bound of a fused launch
constexpr int kMaxJobs = 2 * kMaxSlots + 2;
constexpr int kGroup = 128;               // group size of the tensor-core path
constexpr int kSliceGroups = 8;           // k-slice of a CTA: 8 groups (1/2/4-bit)
constexpr int kSliceGroupsB3 = 10;        //                   10 groups (3-bit: two 640-wide spans)
constexpr int kRing = 8;                  // 128-bit weight loads in flight per lane
constexpr int kMaxCounters = 8192;        // arrival counters at the head of the workspace
constexpr int kErrWord = kMaxCounters - 1;   // error code of the decode kernels (0 = none)
constexpr int kLimitWord = kMaxCounters - 4; // caller-set poll limit of the layer kernel's bounded waits (0 = built in)
constexpr int kMaxFamilies = 4;           // distinct (wq, scales, zeros) tensor triples per launch
constexpr int kMaxMaps = 3 * kMaxFamilies;

struct GemvJob {
  const uint32_t* wq;      // stacked (or single) packed words
  const __half* scales;
  const __half* zeros;
  const int* nbits;        // [E] or nullptr -> fixed_bits
  const int* wq_strides;   // [E] word offsets or nullptr -> 0
  const int* zs_strides;   // [E] element offsets or nullptr -> e * (K/G) * N
  const long long* idx;    // address of this job's expert id, nullptr -> expert 0
  int n_experts;           // experts in the stacked tensors (0: unknown); ids are clamped into [0, n_experts)
  const __half* xa;        // activation rows [T, K]; with SILU: x1 of this slot
  const __half* xb;        // with SILU: x3 of this slot
  __half* y;               // output rows [T, N] (may be nullptr in combine mode)
  float* h;                // up-pair epilogue: fp32 silu(x1)*x3 of this slot (first job of a pair), or nullptr
  int fixed_bits;
  int N, K;
  int ldx, ldy;
  int col_base;            // first column of this job inside a partial row
  int tile_base;           // first blockIdx.x of this job
  int chunk_base;          // first arrival counter of this job (shared by the jobs of a finish group)
  int map_base;            // persistent kernel: index of this job's wq tensor map (+1 scales, +2 zeros)
  int mask_base;           // persistent kernel: first counter word holding, per column chunk, the set of partial slots in use
  long long wq_rows;       // host: rows of the wq tensor (tensor-map extent)
  long long zs_rows;       // host: rows of the scales / zeros tensors
};

// How a finished column chunk is turned into outputs (persistent kernel).
enum { kEpiStore = 0,   // y = fp16(sum), each job on its own
       kEpiUpPair = 1,  // jobs (2i, 2i+1) = gate/up projection of one slot: x1, x3 and h = silu(x1)*x3
       kEpiCombine = 2  // all jobs: weighted top-k combine (+ unit-weight shared experts)
};

struct alignas(64) GemvParams {
  CUtensorMap maps[kMaxMaps];  // persistent kernel: tiled TMA descriptors of the weight / metadata tensors
  GemvJob jobs[kMaxJobs];
  int n_jobs;
  int T;           // activation rows
  int G;           // group size (generic kernel only; the tensor-core path needs 128)
  int s_max;       // k-slices reserved per column chunk in the tile numbering
  int c_total;     // columns over all jobs = length of one partial row
  int n_chunks;    // arrival counters per token block
  float* partial;  // [s_max][T][c_total]
  int* counters;   // zero on entry, zero on exit
  // Fused top-k combine (decode down projection, T == 1): the CTA that completes a
  // column chunk over ALL jobs writes comb_out = sum_a comb_w[a] * fp16(x2[a]) for the
  // first comb_weighted jobs, then adds the remaining jobs with weight one.
  __half* comb_out;
  const __half* comb_w;
  int comb_weighted;
  int epi;         // kEpi* (persistent kernel)
  int x_f32;       // activations are fp32 vectors (persistent kernel, e.g. h from the up-pair epilogue)
  // The expert ids, bit widths and offsets the jobs point to were final before the previous
  // kernel of the stream started: the persistent kernel may resolve them while that kernel
  // still runs, ahead of its dependency wait.
  int plan_early;
};

struct ResolvedJob {
  const uint32_t* wq;
  const __half* scales;
  const __half* zeros;
  int bits;
  int slices;
};

__device__ __forceinline__ int slice_groups(int bits) { return bits == 3 ? kSliceGroupsB3 : kSliceGroups; }

__device__ __forceinline__ ResolvedJob resolve_job(const GemvJob& J, int G) {
  ResolvedJob R;
  int e = J.idx ? static_cast<int>(*J.idx) : 0;
  if (J.n_experts > 0) e = e < 0 ? 0 : (e >= J.n_experts ? J.n_experts - 1 : e);
  R.bits = J.nbits ? J.nbits[e] : J.fixed_bits;
  const int ngroups = J.K / G;
  const size_t zoff = J.zs_strides ? static_cast<size_t>(J.zs_strides[e])
                                   : static_cast<size_t>(e) * ngroups * J.N;
  R.wq = J.wq + (J.wq_strides ? static_cast<size_t>(J.wq_strides[e]) : 0);
  R.scales = J.scales + zoff;
  R.zeros = J.zeros + zoff;
  R.slices = cdiv(ngroups, slice_groups(R.bits));
  return R;
}

// Launch the jobs in P (tensor-core path when every job qualifies, generic kernel
// otherwise).  Defined in gemv.cu.
int run_gemv_jobs(GemvParams& P, bool silu, int G, void* workspace, size_t workspace_bytes, cudaStream_t stream);
size_t gemv_workspace_bytes(int total_cols, int max_k, int tokens);
// Persistent bulk-copy kernel for one activation row (gemv_stream.cu).
int launch_stream(GemvParams& P, float* partial, size_t partial_floats, int* counters, cudaStream_t stream);
int silu_mul_f32(const __half* x1, const __half* x3, float* h, int n, cudaStream_t stream);

}  // namespace gemq
