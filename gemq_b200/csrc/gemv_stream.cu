// Persistent, TMA fed dequant GEMV for one activation row (decode batch 1).
//
// One CTA per SM.  The launch's work is cut into units of 64 packed word rows x 128
// output columns of one job (32 KB of codes plus the group metadata: 2048 / 1024 / 640 /
// 512 reduction elements at 1 / 2 / 3 / 4 bits).  Units are ordered job-major, column
// chunk-major, k-slice-minor and dealt to the CTAs in contiguous, byte-balanced ranges, so
// a CTA usually owns several slices of a chunk and keeps their running sum in registers.
// Inside a CTA four roles run concurrently:
//   * a producer warp streams the units into a 4-stage shared-memory ring with tiled TMA
//     (cp.async.bulk.tensor.2d on the [word rows, N] tensors as they are: four 128B-swizzled
//     boxes of 64 rows x 32 columns plus 4-row boxes of scales and offsets per unit,
//     completion through mbarrier transaction counts);
//   * two table warps (alternate units) turn the activation slice of each unit into the
//     operand table of that unit, in a six-slot ring of its own: signed base-256 digit planes
//     for the integer MMA of the 1/2/4-bit units, pre-scaled fp16 values for the 3-bit ones;
//   * sixteen consumer warps in two groups that take alternate units (4 column strips x 2 row
//     halves each) feed the packed words, masked in place, to mma.sync as the A operand and
//     accumulate over the consecutive slices of a part in registers;
//   * a finisher warp adds the four row parts in a fixed order and writes the result:
//     directly when this CTA covered the whole reduction of a plain GEMV, otherwise through
//     zero-restoring fp32 partial slots, a per-chunk set of slots in use and an arrival counter
//     (the warp that completes a finish group adds the slots in order and runs the epilogue).
//     Global-memory latency of this protocol never stalls the consumers.
// Every wait is bounded: on expiry the kernel records an error code and keeps going.
#include "gemv.cuh"
#include "ptx.cuh"

namespace gemq {

constexpr int kSConsumers = 16;
constexpr int kWarpProducer = kSConsumers;
constexpr int kWarpTable = kSConsumers + 1;   // first of kTableWarps table warps (they take alternate units)
constexpr int kTableWarps = 2;
constexpr int kWarpFinisher = kWarpTable + kTableWarps;
constexpr int kSWarps = kWarpFinisher + 1;
constexpr int kSThreads = 32 * kSWarps;
constexpr int kSStages = 4;
constexpr int kTabSlots = 6;
constexpr int kRedSlots = 4;
constexpr int kUnitRows = 64;
constexpr int kStripBytes = kUnitRows * 128;  // one TMA box: 64 word rows x 32 columns, 128B-swizzled
constexpr int kMaxUnitGroups = 16;
constexpr int kErrSlot = kErrWord;


enum { kErrBadExpert = 7, kErrFullWait = 1, kErrEmptyWait = 2, kErrRedFullWait = 3, kErrRedEmptyWait = 4, kErrTabFullWait = 5, kErrTabEmptyWait = 6 };

struct StageBuf {
  alignas(1024) unsigned char words[4 * kStripBytes];
  alignas(16) __half scales[kMaxUnitGroups][128];
  alignas(16) __half zeros[kMaxUnitGroups][128];
};

// Activation operand table of one unit.  The tables sit in a ring of their own, deeper than the
// data ring, so that building one (a few hundred dependent instructions on a single warp that
// shares its scheduler with four busy consumer warps) is never on the refill path of a stage.
struct TableBuf {
  // 1/2/4-bit: [3 digit planes][64 rows][8/B words of s8 digits], planes padded apart (kPlaneStride);
  // 3-bit: [2 variants][64 rows][16 halves]
  alignas(16) uint32_t tab[1536 + 16];
  float xsum[kMaxUnitGroups];       // sum of the activations of each group
  float fin[kMaxUnitGroups];        // power of two that undoes the operand scaling of each group
};

struct JobInfo {
  int wq_row0, zs_row0;  // first row of the job's expert inside the stacked tensors
  int map_base;
  int bits, slices, nch, groups_per_unit, ngroups, kw;
};

struct Range {
  int job, ulo, uhi;
  int rev;  // walk the range from its last chunk to its first
};

struct StreamSmem {
  StageBuf stage[kSStages];
  TableBuf table[kTabSlots];
  alignas(16) float red[kRedSlots][4][128];
  alignas(16) uint32_t zero_row[16];
  alignas(8) unsigned long long full[kSStages], empty[kSStages], tfull[kTabSlots], tempty[kTabSlots], redfull[kRedSlots],
      redempty[kRedSlots];
  JobInfo info[kMaxJobs];
  Range ranges[kMaxJobs];
  int n_ranges;
};

struct Unit {
  int job, slice, chunk, bits;
  int n0, ncols, g0, ng, wr0, nrows;
};

// A run of consecutive k-slices [sa, sb) of one column chunk of one job.
struct Part {
  int job, chunk, sa, sb;
};

__device__ __forceinline__ void mma16816s(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- unit geometry and the per-CTA plan -------------------------------------------------
__device__ __forceinline__ int unit_groups(int bits) { return bits == 3 ? 5 : 16 / bits; }

__device__ __forceinline__ void make_unit(const GemvJob& J, const JobInfo& I, int job, int slice, int chunk, Unit& U) {
  U.job = job; U.slice = slice; U.chunk = chunk; U.bits = I.bits;
  U.n0 = chunk * 128;
  U.ncols = min(128, J.N - U.n0);
  U.g0 = slice * I.groups_per_unit;
  U.ng = min(I.groups_per_unit, I.ngroups - U.g0);
  U.wr0 = slice * kUnitRows;
  U.nrows = I.bits == 3 ? min(kUnitRows, I.kw - U.wr0) : U.ng * (4 * I.bits);
}

// Walks this CTA's parts in order; identical in every role.  The ranges of odd jobs of a fused
// launch are walked backwards: the chunks of a finish group (gate and up member, or the experts
// of a combine) are then completed about as often by the even job's CTA as by the odd job's, and
// with them the draining of the partial slots, which otherwise piles up on the odd jobs' CTAs.
struct PartWalk {
  int r, u;
  __device__ __forceinline__ static int first(const Range& R) { return R.rev ? R.uhi : R.ulo; }
  __device__ __forceinline__ void begin(const StreamSmem& S) {
    r = 0;
    u = S.n_ranges > 0 ? first(S.ranges[0]) : 0;
  }
  __device__ __forceinline__ bool next(const StreamSmem& S, Part& Pt) {
    while (r < S.n_ranges && (S.ranges[r].rev ? u <= S.ranges[r].ulo : u >= S.ranges[r].uhi)) {
      ++r;
      if (r < S.n_ranges) u = first(S.ranges[r]);
    }
    if (r >= S.n_ranges) return false;
    const Range& R = S.ranges[r];
    const int sl = S.info[R.job].slices;
    Pt.job = R.job;
    if (R.rev) {
      Pt.chunk = (u - 1) / sl;
      const int lo = max(R.ulo, Pt.chunk * sl);
      Pt.sa = lo - Pt.chunk * sl;
      Pt.sb = u - Pt.chunk * sl;
      u = lo;
    } else {
      Pt.chunk = u / sl;
      Pt.sa = u - Pt.chunk * sl;
      Pt.sb = min(sl, Pt.sa + (R.uhi - u));
      u += Pt.sb - Pt.sa;
    }
    return true;
  }
};

// The launch parameters a plan lane needs.  They sit in the constant bank, cold at kernel
// start, and do not depend on earlier kernels: they are read ahead of the dependency wait.
struct PlanArgs {
  const long long* idx;
  const int* nbits;
  const int* wq_strides;
  const int* zs_strides;
  int fixed_bits, N, K, map_base, n_experts;
};

__device__ __forceinline__ void read_plan_args(const GemvParams& P, PlanArgs& A) {
  const int lane = threadIdx.x & 31;
  if (lane < P.n_jobs) {
    const GemvJob& J = P.jobs[lane];
    A.idx = J.idx; A.nbits = J.nbits; A.wq_strides = J.wq_strides; A.zs_strides = J.zs_strides;
    A.fixed_bits = J.fixed_bits; A.N = J.N; A.K = J.K; A.map_base = J.map_base; A.n_experts = J.n_experts;
  }
}

// Warp 0: one lane per job resolves the expert (two dependent global loads) and sizes the
// job; a warp scan of the byte costs then gives this CTA its contiguous unit range per job.
__device__ void make_plan(StreamSmem& S, const GemvParams& P, const PlanArgs& J) {
  const int lane = threadIdx.x & 31;
  unsigned n_units = 0, unit_cost = 1;
  if (lane < P.n_jobs) {
    int e = J.idx ? static_cast<int>(*J.idx) : 0;
    if (J.n_experts > 0 && (e < 0 || e >= J.n_experts)) {  // never index the tables with a bad id
      atomicExch(P.counters + kErrSlot, kErrBadExpert);
      e = e < 0 ? 0 : J.n_experts - 1;
    }
    const int bits = J.nbits ? J.nbits[e] : J.fixed_bits;
    JobInfo I;
    I.ngroups = J.K / kGroup;
    I.wq_row0 = J.wq_strides ? J.wq_strides[e] / J.N : 0;
    I.zs_row0 = J.zs_strides ? J.zs_strides[e] / J.N : e * I.ngroups;
    I.map_base = J.map_base;
    I.bits = bits < 1 ? 1 : (bits > 4 ? 4 : bits);
    I.groups_per_unit = unit_groups(I.bits);
    I.slices = cdiv(I.ngroups, I.groups_per_unit);
    I.nch = cdiv(J.N, 128);
    I.kw = cdiv(J.K, 32 / I.bits);
    S.info[lane] = I;
    Unit U;
    make_unit(P.jobs[lane], I, lane, I.slices - 1, 0, U);
    const unsigned chunk_cost = (I.slices - 1) * (kUnitRows + I.groups_per_unit) + U.nrows + U.ng;  // x 512 B
    unit_cost = max(1u, chunk_cost / I.slices);
    n_units = static_cast<unsigned>(I.nch) * I.slices;
  }
  const unsigned w = n_units * unit_cost;
  unsigned incl = w;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  const unsigned total = __shfl_sync(0xffffffffu, incl, 31);
  const unsigned prefix = incl - w;
  unsigned lo, hi;
  if (total < 0xffffffffu / (gridDim.x + 1)) {  // the usual case: no 64-bit division on the critical path
    lo = total * blockIdx.x / gridDim.x;
    hi = total * (blockIdx.x + 1) / gridDim.x;
  } else {
    lo = static_cast<unsigned>(static_cast<unsigned long long>(total) * blockIdx.x / gridDim.x);
    hi = static_cast<unsigned>(static_cast<unsigned long long>(total) * (blockIdx.x + 1) / gridDim.x);
  }
  unsigned ulo = lo <= prefix ? 0u : (lo - prefix + unit_cost - 1) / unit_cost;
  unsigned uhi = hi <= prefix ? 0u : (hi - prefix + unit_cost - 1) / unit_cost;
  ulo = min(ulo, n_units);
  uhi = min(uhi, n_units);
  const bool have = uhi > ulo;
  const unsigned ballot = __ballot_sync(0xffffffffu, have);
  if (have) {
    Range R;
    R.job = lane; R.ulo = static_cast<int>(ulo); R.uhi = static_cast<int>(uhi);
    R.rev = (P.epi != kEpiStore) && (lane & 1);
    S.ranges[__popc(ballot & ((1u << lane) - 1u))] = R;
  }
  if (lane == 0) S.n_ranges = __popc(ballot);
}

// ---- producer ---------------------------------------------------------------------------
__device__ void producer_role(StreamSmem& S, const GemvParams& P, int* err) {
  const int lane = threadIdx.x & 31;
  PartWalk W;
  W.begin(S);
  Part Pt;
  int it = 0;
  while (W.next(S, Pt)) {
    const GemvJob& J = P.jobs[Pt.job];
    const JobInfo& I = S.info[Pt.job];
    for (int sl = Pt.sa; sl < Pt.sb; ++sl, ++it) {
      Unit U;
      make_unit(J, I, Pt.job, sl, Pt.chunk, U);
      const int st = it % kSStages;
      const uint32_t par = (it / kSStages) & 1;
      StageBuf& B = S.stage[st];
      mbar_wait(&S.empty[st], par ^ 1, err, kErrEmptyWait);
      const int nstrips = U.ncols / 32, nmeta = (U.ng + 3) / 4;
      if (lane == 0) mbar_arrive_expect_tx(&S.full[st], nstrips * kStripBytes + 2 * nmeta * 1024);
      __syncwarp();
      if (lane < nstrips) {
        tma_load_2d(B.words + lane * kStripBytes, &P.maps[I.map_base], U.n0 + 32 * lane, I.wq_row0 + U.wr0,
                    &S.full[st]);
      } else if (lane >= 4 && lane < 4 + 2 * nmeta) {
        const int t = (lane - 4) & 1, q = (lane - 4) >> 1;
        tma_load_2d(t ? static_cast<void*>(B.zeros[4 * q]) : static_cast<void*>(B.scales[4 * q]),
                    &P.maps[I.map_base + 1 + t], U.n0, I.zs_row0 + U.g0 + 4 * q, &S.full[st]);
      }
    }
  }
}

// ---- activation tables ----------------------------------------------------------------
// c = 14 - floor(log2(max|x|)) of a group: the largest value lands in [2^14, 2^15).
__device__ __forceinline__ int scale_exponent(float mx) {
  int c = 14 - (static_cast<int>((__float_as_uint(mx) >> 23) & 0xffu) - 127);
  return c < -15 ? -15 : (c > 40 ? 40 : c);
}

// ---- 1/2/4-bit units: integer operands ------------------------------------------------------
// A word ANDed with a per-byte mask is a ready u8 A operand of mma.sync.m16n8k32 (u8 x s8 ->
// s32) with four codes in it, each shifted left by its position inside the byte: code j of a
// word (bit B*j) sits in byte j / (8/B) at in-byte position B * (j % (8/B)); operand q of a
// word collects the codes {y * 8/B + q : y = 0..3}, all at position pos = B*q.  One AND per
// four codes, no shifts.
// The activations of a group are scaled by 2^(c - pos) so that the largest lies in
// [2^20, 2^21), rounded to an integer and split into three balanced base-256 digits
// (each in [-128, 127]).  Digit plane pl of the table is an s8 B operand worth 256^pl; the
// planes of two consecutive groups occupy MMA columns 0..2 and 4..6.  The integer
// accumulation is exact.  (mma.sync with e4m3 operands would need half as many planes, but
// on sm_100a it costs 23 to 44 issue cycles once its operands change between instructions,
// against 8 for the integer form; the 4-bit integer forms are slower still.)
template <int B>
struct I8Fmt {
  static constexpr int kCpb = 8 / B;      // codes per byte = operands per word
  static constexpr int kWin = 2 * B;      // loop iterations per pair of groups
  static constexpr int kPlaneStride = 64 * kCpb + (B == 1 ? 4 : (B == 2 ? 16 : 8));  // words; the pad spreads the planes over the banks
  static constexpr uint32_t kMask = ((1u << B) - 1u) * 0x01010101u;
  __device__ static __forceinline__ uint32_t operand(uint32_t w, int q) { return w & (kMask << (B * q)); }
};

// c = 20 - floor(log2(max|x|)) of a group: the largest scaled value lands in [2^20, 2^21).
__device__ __forceinline__ int scale_exponent_i8(float mx) {
  int c = 20 - (static_cast<int>((__float_as_uint(mx) >> 23) & 0xffu) - 127);
  return c < -60 ? -60 : (c > 60 ? 60 : c);
}

// Rounds v (|v| < 2^21) to an integer iv and returns a word whose bytes 0 and 1 are the two low
// balanced digits of iv plus 128 and whose byte 2 is 64 plus the top digit: adding
// 1.5 * 2^23 + 0x8080 leaves iv + 0x8080 in the low mantissa bits.
__device__ __forceinline__ uint32_t digits_word(float x, float f) { return __float_as_uint(fmaf(x, f, 12615808.0f)); }

// Lane handles word rows `lane` and `lane + 32`.  A group is 4*B consecutive rows, so its
// maximum and sum are reductions over 4*B neighbouring lanes.
template <int B>
__device__ __forceinline__ void build_table_i8(TableBuf& T, const void* x, const Unit& U, bool XF32) {
  using F = I8Fmt<B>;
  constexpr int EPS = 32 / B, CPB = F::kCpb, LPG = 4 * B;
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int row = lane + 32 * rr;
    const bool on = row < U.nrows;
    float xv[EPS];
    if (on) {
      const size_t k = static_cast<size_t>(U.g0) * kGroup + static_cast<size_t>(row) * EPS;
      if (XF32) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(x) + k);
#pragma unroll
        for (int i = 0; i < EPS / 4; ++i) {
          const float4 t = p[i];
          xv[4 * i] = t.x; xv[4 * i + 1] = t.y; xv[4 * i + 2] = t.z; xv[4 * i + 3] = t.w;
        }
      } else {
        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const __half*>(x) + k);
#pragma unroll
        for (int i = 0; i < EPS / 8; ++i) {
          const uint4 t = p[i];
          const __half2* h = reinterpret_cast<const __half2*>(&t);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = __half22float2(h[q]);
            xv[8 * i + 2 * q] = f.x; xv[8 * i + 2 * q + 1] = f.y;
          }
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < EPS; ++i) xv[i] = 0.f;
    }
    float mx = 0.f, sm = 0.f;
#pragma unroll
    for (int i = 0; i < EPS; ++i) { mx = fmaxf(mx, fabsf(xv[i])); sm += xv[i]; }
#pragma unroll
    for (int o = 1; o < LPG; o <<= 1) {
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      sm += __shfl_xor_sync(0xffffffffu, sm, o);
    }
    const int c = scale_exponent_i8(mx);
    if (on && (lane % LPG) == 0) {
      T.xsum[row / LPG] = sm;
      T.fin[row / LPG] = pow2i(-c);
    }
    if (on) {
      constexpr int QB = CPB >= 4 ? 4 : CPB;  // operands per store
      const float fb = pow2i(c);
#pragma unroll
      for (int q0 = 0; q0 < CPB; q0 += QB) {
        uint32_t pl[3][QB];
#pragma unroll
        for (int qq = 0; qq < QB; ++qq) {
          const int q = q0 + qq;
          const float f = fb * (1.0f / static_cast<float>(1 << (B * q)));
          uint32_t e[4];
#pragma unroll
          for (int y = 0; y < 4; ++y) e[y] = digits_word(xv[y * CPB + q], f);
          // digit d of the four values goes to byte y of plane word d
          const uint32_t x01 = __byte_perm(e[0], e[1], 0x5410), x23 = __byte_perm(e[2], e[3], 0x5410);
          pl[0][qq] = __byte_perm(x01, x23, 0x6420) ^ 0x80808080u;
          pl[1][qq] = __byte_perm(x01, x23, 0x7531) ^ 0x80808080u;
          const uint32_t t = __byte_perm(__byte_perm(e[0], e[1], 0x0062), __byte_perm(e[2], e[3], 0x0062), 0x5410) ^ 0x40404040u;
          pl[2][qq] = t | ((t & 0x40404040u) << 1);  // sign-extend the 7-bit top digit
        }
#pragma unroll
        for (int p = 0; p < 3; ++p) {
          uint32_t* dst = T.tab + p * F::kPlaneStride + row * CPB + q0;
          if (QB == 4) *reinterpret_cast<uint4*>(dst) = make_uint4(pl[p][0], pl[p][1], pl[p][2], pl[p][3]);
          else *reinterpret_cast<uint2*>(dst) = make_uint2(pl[p][0], pl[p][1]);
        }
      }
    }
  }
}

// 3-bit: element-wise, one group (128 elements, 4 per lane) at a time.
__device__ __forceinline__ void build_table_b3(TableBuf& T, const void* x, const Unit& U, bool XF32) {
  const int lane = threadIdx.x & 31;
  uint4* z4 = reinterpret_cast<uint4*>(T.tab);
#pragma unroll
  for (int i = 0; i < 8; ++i) z4[lane + 32 * i] = make_uint4(0u, 0u, 0u, 0u);
  __syncwarp();
  __half* tab = reinterpret_cast<__half*>(T.tab);
  for (int gq = 0; gq < U.ng; ++gq) {
    float xv[4];
    float mx = 0.f, sm = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const size_t k = static_cast<size_t>(U.g0 + gq) * kGroup + i * 32 + lane;
      xv[i] = XF32 ? static_cast<const float*>(x)[k] : __half2float(static_cast<const __half*>(x)[k]);
      mx = fmaxf(mx, fabsf(xv[i]));
      sm += xv[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      sm += __shfl_xor_sync(0xffffffffu, sm, o);
    }
    const int c = scale_exponent(mx);
    if (lane == 0) {
      T.xsum[gq] = sm;
      T.fin[gq] = pow2i(24 - c);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = gq * kGroup + i * 32 + lane;
      const int row = e / 10, j = e - row * 10;
      const int hi = j >= 5 ? 1 : 0, q = j - 5 * hi;
      const int variant = (gq != ((row * 10) >> 7)) ? 1 : 0;
      const int pos = 3 * (q < 3 ? q : q - 3);
      tab[variant * 1024 + row * 16 + 2 * q + hi] = __float2half_rn(xv[i] * pow2i(c - pos));
    }
  }
}

// One kernel serves fp16 and fp32 activations (a run-time branch in the table builders): the
// gate/up and down launches of a layer then share their code in the instruction caches.
__device__ void table_role(StreamSmem& S, const GemvParams& P, int* err, int tw) {
  const bool XF32 = P.x_f32 != 0;
  const int lane = threadIdx.x & 31;
  PartWalk W;
  W.begin(S);
  Part Pt;
  int it = 0;
  while (W.next(S, Pt)) {
    const GemvJob& J = P.jobs[Pt.job];
    const JobInfo& I = S.info[Pt.job];
    for (int sl = Pt.sa; sl < Pt.sb; ++sl, ++it) {
      if (it % kTableWarps != tw) continue;  // a single warp is latency-bound at about one unit per microsecond
      Unit U;
      make_unit(J, I, Pt.job, sl, Pt.chunk, U);
      const int ts = it % kTabSlots;
      mbar_wait(&S.tempty[ts], ((it / kTabSlots) & 1) ^ 1, err, kErrTabEmptyWait);
      TableBuf& T = S.table[ts];
      if (U.bits == 1) build_table_i8<1>(T, J.xa, U, XF32);
      else if (U.bits == 2) build_table_i8<2>(T, J.xa, U, XF32);
      else if (U.bits == 3) build_table_b3(T, J.xa, U, XF32);
      else build_table_i8<4>(T, J.xa, U, XF32);
      __syncwarp();
      if (lane == 0) mbar_arrive(&S.tfull[ts]);
    }
  }
}

// ---- consumers --------------------------------------------------------------------------
__device__ __forceinline__ void apply_group(const StageBuf& Sg, const TableBuf& Tb, int gu, int col, float xs, const float (&acc)[2][4],
                                            int p, float (&vs)[2][4]) {
  const uint2 sr = *reinterpret_cast<const uint2*>(&Sg.scales[gu][col]);
  const uint2 zr = *reinterpret_cast<const uint2*>(&Sg.zeros[gu][col]);
  const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sr.x));
  const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sr.y));
  const float2 z01 = __half22float2(*reinterpret_cast<const __half2*>(&zr.x));
  const float2 z23 = __half22float2(*reinterpret_cast<const __half2*>(&zr.y));
  const float fin = Tb.fin[gu];
  vs[0][p] += fmaf(s01.x * fin, acc[0][p], z01.x * xs);
  vs[0][2 + p] += fmaf(s01.y * fin, acc[0][2 + p], z01.y * xs);
  vs[1][p] += fmaf(s23.x * fin, acc[1][p], z23.x * xs);
  vs[1][2 + p] += fmaf(s23.y * fin, acc[1][2 + p], z23.y * xs);
}

// Word (row, 16-byte chunk ch) of column strip cw inside the 128B-swizzled box.
__device__ __forceinline__ const uint4* strip_word(const StageBuf& Sg, int cw, int row, int ch) {
  return reinterpret_cast<const uint4*>(Sg.words + cw * kStripBytes + row * 128 + ((ch ^ (row & 7)) << 4));
}

// 16-byte chunk of the strip (= 4 output columns) read by the lanes of MMA row pair g.  The
// two row pairs of a quarter warp must differ in the chunk bit the swizzle does not cover:
// bit 2 for the 1/2/4-bit access pattern (rows r+c), bit 0 for the 3-bit one (rows r+2c).
__device__ __forceinline__ int lane_chunk(int bits, int g) { return bits == 3 ? g : ((g >> 1) | ((g & 1) << 2)); }

// The sixteen consumer warps form two groups of eight that take alternate units, so that one
// group's MMA phase overlaps the other's load / scale phases.  Inside a group a warp owns one
// of 4 column strips and one of 2 row halves.
constexpr int kConsumerGroups = 2;
constexpr int kGroupWarps = kSConsumers / kConsumerGroups;
constexpr int kRowsPerWarp = kUnitRows / (kGroupWarps / 4);  // 32

__device__ __forceinline__ void mma16832u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Rows [32*kp, 32*kp+32) of the unit, columns of strip cw chunk ch; adds into vs.
// B-operand lane group g feeds MMA column g: digit plane g & 3 (plane 3 is empty) of the even
// (g < 4) or odd (g >= 4) group of the current pair of groups; rows of the other group see zeros.
template <int B>
__device__ __forceinline__ void consume_i8(const StageBuf& Sg, const TableBuf& Tb, const uint32_t* zero_row, int nrows, int ng, int cw,
                                           int kp, float (&vs)[2][4]) {
  using F = I8Fmt<B>;
  constexpr int CPB = F::kCpb;
  constexpr int NI = kRowsPerWarp / 4;        // loop iterations: 4 word rows (one per c) each
  constexpr int GPH = kRowsPerWarp / (4 * B); // groups inside this warp's rows
  constexpr int CH = B == 1 ? 2 : 4;          // word loads in flight (register budget)
  const int lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  const int ch = lane_chunk(B, g);
  const int r0 = kRowsPerWarp * kp;
  const bool plane_on = (g & 3) < 3;
  const uint32_t* tp = Tb.tab + (g & 3) * F::kPlaneStride;
  const int delta = g >> 2;
  int acc[2][4];
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[s][e] = 0;
#pragma unroll
  for (int i0 = 0; i0 < NI; i0 += CH) {
    uint4 w4[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i)
      if (r0 + 4 * (i0 + i) < nrows) w4[i] = *strip_word(Sg, cw, r0 + 4 * (i0 + i) + c, ch);
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int it = i0 + i;
      if (r0 + 4 * it < nrows) {
        const int row = r0 + 4 * it + c;
        const uint32_t* bp = (plane_on && delta == ((it / B) & 1)) ? tp + row * CPB : zero_row;
        uint32_t bf[CPB];
        if (CPB >= 4) {
#pragma unroll
          for (int q4 = 0; q4 < CPB / 4; ++q4) {
            const uint4 t = *reinterpret_cast<const uint4*>(bp + 4 * q4);
            bf[4 * q4 + 0] = t.x; bf[4 * q4 + 1] = t.y; bf[4 * q4 + 2] = t.z; bf[4 * q4 + 3] = t.w;
          }
        } else {
          const uint2 t = *reinterpret_cast<const uint2*>(bp);
          bf[0] = t.x; bf[1] = t.y;
        }
        const uint32_t wv[4] = {w4[i].x, w4[i].y, w4[i].z, w4[i].w};
#pragma unroll
        for (int m = 0; m < CPB / 2; ++m)
#pragma unroll
          for (int s = 0; s < 2; ++s)
            mma16832u8s8(acc[s], F::operand(wv[2 * s], 2 * m), F::operand(wv[2 * s + 1], 2 * m),
                         F::operand(wv[2 * s], 2 * m + 1), F::operand(wv[2 * s + 1], 2 * m + 1), bf[2 * m],
                         bf[2 * m + 1]);
      }
      if ((it + 1) % F::kWin == 0) {
        // C columns 2c, 2c+1 carry digit planes 2(c&1), 2(c&1)+1 of group (c >> 1) of this pair
        const int gu = kp * GPH + (it / F::kWin) * 2 + (c >> 1);
        if (gu < ng) {
          const int col = 32 * cw + 4 * ch;
          const uint2 sr = *reinterpret_cast<const uint2*>(&Sg.scales[gu][col]);
          const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sr.x));
          const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sr.y));
          const float f0 = Tb.fin[gu] * ((c & 1) ? 65536.0f : 1.0f), f1 = f0 * 256.0f;
          // planes 0+1 (or 2 alone: plane 3 is empty) of one output column, then the scale
          const float t00 = fmaf(f1, __int2float_rn(acc[0][1]), f0 * __int2float_rn(acc[0][0]));
          const float t01 = fmaf(f1, __int2float_rn(acc[0][3]), f0 * __int2float_rn(acc[0][2]));
          const float t10 = fmaf(f1, __int2float_rn(acc[1][1]), f0 * __int2float_rn(acc[1][0]));
          const float t11 = fmaf(f1, __int2float_rn(acc[1][3]), f0 * __int2float_rn(acc[1][2]));
          vs[0][0] = fmaf(s01.x, t00, vs[0][0]);
          vs[0][2] = fmaf(s01.y, t01, vs[0][2]);
          vs[1][0] = fmaf(s23.x, t10, vs[1][0]);
          vs[1][2] = fmaf(s23.y, t11, vs[1][2]);
          if ((c & 1) == 0) {  // the offset term z * sum(x), once per group and column
            const uint2 zr = *reinterpret_cast<const uint2*>(&Sg.zeros[gu][col]);
            const float2 z01 = __half22float2(*reinterpret_cast<const __half2*>(&zr.x));
            const float2 z23 = __half22float2(*reinterpret_cast<const __half2*>(&zr.y));
            const float xs = Tb.xsum[gu];
            vs[0][1] = fmaf(z01.x, xs, vs[0][1]); vs[0][3] = fmaf(z01.y, xs, vs[0][3]);
            vs[1][1] = fmaf(z23.x, xs, vs[1][1]); vs[1][3] = fmaf(z23.y, xs, vs[1][3]);
          }
        }
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[s][e] = 0;
      }
    }
  }
}

// 3-bit: 10 codes per word; a 640-wide unit is word aligned, its five groups ride in MMA
// columns 0..4.  A word that straddles two groups appears in two table variants.
struct S3Fmt {
  __device__ static __forceinline__ uint32_t merge(uint32_t w) { return (w & 0x00007fffu) | ((w << 1) & 0x7fff0000u); }
  __device__ static __forceinline__ uint32_t operand(uint32_t t, int q) {
    return q < 3 ? (t & (0x00070007u << (3 * q))) : ((t >> 9) & (0x00070007u << (3 * (q - 3))));
  }
};

__device__ __forceinline__ void consume_b3(const StageBuf& Sg, const TableBuf& Tb, const uint32_t* zero_row, int nrows, int ng, int cw,
                                           int kp, float (&vs)[2][4]) {
  const int lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  const int r0 = kRowsPerWarp * kp;
  float acc[2][4];
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[s][e] = 0.f;
#pragma unroll
  for (int i = 0; i < kRowsPerWarp / 8; ++i) {
    if (r0 + 8 * i < nrows) {
      uint32_t mw[2][4];
      uint32_t bf[10];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int row = r0 + 8 * i + 2 * c + r;
        uint4 w = make_uint4(0u, 0u, 0u, 0u);
        if (row < nrows) w = *strip_word(Sg, cw, row, g);
        mw[r][0] = S3Fmt::merge(w.x); mw[r][1] = S3Fmt::merge(w.y);
        mw[r][2] = S3Fmt::merge(w.z); mw[r][3] = S3Fmt::merge(w.w);
        const int d0 = (row * 10) >> 7;
        const uint32_t* bp = zero_row;
        if (g == d0) bp = Tb.tab + row * 8;
        else if (g == d0 + 1) bp = Tb.tab + 512 + row * 8;
        const uint4 t4 = *reinterpret_cast<const uint4*>(bp);
        bf[5 * r + 0] = t4.x; bf[5 * r + 1] = t4.y; bf[5 * r + 2] = t4.z; bf[5 * r + 3] = t4.w;
        bf[5 * r + 4] = bp[4];
      }
#pragma unroll
      for (int m = 0; m < 5; ++m)
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const int s0 = 2 * m, s1 = 2 * m + 1;
          const uint32_t a0 = s0 < 5 ? S3Fmt::operand(mw[0][2 * s], s0) : S3Fmt::operand(mw[1][2 * s], s0 - 5);
          const uint32_t a1 = s0 < 5 ? S3Fmt::operand(mw[0][2 * s + 1], s0) : S3Fmt::operand(mw[1][2 * s + 1], s0 - 5);
          const uint32_t a2 = s1 < 5 ? S3Fmt::operand(mw[0][2 * s], s1) : S3Fmt::operand(mw[1][2 * s], s1 - 5);
          const uint32_t a3 = s1 < 5 ? S3Fmt::operand(mw[0][2 * s + 1], s1) : S3Fmt::operand(mw[1][2 * s + 1], s1 - 5);
          mma16816s(acc[s], a0, a1, a2, a3, bf[s0], bf[s1]);
        }
    }
  }
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const int d = 2 * c + p;  // unit-local group carried by C column d
    // groups are not aligned to the row halves: the offset term is added once, by half 0
    if (d < 5 && d < ng) apply_group(Sg, Tb, d, 32 * cw + 4 * g, kp == 0 ? Tb.xsum[d] : 0.f, acc, p, vs);  // chunk = g
  }
}

__device__ void consumer_role(StreamSmem& S, const GemvParams& P, int* err) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = warp / kGroupWarps, wl = warp % kGroupWarps;
  const int cw = wl & 3, kp = wl >> 2;
  const int g = lane >> 2, c = lane & 3;
  PartWalk W;
  W.begin(S);
  Part Pt;
  int it = 0, pc = 0;
  while (W.next(S, Pt)) {
    const GemvJob& J = P.jobs[Pt.job];
    const JobInfo& I = S.info[Pt.job];
    const int ncols = min(128, J.N - Pt.chunk * 128);
    const bool strip_on = 32 * cw < ncols;
    float vs[2][4];
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int e = 0; e < 4; ++e) vs[s][e] = 0.f;
    for (int sl = Pt.sa; sl < Pt.sb; ++sl, ++it) {
      if ((it & (kConsumerGroups - 1)) != grp) continue;  // the other group's unit
      const int ng = min(I.groups_per_unit, I.ngroups - sl * I.groups_per_unit);
      const int nrows = I.bits == 3 ? min(kUnitRows, I.kw - sl * kUnitRows) : ng * (4 * I.bits);
      const int st = it % kSStages;
      const int ts = it % kTabSlots;
      const StageBuf& B = S.stage[st];
      const TableBuf& T = S.table[ts];
      mbar_wait(&S.tfull[ts], (it / kTabSlots) & 1, err, kErrTabFullWait);
      mbar_wait(&S.full[st], (it / kSStages) & 1, err, kErrFullWait);
      if (strip_on && kRowsPerWarp * kp < nrows) {
        if (I.bits == 1) consume_i8<1>(B, T, S.zero_row, nrows, ng, cw, kp, vs);
        else if (I.bits == 2) consume_i8<2>(B, T, S.zero_row, nrows, ng, cw, kp, vs);
        else if (I.bits == 3) consume_b3(B, T, S.zero_row, nrows, ng, cw, kp, vs);
        else consume_i8<4>(B, T, S.zero_row, nrows, ng, cw, kp, vs);
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&S.empty[st]);
        mbar_arrive(&S.tempty[ts]);
      }
    }
    // end of the part: sum the 8 MMA columns (= groups) and hand the strip to the finisher
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      vs[s][0] += vs[s][1];
      vs[s][2] += vs[s][3];
#pragma unroll
      for (int o = 1; o <= 2; o <<= 1) {
        vs[s][0] += __shfl_xor_sync(0xffffffffu, vs[s][0], o);
        vs[s][2] += __shfl_xor_sync(0xffffffffu, vs[s][2], o);
      }
    }
    const int slot = pc % kRedSlots;
    mbar_wait(&S.redempty[slot], ((pc / kRedSlots) & 1) ^ 1, err, kErrRedEmptyWait);
    if (c == 0)
      *reinterpret_cast<float4*>(&S.red[slot][grp * 2 + kp][32 * cw + 4 * lane_chunk(I.bits, g)]) =
          make_float4(vs[0][0], vs[0][2], vs[1][0], vs[1][2]);
    __syncwarp();
    if (lane == 0) mbar_arrive(&S.redfull[slot]);
    ++pc;
  }
}

// ---- finisher -----------------------------------------------------------------------------
// Sum the partial slots of one job's chunk columns n..n+3 in slice order and restore them to zero.
// A word per (job, chunk) records which slots hold a partial (one bit per part, at the part's
// first slice): only those are read, a few at a time so that their latencies overlap.  Jobs
// with more than 32 slices scan every slot.
// (Arguments by value: a reference to the kernel parameters would turn every access into a generic load.)
__device__ __noinline__ float4 drain_slots(float* src, size_t c_total, const unsigned* slot_set, int slices) {
  constexpr int kBatch = 4;
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
  if (slices <= 32) {
    unsigned m = __ldcg(slot_set);
    while (m) {
      float4 t[kBatch];
      float4* q[kBatch];
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        q[i] = nullptr;
        if (m) {
          const int s = __ffs(m) - 1;
          m &= m - 1;
          q[i] = reinterpret_cast<float4*>(src + static_cast<size_t>(s) * c_total);
          t[i] = __ldcg(q[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < kBatch; ++i)
        if (q[i]) {
          sum.x += t[i].x; sum.y += t[i].y; sum.z += t[i].z; sum.w += t[i].w;
          __stcg(q[i], make_float4(0.f, 0.f, 0.f, 0.f));
        }
    }
    return sum;
  }
  for (int s0 = 0; s0 < slices; s0 += kBatch) {
    float4 t[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i)
      if (s0 + i < slices) t[i] = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(s0 + i) * c_total));
#pragma unroll
    for (int i = 0; i < kBatch; ++i)
      if (s0 + i < slices) {
        sum.x += t[i].x; sum.y += t[i].y; sum.z += t[i].z; sum.w += t[i].w;
        __stcg(reinterpret_cast<float4*>(src + static_cast<size_t>(s0 + i) * c_total), make_float4(0.f, 0.f, 0.f, 0.f));
      }
  }
  return sum;
}

__device__ __forceinline__ void store_half4(__half* dst, const float4& v) {
  const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
  uint2 o;
  o.x = *reinterpret_cast<const uint32_t*>(&lo);
  o.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = o;
}

__device__ __forceinline__ float4 round_half4(const float4& v) {
  return make_float4(__half2float(__float2half_rn(v.x)), __half2float(__float2half_rn(v.y)),
                     __half2float(__float2half_rn(v.z)), __half2float(__float2half_rn(v.w)));
}

__device__ void finish_group(const StreamSmem& S, const GemvParams& P, const Part& Pt, int n) {
  if (P.epi == kEpiStore) {
    const GemvJob& J = P.jobs[Pt.job];
    store_half4(J.y + n, drain_slots(P.partial + J.col_base + n, P.c_total, reinterpret_cast<const unsigned*>(P.counters + J.mask_base + Pt.chunk), S.info[Pt.job].slices));
  } else if (P.epi == kEpiUpPair) {
    const int j1 = Pt.job & ~1, j3 = j1 + 1;
    const GemvJob& J1 = P.jobs[j1];
    const GemvJob& J3 = P.jobs[j3];
    const float4 a = round_half4(drain_slots(P.partial + J1.col_base + n, P.c_total, reinterpret_cast<const unsigned*>(P.counters + J1.mask_base + Pt.chunk), S.info[j1].slices));
    const float4 b = round_half4(drain_slots(P.partial + J3.col_base + n, P.c_total, reinterpret_cast<const unsigned*>(P.counters + J3.mask_base + Pt.chunk), S.info[j3].slices));
    if (J1.y) store_half4(J1.y + n, a);
    if (J3.y) store_half4(J3.y + n, b);
    if (J1.h)
      *reinterpret_cast<float4*>(J1.h + n) =
          make_float4(silu_f32(a.x) * b.x, silu_f32(a.y) * b.y, silu_f32(a.z) * b.z, silu_f32(a.w) * b.w);
  } else {
    float4 accw = make_float4(0.f, 0.f, 0.f, 0.f), res = accw;
    for (int i = 0; i < P.n_jobs; ++i) {
      const GemvJob& Ji = P.jobs[i];
      const float4 x2 = round_half4(drain_slots(P.partial + Ji.col_base + n, P.c_total, reinterpret_cast<const unsigned*>(P.counters + Ji.mask_base + Pt.chunk), S.info[i].slices));
      if (Ji.y) store_half4(Ji.y + n, x2);
      if (i < P.comb_weighted) {
        const float wgt = __half2float(P.comb_w[i]);
        accw.x = fmaf(wgt, x2.x, accw.x); accw.y = fmaf(wgt, x2.y, accw.y);
        accw.z = fmaf(wgt, x2.z, accw.z); accw.w = fmaf(wgt, x2.w, accw.w);
        if (i == P.comb_weighted - 1) res = round_half4(accw);
      } else {
        res = round_half4(make_float4(res.x + x2.x, res.y + x2.y, res.z + x2.z, res.w + x2.w));
      }
    }
    store_half4(P.comb_out + n, res);
  }
}

__device__ void finisher_role(StreamSmem& S, const GemvParams& P, int* err) {
  const int lane = threadIdx.x & 31;
  PartWalk W;
  W.begin(S);
  Part Pt;
  for (int pc = 0; W.next(S, Pt); ++pc) {
    const GemvJob& J = P.jobs[Pt.job];
    const JobInfo& I = S.info[Pt.job];
    const int slot = pc % kRedSlots;
    mbar_wait(&S.redfull[slot], (pc / kRedSlots) & 1, err, kErrRedFullWait);
    float4 r = *reinterpret_cast<const float4*>(&S.red[slot][0][4 * lane]);
#pragma unroll
    for (int q = 1; q < 4; ++q) {
      const float4 t = *reinterpret_cast<const float4*>(&S.red[slot][q][4 * lane]);
      r.x += t.x; r.y += t.y; r.z += t.z; r.w += t.w;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&S.redempty[slot]);

    const int n0 = Pt.chunk * 128;
    const int ncols = min(128, J.N - n0);
    const bool col_on = 4 * lane < ncols;
    const int n = n0 + 4 * lane;
    const bool whole = Pt.sa == 0 && Pt.sb == I.slices;
    if (whole && P.epi == kEpiStore) {
      if (col_on) store_half4(J.y + n, r);
      continue;
    }
    if (col_on) __stcg(reinterpret_cast<float4*>(P.partial + static_cast<size_t>(Pt.sa) * P.c_total + J.col_base + n), r);
    if (lane == 0) atomicOr(reinterpret_cast<unsigned*>(P.counters + J.mask_base + Pt.chunk), 1u << (Pt.sa & 31));
    __threadfence();
    __syncwarp();
    int last = 0;
    if (lane == 0) {
      int expected = I.slices;
      int* ctr = P.counters + J.chunk_base + Pt.chunk;
      if (P.epi == kEpiUpPair) expected = S.info[Pt.job & ~1].slices + S.info[(Pt.job & ~1) + 1].slices;
      if (P.epi == kEpiCombine) {
        expected = 0;
        for (int i = 0; i < P.n_jobs; ++i) expected += S.info[i].slices;
      }
      const int add = Pt.sb - Pt.sa;
      const int old = atomicAdd(ctr, add);
      last = (old + add == expected);
      if (last) *ctr = 0;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      __threadfence();
      if (col_on) finish_group(S, P, Pt, n);
      __syncwarp();
      if (lane == 0) {  // every lane has read the slot sets of the jobs it drained: clear them
        const int j0 = P.epi == kEpiStore ? Pt.job : (P.epi == kEpiUpPair ? (Pt.job & ~1) : 0);
        const int j1 = P.epi == kEpiStore ? Pt.job + 1 : (P.epi == kEpiUpPair ? j0 + 2 : P.n_jobs);
        for (int j = j0; j < j1; ++j) P.counters[P.jobs[j].mask_base + Pt.chunk] = 0;
      }
    }
  }
}

__global__ void __launch_bounds__(kSThreads, 1) gemv_stream_kernel(const __grid_constant__ GemvParams P) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  StreamSmem& S = *reinterpret_cast<StreamSmem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  int* err = P.counters + kErrSlot;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSStages; ++s) {
      mbar_init(&S.full[s], 1);             // producer, with the byte count
      mbar_init(&S.empty[s], kGroupWarps);  // only the group that owns the unit releases its stage
    }
    for (int s = 0; s < kTabSlots; ++s) {
      mbar_init(&S.tfull[s], 1);            // the table warp that built it
      mbar_init(&S.tempty[s], kGroupWarps);
    }
    for (int s = 0; s < kRedSlots; ++s) {
      mbar_init(&S.redfull[s], kSConsumers);
      mbar_init(&S.redempty[s], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 16) S.zero_row[threadIdx.x] = 0u;
  if (warp == kWarpProducer && (threadIdx.x & 31) < kMaxMaps)  // descriptor fetch overlaps the plan
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<unsigned long long>(&P.maps[threadIdx.x & 31])) : "memory");
  // Let the next kernel of the stream start its own prologue as SMs free up, then wait until
  // the previous kernel's results (expert ids, activations, zeroed workspace) are visible.  The
  // plan runs ahead of the wait when the launch says its inputs are older than that kernel.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  PlanArgs plan_args;
  if (warp == 0) {
    read_plan_args(P, plan_args);
    if (P.plan_early) make_plan(S, P, plan_args);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (warp == 0 && !P.plan_early) make_plan(S, P, plan_args);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  if (warp < kSConsumers) consumer_role(S, P, err);
  else if (warp == kWarpProducer) producer_role(S, P, err);
  else if (warp < kWarpFinisher) table_role(S, P, err, warp - kWarpTable);
  else finisher_role(S, P, err);
  __syncthreads();
}

// h[i] = silu(x1[i]) * x3[i] in fp32 (gemq/triton_kernels/fused_dequant_bmm.py:237-239)
__global__ void silu_mul_kernel(const __half* __restrict__ x1, const __half* __restrict__ x3, float* __restrict__ h, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) h[i] = silu_f32(__half2float(x1[i])) * __half2float(x3[i]);
}

// ---- host ---------------------------------------------------------------------------------
// Descriptor of a row-major [rows, N] tensor: uint32 words with 64 x 32 boxes (128B swizzle)
// or fp16 metadata with 4 x 128 boxes.
static bool tensor_map(CUtensorMap* out, const void* base, int N, long long rows, bool weights) {
  return weights ? tensor_map_2d(out, base, 4, N, rows, 32, kUnitRows, true)
                 : tensor_map_2d(out, base, 2, N, rows, 128, 4, false);
}

static int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

static int launch_stream_t(GemvParams& P, cudaStream_t stream, int units_bound) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  const size_t smem = sizeof(StreamSmem) + 1024;
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(gemv_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return GEMQ_ERR_LAUNCH;
    attr_set[dev] = true;
  }
  const int sms = sm_count();
  if (sms <= 0) return GEMQ_ERR_LAUNCH;
  const int grid = units_bound < sms ? units_bound : sms;
  // Programmatic dependent launch: this grid may be scheduled while the previous kernel of the
  // stream drains; everything that reads that kernel's results sits behind griddepcontrol.wait.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kSThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, gemv_stream_kernel, P) != cudaSuccess) return GEMQ_ERR_LAUNCH;
  return launch_status();
}

int silu_mul_f32(const __half* x1, const __half* x3, float* h, int n, cudaStream_t stream) {
  silu_mul_kernel<<<cdiv(n, 256), 256, 0, stream>>>(x1, x3, h, n);
  return launch_status();
}

// One activation row; every job N % 32 == 0, K % 128 == 0, group 128, activations 16-byte
// aligned.  P.epi / P.x_f32 select epilogue and activation type; kEpiUpPair expects the
// jobs in (gate, up) pairs.
int launch_stream(GemvParams& P, float* partial, size_t partial_floats, int* counters, cudaStream_t stream) {
  int cols = 0, chunks = 0, max_slices = 0, units = 0, families = 0;
  for (int i = 0; i < P.n_jobs; ++i) {
    GemvJob& J = P.jobs[i];
    // tensor maps: jobs reading the same (wq, scales, zeros) tensors share one family
    J.map_base = -1;
    for (int k = 0; k < i; ++k)
      if (P.jobs[k].wq == J.wq && P.jobs[k].scales == J.scales && P.jobs[k].zeros == J.zeros && P.jobs[k].N == J.N)
        J.map_base = P.jobs[k].map_base;
    if (J.map_base < 0) {
      if (families == kMaxFamilies) return GEMQ_ERR_BAD_SHAPE;
      J.map_base = 3 * families++;
      if (!tensor_map(&P.maps[J.map_base], J.wq, J.N, J.wq_rows, true) ||
          !tensor_map(&P.maps[J.map_base + 1], J.scales, J.N, J.zs_rows, false) ||
          !tensor_map(&P.maps[J.map_base + 2], J.zeros, J.N, J.zs_rows, false))
        return GEMQ_ERR_LAUNCH;
    }
    const int nch = cdiv(J.N, 128);
    J.col_base = cols;
    J.tile_base = 0;
    cols += J.N;
    if (P.epi == kEpiStore) {
      J.chunk_base = chunks;
      chunks += nch;
    } else if (P.epi == kEpiUpPair) {
      J.chunk_base = chunks;
      if (i & 1) chunks += nch;
    } else {
      J.chunk_base = 0;
      chunks = nch;
    }
    const int slices = cdiv(J.K / kGroup, 4);  // 4-bit units are the shortest: 4 groups
    max_slices = slices > max_slices ? slices : max_slices;
    units += nch * cdiv(J.K / kGroup, 16);     // at least this many (1-bit units: 16 groups)
  }
  if (P.epi == kEpiUpPair && (P.n_jobs & 1)) return GEMQ_ERR_BAD_ARG;
  int words = chunks;  // arrival counters, then one slot-set word per job and column chunk
  for (int i = 0; i < P.n_jobs; ++i) {
    P.jobs[i].mask_base = words;
    words += cdiv(P.jobs[i].N, 128);
  }
  if (words >= kMaxCounters - 4) return GEMQ_ERR_WORKSPACE;  // the last words are reserved (error code, wait limit, exit count)
  if (static_cast<size_t>(max_slices) * cols > partial_floats) return GEMQ_ERR_WORKSPACE;
  P.c_total = cols;
  P.n_chunks = chunks;
  P.s_max = max_slices;
  P.G = kGroup;
  P.partial = partial;
  P.counters = counters;
  return launch_stream_t(P, stream, units);
}

}  // namespace gemq

