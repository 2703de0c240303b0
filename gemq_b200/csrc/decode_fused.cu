// One-token forward of a quantised MoE layer in ONE persistent launch (one CTA per SM):
// router, fused gate/up projections, SiLU*mul, down projections and the weighted top-k combine
// (+ shared experts), gemq/inference/moe_block.py:200-235 and :488-531.
//
// Work.  Every matrix is cut into quanta of 4 quantisation groups (5 for 3-bit: 640 reduction
// elements = 64 whole packed rows) times 128 output columns.  Phase 0 lists the quanta of the
// gate and up projections of the selected experts (slot-major, column chunk, gate|up, k), phase 1
// those of the down projections; each phase is dealt to the CTAs in contiguous byte-balanced
// ranges, so the launch streams every selected weight exactly once and all SMs end together.
// A maximal run of quanta of one (matrix, column chunk) inside a range is a "part".
//
// Inside a CTA twelve consumer warps split the reduction dimension of a part (run lanes); each
// streams its own packed rows straight from global memory through a private ring of
// asynchronous copies (cp.async).  A task is 4 packed rows x 128 columns: four 512-byte row
// segments, each fetched by one warp instruction -- the access pattern that reaches the copy
// bandwidth of the part (128-byte pieces per row stay at half of it); five tasks = 10 KB in
// flight per warp.  The copies land in shared memory with a 16-byte swizzle so that the
// MMA-shaped reads (lane = 4 columns of one row) are conflict free.  The scales and offsets of a
// run travel through the same ring behind its packed rows.  The codes are never de-quantised:
//   1/2/4-bit: `word & mask` leaves four codes, one per byte, each shifted by its position in the
//     byte: a ready u8 A operand of mma.sync.m16n8k32.s32.u8.s8.  The B operand is the
//     activation, per group scaled to 21 bits and split into three balanced base-256 digit planes;
//     it is loaded once per task and used for all eight 16-column tiles.  Two consecutive groups
//     ride in MMA columns 0..2 and 4..6 and are folded into the fp32 result with their scales and
//     offsets every two groups.
//   3-bit: ten codes per word at bits 0, 3, .., 27; three masks (one after a shift of the word,
//     for the two codes that straddle byte boundaries) give u8 operands of the same MMA, five
//     operand registers per two words.  A run is 64 packed rows = five groups; the group a code
//     belongs to is a fixed function of the row's position in the run, rows whose codes fall into
//     two groups are masked per half of the MMA columns, and a group is folded when the 16-row
//     quad in which it ends is done.
// The activation tables (digit planes of x for a bit width, of h = silu(x1)*x3 for a slot) are
// built once per CTA and kept in shared memory.
// Four finisher warps (parts round robin) add the twelve run lanes of a part and run the
// cross-CTA protocol: fp32 partial slots that are restored to zero and one 64-bit word per column
// chunk that carries the arrival count and the set of slots in use, so that the CTA that
// completes a chunk knows which slots to add (in slice order: bit-reproducible) and applies the
// epilogue (h = silu(x1)*x3 in fp32, or the weighted combine).  In the gate/up phase a part
// arrives before it publishes its row: the part that completes a chunk whose other rows are all
// published keeps its own sums in registers.  An h chunk is a
// reduction group of the down projections: a flag per chunk lets a CTA build its phase-1 table
// group by group while the last gate/up chunks are still being finished, and the weight copies of
// phase 1 are in flight long before.  Every wait is bounded and records an error code.
#include "gemv.cuh"
#include "ptx.cuh"

namespace gemq {
namespace fused {

constexpr int kLanes = 12;                // run lanes of a part: the reduction dimension is dealt to them round robin
constexpr int kCons = kLanes;             // consumer warps, one per run lane (three per SM sub-partition)
constexpr int kFin = 4;                   // finisher warps, one per reduction slot
constexpr int kWarps = kCons + kFin;
constexpr int kThreads = 32 * kWarps;
constexpr int kConsThreads = 32 * kCons;
constexpr int kRing = 6;                  // ring slots per consumer warp (five tasks in flight)
constexpr int kSlotBytes = 2048;          // a task: 4 packed rows x 128 columns, or the scales | offsets of four groups
constexpr int kRedSlots = kFin;
constexpr int kMaxS = kMaxSlots + 1;      // routed slots + merged shared expert
constexpr int kMaxK = 14336;
constexpr int kMaxGroups = kMaxK / kGroup;
constexpr int kMaxParts = 40;
constexpr int kRouteMaxE = 32;
constexpr int kMetaE = 64;
constexpr int kErrSlot = kErrWord;
constexpr int kExitSlot = kMaxCounters - 3;  // CTAs that left this launch
// words of activation tables: three digit planes of kMaxK bytes (+ padding), or the 3-bit
// tables (16 halves per packed row + 16 per group for the rows that straddle two groups)
constexpr int kTabWordsI8 = 3 * (kMaxK / 4 + 16);
// 3-bit: per digit plane two words per packed row (rows rounded up to whole 64-row runs) and one
// word per pair of rows, plus the pads that spread the planes over the banks
constexpr int kB3RowsMax = (((kMaxK + 9) / 10 + 63) / 64) * 64;
constexpr int kTabWordsB3 = 3 * (2 * kB3RowsMax + 8) + 3 * (kB3RowsMax / 2 + 4);
constexpr int kTabWords = kTabWordsI8 > kTabWordsB3 ? kTabWordsI8 : kTabWordsB3;

enum { kErrBadExpert = 7, kErrRedFull = 11, kErrRedEmpty = 12, kErrPhase = 13 };


struct Mat3 {
  const uint32_t* wq;
  const __half* sc;
  const __half* zr;
};

struct FusedParams {
  const __half* x;       // [D]
  const __half* gate;    // [E, D]
  __half* out;           // [D]
  long long* idx;        // [A]
  __half* w;             // [A]
  int D, F, E, A, SF, S;
  int do_route, route_mode, renorm;
  Mat3 w1, w3, w2;       // stacked experts
  const int* nbits1; const int* wqs1; const int* zss1; const int* zss3;
  const int* nbits2; const int* wqs2; const int* zss2;
  Mat3 s1, s3, s2;       // merged shared expert (SF > 0)
  int sbits;
  float* partial;        // [slices][c_total], zero between launches
  int* counters;         // zero between launches
  float* h;              // [A*F + SF]
  int c_total;           // columns of a partial row: gate/up columns of all slots, then the down columns
  int up_cols;
  long long wq_bytes[3]; // extent of the stacked gate / up / down code tensors (0: unknown)
};

struct SlotInfo {
  const uint32_t* wq[3];  // gate, up, down matrix of the slot's expert (row 0)
  const __half* sc[3];
  const __half* zr[3];
  int bits[2];            // gate/up, down
  int F;                  // gate/up columns = down reduction length
  int hoff;               // first h element of the slot
  int nq[2], nch[2];      // quanta per (matrix, chunk); column chunks, per phase
  int colb[2];            // first partial column of the slot, per phase
  int ctrb;               // phase 0: first pair counter
  int maskb[2];           // first slot-set word, per phase
};

struct PartDesc {
  const uint32_t* w;      // row 0 of the matrix, first column of the chunk
  const __half* sc;
  const __half* zr;
  int N, B, kw, ngroups;
  int run_lo, run_hi;     // flush runs (2 groups; 5 for 3-bit) of this part
  int roff;               // run lane that takes run_lo: the runs of all parts go round the lanes in one sequence
  int ncols;
  int tab;                // activation table the part needs: bit width (phase 0) or 8 + slot (phase 1)
  int phase, s, c;
  int qa, qb;             // quanta [qa, qb) of the chunk
  int ctr, expected, mask, colp;
};

struct Tables {
  float xsum[kMaxGroups];
  float fin[kMaxGroups];
  alignas(16) uint32_t tab[kTabWords];
};

struct Smem {
  alignas(128) unsigned char ring[kCons][kRing][kSlotBytes];
  Tables T;
  alignas(16) float red[kRedSlots][kLanes][128];
  alignas(8) unsigned long long redfull[kRedSlots], redempty[kRedSlots];
  SlotInfo slot[kMaxS];
  PartDesc parts[kMaxParts];
  int n_parts, expected1, pairs_total, overflow;
  int spin;  // polls a bounded wait may take
  int sel_e[kMaxS];
  __half sel_w[kMaxS];
  float logit[kRouteMaxE];
  float part_sum[kRouteMaxE][8];
  int emeta[7][kMetaE];  // nbits / stride tables of the experts, fetched ahead of the dependency wait
};

static_assert(sizeof(Smem) <= 227 * 1024 - 64, "shared memory of the layer kernel exceeds the per-CTA limit");
static_assert(kMaxGroups <= 32 * kCons, "the 3-bit table builder deals a warp at most one group per lane");

// ---- small helpers ----------------------------------------------------------------------
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bar_consumers() { asm volatile("bar.sync 1, %0;" ::"n"(kConsThreads) : "memory"); }

__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ int clamp_bits(int b) { return b < 1 ? 1 : (b > 4 ? 4 : b); }
__device__ __forceinline__ int quantum_groups(int bits) { return bits == 3 ? 5 : 4; }
// relative cost of a quantum, for the byte/issue balanced deal of the quanta to the CTAs
// (relative time of a quantum measured in place: the low bit widths are bound by the MMA and
// logic issue rate, not by their bytes)
__device__ __forceinline__ unsigned quantum_cost(int bits) {
  return bits == 1 ? 32u : (bits == 2 ? 39u : (bits == 3 ? 86u : 54u));
}

__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// ---- integer operand format (1/2/4-bit) ---------------------------------------------------
template <int B>
struct I8 {
  static constexpr int kEps = 32 / B;
  static constexpr int kCpb = 8 / B;  // codes per byte = operands per word
  static constexpr int kPad = B == 1 ? 4 : (B == 2 ? 16 : 8);  // words between the planes (bank spread)
  static constexpr uint32_t kMask = ((1u << B) - 1u) * 0x01010101u;
  __device__ static __forceinline__ uint32_t operand(uint32_t w, int q) { return w & (kMask << (B * q)); }
  __device__ static __forceinline__ int plane_stride(int K) { return K / 4 + kPad; }
};

// c = 20 - floor(log2(max|x|)): the largest scaled value of a group lands in [2^20, 2^21).
__device__ __forceinline__ int scale_exp_i8(float mx) {
  int c = 20 - (static_cast<int>((__float_as_uint(mx) >> 23) & 0xffu) - 127);
  return c < -60 ? -60 : (c > 60 ? 60 : c);
}
// round(x * f) + 0x8080 in the low mantissa bits: bytes 0, 1 = low balanced digits + 128, byte 2 = top digit + 64
__device__ __forceinline__ uint32_t digits_word(float x, float f) { return __float_as_uint(fmaf(x, f, 12615808.0f)); }

// Wait until the h chunks (= reduction groups of phase 1) [g0, g1) of a slot are complete.  The
// flags are written by the finisher that completed the chunk, after a fence.  Every lane polls a
// flag of its own, so the wait costs one L2 round trip however many chunks it covers.
__device__ __forceinline__ void poll_flag(const int* flag, int* err, int spin) {
  int i = 0;
  while (ld_acquire(flag) == 0) {
    if (++i > spin) { atomicExch(err, kErrPhase); break; }
    __nanosleep(32);
  }
}
__device__ __forceinline__ void wait_groups(const int* flags, int g0, int g1, int* err, int spin) {
  if (flags) {
    for (int gq = g0 + static_cast<int>(threadIdx.x & 31); gq < g1; gq += 32) poll_flag(flags + gq, err, spin);
    __syncwarp();
  }
}

// Digit-plane table of the activation vector for B-bit matrices; the consumer warps take the
// wanted 32-row blocks round robin.  A group is 4*B consecutive rows (= lanes).
template <int B>
__device__ __forceinline__ void build_i8(Tables& T, const void* x, bool xf32, int K, unsigned need, const int* flags,
                                         int* err, int spin, int warp, int lane) {
  using F = I8<B>;
  constexpr int EPS = F::kEps, CPB = F::kCpb, LPG = 4 * B;
  const int rows = K / EPS;
  const int ps = F::plane_stride(K);
  int taken = 0;
  for (int row0 = 0; row0 < rows; row0 += 32) {
    const int q0 = (row0 / LPG) >> 2, q1 = ((row0 + 31) / LPG) >> 2;
    if (q0 < 32 && !((need >> q0) & 1u) && !((need >> (q1 < 32 ? q1 : 31)) & 1u)) continue;
    if ((taken++ % kCons) != warp) continue;
    wait_groups(flags, row0 / LPG, min(rows, row0 + 32) / LPG, err, spin);
    const int row = row0 + lane;
    const bool on = row < rows;
    float xv[EPS];
    if (on) {
      const size_t k = static_cast<size_t>(row) * EPS;
      if (xf32) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(x) + k);
#pragma unroll
        for (int i = 0; i < EPS / 4; ++i) {
          const float4 t = __ldcg(p + i);
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
    const int c = scale_exp_i8(mx);
    if (on && (lane % LPG) == 0) {
      T.xsum[row / LPG] = sm;
      T.fin[row / LPG] = pow2i(-c);
    }
    if (on) {
      constexpr int QB = CPB >= 4 ? 4 : CPB;
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
          const uint32_t x01 = __byte_perm(e[0], e[1], 0x5410), x23 = __byte_perm(e[2], e[3], 0x5410);
          pl[0][qq] = __byte_perm(x01, x23, 0x6420) ^ 0x80808080u;
          pl[1][qq] = __byte_perm(x01, x23, 0x7531) ^ 0x80808080u;
          const uint32_t t =
              __byte_perm(__byte_perm(e[0], e[1], 0x0062), __byte_perm(e[2], e[3], 0x0062), 0x5410) ^ 0x40404040u;
          pl[2][qq] = t | ((t & 0x40404040u) << 1);  // sign-extend the 7-bit top digit
        }
#pragma unroll
        for (int p = 0; p < 3; ++p) {
          uint32_t* dst = T.tab + p * ps + row * CPB + q0;
          if (QB == 4) *reinterpret_cast<uint4*>(dst) = make_uint4(pl[p][0], pl[p][1], pl[p][2], pl[p][3]);
          else *reinterpret_cast<uint2*>(dst) = make_uint2(pl[p][0], pl[p][1]);
        }
      }
    }
  }
}

// 3-bit matrices on the integer path.  A packed word holds ten codes at bits 0, 3, .., 27; three
// masks turn it into u8 operands: kind 0 = codes 0, 3, 6, 8 (one per byte, shifted left by
// 0, 1, 2, 0 inside their bytes), kind 1 = codes 1, 4, 7, 9 (shifts 3, 4, 5, 3), kind 2 = codes 2
// and 5, which straddle byte boundaries and are brought into bytes 0, 1 by a shift of the word
// (shifts 0, 1); the kind-2 operands of two rows share a register.  The table holds, per digit
// plane, two words per packed row (kinds 0, 1) and one word per row pair (r, r + 4: kind 2 of
// both), every code scaled with its own group's exponent; a row whose codes fall into two groups
// is masked when it is used.  A run is 64 rows = 640 k = 5 groups, so the group a code belongs
// to is a fixed function of the row's position in the run.
__device__ __forceinline__ int b3_rows(int K) { return (K + 9) / 10; }
__device__ __forceinline__ int b3_rows_padded(int K) { return ((b3_rows(K) + 63) >> 6) << 6; }
__device__ __forceinline__ int b3_stride_a(int K) { return 2 * b3_rows_padded(K) + 8; }
__device__ __forceinline__ int b3_stride_k2(int K) { return b3_rows_padded(K) / 2 + 4; }

// four digit words -> the three plane words of their four codes (byte i = code i)
__device__ __forceinline__ void planes_of4(const uint32_t (&e)[4], uint32_t (&pl)[3]) {
  const uint32_t x01 = __byte_perm(e[0], e[1], 0x5410), x23 = __byte_perm(e[2], e[3], 0x5410);
  pl[0] = __byte_perm(x01, x23, 0x6420) ^ 0x80808080u;
  pl[1] = __byte_perm(x01, x23, 0x7531) ^ 0x80808080u;
  const uint32_t t = __byte_perm(__byte_perm(e[0], e[1], 0x0062), __byte_perm(e[2], e[3], 0x0062), 0x5410) ^ 0x40404040u;
  pl[2] = t | ((t & 0x40404040u) << 1);  // sign-extend the 7-bit top digit
}

__device__ __forceinline__ void build_b3(Tables& T, const void* x, bool xf32, int K, unsigned need, const int* flags,
                                         int* err, int spin, int warp, int lane) {
  const int ngroups = K / kGroup;
  const int nruns = b3_rows_padded(K) >> 6;  // < 32: bit q of `need` = run q
  need &= nruns >= 32 ? 0xffffffffu : ((1u << nruns) - 1u);
  const int nwant = __popc(need);
  // pass 1: exponent and sum of every group of the wanted runs.  Eight lanes per group, four
  // groups per warp and batch: their flags are polled together, their loads are in flight together.
  {
    const int sub = lane >> 3, l8 = lane & 7;
#pragma unroll 1
    for (int i0 = 4 * warp; i0 < 5 * nwant; i0 += 4 * kCons) {
      const int i = i0 + sub;
      int my_g = -1;
      if (i < 5 * nwant) {
        const int run = __fns(need, 0, i / 5 + 1);
        const int gq = 5 * run + i % 5;
        if (gq < ngroups) my_g = gq;
      }
      if (flags) {
        if (my_g >= 0 && l8 == 0) poll_flag(flags + my_g, err, spin);
        __syncwarp();
      }
      float mx = 0.f, sm = 0.f;
      if (my_g >= 0) {
        const size_t k = static_cast<size_t>(my_g) * kGroup + 16 * l8;
        if (xf32) {
          const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(x) + k);
          float4 t[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) t[u] = __ldcg(p + u);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            mx = fmaxf(fmaxf(mx, fmaxf(fabsf(t[u].x), fabsf(t[u].y))), fmaxf(fabsf(t[u].z), fabsf(t[u].w)));
            sm += (t[u].x + t[u].y) + (t[u].z + t[u].w);
          }
        } else {
          const uint4* p = reinterpret_cast<const uint4*>(static_cast<const __half*>(x) + k);
          uint4 t[2] = {p[0], p[1]};
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const __half2* h = reinterpret_cast<const __half2*>(&t[u]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 f = __half22float2(h[q]);
              mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
              sm += f.x + f.y;
            }
          }
        }
      }
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) {
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        sm += __shfl_xor_sync(0xffffffffu, sm, o);
      }
      if (my_g >= 0 && l8 == 0) {
        T.xsum[my_g] = sm;
        T.fin[my_g] = pow2i(-scale_exp_i8(mx));
      }
    }
  }
  bar_consumers();
  // pass 2: a lane per packed row, the 32-row halves of the wanted runs round robin over the warps
  const int sa = b3_stride_a(K), sk = b3_stride_k2(K);
  uint32_t* tab_k2 = T.tab + 3 * sa;
#pragma unroll 1
  for (int i = warp; i < 2 * nwant; i += kCons) {
    const int row = 64 * __fns(need, 0, (i >> 1) + 1) + 32 * (i & 1) + lane;
    const int k0 = 10 * row;
    const int g_lo = k0 >> 7;
    const int j_hi = 128 * (g_lo + 1) - k0;  // first code of the row that belongs to the next group
    const float f_lo = g_lo < ngroups ? __uint_as_float(0x7f000000u - __float_as_uint(T.fin[g_lo])) : 0.f;
    const float f_hi = (j_hi < 10 && g_lo + 1 < ngroups) ? __uint_as_float(0x7f000000u - __float_as_uint(T.fin[g_lo + 1])) : 0.f;
    float v[10];
#pragma unroll
    for (int j = 0; j < 10; ++j) {
      const int k = k0 + j;
      v[j] = 0.f;
      if (k < K) v[j] = xf32 ? __ldcg(static_cast<const float*>(x) + k) : __half2float(static_cast<const __half*>(x)[k]);
    }
    uint32_t e[10];
#pragma unroll
    for (int j = 0; j < 10; ++j) {
      // position of code j inside its byte: kind 0 = codes 0,3,6,8 at 0,1,2,0; kind 1 = 1,4,7,9 at 3,4,5,3; kind 2 = 2,5 at 0,1
      constexpr int sh[10] = {0, 3, 0, 1, 4, 1, 2, 5, 0, 3};
      e[j] = digits_word(v[j], (j < j_hi ? f_lo : f_hi) * (1.0f / static_cast<float>(1 << sh[j])));
    }
    uint32_t pl[3];
    {
      const uint32_t k0e[4] = {e[0], e[3], e[6], e[8]}, k1e[4] = {e[1], e[4], e[7], e[9]};
      uint32_t p1[3];
      planes_of4(k0e, pl);
      planes_of4(k1e, p1);
#pragma unroll
      for (int p = 0; p < 3; ++p) *reinterpret_cast<uint2*>(T.tab + p * sa + 2 * row) = make_uint2(pl[p], p1[p]);
    }
    const uint32_t e2p = __shfl_down_sync(0xffffffffu, e[2], 4), e5p = __shfl_down_sync(0xffffffffu, e[5], 4);
    if ((lane & 4) == 0) {
      const uint32_t k2e[4] = {e[2], e[5], e2p, e5p};
      planes_of4(k2e, pl);
#pragma unroll
      for (int p = 0; p < 3; ++p) tab_k2[p * sk + 4 * (row >> 3) + (row & 3)] = pl[p];
    }
  }
}

// All consumer warps: wait until nobody reads the old table, build the new one, publish it.
// `need`: bit q set = quantum q (4 groups; 5 for 3-bit) of the vector is wanted.  `flags`: one
// word per group that turns non-zero when the group's slice of the vector exists (h in phase 1),
// or nullptr.
__device__ __noinline__ void build_table(Tables* T, const void* x, int xf32, int K, int B, unsigned need, const int* flags,
                                         int* err, int spin, int warp, int lane) {
  bar_consumers();
  if (B == 1) build_i8<1>(*T, x, xf32 != 0, K, need, flags, err, spin, warp, lane);
  else if (B == 2) build_i8<2>(*T, x, xf32 != 0, K, need, flags, err, spin, warp, lane);
  else if (B == 3) build_b3(*T, x, xf32 != 0, K, need, flags, err, spin, warp, lane);
  else build_i8<4>(*T, x, xf32 != 0, K, need, flags, err, spin, warp, lane);
  bar_consumers();
}

// ---- router (same arithmetic as route_kernel: identical ids and weights in every CTA) --------
__device__ __forceinline__ float dot8h(const uint4& a, const uint4& b) {
  const __half* pa = reinterpret_cast<const __half*>(&a);
  const __half* pb = reinterpret_cast<const __half*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s = fmaf(__half2float(pa[i]), __half2float(pb[i]), s);
  return s;
}
__device__ __forceinline__ float round_h(float v) { return __half2float(__float2half_rn(v)); }

__device__ void route_cta(Smem& S, const FusedParams& P) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int E = P.E, D = P.D, A = P.A, mode = P.route_mode;
  int parts = E >= 32 ? 1 : 32 / E;
  parts = parts > 8 ? 8 : parts;
  while (parts > 1 && (D % (parts * 256)) != 0) parts >>= 1;
  const int seg = D / parts;
  // Two (expert, segment) tasks per pass, the loads of both in flight together; each task keeps its
  // own summation order, so the logits do not depend on how the tasks are batched.  Every CTA
  // reads the whole router matrix: the CTAs start at different tasks so that at any moment they
  // pull different lines out of L2 instead of all queueing at the same slices.
  const int rot = static_cast<int>(blockIdx.x % static_cast<unsigned>(E * parts));
#pragma unroll 1
  for (int task0 = warp; task0 < E * parts; task0 += 2 * kWarps) {
    float acc[2] = {0.f, 0.f};
#pragma unroll 1
    for (int k0 = 0; k0 < seg; k0 += 4 * 256) {
      uint4 gq[2][4], xq[2][4];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (task0 + u * kWarps < E * parts) {
          const int task = (task0 + u * kWarps + rot) % (E * parts);
          const int e = task / parts, sg = task - e * parts;
          const __half* ge = P.gate + static_cast<size_t>(e) * D + static_cast<size_t>(sg) * seg;
          const __half* xs = P.x + static_cast<size_t>(sg) * seg;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int k = k0 + (i * 32 + lane) * 8;
            if (k < seg) {
              gq[u][i] = *reinterpret_cast<const uint4*>(ge + k);
              xq[u][i] = *reinterpret_cast<const uint4*>(xs + k);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (task0 + u * kWarps < E * parts) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (k0 + (i * 32 + lane) * 8 < seg) acc[u] += dot8h(xq[u][i], gq[u][i]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (task0 + u * kWarps < E * parts) {
        const int task = (task0 + u * kWarps + rot) % (E * parts);
        const int e = task / parts, sg = task - e * parts;
        float s = acc[u];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) S.part_sum[e][sg] = s;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < E) {
    float s = 0.f;
    for (int q = 0; q < parts; ++q) s += S.part_sum[threadIdx.x][q];
    if (mode != 2) s = round_h(s);
    S.logit[threadIdx.x] = s;
  }
  __syncthreads();
  if (warp != 0) return;
  float p = lane < E ? S.logit[lane] : -INFINITY;
  float mx = p;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  p = lane < E ? expf(p - mx) : 0.f;
  float sum = p;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  p = p / sum;
  if (mode == 0) p = round_h(p);
  if (lane >= E) p = -1.f;
  float my_w = 0.f;
  int my_i = 0;
  // top-k: the largest probability, the lowest expert id among equals.  Probabilities are >= +0,
  // so their bit patterns order like unsigned integers: one warp-wide integer max and one ballot per
  // pick instead of a shuffle tree over (value, index) pairs.
#pragma unroll 1
  for (int a = 0; a < A; ++a) {
    const unsigned key = p >= 0.f ? __float_as_uint(p) + 1u : 0u;  // 0: not a candidate (beyond E, or taken)
    const unsigned kmax = __reduce_max_sync(0xffffffffu, key);
    const int bi = __ffs(__ballot_sync(0xffffffffu, key == kmax)) - 1;
    const float bv = __uint_as_float(kmax - 1u);
    if (lane == a) { my_w = bv; my_i = bi; }
    if (lane == bi) p = -3.f;
  }
  float tot = 0.f;
  for (int a = 0; a < A; ++a) tot += __shfl_sync(0xffffffffu, my_w, a);
  if (mode == 0) tot = round_h(tot);
  if (lane < A) {
    const __half wv = __float2half_rn(P.renorm ? my_w / tot : my_w);
    S.sel_e[lane] = my_i;
    S.sel_w[lane] = wv;
    if (blockIdx.x == 0) {
      P.idx[lane] = my_i;
      P.w[lane] = wv;
    }
  }
}

// ---- plan (warp 0) ----------------------------------------------------------------------------
// a / b for a < 2^24, b > 0: one approximate reciprocal and a correction instead of the integer
// division sequence (the plan is a single warp's chain of dependent instructions).
__device__ __forceinline__ unsigned small_div(unsigned a, unsigned b) {
  unsigned q = __float2uint_rz(__fdividef(__uint2float_rz(a), __uint2float_rz(b)));
  if (q * b > a) --q;
  if ((q + 1) * b <= a) ++q;
  return q;
}
__device__ __forceinline__ int quanta_of(int groups, int bits) { return bits == 3 ? (groups + 4) / 5 : (groups + 3) >> 2; }

__device__ void make_plan(Smem& S, const FusedParams& P) {
  const int lane = threadIdx.x & 31;
  const int Sn = P.S;
  // slots
  int Fs = 0, b1 = 1, b2 = 1;
  if (lane < Sn) {
    SlotInfo I;
    if (lane < P.A) {
      int e = S.sel_e[lane];
      if (e < 0 || e >= P.E) {  // caller-supplied routing with an id out of range: never index with it
        atomicExch(P.counters + kErrSlot, kErrBadExpert);
        e = e < 0 ? 0 : P.E - 1;
      }
      const bool pre = P.E <= kMetaE;  // tables staged in shared memory ahead of the dependency wait
      b1 = clamp_bits(pre ? S.emeta[0][e] : P.nbits1[e]);
      b2 = clamp_bits(pre ? S.emeta[1][e] : P.nbits2[e]);
      Fs = P.F;
      const size_t o1 = static_cast<size_t>(pre ? S.emeta[2][e] : P.wqs1[e]);
      const size_t o2 = static_cast<size_t>(pre ? S.emeta[3][e] : P.wqs2[e]);
      const size_t z1 = P.zss1 ? static_cast<size_t>(pre ? S.emeta[4][e] : P.zss1[e])
                               : static_cast<size_t>(e) * (P.D / kGroup) * P.F;
      const size_t z3 = P.zss3 ? static_cast<size_t>(pre ? S.emeta[5][e] : P.zss3[e]) : z1;
      const size_t z2 = P.zss2 ? static_cast<size_t>(pre ? S.emeta[6][e] : P.zss2[e])
                               : static_cast<size_t>(e) * (P.F / kGroup) * P.D;
      I.wq[0] = P.w1.wq + o1; I.wq[1] = P.w3.wq + o1; I.wq[2] = P.w2.wq + o2;
      I.sc[0] = P.w1.sc + z1; I.zr[0] = P.w1.zr + z1;
      I.sc[1] = P.w3.sc + z3; I.zr[1] = P.w3.zr + z3;
      I.sc[2] = P.w2.sc + z2; I.zr[2] = P.w2.zr + z2;
    } else {
      b1 = b2 = clamp_bits(P.sbits);
      Fs = P.SF;
      I.wq[0] = P.s1.wq; I.wq[1] = P.s3.wq; I.wq[2] = P.s2.wq;
      I.sc[0] = P.s1.sc; I.zr[0] = P.s1.zr;
      I.sc[1] = P.s3.sc; I.zr[1] = P.s3.zr;
      I.sc[2] = P.s2.sc; I.zr[2] = P.s2.zr;
    }
    I.bits[0] = b1; I.bits[1] = b2;
    I.F = Fs;
    I.nq[0] = quanta_of(P.D / kGroup, b1);
    I.nq[1] = quanta_of(Fs / kGroup, b2);
    I.nch[0] = cdiv(Fs, 128);
    I.nch[1] = cdiv(P.D, 128);
    S.slot[lane] = I;
  }
  // exclusive prefix sums over the slots: h / partial offsets, pair counters, down quanta
  int nch0 = lane < Sn ? cdiv(Fs, 128) : 0;
  int fs = lane < Sn ? Fs : 0;
  int nq1 = lane < Sn ? quanta_of(Fs / kGroup, b2) : 0;
  int in_nch = nch0, in_fs = fs, in_nq1 = nq1;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, in_nch, o), b = __shfl_up_sync(0xffffffffu, in_fs, o),
              c = __shfl_up_sync(0xffffffffu, in_nq1, o);
    if (lane >= o) { in_nch += a; in_fs += b; in_nq1 += c; }
  }
  const int pairs_total = __shfl_sync(0xffffffffu, in_nch, 31);
  const int expected1 = __shfl_sync(0xffffffffu, in_nq1, 31);
  const int nch1 = cdiv(P.D, 128);
  const int base1 = 3 * pairs_total;
  if (lane < Sn) {
    SlotInfo& I = S.slot[lane];
    I.hoff = in_fs - fs;
    I.ctrb = in_nch - nch0;
    I.colb[0] = 2 * (in_fs - fs);
    I.colb[1] = P.up_cols + lane * P.D;  // the phases overlap in time: their partial columns must not
    I.maskb[0] = pairs_total + 2 * (in_nch - nch0);
    I.maskb[1] = base1 + nch1 + lane * nch1;
  }
  if (lane == 0) {
    S.pairs_total = pairs_total;
    S.expected1 = expected1;
    S.overflow = 0;
  }
  __syncwarp();
  // ranges and parts of the two phases
  int pbase = 0;
#pragma unroll 1
  for (int ph = 0; ph < 2; ++ph) {
    unsigned n_units = 0, cost = 1;
    int nq = 1;
    if (lane < Sn) {
      const SlotInfo& I = S.slot[lane];
      nq = I.nq[ph];
      n_units = static_cast<unsigned>(I.nch[ph]) * (ph ? 1u : 2u) * nq;
      cost = quantum_cost(I.bits[ph]);
    }
    const unsigned wgt = n_units * cost;
    unsigned incl = wgt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const unsigned total = __shfl_sync(0xffffffffu, incl, 31);
    const unsigned prefix = incl - wgt;
    // cut points: any monotone function of the CTA index evaluated the same way by both neighbours
    const float per_cta = static_cast<float>(total) / static_cast<float>(gridDim.x);
    const unsigned lo = blockIdx.x == 0 ? 0u : min(total, static_cast<unsigned>(per_cta * static_cast<float>(blockIdx.x)));
    const unsigned hi = blockIdx.x + 1 == gridDim.x ? total
                                                    : min(total, static_cast<unsigned>(per_cta * static_cast<float>(blockIdx.x + 1)));
    const bool small = total < (1u << 23);  // always, for the layers this kernel takes; the exact form stays as the guard
    unsigned ulo = lo <= prefix ? 0u : (small ? small_div(lo - prefix + cost - 1, cost) : (lo - prefix + cost - 1) / cost);
    unsigned uhi = hi <= prefix ? 0u : (small ? small_div(hi - prefix + cost - 1, cost) : (hi - prefix + cost - 1) / cost);
    ulo = min(ulo, n_units);
    uhi = min(uhi, n_units);
    const unsigned cm_lo = small ? small_div(ulo, nq) : ulo / nq;
    const int np = uhi > ulo ? static_cast<int>((small ? small_div(uhi - 1, nq) : (uhi - 1) / nq) - cm_lo + 1) : 0;
    int inp = np;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, inp, o);
      if (lane >= o) inp += t;
    }
    const int np_total = __shfl_sync(0xffffffffu, inp, 31);
    int pi = pbase + inp - np;
    if (pbase + np_total > kMaxParts) {
      if (lane == 0) S.overflow = 1;
    } else if (np > 0) {
      const SlotInfo& I = S.slot[lane];
      const int B = I.bits[ph];
      const int K = ph ? I.F : P.D, N = ph ? P.D : I.F;
      const int ngroups = K / kGroup;
      const int first_cm = static_cast<int>(cm_lo);
#pragma unroll 1
      for (int k = 0; k < np; ++k, ++pi) {
        const int cm = first_cm + k;
        const int c = ph ? cm : (cm >> 1), m = ph ? 0 : (cm & 1), mi = ph ? 2 : m;
        const int qa = max(static_cast<int>(ulo), cm * nq) - cm * nq;
        const int qb = min(static_cast<int>(uhi), (cm + 1) * nq) - cm * nq;
        PartDesc d;
        const int n0 = c * 128;
        d.w = I.wq[mi] + n0;
        d.sc = I.sc[mi] + n0;
        d.zr = I.zr[mi] + n0;
        d.N = N; d.B = B; d.ngroups = ngroups;
        d.kw = B == 3 ? b3_rows(K) : (K * B) >> 5;
        if (B == 3) { d.run_lo = qa; d.run_hi = min(qb, nq); }
        else { d.run_lo = 2 * qa; d.run_hi = min(2 * qb, cdiv(ngroups, 2)); }
        d.ncols = min(128, N - n0);
        d.tab = ph ? 8 + lane : B;
        d.phase = ph; d.s = lane; d.c = c;
        d.qa = qa; d.qb = qb;
        if (ph) {
          d.ctr = base1 + c;
          d.expected = expected1;
          d.mask = I.maskb[1] + c;
          d.colp = I.colb[1] + n0;
        } else {
          d.ctr = I.ctrb + c;  // index of a 64-bit word
          d.expected = 2 * nq;
          d.mask = m;          // phase 0: which half of the slot set this part's bit goes to
          d.colp = I.colb[0] + m * I.F + n0;
        }
        S.parts[pi] = d;
      }
    }
    pbase += np_total;
  }
  __syncwarp();
  if (lane == 0) {
    const int n = S.overflow ? 0 : pbase;
    int runs = 0;
    for (int p = 0; p < n; ++p) {
      S.parts[p].roff = runs % kLanes;
      runs += S.parts[p].run_hi - S.parts[p].run_lo;
    }
    S.n_parts = n;
  }
}

// ---- the load side of a consumer warp: walks the warp's tasks ahead of the compute side ------
// A flush run of a 1/2/4-bit matrix (two groups) is a sequence of ring tasks: nt weight tasks of 4
// packed rows x 128 columns, then a "meta" task carrying the scales | offsets (256 + 256 bytes per
// group) of the run's groups; the run is folded when the meta task arrives, reading the scales
// straight from the ring.  A 3-bit run (64 packed rows, five groups) is a sequence of quads: four
// weight tasks (16 rows) and a meta task with the group that ends inside the quad (the last quad
// of a run: the two groups that end there), so that a group is folded as soon as it is complete.
struct Loader {
  const uint32_t* w;    // lane's 16 bytes in row 0 of the next weight task
  int i, nt, ntot;      // next task of the run; weight tasks (3-bit: quads); weight + meta tasks
  int b3;               // 3-bit run layout
  int N;                // row pitch of the part's matrix (words, = halves of the scale rows)
  int rows_left;        // 3-bit: valid packed rows from the next weight task on (other widths: unused)
  int run, p;           // current run, part
  int slot;             // ring slot of the next task
  uint32_t ring;        // shared address of the warp's ring
  uint32_t roff[4];     // lane's position inside a weight task, per row
};
// What a step needs once per run is read from the part in shared memory instead of being carried
// in registers (the kernel sits at its register limit): the lane's scales (lanes 0..15) or offsets
// (lanes 16..31) of group 0 of the run, and the groups of the run.
__device__ __forceinline__ const __half* loader_meta(const Loader& L, const PartDesc& d, int lane) {
  return ((lane & 16) ? d.zr : d.sc) + static_cast<size_t>((L.b3 ? 5 : 2) * L.run) * d.N + 8 * (lane & 15);
}

__device__ __forceinline__ int run_groups(int B, int run, int ngroups) {
  return B == 3 ? min(5, ngroups - 5 * run) : min(2, ngroups - 2 * run);
}
__device__ __forceinline__ int run_weight_tasks(int B, int run, int ngroups) { return min(2, ngroups - 2 * run) * B; }
// quads (16 packed rows) of a 3-bit run
__device__ __forceinline__ int b3_run_quads(int run, int kw) { return (min(64, kw - 64 * run) + 15) >> 4; }
// first run of run lane kq in a part
__device__ __forceinline__ int first_run(const PartDesc& d, int kq) { return d.run_lo + (kq + kLanes - d.roff) % kLanes; }

// Ring position of the 16 bytes of column quad q (4 columns) of task row r: quads are permuted
// inside groups of eight so that lanes reading different rows hit different banks.
__device__ __forceinline__ int ring_off(int r, int q) { return r * 512 + (((q & 24) | ((q ^ (2 * r)) & 7)) << 4); }

__device__ __forceinline__ void cp_async16s(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

// Move the loader to the first task of its next run.
__device__ __forceinline__ void loader_next_run(Loader* Lp, const Smem* Sp, int kq, int lane, int first) {
  Loader& L = *Lp;
  const Smem& S = *Sp;
  if (!first) L.run += kLanes;
  while (L.p < 0 || L.run >= S.parts[L.p].run_hi) {
    if (++L.p >= S.n_parts) { L.ntot = 0; L.i = 0; return; }
    L.run = first_run(S.parts[L.p], kq);
  }
  const PartDesc& d = S.parts[L.p];
  const int B = d.B;
  L.N = d.N;
  L.b3 = B == 3;
  if (B == 3) {
    L.nt = b3_run_quads(L.run, d.kw);
    L.ntot = 5 * L.nt;
  } else {
    L.nt = run_weight_tasks(B, L.run, d.ngroups);
    L.ntot = L.nt + 1;
  }
  L.i = 0;
  const int row0 = (B == 3 ? 64 : 8 * B) * L.run;
  L.rows_left = B == 3 ? d.kw - row0 : (1 << 30);
  L.w = d.w + static_cast<size_t>(row0) * d.N + 4 * lane;
}

// Issue the copies of the loader's next task (one commit group per call, empty when the warp
// has run out of tasks) and step to the task after it.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// (The loader runs ahead of the compute side: the form of ITS run decides, not the part being computed.)
__device__ __forceinline__ void loader_step(Loader& L, const Smem& S, int kq, int lane) {
  if (L.i < L.ntot) {
    const uint32_t dst = L.ring + L.slot * kSlotBytes;
    if (!L.b3) {
      if (L.i < L.nt) {
        const char* src = reinterpret_cast<const char*>(L.w);
        const size_t pitch = static_cast<size_t>(L.N) * 4;
#pragma unroll
        for (int r = 0; r < 4; ++r) cp_async16(dst + L.roff[r], src + r * pitch);
        L.w += 4 * static_cast<size_t>(L.N);
      } else {
        // lanes 0..15 copy the 256 bytes of scales of a group, lanes 16..31 its offsets
        const PartDesc& d = S.parts[L.p];
        const __half* m = loader_meta(L, d, lane);
        cp_async16(dst + 16 * lane, m);
        if (d.ngroups - 2 * L.run > 1) cp_async16(dst + 512 + 16 * lane, m + L.N);
      }
    } else {
      const int quad = L.i / 5, qpos = L.i - 5 * quad;  // position in the quad sequence
      if (qpos < 4) {
        if (L.rows_left >= 4) {
          const char* src = reinterpret_cast<const char*>(L.w);
          const size_t pitch = static_cast<size_t>(L.N) * 4;
#pragma unroll
          for (int r = 0; r < 4; ++r) cp_async16(dst + L.roff[r], src + r * pitch);
        } else {
          // rows past the end of a 3-bit matrix are zero-filled; their source stays on the last valid row
          const uint32_t* src = L.rows_left > 0 ? L.w : S.parts[L.p].w + 4 * lane;
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            cp_async16s(dst + L.roff[r], src, r < L.rows_left ? 16 : 0);
            if (r < 3 && r + 1 < L.rows_left) src += L.N;
          }
        }
        L.rows_left -= 4;
        L.w += 4 * static_cast<size_t>(L.N);
      } else {
        // the group that ends in this quad, and the next one after the last quad of the run
        const PartDesc& d = S.parts[L.p];
        const int ng = min(5, d.ngroups - 5 * L.run);
        const __half* src = loader_meta(L, d, lane) + static_cast<size_t>(quad) * L.N;
        if (quad < ng) cp_async16(dst + 16 * lane, src);
        if (quad == L.nt - 1 && quad + 1 < ng) cp_async16(dst + 512 + 16 * lane, src + L.N);
      }
    }
    if (++L.i == L.ntot) loader_next_run(&L, &S, kq, lane, 0);
  }
  cp_async_commit();
  L.slot = L.slot + 1 == kRing ? 0 : L.slot + 1;
}

// ---- compute side -------------------------------------------------------------------------------
struct RunState {
  int acc[4][2][4];   // [column quad group j][tile s][C fragment]: columns 4(g+8j) + 2s, + 2s+1
  float vs[4][2][2];  // running sums of those two columns over the runs of the part
};

__device__ __forceinline__ void unpack4(const uint2& r, float (&f)[4]) {
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// Weight task of a 1/2/4-bit run: `wp` = lane's row c, quad g in the ring slot, `bp` = lane's B
// operand words of that row, `on` = the lane's MMA column is fed by the task's group (else zeros).
template <int B>
__device__ __forceinline__ void task_i8(RunState& R, const unsigned char* wp, const uint32_t* bp, bool on) {
  using F = I8<B>;
  constexpr int CPB = F::kCpb;
  uint32_t bf[CPB];
  if (CPB >= 4) {
#pragma unroll
    for (int q4 = 0; q4 < CPB / 4; ++q4) {
      const uint4 t = *reinterpret_cast<const uint4*>(bp + 4 * q4);
      bf[4 * q4] = t.x; bf[4 * q4 + 1] = t.y; bf[4 * q4 + 2] = t.z; bf[4 * q4 + 3] = t.w;
    }
  } else {
    const uint2 t = *reinterpret_cast<const uint2*>(bp);
    bf[0] = t.x; bf[1] = t.y;
  }
#pragma unroll
  for (int q = 0; q < CPB; ++q) bf[q] = on ? bf[q] : 0u;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 w = *reinterpret_cast<const uint4*>(wp + 128 * j);
    const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int mm = 0; mm < CPB / 2; ++mm)
#pragma unroll
      for (int s = 0; s < 2; ++s)
        mma_u8s8(R.acc[j][s], F::operand(wv[2 * s], 2 * mm), F::operand(wv[2 * s + 1], 2 * mm),
                 F::operand(wv[2 * s], 2 * mm + 1), F::operand(wv[2 * s + 1], 2 * mm + 1), bf[2 * mm], bf[2 * mm + 1]);
  }
}

// Fold a 1/2/4-bit run into the running sums; `mp` = the run's meta task in the ring.
// C columns 2c, 2c+1 hold digit planes 2(c&1), 2(c&1)+1 of group (c >> 1) of the pair.
__device__ __forceinline__ void fold_i8(RunState* Rp, const Tables* Tp, const unsigned char* mp, int run, int ng, int lane) {
  RunState& R = *Rp;
  const Tables& T = *Tp;
  const int g = lane >> 2, c = lane & 3;
  const int gu = c >> 1;
  if (gu < ng) {
    const int grp = 2 * run + gu;
    const float f0 = T.fin[grp] * ((c & 1) ? 65536.0f : 1.0f), f1 = f0 * 256.0f;
    const float xs = (c & 1) ? 0.f : T.xsum[grp];  // the offset term z * sum(x), once per group and column
    const unsigned char* gp = mp + 512 * gu + 8 * g;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float sc[4], zr[4];
      unpack4(*reinterpret_cast<const uint2*>(gp + 64 * j), sc);
      unpack4(*reinterpret_cast<const uint2*>(gp + 256 + 64 * j), zr);
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const float ta = fmaf(f1, __int2float_rn(R.acc[j][s][1]), f0 * __int2float_rn(R.acc[j][s][0]));
        const float tb = fmaf(f1, __int2float_rn(R.acc[j][s][3]), f0 * __int2float_rn(R.acc[j][s][2]));
        R.vs[j][s][0] += fmaf(sc[2 * s], ta, zr[2 * s] * xs);
        R.vs[j][s][1] += fmaf(sc[2 * s + 1], tb, zr[2 * s + 1] * xs);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int e = 0; e < 4; ++e) R.acc[j][s][e] = 0;
}

// A pair of 3-bit weight tasks (8 packed rows): lane c takes row c of the even task (`ep`) and
// row c of the odd one (`op`), i.e. rows i and i + 4 of the pair.  Per column pair three MMAs:
// kinds 0 | 1 of each row, then the kind-2 operands of both rows in one register.  `b` = the
// lane's B words (already masked to the group its MMA column serves): kinds 0, 1 of the even
// row, of the odd row, kind 2 of the pair.
__device__ __forceinline__ void pair_b3(RunState& R, const unsigned char* ep, const unsigned char* op, const uint32_t (&b)[5]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 we = *reinterpret_cast<const uint4*>(ep + 128 * j);
    const uint4 wo = *reinterpret_cast<const uint4*>(op + 128 * j);
    const uint32_t ev[4] = {we.x, we.y, we.z, we.w}, ov[4] = {wo.x, wo.y, wo.z, wo.w};
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const uint32_t e0 = ev[2 * s], e1 = ev[2 * s + 1], o0 = ov[2 * s], o1 = ov[2 * s + 1];
      mma_u8s8(R.acc[j][s], e0 & 0x071c0e07u, e1 & 0x071c0e07u, e0 & 0x38e07038u, e1 & 0x38e07038u, b[0], b[1]);
      mma_u8s8(R.acc[j][s], o0 & 0x071c0e07u, o1 & 0x071c0e07u, o0 & 0x38e07038u, o1 & 0x38e07038u, b[2], b[3]);
      const uint32_t x0 = ((e0 >> 6) & 0x00000e07u) | ((o0 << 10) & 0x0e070000u);
      const uint32_t x1 = ((e1 >> 6) & 0x00000e07u) | ((o1 << 10) & 0x0e070000u);
      mma_u8s8(R.acc[j][s], x0, x1, 0u, 0u, b[4], 0u);
    }
  }
}

// Fold the MMA columns of one or both groups of a 3-bit quad into the running sums.  C columns
// 2c, 2c+1 of lane c hold digit planes 2(c&1), 2(c&1)+1 of the group served by half c >> 1 of the
// MMA columns; `grp` = that group, `slot` = its place in the meta task `mp`, `on` = fold it now.
__device__ __forceinline__ void fold_b3(RunState* Rp, const Tables* Tp, const unsigned char* mp, int grp, int slot, bool on,
                                        int lane) {
  RunState& R = *Rp;
  const Tables& T = *Tp;
  const int g = lane >> 2, c = lane & 3;
  if (on) {
    const float f0 = T.fin[grp] * ((c & 1) ? 65536.0f : 1.0f), f1 = f0 * 256.0f;
    const float xs = (c & 1) ? 0.f : T.xsum[grp];
    const unsigned char* gp = mp + 512 * slot + 8 * g;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float sc[4], zr[4];
      unpack4(*reinterpret_cast<const uint2*>(gp + 64 * j), sc);
      unpack4(*reinterpret_cast<const uint2*>(gp + 256 + 64 * j), zr);
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const float ta = fmaf(f1, __int2float_rn(R.acc[j][s][1]), f0 * __int2float_rn(R.acc[j][s][0]));
        const float tb = fmaf(f1, __int2float_rn(R.acc[j][s][3]), f0 * __int2float_rn(R.acc[j][s][2]));
        R.vs[j][s][0] += fmaf(sc[2 * s], ta, zr[2 * s] * xs);
        R.vs[j][s][1] += fmaf(sc[2 * s + 1], tb, zr[2 * s + 1] * xs);
#pragma unroll
        for (int e = 0; e < 4; ++e) R.acc[j][s][e] = 0;
      }
    }
  }
}

// The compute side's position in its ring.
struct Cursor {
  const unsigned char* ring;  // the warp's ring
  int slot;                   // slot of the next task
};
__device__ __forceinline__ const unsigned char* cursor_take(Cursor& C) {
  cp_async_wait<kRing - 2>();
  __syncwarp();
  const unsigned char* p = C.ring + C.slot * kSlotBytes;
  C.slot = C.slot + 1 == kRing ? 0 : C.slot + 1;
  return p;
}

// All runs of run lane kq in a 1/2/4-bit part.
template <int B>
__device__ __forceinline__ void part_i8(RunState& R, Loader& L, Cursor& C, const Smem& S, const PartDesc& d, int kq, int lane) {
  using F = I8<B>;
  const int g = lane >> 2, c = lane & 3;
  const int K = d.ngroups * kGroup;
  const int woff = ring_off(c, g);
  // this lane's MMA column: digit plane (g & 3) of the first (g < 4) or second group of a run; column 3 / 7 stays empty
  const uint32_t* plane = S.T.tab + min(g & 3, 2) * F::plane_stride(K) + c * F::kCpb;  // columns 3 / 7: switched off below
  const bool feeds = (g & 3) < 3;
  const int run_hi = d.run_hi;
#pragma unroll 1
  for (int run = first_run(d, kq); run < run_hi; run += kLanes) {
    const int ng = min(2, d.ngroups - 2 * run);
    const uint32_t* bp = plane + 8 * B * run * F::kCpb;
#pragma unroll 1
    for (int gi = 0; gi < ng; ++gi) {
      const bool on = feeds && (g >> 2) == gi;
#pragma unroll 1
      for (int ii = 0; ii < B; ++ii) {
        const unsigned char* slotp = cursor_take(C);
        task_i8<B>(R, slotp + woff, bp, on);
        bp += 4 * F::kCpb;
        loader_step(L, S, kq, lane);
      }
    }
    const unsigned char* mp = cursor_take(C);
    fold_i8(&R, &S.T, mp, run, ng, lane);
    loader_step(L, S, kq, lane);
  }
}

// All runs of run lane kq in a 3-bit part.
__device__ __forceinline__ void part_b3(RunState& R, Loader& L, Cursor& C, const Smem& S, const PartDesc& d, int kq, int lane) {
  const int K = d.ngroups * kGroup;
  const int g = lane >> 2, c = lane & 3;
  const int woff = ring_off(c, g);
  // this lane's MMA column: digit plane (g & 3) for the even (g < 4) or odd group of the quad; column 3 / 7 stays empty
  const bool feeds = (g & 3) < 3;
  const uint32_t* tab_a = S.T.tab + (g & 3) * b3_stride_a(K);
  const uint32_t* tab_k2 = S.T.tab + 3 * b3_stride_a(K) + (g & 3) * b3_stride_k2(K);
  const int run_hi = d.run_hi;
#pragma unroll 1
  for (int run = first_run(d, kq); run < run_hi; run += kLanes) {
    const int ng = min(5, d.ngroups - 5 * run);
    const int nquads = b3_run_quads(run, d.kw);
#pragma unroll 1
    for (int quad = 0; quad < nquads; ++quad) {
      // groups of the quad: ga ends at local row 12 - 3 * quad, whose codes from 8 - 2 * quad on belong to ga + 1
      const int ga = 5 * run + quad;
      const bool is_a = ((ga ^ (g >> 2)) & 1) == 0;  // does this lane's half of the MMA columns serve ga
      const int brow = 12 - 3 * quad;
      // bytes of the boundary row that belong to ga + 1, per kind (codes 0,3,6,8 | 1,4,7,9 | 2,5)
      const uint32_t mb0 = quad == 0 ? 0xff000000u : (quad == 3 ? 0xffffff00u : 0xffff0000u);
      const uint32_t mb1 = quad == 0 ? 0xff000000u : (quad == 1 ? 0xffff0000u : 0xffffff00u);
      const uint32_t mb2 = quad < 2 ? 0u : (quad == 2 ? 0xff00u : 0xffffu);
      const unsigned char* prev = nullptr;
#pragma unroll 1
      for (int t = 0; t < 4; ++t) {
        const unsigned char* slotp = cursor_take(C);
        if (t & 1) {
          const int row = 64 * run + 16 * quad + 4 * (t - 1) + c;  // even task's row; the odd one's is row + 4
          uint32_t b[5] = {0u, 0u, 0u, 0u, 0u};
          if (feeds) {
            const uint2 be = *reinterpret_cast<const uint2*>(tab_a + 2 * row);
            const uint2 bo = *reinterpret_cast<const uint2*>(tab_a + 2 * (row + 4));
            const uint32_t bk = tab_k2[4 * (row >> 3) + (row & 3)];
            const int ie = 4 * (t - 1) + c, io = ie + 4;  // local rows in the quad
            // mask of the bytes that belong to this lane's group, for the even and the odd row
            const uint32_t full = is_a ? 0xffffffffu : 0u;
            const uint32_t me0 = ie < brow ? full : (ie > brow ? ~full : (is_a ? ~mb0 : mb0));
            const uint32_t me1 = ie < brow ? full : (ie > brow ? ~full : (is_a ? ~mb1 : mb1));
            const uint32_t me2 = ie < brow ? full : (ie > brow ? ~full : (is_a ? ~mb2 : mb2));
            const uint32_t mo0 = io < brow ? full : (io > brow ? ~full : (is_a ? ~mb0 : mb0));
            const uint32_t mo1 = io < brow ? full : (io > brow ? ~full : (is_a ? ~mb1 : mb1));
            const uint32_t mo2 = io < brow ? full : (io > brow ? ~full : (is_a ? ~mb2 : mb2));
            b[0] = be.x & me0; b[1] = be.y & me1;
            b[2] = bo.x & mo0; b[3] = bo.y & mo1;
            b[4] = bk & ((me2 & 0xffffu) | (mo2 << 16));
          }
          pair_b3(R, prev + woff, slotp + woff, b);
          __syncwarp();  // every lane is done with `prev` before its slot is refilled
        }
        prev = slotp;
        loader_step(L, S, kq, lane);
      }
      const unsigned char* mp = cursor_take(C);
      // the group that ends in this quad; after the last quad of the run also the one after it
      // (the lane's accumulator columns 2c, 2c+1 lie in half c >> 1 of the MMA columns)
      const bool last = quad == nquads - 1;
      const bool acc_a = ((ga ^ (c >> 1)) & 1) == 0;
      const int grp = acc_a ? ga : ga + 1;
      const bool on = (acc_a || last) && grp - 5 * run < ng;
      fold_b3(&R, &S.T, mp, grp, acc_a ? 0 : 1, on, lane);
      loader_step(L, S, kq, lane);
    }
  }
}

__device__ void consumer_role(Smem& S, const FusedParams& P, int* err) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kq = warp;
  const int g = lane >> 2, c = lane & 3;
  Loader L;
  L.p = -1; L.run = 0; L.i = 0; L.nt = 0; L.ntot = 0; L.N = 0; L.rows_left = 0; L.b3 = 0;
  L.w = nullptr;
  L.slot = 0;
  L.ring = smem_u32(S.ring[warp][0]);
#pragma unroll
  for (int r = 0; r < 4; ++r) L.roff[r] = ring_off(r, lane);
  loader_next_run(&L, &S, kq, lane, 1);
  // The weights do not depend on the tables: start filling the ring first.  Only part of it:
  // the copies queue up behind the memory system's limit on requests in flight, and the first
  // table should be built while they travel, not after the last one was accepted.
  constexpr int kEarly = 2;
#pragma unroll 1
  for (int k = 0; k < kEarly; ++k) loader_step(L, S, kq, lane);
  Cursor C;
  C.ring = S.ring[warp][0];
  C.slot = 0;
  RunState R;
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int s = 0; s < 2; ++s) {
#pragma unroll
      for (int e = 0; e < 4; ++e) R.acc[j][s][e] = 0;
      R.vs[j][s][0] = 0.f; R.vs[j][s][1] = 0.f;
    }

  int cur_tab = -1;
  const int n_parts = S.n_parts;
#pragma unroll 1
  for (int p = 0; p < n_parts; ++p) {
    const PartDesc& d = S.parts[p];
    const int B = d.B;
    if (d.tab != cur_tab) {
      const void* xsrc = d.phase ? static_cast<const void*>(P.h + S.slot[d.s].hoff) : static_cast<const void*>(P.x);
      // phase 1 needs the digits of the quanta this CTA's parts of the slot cover, not the whole vector
      unsigned need = 0xffffffffu;
      if (d.phase) {
        need = 0u;
        for (int pp = p; pp < n_parts && S.parts[pp].tab == d.tab; ++pp)
          need |= (S.parts[pp].qb >= 32 ? 0xffffffffu : ((1u << S.parts[pp].qb) - 1u)) & ~((1u << S.parts[pp].qa) - 1u);
      }
      // the h chunks of a slot are the reduction groups of its down projection: their flags gate the build
      const int* flags = d.phase ? P.counters + 2 * S.pairs_total + S.slot[d.s].ctrb : nullptr;
      build_table(&S.T, xsrc, d.phase, d.ngroups * kGroup, B, need, flags, err, S.spin, warp, lane);
      if (cur_tab < 0) {
#pragma unroll 1
        for (int k = kEarly; k < kRing - 1; ++k) loader_step(L, S, kq, lane);
      }
      cur_tab = d.tab;
    }
    if (B == 1) part_i8<1>(R, L, C, S, d, kq, lane);
    else if (B == 2) part_i8<2>(R, L, C, S, d, kq, lane);
    else if (B == 4) part_i8<4>(R, L, C, S, d, kq, lane);
    else part_b3(R, L, C, S, d, kq, lane);
    // end of the part: fold the MMA columns of the four lanes of a row, hand the columns to the finisher
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int s = 0; s < 2; ++s)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          R.vs[j][s][e] += __shfl_xor_sync(0xffffffffu, R.vs[j][s][e], 1);
          R.vs[j][s][e] += __shfl_xor_sync(0xffffffffu, R.vs[j][s][e], 2);
        }
    const int rs = p % kRedSlots;
    mbar_wait(&S.redempty[rs], ((p / kRedSlots) & 1) ^ 1, err, kErrRedEmpty, 64, S.spin);
    if (c == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<float4*>(&S.red[rs][kq][4 * (g + 8 * j)]) =
            make_float4(R.vs[j][0][0], R.vs[j][0][1], R.vs[j][1][0], R.vs[j][1][1]);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&S.redfull[rs]);
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int s = 0; s < 2; ++s) { R.vs[j][s][0] = 0.f; R.vs[j][s][1] = 0.f; }
  }
  cp_async_wait<0>();
}

// ---- finisher ---------------------------------------------------------------------------------
// Sum the partial slots of columns n..n+3 in slice order and restore them to zero; `slot_set`
// says which slots hold a partial (one bit per part, at the part's first quantum).
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

// Two jobs at once (gate and up partials of a column chunk), slot sets given by value: up to
// four slots of each job are in flight together (one L2 round trip for a strip cut in up to four);
// each job is summed in slice order.
__device__ __noinline__ void drain_pair(float* sa, float* sb, size_t c_total, unsigned ma, unsigned mb, float4& a,
                                           float4& b) {
  constexpr int kB = 4;
  a = make_float4(0.f, 0.f, 0.f, 0.f);
  b = a;
  const float4 zero = a;
  while (ma | mb) {
    float4* qa[kB];
    float4* qb[kB];
    float4 ta[kB], tb[kB];
#pragma unroll
    for (int i = 0; i < kB; ++i) {
      qa[i] = nullptr;
      qb[i] = nullptr;
      if (ma) {
        qa[i] = reinterpret_cast<float4*>(sa + static_cast<size_t>(__ffs(ma) - 1) * c_total);
        ma &= ma - 1;
        ta[i] = __ldcg(qa[i]);
      }
      if (mb) {
        qb[i] = reinterpret_cast<float4*>(sb + static_cast<size_t>(__ffs(mb) - 1) * c_total);
        mb &= mb - 1;
        tb[i] = __ldcg(qb[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < kB; ++i) {
      if (qa[i]) { a.x += ta[i].x; a.y += ta[i].y; a.z += ta[i].z; a.w += ta[i].w; __stcg(qa[i], zero); }
      if (qb[i]) { b.x += tb[i].x; b.y += tb[i].y; b.z += tb[i].z; b.w += tb[i].w; __stcg(qb[i], zero); }
    }
  }
}

// Continue a slice-order sum: add the partial slots of `mask` (up to four loads in flight) and
// restore them to zero.
__device__ __noinline__ void drain_more(float* s, size_t c_total, unsigned mask, float4& acc) {
  constexpr int kB = 4;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  while (mask) {
    float4* q[kB];
    float4 t[kB];
#pragma unroll
    for (int i = 0; i < kB; ++i) {
      q[i] = nullptr;
      if (mask) {
        q[i] = reinterpret_cast<float4*>(s + static_cast<size_t>(__ffs(mask) - 1) * c_total);
        mask &= mask - 1;
        t[i] = __ldcg(q[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < kB; ++i)
      if (q[i]) { acc.x += t[i].x; acc.y += t[i].y; acc.z += t[i].z; acc.w += t[i].w; __stcg(q[i], zero); }
  }
}

__device__ __forceinline__ unsigned long long ld_acquire64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void store_half4(__half* dst, const float4& v) {
  const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
  uint2 o;
  o.x = *reinterpret_cast<const uint32_t*>(&lo);
  o.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = o;
}
__device__ __forceinline__ float4 round_half4(const float4& v) {
  return make_float4(round_h(v.x), round_h(v.y), round_h(v.z), round_h(v.w));
}

// Finisher warp f takes the parts p = f, f + kFin, ...: it owns reduction slot f.
__device__ void finisher_role(Smem& S, const FusedParams& P, int* err) {
  const int lane = threadIdx.x & 31;
  const int n_parts = S.n_parts;
  unsigned* cw = reinterpret_cast<unsigned*>(P.counters);
  const int rs = (threadIdx.x >> 5) - kCons;
  for (int p = rs; p < n_parts; p += kFin) {
    const PartDesc& d = S.parts[p];
    mbar_wait(&S.redfull[rs], (p / kRedSlots) & 1, err, kErrRedFull, 64, S.spin);
    float4 r = *reinterpret_cast<const float4*>(&S.red[rs][0][4 * lane]);
#pragma unroll
    for (int q = 1; q < kLanes; ++q) {
      const float4 t = *reinterpret_cast<const float4*>(&S.red[rs][q][4 * lane]);
      r.x += t.x; r.y += t.y; r.z += t.z; r.w += t.w;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&S.redempty[rs]);

    const bool col_on = 4 * lane < d.ncols;
    const size_t ct = static_cast<size_t>(P.c_total);
    float4* my_slot = reinterpret_cast<float4*>(P.partial + static_cast<size_t>(d.qa) * ct + d.colp + 4 * lane);
    const int n = d.c * 128 + 4 * lane;
    if (d.phase == 0) {
      // One 64-bit word per (slot, column chunk): quanta arrived (bits 0..7), quanta whose partial
      // row is published (bits 8..15), the set of published partial slots (gate: bits 32..47, up:
      // 48..63).  A part arrives first.  If it is the last to arrive and every other row is already
      // published (the rule at the end of the gate/up phase, which is what the down phase waits
      // for), it completes the pair with its own sums still in registers: no store, no fence, no
      // second round trip on that path.  Otherwise it publishes its row like the others, and
      // whoever publishes last completes the pair from memory.  Nobody waits for anybody, and the
      // sums are formed in slice order on either path.
      const int mine_q = d.qb - d.qa;
      unsigned long long* c64 = reinterpret_cast<unsigned long long*>(P.counters) + d.ctr;
      const unsigned long long my_bit = 1ull << (32 + 16 * d.mask + d.qa);
      unsigned long long word = 0ull;
      int path = 0;  // 0: not the completer, 1: completes from registers, 2: completes from memory
      if (lane == 0) {
        word = atomicAdd(c64, static_cast<unsigned long long>(mine_q));
        if (static_cast<int>(word & 0xffull) + mine_q == d.expected && static_cast<int>((word >> 8) & 0xffull) == d.expected - mine_q)
          path = 1;
      }
      path = __shfl_sync(0xffffffffu, path, 0);
      if (path == 0) {
        if (col_on) __stcg(my_slot, r);
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          word = atomicAdd(c64, (static_cast<unsigned long long>(mine_q) << 8) | my_bit) | my_bit;
          if (static_cast<int>((word >> 8) & 0xffull) + mine_q == d.expected) path = 2;
        }
        path = __shfl_sync(0xffffffffu, path, 0);
        if (path == 0) continue;
      }
      if (lane == 0) *c64 = 0ull;
      const unsigned hi = __shfl_sync(0xffffffffu, static_cast<unsigned>(word >> 32), 0);
      __threadfence();
      const SlotInfo& I = S.slot[d.s];
      if (col_on) {
        float* sa = P.partial + I.colb[0] + n;
        float* sb = sa + I.F;
        const unsigned ma = hi & 0xffffu, mb = hi >> 16;
        float4 a, b;
        if (path == 2) {
          drain_pair(sa, sb, ct, ma, mb, a, b);
        } else {
          // slots below this part's slice of its own matrix and every slot of the other matrix,
          // then this part's sums, then the slots above
          const unsigned below = (1u << d.qa) - 1u;
          if (d.mask == 0) {
            drain_pair(sa, sb, ct, ma & below, mb, a, b);
            a.x += r.x; a.y += r.y; a.z += r.z; a.w += r.w;
            drain_more(sa, ct, ma & ~below, a);
          } else {
            drain_pair(sa, sb, ct, ma, mb & below, a, b);
            b.x += r.x; b.y += r.y; b.z += r.z; b.w += r.w;
            drain_more(sb, ct, mb & ~below, b);
          }
        }
        a = round_half4(a);
        b = round_half4(b);
        *reinterpret_cast<float4*>(P.h + I.hoff + n) =
            make_float4(silu_f32(a.x) * b.x, silu_f32(a.y) * b.y, silu_f32(a.z) * b.z, silu_f32(a.w) * b.w);
      }
      __threadfence();
      __syncwarp();
      if (lane == 0) *reinterpret_cast<volatile int*>(P.counters + 2 * S.pairs_total + d.ctr) = 1;  // h chunk complete
      continue;
    }
    if (col_on) __stcg(my_slot, r);
    if (P.S <= 2) {
      // Down projections of at most two slots: the slot sets of both (28 bits each, one bit per
      // quantum) ride above an 8-bit arrival count in one 64-bit word per column chunk.
      __threadfence();
      __syncwarp();
      unsigned cnt = 0, m0 = 0, m1 = 0;
      if (lane == 0) {
        unsigned long long* c64 = reinterpret_cast<unsigned long long*>(P.counters) + ((3 * S.pairs_total + 1) >> 1) + d.c;
        const unsigned long long mine = 1ull << (8 + 28 * d.s + d.qa);
        const unsigned long long old = atomicAdd(c64, static_cast<unsigned long long>(d.qb - d.qa) | mine);
        cnt = static_cast<unsigned>(old & 0xffu) + static_cast<unsigned>(d.qb - d.qa);
        const unsigned long long m = (old | mine) >> 8;
        m0 = static_cast<unsigned>(m) & 0xfffffffu;
        m1 = static_cast<unsigned>(m >> 28) & 0xfffffffu;
        if (static_cast<int>(cnt) == d.expected) *c64 = 0ull;
      }
      cnt = __shfl_sync(0xffffffffu, cnt, 0);
      m0 = __shfl_sync(0xffffffffu, m0, 0);
      m1 = __shfl_sync(0xffffffffu, m1, 0);
      if (static_cast<int>(cnt) != d.expected) continue;
      __threadfence();
      if (col_on) {
        float4 x2[2];
        drain_pair(P.partial + S.slot[0].colb[1] + n, P.partial + S.slot[P.S - 1].colb[1] + n, ct, m0, P.S > 1 ? m1 : 0u,
                   x2[0], x2[1]);
        float4 accw = make_float4(0.f, 0.f, 0.f, 0.f), res = accw;
#pragma unroll
        for (int s = 0; s < 2; ++s)
          if (s < P.S) {
            const float4 v = round_half4(x2[s]);
            if (s < P.A) {
              const float wgt = __half2float(S.sel_w[s]);
              accw.x = fmaf(wgt, v.x, accw.x); accw.y = fmaf(wgt, v.y, accw.y);
              accw.z = fmaf(wgt, v.z, accw.z); accw.w = fmaf(wgt, v.w, accw.w);
              if (s == P.A - 1) res = round_half4(accw);
            } else {
              res = round_half4(make_float4(res.x + v.x, res.y + v.y, res.z + v.z, res.w + v.w));
            }
          }
        store_half4(P.out + n, res);
      }
      continue;
    }
    if (lane == 0) atomicOr(cw + d.mask, 1u << (d.qa & 31));
    __threadfence();
    __syncwarp();
    int last = 0;
    if (lane == 0) {
      const int add = d.qb - d.qa;
      const int old = atomicAdd(P.counters + d.ctr, add);
      last = (old + add == d.expected);
      if (last) P.counters[d.ctr] = 0;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) continue;
    __threadfence();
    {
      if (col_on) {
        float4 accw = make_float4(0.f, 0.f, 0.f, 0.f), res = accw;
        for (int s = 0; s < P.S; ++s) {
          const SlotInfo& I = S.slot[s];
          const float4 x2 = round_half4(drain_slots(P.partial + I.colb[1] + n, ct, cw + I.maskb[1] + d.c, I.nq[1]));
          if (s < P.A) {
            const float wgt = __half2float(S.sel_w[s]);
            accw.x = fmaf(wgt, x2.x, accw.x); accw.y = fmaf(wgt, x2.y, accw.y);
            accw.z = fmaf(wgt, x2.z, accw.z); accw.w = fmaf(wgt, x2.w, accw.w);
            if (s == P.A - 1) res = round_half4(accw);
          } else {
            res = round_half4(make_float4(res.x + x2.x, res.y + x2.y, res.z + x2.z, res.w + x2.w));
          }
        }
        store_half4(P.out + n, res);
      }
      __syncwarp();
      if (lane == 0)
        for (int s = 0; s < P.S; ++s) cw[S.slot[s].maskb[1] + d.c] = 0u;
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1) moe_decode_kernel(const __grid_constant__ FusedParams P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Smem& S = *reinterpret_cast<Smem*>(smem_raw);
  const int warp = threadIdx.x >> 5;
  int* err = P.counters + kErrSlot;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kRedSlots; ++s) {
      mbar_init(&S.redfull[s], kCons);
      mbar_init(&S.redempty[s], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Ahead of the dependency wait: what does not depend on earlier kernels.  The per-expert bit
  // widths and offsets go to shared memory, the router matrix is pulled into L2.
  if (P.E <= kMetaE) {
    for (int i = threadIdx.x; i < 7 * P.E; i += kThreads) {
      const int a = i / P.E, e = i - a * P.E;
      const int* src = a == 0 ? P.nbits1 : a == 1 ? P.nbits2 : a == 2 ? P.wqs1 : a == 3 ? P.wqs2
                     : a == 4 ? P.zss1 : a == 5 ? P.zss3 : P.zss2;
      S.emeta[a][e] = src ? src[e] : 0;
    }
  }
  if (P.do_route) {
    const size_t lines = (static_cast<size_t>(P.E) * P.D * sizeof(__half) + 127) / 128;
    for (size_t i = threadIdx.x; i < lines; i += kThreads)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(P.gate) + i * 128));
  }
  // the activation's lines too: whoever writes them later writes into L2, where they then already are
  for (size_t i = threadIdx.x; i < (static_cast<size_t>(P.D) * sizeof(__half) + 127) / 128; i += kThreads)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(P.x) + i * 128));
  // One line of every 2 MB page of the expert matrices: the address translations are resolved
  // while the previous kernel drains, not when all CTAs ask for their first rows at once.
  {
    constexpr long long kPage = 2ll << 20;
    const char* base[3] = {reinterpret_cast<const char*>(P.w1.wq), reinterpret_cast<const char*>(P.w3.wq),
                           reinterpret_cast<const char*>(P.w2.wq)};
#pragma unroll
    for (int m = 0; m < 3; ++m) {
      const long long pages = (P.wq_bytes[m] + kPage - 1) / kPage;
      for (long long i = blockIdx.x * kThreads + threadIdx.x; i < pages; i += static_cast<long long>(gridDim.x) * kThreads)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base[m] + i * kPage));
    }
  }
  // The next kernel of the stream may start its prologue; everything below reads results of
  // the previous kernel (the activation, the zeroed workspace) and therefore waits for it.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) {
    const int lim = P.counters[kLimitWord];
    S.spin = lim > 0 ? lim : kSpinLimit;
  }
  if (P.do_route) {
    route_cta(S, P);
  } else if (threadIdx.x < P.A) {
    S.sel_e[threadIdx.x] = static_cast<int>(P.idx[threadIdx.x]);
    S.sel_w[threadIdx.x] = P.w[threadIdx.x];
  }
  __syncthreads();
  if (warp == 0) make_plan(S, P);
  __syncthreads();
  if (S.overflow && threadIdx.x == 0) atomicExch(err, 14);
  if (warp < kCons) consumer_role(S, P, err);
  else finisher_role(S, P, err);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int old = atomicAdd(P.counters + kExitSlot, 1);
    S.overflow = old == static_cast<int>(gridDim.x) - 1;  // the last CTA: nobody reads the h flags any more
  }
  __syncthreads();
  if (S.overflow) {
    for (int i = threadIdx.x; i < S.pairs_total; i += kThreads) P.counters[2 * S.pairs_total + i] = 0;
    if (threadIdx.x == 0) P.counters[kExitSlot] = 0;
  }
}

}  // namespace fused

// ---- host ----------------------------------------------------------------------------------------
static int fused_sm_count() {
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

static fused::Mat3 mat_of(const gemq_stacked_t& W) {
  return {reinterpret_cast<const uint32_t*>(W.wq), static_cast<const __half*>(W.scales), static_cast<const __half*>(W.zeros)};
}
static fused::Mat3 mat_of(const gemq_single_t& W) {
  return {reinterpret_cast<const uint32_t*>(W.wq), static_cast<const __half*>(W.scales), static_cast<const __half*>(W.zeros)};
}
static bool mat_aligned(const fused::Mat3& m) { return aligned16(m.wq) && aligned16(m.sc) && aligned16(m.zr); }

// True when the fused kernel takes this layer; the limits are the table sizes (reduction
// lengths up to kMaxK), the counter words and the per-CTA part list.
bool decode_fused_ok(const gemq_moe_layer_t* L, size_t partial_floats) {
  using namespace fused;
  const int D = L->hidden, F = L->ffn, A = L->top_k, SF = L->shared_ffn;
  if (L->group_size != kGroup || D % 128 || F % 128 || SF % 128) return false;
  if (D > kMaxK || F > kMaxK || SF > kMaxK || A > kMaxSlots) return false;
  if (D > 8192) return false;  // the slot set of a gate / up chunk (one bit per quantum) must fit 16 bits
  if (SF > 0 && (L->s1.group_size != kGroup || L->s3.group_size != kGroup || L->s2.group_size != kGroup)) return false;
  if (!mat_aligned(mat_of(L->w1)) || !mat_aligned(mat_of(L->w3)) || !mat_aligned(mat_of(L->w2))) return false;
  if (SF > 0 && (!mat_aligned(mat_of(L->s1)) || !mat_aligned(mat_of(L->s3)) || !mat_aligned(mat_of(L->s2)))) return false;
  const int S = A + (SF > 0 ? 1 : 0);
  const int pairs = A * (F / 128) + SF / 128, nch1 = D / 128;
  if (3 * pairs + (S + 1) * nch1 + 8 >= kMaxCounters) return false;
  const int maxf = F > SF ? F : SF;
  const size_t c_total = static_cast<size_t>(2 * (A * F + SF) + S * D);
  const size_t slices = static_cast<size_t>(cdiv(cdiv(D > maxf ? D : maxf, kGroup), 4));
  if (slices * c_total > partial_floats) return false;
  // parts per CTA (a part is a run of quanta of one matrix and column chunk): bound for any bit widths
  int sms = fused_sm_count();
  if (sms <= 0) return false;
  const int u0 = pairs * 2 * cdiv(D / kGroup, 4), u1 = nch1 * (A * cdiv(F / kGroup, 4) + cdiv(SF / kGroup, 4));
  const int grid = (u0 > u1 ? u0 : u1) < sms ? (u0 > u1 ? u0 : u1) : sms;
  const int nq0 = cdiv(D / kGroup, 5), nq1 = cdiv((SF > 0 && SF < F ? SF : F) / kGroup, 5);
  const int parts = cdiv(cdiv(u0, grid) + S, nq0) + cdiv(cdiv(u1, grid) + S, nq1) + 4 * S + 4;
  return parts <= kMaxParts;
}

// Launch the fused layer kernel for one token.  `route_in_kernel`: the router runs inside the
// launch (E <= 32, D % 256 == 0); otherwise idx / w hold the routing already.
int launch_decode_fused(const gemq_moe_layer_t* L, const __half* x, __half* out, int64_t* idx, __half* w,
                        int route_in_kernel, int route_mode, float* partial, int* counters, float* h,
                        cudaStream_t stream) {
  using namespace fused;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  const size_t smem = sizeof(Smem);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(moe_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
        cudaSuccess)
      return GEMQ_ERR_LAUNCH;
    attr_set[dev] = true;
  }
  const int sms = fused_sm_count();
  if (sms <= 0) return GEMQ_ERR_LAUNCH;
  FusedParams P = {};
  P.x = x; P.gate = static_cast<const __half*>(L->gate); P.out = out;
  P.idx = reinterpret_cast<long long*>(idx); P.w = w;
  P.D = L->hidden; P.F = L->ffn; P.E = L->n_experts; P.A = L->top_k; P.SF = L->shared_ffn;
  P.S = P.A + (P.SF > 0 ? 1 : 0);
  P.do_route = route_in_kernel; P.route_mode = route_mode; P.renorm = L->renorm;
  P.w1 = mat_of(L->w1); P.w3 = mat_of(L->w3); P.w2 = mat_of(L->w2);
  P.nbits1 = L->w1.nbits; P.wqs1 = L->w1.wq_strides; P.zss1 = L->w1.zs_strides; P.zss3 = L->w3.zs_strides;
  P.nbits2 = L->w2.nbits; P.wqs2 = L->w2.wq_strides; P.zss2 = L->w2.zs_strides;
  if (P.SF > 0) {
    P.s1 = mat_of(L->s1); P.s3 = mat_of(L->s3); P.s2 = mat_of(L->s2);
    P.sbits = L->s1.nbits;
  }
  P.partial = partial; P.counters = counters; P.h = h;
  P.wq_bytes[0] = L->w1.wq_rows * static_cast<long long>(P.F) * 4;
  P.wq_bytes[1] = L->w3.wq_rows * static_cast<long long>(P.F) * 4;
  P.wq_bytes[2] = L->w2.wq_rows * static_cast<long long>(P.D) * 4;
  const int up_cols = 2 * (P.A * P.F + P.SF), down_cols = P.S * P.D;
  P.c_total = up_cols + down_cols;
  P.up_cols = up_cols;
  // at least one quantum per CTA in the larger phase (a quantum is at most 5 groups)
  const int u0 = (P.A * (P.F / 128) + P.SF / 128) * 2 * cdiv(P.D / kGroup, 5);
  const int u1 = (P.D / 128) * (P.A * cdiv(P.F / kGroup, 5) + (P.SF > 0 ? cdiv(P.SF / kGroup, 5) : 0));
  const int units = u0 > u1 ? u0 : u1;
  const int grid = units < sms ? (units < 1 ? 1 : units) : sms;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, moe_decode_kernel, P) != cudaSuccess) return GEMQ_ERR_LAUNCH;
  return launch_status();
}

}  // namespace gemq

