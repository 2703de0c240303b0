// Dequant-fused GEMV for decode (1..8 activation rows per pass) on sm_100a.
//
// The packed words never pass through shared memory.  Each lane loads 128 bits
// (four neighbouring output columns of one word row), masks code pairs IN PLACE into
// the mantissa of two fp16 lanes -- an fp16 whose exponent field is zero is the
// subnormal m * 2^-24, so `word & mask` IS a valid fp16x2 operand holding the integer
// codes (times 2^pos for a code that sits `pos` bits up) -- and feeds them to
// mma.sync.m16n8k16 as the A operand.  The B operand is the activation, pre-scaled
// per k by 2^(c-pos) and stored once per CTA in shared memory in fragment order.
// Products are exact in fp32; sum_k q*x is accumulated per quantisation group and the
// group scale/offset are applied in fp32:
//     y[n] = sum_g  s[g,n] * (sum_{k in g} q[k,n] x[k])  +  z[g,n] * (sum_{k in g} x[k])
// With one activation row the 8 MMA columns carry 8 different groups (the B lane of
// column d supplies x only while the loop is inside group d), so scales are applied
// once per 8 groups.  With TT rows the columns are (group, row) pairs.
//
// Work split: one CTA = 128 output columns x one k-slice (8 groups; 10 for 3-bit) of
// one job.  Split-K partials go to an fp32 workspace; the CTA that arrives last at a
// column chunk adds them in slice order (deterministic) and runs the epilogue.
#include "gemv.cuh"

namespace gemq {

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ----------------------------------------------------------------------------------
// Shared-memory state of one CTA
// ----------------------------------------------------------------------------------
template <int TT>
struct TileSmem {
  // Activation table.  1/2/4-bit: [TT][word row][eps halves] (<= 1024 halves per row of x).
  // 3-bit: [2 variants][128 word rows][16 halves].
  static constexpr int kTabWords = (TT * 512 > 2048) ? TT * 512 : 2048;
  uint32_t tab[kTabWords];
  uint32_t zero_row[16];
  float xsum[TT][kSliceGroupsB3];  // sum of x over each group of the slice
  float fin[TT];                   // 2^(24 - c): undoes the subnormal and activation scaling
  int cshift[TT];                  // c
  float red_sum[kCtaWarps][TT][kSliceGroupsB3];
  float red_max[kCtaWarps][TT];
  int last;
};

template <bool SILU>
__device__ __forceinline__ float load_act(const GemvJob& J, int t, int k) {
  if (SILU) {
    const float a = __half2float(J.xa[static_cast<size_t>(t) * J.ldx + k]);
    const float b = __half2float(J.xb[static_cast<size_t>(t) * J.ldx + k]);
    return silu_f32(a) * b;
  }
  return __half2float(J.xa[static_cast<size_t>(t) * J.ldx + k]);
}

// Group sums and the power-of-two scaling of up to TT activation rows over the k-range
// [k0, k0 + ng*128).  Thread `tid` owns element tid of every group.
template <int TT, bool SILU>
__device__ __forceinline__ void act_stats(TileSmem<TT>& S, const GemvJob& J, int t0, int nt, int k0, int ng) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int tc = 0; tc < TT; ++tc) {
    float mx = 0.f;
#pragma unroll
    for (int i = 0; i < kSliceGroupsB3; ++i) {
      float v = 0.f;
      if (tc < nt && i < ng) v = load_act<SILU>(J, t0 + tc, k0 + i * kGroup + tid);
      mx = fmaxf(mx, fabsf(v));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) S.red_sum[warp][tc][i] = v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) S.red_max[warp][tc] = mx;
  }
  __syncthreads();
  if (tid < TT * kSliceGroupsB3) {
    const int tc = tid / kSliceGroupsB3, i = tid % kSliceGroupsB3;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kCtaWarps; ++w) s += S.red_sum[w][tc][i];
    S.xsum[tc][i] = s;
  }
  if (tid < TT) {
    float mx = 0.f;
#pragma unroll
    for (int w = 0; w < kCtaWarps; ++w) mx = fmaxf(mx, S.red_max[w][tid]);
    // c puts the largest |x| of the slice into [2^14, 2^15): full fp16 precision for x
    // down to 2^-20 of the maximum even after the 2^-9 shift of the highest code lane.
    int e = static_cast<int>((__float_as_uint(mx) >> 23) & 0xffu) - 127;
    int c = 14 - e;
    c = c < -15 ? -15 : (c > 40 ? 40 : c);
    S.cshift[tid] = c;
    S.fin[tid] = pow2i(24 - c);
  }
  if (tid < 16) S.zero_row[tid] = 0u;
  __syncthreads();
}

// ----------------------------------------------------------------------------------
// 1-, 2- and 4-bit tiles
// ----------------------------------------------------------------------------------
template <int B>
struct Pow2Fmt {
  static constexpr int kEps = 32 / B;       // codes per word
  static constexpr int kPairs = kEps / 2;   // fp16x2 operands per word: codes (j, j + eps/2)
  static constexpr int kPos = 10 / B;       // codes per half that fit the 10 mantissa bits in place
  static constexpr int kMma = kEps / 4;     // MMAs per word row and row pair
  static constexpr uint32_t kMask = ((1u << B) - 1u) * 0x00010001u;
  // A operand number q of a word: codes j = q (low half) and q + eps/2 (high half).
  __device__ static __forceinline__ uint32_t operand(uint32_t w, int q) {
    const int stage = q / kPos, jj = q % kPos;
    return (w >> (stage * kPos * B)) & (kMask << (B * jj));
  }
  __device__ static __forceinline__ int pos_of_pair(int q) { return B * (q % kPos); }
};

template <int B, int TT, bool SILU>
__device__ __forceinline__ void build_table_pow2(TileSmem<TT>& S, const GemvJob& J, int t0, int nt, int k0, int ng) {
  using F = Pow2Fmt<B>;
  const int tid = threadIdx.x;
  __half* tab = reinterpret_cast<__half*>(S.tab);
#pragma unroll
  for (int tc = 0; tc < TT; ++tc) {
    if (tc < nt) {
      const int c = S.cshift[tc];
#pragma unroll
      for (int i = 0; i < kSliceGroups; ++i) {
        if (i < ng) {
          const int kl = i * kGroup + tid;
          const float v = load_act<SILU>(J, t0 + tc, k0 + kl);
          const int row = kl / F::kEps, j = kl % F::kEps;
          const int hi = j / F::kPairs, q = j % F::kPairs;
          tab[tc * 1024 + row * F::kEps + 2 * q + hi] = __float2half_rn(v * pow2i(c - F::pos_of_pair(q)));
        }
      }
    }
  }
}

// One CTA tile for B in {1,2,4}: columns [n0w, n0w+32) per warp, groups [g0, g1).
// Leaves this lane's four column results per token pair in v[set][e].
template <int B, int TT, bool SILU>
__device__ __forceinline__ void tile_pow2(TileSmem<TT>& S, const GemvJob& J, const ResolvedJob& R,
                                          int t0, int nt, int g0, int g1, int n_lane, bool warp_on,
                                          float (&v)[2][4]) {
  using F = Pow2Fmt<B>;
  constexpr int WG = 8 / TT;       // groups per accumulation window
  constexpr int IPW = WG * B;      // loop iterations per window (B iterations of 4 word rows per group)
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int N = J.N;
  const int ng = g1 - g0;
  const int iters = warp_on ? ng * B : 0;
  const int wr0 = g0 * (kGroup / F::kEps);
  const size_t rs = static_cast<size_t>(4) * N;  // words per loop iteration
  const uint32_t* wp = R.wq + static_cast<size_t>(wr0 + c) * N + n_lane;

  uint4 ring[kRing];
#pragma unroll
  for (int u = 0; u < kRing; ++u)
    if (u < iters) ring[u] = ld_stream_v4(wp + u * rs);

  act_stats<TT, SILU>(S, J, t0, nt, g0 * kGroup, ng);
  build_table_pow2<B, TT, SILU>(S, J, t0, nt, g0 * kGroup, ng);
  __syncthreads();

  const int tcol = g % TT, dcol = g / TT;
  const bool tok_ok = tcol < nt;
  const uint32_t* my_tab = S.tab + tcol * 512 + c * F::kPairs;
  const __half* sc = R.scales + static_cast<size_t>(g0) * N + n_lane;
  const __half* zr = R.zeros + static_cast<size_t>(g0) * N + n_lane;

  float acc[2][4], out[2][4], outz[2][4];
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[s][e] = out[s][e] = outz[s][e] = 0.f;
  uint2 sreg[2], zreg[2];
  sreg[0] = sreg[1] = zreg[0] = zreg[1] = make_uint2(0u, 0u);

  for (int it0 = 0; it0 < iters; it0 += kRing) {
#pragma unroll
    for (int u = 0; u < kRing; ++u) {
      const int it = it0 + u;
      if (it < iters) {
        const uint4 w4 = ring[u];
        if (it + kRing < iters) ring[u] = ld_stream_v4(wp + static_cast<size_t>(it + kRing) * rs);
        const int wi = it % IPW, wnd = it / IPW;
        if (wi == 0) {
#pragma unroll
          for (int p = 0; p < 2; ++p) {
            const int gl = wnd * WG + (2 * c + p) / TT;  // slice-local group of C column 2c+p
            if (gl < ng) {
              sreg[p] = *reinterpret_cast<const uint2*>(sc + static_cast<size_t>(gl) * N);
              zreg[p] = *reinterpret_cast<const uint2*>(zr + static_cast<size_t>(gl) * N);
            }
          }
        }
        const int gi = wi / B;
        const uint32_t* bp = (tok_ok && dcol == gi) ? my_tab + it * (4 * F::kPairs) : S.zero_row;
        uint32_t bf[F::kPairs];
#pragma unroll
        for (int q4 = 0; q4 < F::kPairs / 4; ++q4) {
          const uint4 t = *reinterpret_cast<const uint4*>(bp + 4 * q4);
          bf[4 * q4 + 0] = t.x; bf[4 * q4 + 1] = t.y; bf[4 * q4 + 2] = t.z; bf[4 * q4 + 3] = t.w;
        }
        const uint32_t wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
        for (int m = 0; m < F::kMma; ++m) {
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            mma16816(acc[s], F::operand(wv[2 * s], 2 * m), F::operand(wv[2 * s + 1], 2 * m),
                     F::operand(wv[2 * s], 2 * m + 1), F::operand(wv[2 * s + 1], 2 * m + 1),
                     bf[2 * m], bf[2 * m + 1]);
          }
        }
        if (wi == IPW - 1 || it == iters - 1) {
#pragma unroll
          for (int p = 0; p < 2; ++p) {
            const int gl = wnd * WG + (2 * c + p) / TT;
            const int tc = (2 * c + p) % TT;
            if (gl < ng) {
              const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sreg[p].x));
              const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sreg[p].y));
              const float2 z01 = __half22float2(*reinterpret_cast<const __half2*>(&zreg[p].x));
              const float2 z23 = __half22float2(*reinterpret_cast<const __half2*>(&zreg[p].y));
              const float xs = S.xsum[tc][gl];
              out[0][p] = fmaf(s01.x, acc[0][p], out[0][p]);
              out[0][2 + p] = fmaf(s01.y, acc[0][2 + p], out[0][2 + p]);
              out[1][p] = fmaf(s23.x, acc[1][p], out[1][p]);
              out[1][2 + p] = fmaf(s23.y, acc[1][2 + p], out[1][2 + p]);
              outz[0][p] = fmaf(z01.x, xs, outz[0][p]);
              outz[0][2 + p] = fmaf(z01.y, xs, outz[0][2 + p]);
              outz[1][p] = fmaf(z23.x, xs, outz[1][p]);
              outz[1][2 + p] = fmaf(z23.y, xs, outz[1][2 + p]);
            }
          }
#pragma unroll
          for (int s = 0; s < 2; ++s)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[s][e] = 0.f;
        }
      }
    }
  }
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int e = 0; e < 4; ++e) v[s][e] = fmaf(out[s][e], S.fin[(2 * c + (e & 1)) % TT], outz[s][e]);
}

// ----------------------------------------------------------------------------------
// 3-bit tiles: 10 codes per word, groups are not word aligned.  A 640-wide span
// (5 groups = 64 word rows) is word aligned; its five groups ride in MMA columns 0..4.
// A word that straddles two groups appears in two table variants (each holding only the
// activations of one of the groups), so no code is ever split.
// ----------------------------------------------------------------------------------
struct B3Fmt {
  __device__ static __forceinline__ uint32_t merge(uint32_t w) {  // codes 0-4 -> low half, 5-9 -> high half
    return (w & 0x00007fffu) | ((w << 1) & 0x7fff0000u);
  }
  __device__ static __forceinline__ uint32_t operand(uint32_t t, int q) {  // codes (q, q+5)
    return q < 3 ? (t & (0x00070007u << (3 * q))) : ((t >> 9) & (0x00070007u << (3 * (q - 3))));
  }
  __device__ static __forceinline__ int pos_of_pair(int q) { return 3 * (q < 3 ? q : q - 3); }
};

template <int TT, bool SILU>
__device__ __forceinline__ void build_table_b3(TileSmem<TT>& S, const GemvJob& J, int t, int k0, int ng) {
  const int tid = threadIdx.x;
  uint4* z4 = reinterpret_cast<uint4*>(S.tab);
#pragma unroll
  for (int i = 0; i < 4; ++i) z4[tid + i * kCtaThreads] = make_uint4(0u, 0u, 0u, 0u);  // 2048 words
  __syncthreads();
  __half* tab = reinterpret_cast<__half*>(S.tab);
  const int c = S.cshift[0];
#pragma unroll
  for (int i = 0; i < kSliceGroupsB3; ++i) {
    if (i < ng) {
      const int kl = i * kGroup + tid;
      const float v = load_act<SILU>(J, t, k0 + kl);
      const int row = kl / 10, j = kl % 10;
      const int hi = j / 5, q = j % 5;
      const int first_group = (row * 10) >> 7;
      const int variant = (i != first_group) ? 1 : 0;
      tab[variant * 2048 + row * 16 + 2 * q + hi] = __float2half_rn(v * pow2i(c - B3Fmt::pos_of_pair(q)));
    }
  }
}

template <int TT, bool SILU>
__device__ __forceinline__ void tile_b3(TileSmem<TT>& S, const GemvJob& J, const ResolvedJob& R,
                                        int t, int g0, int g1, int n_lane, bool warp_on, float (&v)[2][4]) {
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int N = J.N;
  const int ng = g1 - g0;
  const int kw = cdiv(J.K, 10);                 // word rows of the matrix
  const int wr0 = (g0 / 5) * 64;                // first word row of the slice
  const int nwnd = cdiv(ng, 5);
  const int iters = warp_on ? nwnd * 8 : 0;     // lane handles word rows wr0 + 8*it + 2c + {0,1}
  const uint32_t* wp = R.wq + static_cast<size_t>(wr0 + 2 * c) * N + n_lane;
  const size_t rs = static_cast<size_t>(8) * N;

  uint4 ring[kRing];
#pragma unroll
  for (int u = 0; u < kRing; ++u) {
    const int it = u >> 1, r = u & 1;
    ring[u] = make_uint4(0u, 0u, 0u, 0u);
    if (it < iters && wr0 + 8 * it + 2 * c + r < kw) ring[u] = ld_stream_v4(wp + it * rs + static_cast<size_t>(r) * N);
  }

  act_stats<TT, SILU>(S, J, t, 1, g0 * kGroup, ng);
  build_table_b3<TT, SILU>(S, J, t, g0 * kGroup, ng);
  __syncthreads();

  const __half* sc = R.scales + static_cast<size_t>(g0) * N + n_lane;
  const __half* zr = R.zeros + static_cast<size_t>(g0) * N + n_lane;
  float acc[2][4], out[2][4], outz[2][4];
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[s][e] = out[s][e] = outz[s][e] = 0.f;
  uint2 sreg[2], zreg[2];
  sreg[0] = sreg[1] = zreg[0] = zreg[1] = make_uint2(0u, 0u);

  for (int it0 = 0; it0 < iters; it0 += kRing / 2) {
#pragma unroll
    for (int u = 0; u < kRing / 2; ++u) {
      const int it = it0 + u;
      if (it < iters) {
        const uint4 wa = ring[2 * u], wb = ring[2 * u + 1];
        {
          const int nit = it + kRing / 2;
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            ring[2 * u + r] = make_uint4(0u, 0u, 0u, 0u);
            if (nit < iters && wr0 + 8 * nit + 2 * c + r < kw)
              ring[2 * u + r] = ld_stream_v4(wp + nit * rs + static_cast<size_t>(r) * N);
          }
        }
        const int wi = it & 7, wnd = it >> 3;
        if (wi == 0) {
#pragma unroll
          for (int p = 0; p < 2; ++p) {
            const int d = 2 * c + p;
            const int gl = wnd * 5 + d;
            if (d < 5 && gl < ng) {
              sreg[p] = *reinterpret_cast<const uint2*>(sc + static_cast<size_t>(gl) * N);
              zreg[p] = *reinterpret_cast<const uint2*>(zr + static_cast<size_t>(gl) * N);
            }
          }
        }
        // B operands: this lane is MMA column g = group offset inside the window.
        uint32_t bf[10];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int row = 8 * it + 2 * c + r;            // slice-local word row
          const int d0 = ((row * 10) >> 7) - wnd * 5;    // window-local group of the word's first code
          const uint32_t* bp = S.zero_row;
          if (g == d0) bp = S.tab + row * 8;
          else if (g == d0 + 1) bp = S.tab + 1024 + row * 8;
          const uint4 t4 = *reinterpret_cast<const uint4*>(bp);
          bf[5 * r + 0] = t4.x; bf[5 * r + 1] = t4.y; bf[5 * r + 2] = t4.z; bf[5 * r + 3] = t4.w;
          bf[5 * r + 4] = bp[4];
        }
        const uint32_t ma[4] = {B3Fmt::merge(wa.x), B3Fmt::merge(wa.y), B3Fmt::merge(wa.z), B3Fmt::merge(wa.w)};
        const uint32_t mb[4] = {B3Fmt::merge(wb.x), B3Fmt::merge(wb.y), B3Fmt::merge(wb.z), B3Fmt::merge(wb.w)};
#pragma unroll
        for (int m = 0; m < 5; ++m) {
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            // operand slot sl in 0..9: word row A pairs 0..4, then word row B pairs 0..4
            const int s0 = 2 * m, s1 = 2 * m + 1;
            const uint32_t a0 = s0 < 5 ? B3Fmt::operand(ma[2 * s], s0) : B3Fmt::operand(mb[2 * s], s0 - 5);
            const uint32_t a1 = s0 < 5 ? B3Fmt::operand(ma[2 * s + 1], s0) : B3Fmt::operand(mb[2 * s + 1], s0 - 5);
            const uint32_t a2 = s1 < 5 ? B3Fmt::operand(ma[2 * s], s1) : B3Fmt::operand(mb[2 * s], s1 - 5);
            const uint32_t a3 = s1 < 5 ? B3Fmt::operand(ma[2 * s + 1], s1) : B3Fmt::operand(mb[2 * s + 1], s1 - 5);
            mma16816(acc[s], a0, a1, a2, a3, bf[s0], bf[s1]);
          }
        }
        if (wi == 7) {
#pragma unroll
          for (int p = 0; p < 2; ++p) {
            const int d = 2 * c + p;
            const int gl = wnd * 5 + d;
            if (d < 5 && gl < ng) {
              const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sreg[p].x));
              const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sreg[p].y));
              const float2 z01 = __half22float2(*reinterpret_cast<const __half2*>(&zreg[p].x));
              const float2 z23 = __half22float2(*reinterpret_cast<const __half2*>(&zreg[p].y));
              const float xs = S.xsum[0][gl];
              out[0][p] = fmaf(s01.x, acc[0][p], out[0][p]);
              out[0][2 + p] = fmaf(s01.y, acc[0][2 + p], out[0][2 + p]);
              out[1][p] = fmaf(s23.x, acc[1][p], out[1][p]);
              out[1][2 + p] = fmaf(s23.y, acc[1][2 + p], out[1][2 + p]);
              outz[0][p] = fmaf(z01.x, xs, outz[0][p]);
              outz[0][2 + p] = fmaf(z01.y, xs, outz[0][2 + p]);
              outz[1][p] = fmaf(z23.x, xs, outz[1][p]);
              outz[1][2 + p] = fmaf(z23.y, xs, outz[1][2 + p]);
            }
          }
#pragma unroll
          for (int s = 0; s < 2; ++s)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[s][e] = 0.f;
        }
      }
    }
  }
  const float fin = S.fin[0];
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int e = 0; e < 4; ++e) v[s][e] = fmaf(out[s][e], fin, outz[s][e]);
}

// Sum MMA columns that belong to the same activation row.  NC = rows per pass.
template <int NC>
__device__ __forceinline__ void reduce_columns(float (&v)[2][4]) {
  if (NC == 1) {
#pragma unroll
    for (int s = 0; s < 2; ++s) { v[s][0] += v[s][1]; v[s][2] += v[s][3]; }
  }
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (NC <= 2) v[s][e] += __shfl_xor_sync(0xffffffffu, v[s][e], 1);
      if (NC <= 4) v[s][e] += __shfl_xor_sync(0xffffffffu, v[s][e], 2);
    }
}

// Store this lane's results of a pass with NC activation rows (first row t0) as partials.
template <int NC>
__device__ __forceinline__ void store_partials(const GemvParams& P, const GemvJob& J, int slice, int t0, int nt,
                                               int n_lane, const float (&v)[2][4]) {
  const int c = threadIdx.x & 3;
  const bool writer = (NC == 1) ? (c == 0) : (2 * c < NC);
  if (!writer) return;
#pragma unroll
  for (int p = 0; p < (NC == 1 ? 1 : 2); ++p) {
    const int tc = (2 * c + p) % NC;
    if (tc < nt) {
      float* dst = P.partial + (static_cast<size_t>(slice) * P.T + (t0 + tc)) * P.c_total + J.col_base + n_lane;
      *reinterpret_cast<float4*>(dst) = make_float4(v[0][p], v[0][2 + p], v[1][p], v[1][2 + p]);
    }
  }
}

template <int TT, bool SILU>
__global__ void __launch_bounds__(kCtaThreads) gemv_mma_kernel(const __grid_constant__ GemvParams P) {
  __shared__ __align__(16) TileSmem<TT> S;
  const int tid = threadIdx.x;
  const int tile = blockIdx.x;
  int j = 0;
  for (int i = 1; i < P.n_jobs; ++i)
    if (tile >= P.jobs[i].tile_base) j = i;
  const GemvJob& J = P.jobs[j];
  const int local = tile - J.tile_base;
  const int chunk = local / P.s_max, slice = local - chunk * P.s_max;
  const ResolvedJob R = resolve_job(J, kGroup);
  if (slice >= R.slices) return;

  const int t0 = blockIdx.y * TT;
  const int nt = min(TT, P.T - t0);
  const int ngroups = J.K / kGroup;
  const int spg = slice_groups(R.bits);
  const int g0 = slice * spg, g1 = min(g0 + spg, ngroups);
  const int n_warp = chunk * kCtaCols + (tid >> 5) * 32;
  const bool warp_on = n_warp < J.N;
  const int n_lane = n_warp + 4 * ((tid & 31) >> 2);

  float v[2][4];
  if (R.bits == 3) {
    for (int tc = 0; tc < nt; ++tc) {
      if (tc) __syncthreads();
      tile_b3<TT, SILU>(S, J, R, t0 + tc, g0, g1, n_lane, warp_on, v);
      reduce_columns<1>(v);
      if (warp_on) store_partials<1>(P, J, slice, t0 + tc, 1, n_lane, v);
    }
  } else {
    if (R.bits == 1) tile_pow2<1, TT, SILU>(S, J, R, t0, nt, g0, g1, n_lane, warp_on, v);
    else if (R.bits == 2) tile_pow2<2, TT, SILU>(S, J, R, t0, nt, g0, g1, n_lane, warp_on, v);
    else tile_pow2<4, TT, SILU>(S, J, R, t0, nt, g0, g1, n_lane, warp_on, v);
    reduce_columns<TT>(v);
    if (warp_on) store_partials<TT>(P, J, slice, t0, nt, n_lane, v);
  }

  // ---- arrival: the last CTA of a column chunk reduces the slices in order ----
  const bool combine = P.comb_out != nullptr;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int expected = R.slices;
    if (combine) {
      expected = 0;
      for (int i = 0; i < P.n_jobs; ++i) expected += resolve_job(P.jobs[i], kGroup).slices;
    }
    int* ctr = P.counters + blockIdx.y * P.n_chunks + (combine ? 0 : J.chunk_base) + chunk;
    const int old = atomicAdd(ctr, 1);
    S.last = (old == expected - 1);
    if (S.last) *ctr = 0;
  }
  __syncthreads();
  if (!S.last) return;
  __threadfence();
  const int n = chunk * kCtaCols + tid;
  if (n >= J.N) return;
  if (!combine) {
    for (int tc = 0; tc < nt; ++tc) {
      const float* src = P.partial + static_cast<size_t>(t0 + tc) * P.c_total + J.col_base + n;
      float sum = 0.f;
      for (int s = 0; s < R.slices; ++s) {
        float* q = const_cast<float*>(src) + static_cast<size_t>(s) * P.T * P.c_total;
        sum += ld_cg_f32(q);
        __stcg(q, 0.f);  // the partial region is all-zero between launches (the persistent kernel relies on it)
      }
      J.y[static_cast<size_t>(t0 + tc) * J.ldy + n] = __float2half_rn(sum);
    }
  } else {
    float accw = 0.f;
    __half res = __float2half_rn(0.f);
    for (int i = 0; i < P.n_jobs; ++i) {
      const GemvJob& Ji = P.jobs[i];
      const int sl = resolve_job(Ji, kGroup).slices;
      const float* src = P.partial + Ji.col_base + n;
      float sum = 0.f;
      for (int s = 0; s < sl; ++s) {
        float* q = const_cast<float*>(src) + static_cast<size_t>(s) * P.T * P.c_total;
        sum += ld_cg_f32(q);
        __stcg(q, 0.f);
      }
      const __half x2 = __float2half_rn(sum);
      if (Ji.y) Ji.y[n] = x2;
      if (i < P.comb_weighted) {
        accw = fmaf(__half2float(P.comb_w[i]), __half2float(x2), accw);
        if (i == P.comb_weighted - 1) res = __float2half_rn(accw);
      } else {
        res = __float2half_rn(__half2float(res) + __half2float(x2));
      }
    }
    P.comb_out[n] = res;
  }
}

// ----------------------------------------------------------------------------------
// Generic kernel: any group size / extent, one thread per output column, the reference's
// own arithmetic (fp16 fma de-quantisation, fp32 dot).  Used for shapes the tensor-core
// path does not take.
// ----------------------------------------------------------------------------------
template <bool SILU>
__global__ void __launch_bounds__(kCtaThreads) gemv_generic_kernel(const __grid_constant__ GemvParams P) {
  __shared__ float xs[1024];
  const GemvJob& J = P.jobs[blockIdx.y];
  const ResolvedJob R = resolve_job(J, P.G);
  const int t = blockIdx.z;
  const int n = blockIdx.x * kCtaThreads + threadIdx.x;
  if (blockIdx.x * kCtaThreads >= J.N) return;
  const int bits = R.bits, eps = 32 / bits;
  const uint32_t mask = (1u << bits) - 1u;
  const bool on = n < J.N;
  float acc = 0.f;
  for (int kc = 0; kc < J.K; kc += 1024) {
    const int kn = min(1024, J.K - kc);
    __syncthreads();
    for (int i = threadIdx.x; i < kn; i += kCtaThreads) xs[i] = load_act<SILU>(J, t, kc + i);
    __syncthreads();
    if (on) {
      uint32_t w = 0;
      __half s = __float2half_rn(0.f), z = s;
      for (int kk = 0; kk < kn; ++kk) {
        const int k = kc + kk;
        const int jj = k % eps;
        if (jj == 0 || kk == 0) w = R.wq[static_cast<size_t>(k / eps) * J.N + n];
        if (k % P.G == 0 || kk == 0) {
          s = R.scales[static_cast<size_t>(k / P.G) * J.N + n];
          z = R.zeros[static_cast<size_t>(k / P.G) * J.N + n];
        }
        const int q = static_cast<int>((w >> (jj * bits)) & mask);
        const __half wv = __hfma(__int2half_rn(q), s, z);
        acc = fmaf(xs[kk], __half2float(wv), acc);
      }
    }
  }
  if (on) J.y[static_cast<size_t>(t) * J.ldy + n] = __float2half_rn(acc);
}

// ----------------------------------------------------------------------------------
// Host side
// ----------------------------------------------------------------------------------
struct Workspace {
  int* counters;
  float* partial;
  size_t partial_floats;
};

size_t gemv_workspace_bytes(int total_cols, int max_k, int tokens) {
  // the persistent kernel cuts 4-bit matrices into 4-group slices, the shortest of all
  const size_t s_max = static_cast<size_t>(cdiv(cdiv(max_k, kGroup), 4));
  // counters | fp32 partial slots | fp32 activation staging of the SiLU*mul inputs (one row per job)
  return static_cast<size_t>(kMaxCounters) * sizeof(int) +
         s_max * static_cast<size_t>(tokens) * static_cast<size_t>(total_cols) * sizeof(float) +
         static_cast<size_t>(kMaxJobs) * static_cast<size_t>(max_k) * sizeof(float);
}

static bool split_ws(void* ws, size_t bytes, Workspace* out) {
  if (!ws || bytes < kMaxCounters * sizeof(int) || !aligned16(ws)) return false;
  out->counters = static_cast<int*>(ws);
  out->partial = reinterpret_cast<float*>(static_cast<char*>(ws) + kMaxCounters * sizeof(int));
  out->partial_floats = (bytes - kMaxCounters * sizeof(int)) / sizeof(float);
  return true;
}

static bool fast_shape(int N, int K, int G) { return G == kGroup && K % kGroup == 0 && N % 32 == 0 && K > 0 && N > 0; }

// Fill the launch geometry of P.jobs[0..n_jobs) and run the tensor-core kernel.
template <bool SILU>
static int launch_mma(GemvParams& P, const Workspace& W, cudaStream_t stream) {
  int max_k = 0, cols = 0, tiles = 0, chunks = 0;
  for (int i = 0; i < P.n_jobs; ++i) max_k = P.jobs[i].K > max_k ? P.jobs[i].K : max_k;
  P.s_max = cdiv(cdiv(max_k, kGroup), kSliceGroups);
  const bool combine = P.comb_out != nullptr;
  for (int i = 0; i < P.n_jobs; ++i) {
    GemvJob& J = P.jobs[i];
    const int nch = cdiv(J.N, kCtaCols);
    J.col_base = cols;
    J.tile_base = tiles;
    J.chunk_base = chunks;
    cols += J.N;
    tiles += nch * P.s_max;
    if (!combine) chunks += nch;
  }
  if (combine) chunks = cdiv(P.jobs[0].N, kCtaCols);
  P.c_total = cols;
  P.n_chunks = chunks;
  P.G = kGroup;
  const int tt = P.T <= 1 ? 1 : (P.T <= 2 ? 2 : (P.T <= 4 ? 4 : 8));
  const int tblocks = cdiv(P.T, tt);
  if (static_cast<size_t>(chunks) * tblocks >= static_cast<size_t>(kMaxCounters - 1)) return GEMQ_ERR_WORKSPACE;
  if (static_cast<size_t>(P.s_max) * P.T * cols > W.partial_floats) return GEMQ_ERR_WORKSPACE;
  if (tblocks > 65535) return GEMQ_ERR_BAD_SHAPE;
  P.partial = W.partial;
  P.counters = W.counters;
  const dim3 grid(tiles, tblocks);
  switch (tt) {
    case 1: gemv_mma_kernel<1, SILU><<<grid, kCtaThreads, 0, stream>>>(P); break;
    case 2: gemv_mma_kernel<2, SILU><<<grid, kCtaThreads, 0, stream>>>(P); break;
    case 4: gemv_mma_kernel<4, SILU><<<grid, kCtaThreads, 0, stream>>>(P); break;
    default: gemv_mma_kernel<8, SILU><<<grid, kCtaThreads, 0, stream>>>(P); break;
  }
  return launch_status();
}

template <bool SILU>
static int launch_generic(GemvParams& P, int G, cudaStream_t stream) {
  int max_n = 0;
  for (int i = 0; i < P.n_jobs; ++i) max_n = P.jobs[i].N > max_n ? P.jobs[i].N : max_n;
  P.G = G;
  if (P.T > 65535) return GEMQ_ERR_BAD_SHAPE;
  const dim3 grid(cdiv(max_n, kCtaThreads), P.n_jobs, P.T);
  gemv_generic_kernel<SILU><<<grid, kCtaThreads, 0, stream>>>(P);
  return launch_status();
}

int run_gemv_jobs(GemvParams& P, bool silu, int G, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  bool fast = true;
  for (int i = 0; i < P.n_jobs; ++i) {
    const GemvJob& J = P.jobs[i];
    fast = fast && fast_shape(J.N, J.K, G) && aligned16(J.wq) && aligned16(J.scales) && aligned16(J.zeros);
  }
  if (fast) {
    Workspace W;
    if (!split_ws(workspace, workspace_bytes, &W)) return GEMQ_ERR_WORKSPACE;
    bool act_aligned = true;
    for (int i = 0; i < P.n_jobs; ++i) act_aligned = act_aligned && aligned16(P.jobs[i].xa) && aligned16(P.jobs[i].xb);
    if (P.T == 1 && act_aligned) {
      if (silu) {
        // stage h = silu(x1) * x3 in fp32 at the tail of the workspace, one row per job
        int max_k = 0;
        for (int i = 0; i < P.n_jobs; ++i) max_k = P.jobs[i].K > max_k ? P.jobs[i].K : max_k;
        const size_t hfloats = static_cast<size_t>(P.n_jobs) * max_k;
        if (W.partial_floats < hfloats) return GEMQ_ERR_WORKSPACE;
        W.partial_floats -= hfloats;
        float* h = W.partial + W.partial_floats;
        for (int i = 0; i < P.n_jobs; ++i) {
          GemvJob& J = P.jobs[i];
          float* hi = h + static_cast<size_t>(i) * max_k;
          if (int rc = silu_mul_f32(J.xa, J.xb, hi, J.K, stream)) return rc;
          J.xa = reinterpret_cast<const __half*>(hi);
          J.xb = nullptr;
        }
        P.x_f32 = 1;
      }
      return launch_stream(P, W.partial, W.partial_floats, W.counters, stream);
    }
    return silu ? launch_mma<true>(P, W, stream) : launch_mma<false>(P, W, stream);
  }
  if (P.comb_out) return GEMQ_ERR_BAD_SHAPE;
  for (int i = 0; i < P.n_jobs; ++i)
    if (P.jobs[i].K % G != 0) return GEMQ_ERR_BAD_SHAPE;
  return silu ? launch_generic<true>(P, G, stream) : launch_generic<false>(P, G, stream);
}

}  // namespace gemq

using namespace gemq;

extern "C" size_t gemq_gemv_workspace_bytes(int total_cols, int max_k, int tokens) {
  if (total_cols <= 0 || max_k <= 0 || tokens <= 0) return 0;
  return gemv_workspace_bytes(total_cols, max_k, tokens);
}

static bool bits_ok(int b) { return b >= 1 && b <= 4; }

static void job_from_stacked(GemvJob& J, const gemq_stacked_t* W, const int64_t* idx_slot, int N, int K) {
  J.wq = reinterpret_cast<const uint32_t*>(W->wq);
  J.scales = static_cast<const __half*>(W->scales);
  J.zeros = static_cast<const __half*>(W->zeros);
  J.nbits = W->nbits;
  J.wq_strides = W->wq_strides;
  J.zs_strides = W->zs_strides;
  J.idx = reinterpret_cast<const long long*>(idx_slot);
  J.wq_rows = W->wq_rows;
  J.zs_rows = W->zs_rows;
  J.N = N;
  J.K = K;
  J.n_experts = W->n_experts;
}

static bool stacked_ok(const gemq_stacked_t* W) {
  return W && W->wq && W->scales && W->zeros && W->nbits && W->wq_strides && W->wq_rows > 0 && W->zs_rows > 0;
}

extern "C" int gemq_dequant_gemv(const void* x, int ldx, const int32_t* wq, const void* scales, const void* zeros,
                                 void* y, int ldy, int tokens, int N, int K, int nbits, int group_size,
                                 void* workspace, size_t workspace_bytes, gemq_stream_t stream) {
  if (!x || !wq || !scales || !zeros || !y || tokens <= 0 || N <= 0 || K <= 0 || group_size <= 0 || !bits_ok(nbits))
    return GEMQ_ERR_BAD_ARG;
  GemvParams P = {};
  P.n_jobs = 1;
  P.T = tokens;
  GemvJob& J = P.jobs[0];
  J.wq = reinterpret_cast<const uint32_t*>(wq);
  J.scales = static_cast<const __half*>(scales);
  J.zeros = static_cast<const __half*>(zeros);
  J.fixed_bits = nbits;
  J.xa = static_cast<const __half*>(x);
  J.y = static_cast<__half*>(y);
  J.N = N; J.K = K; J.ldx = ldx; J.ldy = ldy;
  J.wq_rows = cdiv(K, 32 / nbits);
  J.zs_rows = K / group_size;
  return run_gemv_jobs(P, false, group_size, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int gemq_dequant_sel_gemv(const void* x, const int64_t* idx, const gemq_stacked_t* w,
                                     void* y, int N, int K, int group_size,
                                     void* workspace, size_t workspace_bytes, gemq_stream_t stream) {
  if (!x || !idx || !stacked_ok(w) || !y || N <= 0 || K <= 0 || group_size <= 0) return GEMQ_ERR_BAD_ARG;
  GemvParams P = {};
  P.n_jobs = 1;
  P.T = 1;
  GemvJob& J = P.jobs[0];
  job_from_stacked(J, w, idx, N, K);
  J.zs_strides = nullptr;
  J.xa = static_cast<const __half*>(x);
  J.y = static_cast<__half*>(y);
  J.ldx = K; J.ldy = N;
  return run_gemv_jobs(P, false, group_size, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int gemq_fused_up_proj(const void* x, const int64_t* idx, int A,
                                  const gemq_stacked_t* w1, const gemq_stacked_t* w3,
                                  void* x1, void* x3, int N, int K, int group_size,
                                  void* workspace, size_t workspace_bytes, gemq_stream_t stream) {
  if (!x || !idx || !stacked_ok(w1) || !stacked_ok(w3) || !x1 || !x3 || A <= 0 || N <= 0 || K <= 0 || group_size <= 0)
    return GEMQ_ERR_BAD_ARG;
  if (A > kMaxSlots) return GEMQ_ERR_BAD_SHAPE;
  GemvParams P = {};
  P.n_jobs = 2 * A;
  P.T = 1;
  for (int a = 0; a < A; ++a) {
    for (int m = 0; m < 2; ++m) {
      GemvJob& J = P.jobs[2 * a + m];
      job_from_stacked(J, m ? w3 : w1, idx + a, N, K);
      J.nbits = w1->nbits;
      J.wq_strides = w1->wq_strides;
      J.zs_strides = nullptr;
      J.xa = static_cast<const __half*>(x);
      J.y = static_cast<__half*>(m ? x3 : x1) + static_cast<size_t>(a) * N;
      J.ldx = K; J.ldy = A * N;
    }
  }
  P.epi = kEpiUpPair;
  return run_gemv_jobs(P, false, group_size, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int gemq_fused_down_proj(const void* x1, const void* x3, const int64_t* idx, int A,
                                    const gemq_stacked_t* w2,
                                    void* x2, int N, int K, int group_size,
                                    void* workspace, size_t workspace_bytes, gemq_stream_t stream) {
  if (!x1 || !x3 || !idx || !stacked_ok(w2) || !x2 || A <= 0 || N <= 0 || K <= 0 || group_size <= 0)
    return GEMQ_ERR_BAD_ARG;
  if (A > kMaxSlots) return GEMQ_ERR_BAD_SHAPE;
  GemvParams P = {};
  P.n_jobs = A;
  P.T = 1;
  for (int a = 0; a < A; ++a) {
    GemvJob& J = P.jobs[a];
    job_from_stacked(J, w2, idx + a, N, K);
    J.zs_strides = nullptr;
    J.xa = static_cast<const __half*>(x1) + static_cast<size_t>(a) * K;
    J.xb = static_cast<const __half*>(x3) + static_cast<size_t>(a) * K;
    J.y = static_cast<__half*>(x2) + static_cast<size_t>(a) * N;
    J.ldx = A * K; J.ldy = A * N;
  }
  return run_gemv_jobs(P, true, group_size, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int gemq_dequant_group_gemv(const void* x, int ldx, const int64_t* indices, int A,
                                       const gemq_stacked_t* w,
                                       void* y, int tokens, int N, int K, int group_size,
                                       void* workspace, size_t workspace_bytes, gemq_stream_t stream) {
  if (!x || !indices || !stacked_ok(w) || !w->zs_strides || !y || A <= 0 || tokens <= 0 || N <= 0 || K <= 0 ||
      group_size <= 0)
    return GEMQ_ERR_BAD_ARG;
  if (A > kMaxJobs) return GEMQ_ERR_BAD_SHAPE;
  GemvParams P = {};
  P.n_jobs = A;
  P.T = tokens;
  for (int a = 0; a < A; ++a) {
    GemvJob& J = P.jobs[a];
    job_from_stacked(J, w, indices + a, N, K);
    J.xa = static_cast<const __half*>(x);
    J.y = static_cast<__half*>(y) + static_cast<size_t>(a) * tokens * N;
    J.ldx = ldx; J.ldy = N;
  }
  return run_gemv_jobs(P, false, group_size, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}
