// Prefill path: expert-sorted grouped GEMM on the 5th-generation tensor cores (tcgen05 / TMEM).
//
//   tokens --route--> (expert, weight) pairs --sort--> rows grouped by expert (Xs)
//   up kernel   : H[r, :]  = silu(Xs[r, :] @ deq(w1[e])) * (Xs[r, :] @ deq(w3[e]))      (both GEMMs in one pass)
//   down kernel : Ys[r, :] = (H[r, :] @ deq(w2[e])) * routing weight
//   combine     : out[t]   = sum over the token's experts, in expert order (index_add_ semantics)
//
// One CTA computes a 256 (rows) x 128 (output columns) tile of one expert, as two M=128
// accumulators that share every de-quantised weight tile.  A 3-stage mbarrier ring over 64-wide
// k-blocks feeds tcgen05.mma (kind::f16, M=128, N=128, K=16 per instruction, fp32 accumulators in
// TMEM: 512 columns for the gate/up pass, 256 otherwise):
//   * a TMA warp loads the activation tile (tiled TMA, 128B swizzle, K-major, box 64 x 256);
//   * sixteen producer warps in two groups that take alternate k-blocks (one thread per output
//     column and 32-element half of the k-block) read the packed words of their column two
//     k-blocks ahead, de-quantise them with the reference's single-rounded fp16 fma (bit-exact
//     weights: the code is extracted in place as the fp16 1024 + q and one hfma2 with the
//     per-position constants 2^-pos and -1024 * 2^-pos gives q exactly), and write the K-major
//     128B-swizzled B tile straight into shared memory; bf16 activations are converted to fp16
//     when the rows are gathered, so the products stay in one format;
//   * one thread of the MMA warp issues the MMAs and commits stage releases;
//   * the producer warps then read the accumulators back with tcgen05.ld and run the epilogue
//     (SiLU-gate product, routing weight, rounding to the activation type).
// Expert of a row tile, its first row and its valid row count come from a tile table built on
// the device, so the routing never reaches the host.  Every wait is bounded.
#include <type_traits>

#include "gemv.cuh"
#include "ptx.cuh"

namespace gemq {

constexpr int kGemmBM = 256, kGemmBN = 128, kGemmBK = 64;  // CTA tile; two M=128 MMAs share every B tile
constexpr int kMmaM = 128;
constexpr int kGemmStages = 3;
constexpr int kGemmProducerWarps = 16;
constexpr int kGemmThreads = 32 * (kGemmProducerWarps + 2);  // de-quantise/epilogue warps + TMA warp + MMA warp
constexpr int kTileBytes = kGemmBN * kGemmBK * 2;  // 16 KB: a B tile, or one 128-row half of the A tile

enum { kErrGemmAFull = 11, kErrGemmBFull = 12, kErrGemmEmpty = 13, kErrGemmAcc = 14 };


struct alignas(64) GemmParams {
  CUtensorMap a_map;        // activations [rows, K] (16-bit), box 64 x 256, 128B swizzle
  const uint32_t* wq[2];    // stacked packed words ([0] only unless UP)
  const __half* scales[2];
  const __half* zeros[2];
  const int* nbits;         // [E] or nullptr -> fixed_bits
  const int* wq_strides;    // [E] or nullptr
  const int* zs_strides;    // [E] or nullptr -> e * (K/G) * N
  int fixed_bits;
  const int* tile_expert;   // [n_tiles] or nullptr: one problem, expert 0, rows_single rows
  const int* tile_row0;
  const int* tile_rows;
  const int* n_tiles;
  const long long* single_expert;  // with tile_expert == nullptr: expert id read on the device (or nullptr -> 0)
  int rows_single;
  int N, K, G;
  void* out;                // [rows, N] activation dtype
  const void* row_weight;   // per-row scale (activation dtype) or nullptr
  int* err;
};

struct GemmSmem {
  alignas(1024) unsigned char a[kGemmStages][2 * kTileBytes];
  alignas(1024) unsigned char b[kGemmStages][2][kTileBytes];
  alignas(8) unsigned long long a_full[kGemmStages], b_full[kGemmStages], empty[kGemmStages], acc_full;
  uint32_t tmem_base;
};

// ---- de-quantisation of one output column's 64 reduction elements into a swizzled B row ------
template <bool BF16>
__device__ __forceinline__ uint32_t pack_act2(__half2 v) {
  if (BF16) {
    const float2 f = __half22float2(v);
    const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
    return *reinterpret_cast<const uint32_t*>(&b);
  }
  return *reinterpret_cast<const uint32_t*>(&v);
}

// W^T[k, n] = fp16(fma(fp16(q), s, z)) (gemq/triton_kernels/utils.py:206-210) for the 32
// reduction elements [k0, k0+32) of one output column, written as four 16-byte chunks
// (chunk0 .. chunk0+3) of the column's swizzled 128-byte B row.
//
// 1/2/4-bit: `(w & mask) | 0x6400` leaves 1024 + q*2^pos in each fp16 half (codes j and
// j + eps/2 of the word, in place); minus 1024 and times 2^-pos are exact, so the fma sees the
// exact integer code.  A byte permute then pairs neighbouring k.
template <bool BF16, int B>
__device__ __forceinline__ void dequant32_pow2(unsigned char* brow, int swz, int chunk0, const uint32_t* w,
                                               __half2 s2, __half2 z2) {
  constexpr int EPS = 32 / B, PAIRS = EPS / 2, NPOS = 10 / B, NW = 32 / EPS;
  constexpr uint32_t MASK = ((1u << B) - 1u) * 0x00010001u;
  uint32_t outw[16];
  const __half2 k1024 = __float2half2_rn(1024.f);
#pragma unroll
  for (int i = 0; i < NW; ++i) {
    __half2 v[PAIRS];
#pragma unroll
    for (int q = 0; q < PAIRS; ++q) {
      const int stage = q / NPOS, jj = q % NPOS;
      const uint32_t bits = ((w[i] >> (stage * NPOS * B)) & (MASK << (B * jj))) | 0x64006400u;
      // (1024 + q*2^pos) * 2^-pos - 1024 * 2^-pos = q, exactly, in one fma
      constexpr float kInv[10] = {1.f, 1.f / 2, 1.f / 4, 1.f / 8, 1.f / 16, 1.f / 32, 1.f / 64, 1.f / 128, 1.f / 256, 1.f / 512};
      const float inv = kInv[B * jj];
      const __half2 c = __hfma2(*reinterpret_cast<const __half2*>(&bits), __float2half2_rn(inv), __float2half2_rn(-1024.f * inv));
      v[q] = __hfma2(c, s2, z2);
    }
#pragma unroll
    for (int q = 0; q < PAIRS; q += 2) {
      const uint32_t a = *reinterpret_cast<const uint32_t*>(&v[q]), bb = *reinterpret_cast<const uint32_t*>(&v[q + 1]);
      const uint32_t lo = __byte_perm(a, bb, 0x5410), hi = __byte_perm(a, bb, 0x7632);
      outw[(i * EPS + q) / 2] = pack_act2<BF16>(*reinterpret_cast<const __half2*>(&lo));
      outw[(i * EPS + PAIRS + q) / 2] = pack_act2<BF16>(*reinterpret_cast<const __half2*>(&hi));
    }
  }
#pragma unroll
  for (int c = 0; c < 4; ++c)
    *reinterpret_cast<uint4*>(brow + (((chunk0 + c) ^ swz) << 4)) =
        make_uint4(outw[4 * c], outw[4 * c + 1], outw[4 * c + 2], outw[4 * c + 3]);
}

// 3-bit: 10 codes per word, so a 32-element window starts at an even code of its first word and
// spans four words.  Per word: fold codes 5..9 into the upper half (code j and j + 5 now sit at
// bit 3*(j % 5) of the two 16-bit halves), extract them in place like the other widths (positions
// 9 and 12 after a shift by 9: the fp16 mantissa has 10 bits), and permute the (j, j + 5) pairs
// into neighbouring-k pairs.  All 20 pairs of the four words are formed; the window is the 16
// that start at pair (k0 mod 10) / 2.
template <bool BF16>
__device__ __forceinline__ void dequant32_b3(unsigned char* brow, int swz, int chunk0, const uint32_t* w, int k0,
                                             __half2 s2, __half2 z2) {
  uint32_t pr[20];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t m = (w[i] & 0x00007fffu) | ((w[i] << 1) & 0x7fff0000u);
    const uint32_t mh = m >> 9;
    uint32_t v[5];
#pragma unroll
    for (int q = 0; q < 5; ++q) {
      const int jj = q < 3 ? q : q - 3;
      const uint32_t bits = ((q < 3 ? m : mh) & (0x00070007u << (3 * jj))) | 0x64006400u;
      constexpr float kInv[3] = {1.f, 1.f / 8, 1.f / 64};
      const float inv = kInv[jj];
      const __half2 c = __hfma2(*reinterpret_cast<const __half2*>(&bits), __float2half2_rn(inv), __float2half2_rn(-1024.f * inv));
      const __half2 d = __hfma2(c, s2, z2);
      v[q] = *reinterpret_cast<const uint32_t*>(&d);
    }
    // v[q] = (code q, code q + 5)  ->  neighbouring codes
    pr[5 * i + 0] = __byte_perm(v[0], v[1], 0x5410);  // codes 0, 1
    pr[5 * i + 1] = __byte_perm(v[2], v[3], 0x5410);  // 2, 3
    pr[5 * i + 2] = __byte_perm(v[4], v[0], 0x7610);  // 4, 5
    pr[5 * i + 3] = __byte_perm(v[1], v[2], 0x7632);  // 6, 7
    pr[5 * i + 4] = __byte_perm(v[3], v[4], 0x7632);  // 8, 9
  }
  if (BF16) {
#pragma unroll
    for (int t = 0; t < 20; ++t) pr[t] = pack_act2<true>(*reinterpret_cast<const __half2*>(&pr[t]));
  }
  const int sh = (k0 % 10) >> 1;  // warp-uniform: all lanes of a warp share k0
  auto store = [&](auto SH) {
    constexpr int O = decltype(SH)::value;
#pragma unroll
    for (int c = 0; c < 4; ++c)
      *reinterpret_cast<uint4*>(brow + (((chunk0 + c) ^ swz) << 4)) =
          make_uint4(pr[O + 4 * c], pr[O + 4 * c + 1], pr[O + 4 * c + 2], pr[O + 4 * c + 3]);
  };
  switch (sh) {
    case 0: store(std::integral_constant<int, 0>{}); break;
    case 1: store(std::integral_constant<int, 1>{}); break;
    case 2: store(std::integral_constant<int, 2>{}); break;
    case 3: store(std::integral_constant<int, 3>{}); break;
    default: store(std::integral_constant<int, 4>{}); break;
  }
}

// ---- B producer loop, specialised for the expert's bit width --------------------------------
// Thread = output column n0 + col and one 32-element half kh of a 64-wide k-block; the two
// groups of 8 warps take alternate k-blocks.  Words and metadata are fetched two of the group's
// k-blocks ahead (register ring of three sets), so the global-load latency is off the critical
// path of the stage ring.  Everything that does not change along k (bit width, expert offsets,
// words per window) is fixed outside the loop: the loop body is loads at constant strides, the
// de-quantisation and one barrier arrival.
template <int NMAT, bool BF16, int B>
__device__ __forceinline__ void produce_loop(GemmSmem& S, const GemmParams& P, int expert, int n0, int KB) {
  constexpr int EPS = B == 3 ? 10 : 32 / B;
  constexpr int NW = B == 3 ? 4 : 32 / EPS;  // words that cover a 32-element window (3-bit: 4 for every even start)
  const int tid = threadIdx.x, lane = tid & 31;
  const int grp = tid >> 8, col = tid & 127, kh = (tid >> 7) & 1;
  const size_t N = P.N;
  const int ngroups = P.K / P.G;
  const size_t woff = P.wq_strides ? static_cast<size_t>(P.wq_strides[expert]) : 0;
  const size_t zoff = P.zs_strides ? static_cast<size_t>(P.zs_strides[expert]) : static_cast<size_t>(expert) * ngroups * N;
  const int gshift = (P.G & (P.G - 1)) == 0 ? __ffs(P.G) - 1 : -1;
  const uint32_t* wp[NMAT];
  const __half* sp[NMAT];
  const __half* zp[NMAT];
#pragma unroll
  for (int m = 0; m < NMAT; ++m) {
    wp[m] = P.wq[m] + woff + n0 + col;
    sp[m] = P.scales[m] + zoff + n0 + col;
    zp[m] = P.zeros[m] + zoff + n0 + col;
  }
  struct WSet { uint32_t w[NMAT][NW]; __half sc[NMAT], zr[NMAT]; };
  WSet ring[3];
  auto fetch = [&](WSet& W, int kb) {
    const int k0 = kb * kGemmBK + 32 * kh;
    const int first = k0 / EPS;  // constant divisor
    const int g = gshift >= 0 ? (kb * kGemmBK) >> gshift : (kb * kGemmBK) / P.G;
#pragma unroll
    for (int m = 0; m < NMAT; ++m) {
      const uint32_t* q = wp[m] + static_cast<size_t>(first) * N;
#pragma unroll
      for (int i = 0; i < NW; ++i) W.w[m][i] = q[static_cast<size_t>(i) * N];
      W.sc[m] = sp[m][static_cast<size_t>(g) * N];
      W.zr[m] = zp[m][static_cast<size_t>(g) * N];
    }
  };
  auto produce = [&](const WSet& W, int kb) {
    const int s = kb % kGemmStages;
    mbar_wait(&S.empty[s], ((kb / kGemmStages) & 1) ^ 1, P.err, kErrGemmEmpty, 32);
#pragma unroll
    for (int m = 0; m < NMAT; ++m) {
      const __half2 s2 = __half2half2(W.sc[m]), z2 = __half2half2(W.zr[m]);
      unsigned char* brow = S.b[s][m] + col * 128;
      if (B == 3) dequant32_b3<BF16>(brow, col & 7, 4 * kh, W.w[m], kb * kGemmBK + 32 * kh, s2, z2);
      else dequant32_pow2<BF16, (B == 3 ? 2 : B)>(brow, col & 7, 4 * kh, W.w[m], s2, z2);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> tensor-core reads
    __syncwarp();
    if (lane == 0) mbar_arrive(&S.b_full[s]);
  };
  if (grp < KB) fetch(ring[0], grp);
  if (grp + 2 < KB) fetch(ring[1], grp + 2);
  for (int kb0 = grp; kb0 < KB; kb0 += 6) {
#pragma unroll
    for (int u = 0; u < 3; ++u) {
      const int kb = kb0 + 2 * u;
      if (kb < KB) {
        if (kb + 4 < KB) fetch(ring[(u + 2) % 3], kb + 4);
        produce(ring[u], kb);
      }
    }
  }
}

template <bool BF16>
__device__ __forceinline__ float act_round(float v) {
  return BF16 ? __bfloat162float(__float2bfloat16_rn(v)) : __half2float(__float2half_rn(v));
}

template <bool BF16>
__device__ __forceinline__ void store_act32(void* dst, const float (&v)[32]) {
  uint32_t w[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if (BF16) {
      const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&b);
    } else {
      const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int i = 0; i < 4; ++i) d[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
}

// MODE kGemmUp: two weight tensors (gate, up), 128 columns of each, epilogue silu(x1) * x3.
// MODE kGemmWide: one tensor, 256 columns per CTA (the second B tile is the same tensor 128
// columns further: twice the work per activation tile, which is what the L2-to-SM traffic of the
// activation tiles asks for); MODE kGemmNarrow: one tensor, 128 columns.  Optional row weight.
enum { kGemmNarrow = 0, kGemmUp = 1, kGemmWide = 2 };

template <int MODE, bool BF16>
__global__ void __launch_bounds__(kGemmThreads, 1) grouped_gemm_kernel(const __grid_constant__ GemmParams P) {
  constexpr bool UP = MODE == kGemmUp;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  GemmSmem& S = *reinterpret_cast<GemmSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mt = blockIdx.y, n0 = blockIdx.x * kGemmBN * (MODE == kGemmWide ? 2 : 1);
  int expert = 0, row0 = mt * kGemmBM, rows = 0;
  if (P.tile_expert) {
    if (mt >= *P.n_tiles) return;  // uniform: before any barrier or TMEM allocation
    expert = P.tile_expert[mt];
    row0 = P.tile_row0[mt];
    rows = P.tile_rows[mt];
  } else {
    rows = min(kGemmBM, P.rows_single - row0);
    if (rows <= 0) return;
    if (P.single_expert) expert = static_cast<int>(*P.single_expert);
  }
  constexpr int NMAT = MODE == kGemmNarrow ? 1 : 2;
  constexpr uint32_t TCOLS = NMAT * 256;  // (row half, matrix) accumulators of 128 columns each
  const int KB = P.K / kGemmBK;

  if (tid == 0) {
    for (int s = 0; s < kGemmStages; ++s) {
      mbar_init(&S.a_full[s], 1);
      mbar_init(&S.b_full[s], kGemmProducerWarps / 2);  // the warp group that owns the k-block
      mbar_init(&S.empty[s], 1);
    }
    mbar_init(&S.acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kGemmProducerWarps + 1) tmem_alloc(&S.tmem_base, TCOLS);
  if (warp == kGemmProducerWarps && lane == 0)
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<unsigned long long>(&P.a_map)) : "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = S.tmem_base;

  if (warp < kGemmProducerWarps) {
    // ---- B producers ---------------------------------------------------------------------------
    const int bits = P.nbits ? P.nbits[expert] : P.fixed_bits;
    if (bits == 1) produce_loop<NMAT, BF16, 1>(S, P, expert, n0, KB);
    else if (bits == 2) produce_loop<NMAT, BF16, 2>(S, P, expert, n0, KB);
    else if (bits == 3) produce_loop<NMAT, BF16, 3>(S, P, expert, n0, KB);
    else produce_loop<NMAT, BF16, 4>(S, P, expert, n0, KB);
    // ---- epilogue: warp w owns TMEM lanes 32w .. 32w+31 = tile rows -------------------------
    mbar_wait(&S.acc_full, 0, P.err, kErrGemmAcc, 64);
    tc_fence_after_sync();
    const int lq = warp & 3, cq = warp >> 2;  // TMEM lane quarter of this warp, 32-column quarter it drains
    for (int hf = 0; hf < 2; ++hf) {
      if (kMmaM * hf >= rows) break;
      const int r = kMmaM * hf + 32 * lq + lane;
      const bool row_on = r < rows;
      float rw = 1.f;
      if (!UP && P.row_weight && row_on)
        rw = BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(P.row_weight)[row0 + r])
                  : __half2float(static_cast<const __half*>(P.row_weight)[row0 + r]);
      unsigned char* orow = static_cast<unsigned char*>(P.out) + (static_cast<size_t>(row0 + r) * P.N + n0) * 2;
      const uint32_t tbase = tmem + (static_cast<uint32_t>(32 * lq) << 16) + hf * NMAT * 128;
      for (int c0 = 32 * cq; c0 < 32 * cq + 32; c0 += 32) {
        uint32_t d1[32];
        float v[32];
        tmem_ld32(tbase + c0, d1);
        if (UP) {
          uint32_t d3[32];
          tmem_ld32(tbase + 128 + c0, d3);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float x1 = act_round<BF16>(__uint_as_float(d1[i])), x3 = act_round<BF16>(__uint_as_float(d3[i]));
            v[i] = act_round<BF16>(silu_f32(x1)) * x3;  // F.silu(x1) * x3 on activation-dtype tensors
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = act_round<BF16>(__uint_as_float(d1[i])) * rw;
        }
        if (row_on) store_act32<BF16>(orow + c0 * 2, v);
        if (MODE == kGemmWide) {  // the second 128 columns
          tmem_ld32(tbase + 128 + c0, d1);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = act_round<BF16>(__uint_as_float(d1[i])) * rw;
          if (row_on) store_act32<BF16>(orow + (kGemmBN + c0) * 2, v);
        }
      }
    }
    tc_fence_before_sync();
  } else if (warp == kGemmProducerWarps) {
    // ---- A producer: one TMA box per k-block ------------------------------------------------
    if (lane == 0) {
      for (int kb = 0; kb < KB; ++kb) {
        const int s = kb % kGemmStages;
        mbar_wait(&S.empty[s], ((kb / kGemmStages) & 1) ^ 1, P.err, kErrGemmEmpty, 32);
        mbar_arrive_expect_tx(&S.a_full[s], 2 * kTileBytes);
        tma_load_2d(S.a[s], &P.a_map, kb * kGemmBK, row0, &S.a_full[s]);
      }
    }
  } else {
    // ---- MMA issuer ---------------------------------------------------------------------------
    if (lane == 0) {
      // Gate/up pass: the two B tiles of a stage are adjacent (256 rows of the same swizzled
      // layout), so one N = 256 instruction per row half covers both and reads A once.
      const uint32_t idesc = umma_idesc_f16(BF16 ? 1 : 0, kMmaM, NMAT * kGemmBN);
      const int halves = rows > kMmaM ? 2 : 1;
      for (int kb = 0; kb < KB; ++kb) {
        const int s = kb % kGemmStages;
        const uint32_t par = (kb / kGemmStages) & 1;
        mbar_wait(&S.a_full[s], par, P.err, kErrGemmAFull, 32);
        mbar_wait(&S.b_full[s], par, P.err, kErrGemmBFull, 32);
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(S.a[s]);
#pragma unroll
        for (int k4 = 0; k4 < kGemmBK / 16; ++k4) {
          const uint64_t bd = umma_desc_k_sw128(smem_u32(S.b[s][0]) + k4 * 32);
          for (int hf = 0; hf < halves; ++hf)
            umma_f16(tmem + hf * NMAT * 128, umma_desc_k_sw128(a_addr + hf * kTileBytes + k4 * 32), bd, idesc,
                     (kb | k4) != 0);
        }
        umma_commit(&S.empty[s]);  // stage is free once these MMAs have read it
      }
      umma_commit(&S.acc_full);
    }
    __syncwarp();
  }
  __syncthreads();
  if (warp == kGemmProducerWarps + 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, TCOLS);
  }
}

}  // namespace gemq

// ==================================================================================================
// Token permutation (device side; replaces one_hot / nonzero / where of gemq/inference/moe_block.py:187-193)
// ==================================================================================================
namespace gemq {

struct PrefillPlan {
  int* counts;       // [E]
  int* cursor;       // [E]
  int* offsets;      // [E + 1]
  int* n_tiles;      // [1]
  int* tile_expert;  // [max_tiles]
  int* tile_row0;
  int* tile_rows;
  int* inv;          // [T * A] sorted row of (token, slot)
};

__global__ void prefill_zero_kernel(PrefillPlan pl, int E) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < E) { pl.counts[i] = 0; pl.cursor[i] = 0; }
}

// Expert ids outside [0, E) (only possible with caller-supplied routing) are left out of the
// permutation and reported through the error word; they contribute nothing to the output.
constexpr int kErrBadExpert = 21;

__global__ void prefill_count_kernel(PrefillPlan pl, const long long* __restrict__ idx, int n, int E, int* err) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long e = idx[i];
  if (e < 0 || e >= E) { atomicExch(err, kErrBadExpert); return; }
  atomicAdd(&pl.counts[static_cast<int>(e)], 1);
}

// One thread: exclusive scan of the expert counts and the row-tile table (E <= 256).
__global__ void prefill_plan_kernel(PrefillPlan pl, int E, int max_tiles) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int off = 0, nt = 0;
  for (int e = 0; e < E; ++e) {
    const int c = pl.counts[e];
    pl.offsets[e] = off;
    for (int r = 0; r < c && nt < max_tiles; r += kGemmBM) {
      pl.tile_expert[nt] = e;
      pl.tile_row0[nt] = off + r;
      pl.tile_rows[nt] = min(kGemmBM, c - r);
      ++nt;
    }
    off += c;
  }
  pl.offsets[E] = off;
  *pl.n_tiles = nt;
}

template <typename T> struct ActT;
template <> struct ActT<__half> {
  static __device__ __forceinline__ float f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half r(float v) { return __float2half_rn(v); }
};
template <> struct ActT<__nv_bfloat16> {
  static __device__ __forceinline__ float f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 r(float v) { return __float2bfloat16_rn(v); }
};

template <typename T>
__device__ __forceinline__ uint4 to_half8(uint4 v) {
  const T* p = reinterpret_cast<const T*>(&v);
  uint4 o;
  __half2* q = reinterpret_cast<__half2*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) q[i] = __floats2half2_rn(ActT<T>::f(p[2 * i]), ActT<T>::f(p[2 * i + 1]));
  return o;
}

// One warp per (token, slot): claim a row in the expert's segment, copy the activation row there.
// bf16 activations are converted to fp16 here: the GEMMs then run entirely in fp16 like the
// reference model does, and the fp16 de-quantised weights need no second rounding.
template <typename T>
__global__ void prefill_scatter_kernel(PrefillPlan pl, const long long* __restrict__ idx, const T* __restrict__ w,
                                       const T* __restrict__ x, __half* __restrict__ xs, __half* __restrict__ row_w,
                                       int n, int A, int D, int E) {
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (i >= n) return;
  int pos = -1;
  if (lane == 0) {
    const long long e = idx[i];
    if (e >= 0 && e < E) {
      pos = pl.offsets[e] + atomicAdd(&pl.cursor[e], 1);
      row_w[pos] = __float2half_rn(ActT<T>::f(w[i]));
    }
    pl.inv[i] = pos;
  }
  pos = __shfl_sync(0xffffffffu, pos, 0);
  if (pos < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(i / A) * D);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(pos) * D);
  for (int k = lane; k < D / 8; k += 32) dst[k] = to_half8<T>(src[k]);
}

template <typename T>
__global__ void to_half_kernel(const T* __restrict__ x, __half* __restrict__ y, size_t n8) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n8) reinterpret_cast<uint4*>(y)[i] = to_half8<T>(reinterpret_cast<const uint4*>(x)[i]);
}

// out[t] = contributions of the token's experts added in increasing expert id, each addition
// rounded to the activation dtype (index_add_ in the loop of moe_block.py:191-195), then the
// shared-expert output (moe_block.py:483).
template <typename T>
__global__ void __launch_bounds__(128) prefill_combine_kernel(const int* __restrict__ inv, const long long* __restrict__ idx,
                                                              const __half* __restrict__ ys, const __half* __restrict__ shared,
                                                              T* __restrict__ out, int tokens, int A, int D) {
  __shared__ int rows[kMaxSlots];
  const int t = blockIdx.x;
  if (threadIdx.x == 0) {
    int order[kMaxSlots];
    for (int a = 0; a < A; ++a) order[a] = a;
    for (int a = 1; a < A; ++a)  // insertion sort of the slots by expert id
      for (int b = a; b > 0 && idx[t * A + order[b]] < idx[t * A + order[b - 1]]; --b) {
        const int tmp = order[b]; order[b] = order[b - 1]; order[b - 1] = tmp;
      }
    for (int a = 0; a < A; ++a) rows[a] = inv[t * A + order[a]];
  }
  __syncthreads();
  // eight columns per thread and step: one 16-byte load per expert row
  for (int i = threadIdx.x; i < D / 8; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int a = 0; a < A; ++a) {
      const int row = rows[a];
      if (row < 0) continue;  // pair with an expert id out of range
      const uint4 v = reinterpret_cast<const uint4*>(ys + static_cast<size_t>(row) * D)[i];
      const __half* h = reinterpret_cast<const __half*>(&v);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float c = ActT<T>::f(ActT<T>::r(__half2float(h[k])));
        acc[k] = ActT<T>::f(ActT<T>::r(acc[k] + c));
      }
    }
    if (shared) {
      const uint4 v = reinterpret_cast<const uint4*>(shared + static_cast<size_t>(t) * D)[i];
      const __half* h = reinterpret_cast<const __half*>(&v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = ActT<T>::f(ActT<T>::r(acc[k] + ActT<T>::f(ActT<T>::r(__half2float(h[k])))));
    }
    uint4 o;
    T* q = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int k = 0; k < 8; ++k) q[k] = ActT<T>::r(acc[k]);
    reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * D)[i] = o;
  }
}

// ---- host ---------------------------------------------------------------------------------------
static bool gemm_shape_ok(int N, int K, int G) { return N % kGemmBN == 0 && K % kGemmBK == 0 && G % kGemmBK == 0 && K % G == 0; }

template <int MODE, bool BF16>
static int launch_gemm_t(GemmParams& P, int n_mtiles_bound, cudaStream_t stream) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  const size_t smem = sizeof(GemmSmem) + 1024;
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(grouped_gemm_kernel<MODE, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return GEMQ_ERR_LAUNCH;
    attr_set[dev] = true;
  }
  if (n_mtiles_bound <= 0 || n_mtiles_bound > 65535) return GEMQ_ERR_BAD_SHAPE;
  const dim3 grid(P.N / (MODE == kGemmWide ? 2 * kGemmBN : kGemmBN), n_mtiles_bound);
  grouped_gemm_kernel<MODE, BF16><<<grid, kGemmThreads, smem, stream>>>(P);
  return launch_status();
}

int launch_gemm(GemmParams& P, bool up, bool bf16, int n_mtiles_bound, cudaStream_t stream) {
  if (up) return bf16 ? launch_gemm_t<kGemmUp, true>(P, n_mtiles_bound, stream) : launch_gemm_t<kGemmUp, false>(P, n_mtiles_bound, stream);
  if (P.N % (2 * kGemmBN) == 0) {  // 256 columns per CTA: the second B tile is the same tensor, 128 columns on
    P.wq[1] = P.wq[0] + kGemmBN;
    P.scales[1] = P.scales[0] + kGemmBN;
    P.zeros[1] = P.zeros[0] + kGemmBN;
    return bf16 ? launch_gemm_t<kGemmWide, true>(P, n_mtiles_bound, stream) : launch_gemm_t<kGemmWide, false>(P, n_mtiles_bound, stream);
  }
  return bf16 ? launch_gemm_t<kGemmNarrow, true>(P, n_mtiles_bound, stream) : launch_gemm_t<kGemmNarrow, false>(P, n_mtiles_bound, stream);
}

}  // namespace gemq

using namespace gemq;

namespace {

size_t up256(size_t v) { return (v + 255) / 256 * 256; }

struct PrefillScratch {
  PrefillPlan plan;
  int* err;
  void* row_w;  // [R] activation dtype
  void* xs;     // [R, D]
  void* h;      // [R, F]
  void* ys;     // [R, D]
  void* hs;     // [T, SF]
  void* yss;    // [T, D]
  void* xh;     // [T, D] fp16 copy of bf16 activations (shared experts)
  int max_tiles;
};

size_t prefill_bytes(const gemq_moe_layer_t* L, int tokens, PrefillScratch* S, char* base) {
  const size_t R = static_cast<size_t>(tokens) * L->top_k;
  const int E = L->n_experts;
  const int max_tiles = static_cast<int>((R + kGemmBM - 1) / kGemmBM) + E;
  size_t off = 0;
  auto take = [&](size_t bytes) { const size_t o = off; off += up256(bytes); return base ? base + o : nullptr; };
  char* counts = take(sizeof(int) * E);
  char* cursor = take(sizeof(int) * E);
  char* offsets = take(sizeof(int) * (E + 1));
  char* ntl = take(sizeof(int) * 2);
  char* te = take(sizeof(int) * max_tiles);
  char* tr0 = take(sizeof(int) * max_tiles);
  char* trn = take(sizeof(int) * max_tiles);
  char* inv = take(sizeof(int) * R);
  char* roww = take(2 * R);
  char* xs = take(2 * R * L->hidden);
  char* h = take(2 * R * L->ffn);
  char* ys = take(2 * R * L->hidden);
  char* hs = take(L->shared_ffn ? 2 * static_cast<size_t>(tokens) * L->shared_ffn : 0);
  char* yss = take(L->shared_ffn ? 2 * static_cast<size_t>(tokens) * L->hidden : 0);
  char* xh = take(L->shared_ffn ? 2 * static_cast<size_t>(tokens) * L->hidden : 0);
  if (S) {
    S->plan.counts = reinterpret_cast<int*>(counts);
    S->plan.cursor = reinterpret_cast<int*>(cursor);
    S->plan.offsets = reinterpret_cast<int*>(offsets);
    S->plan.n_tiles = reinterpret_cast<int*>(ntl);
    S->err = reinterpret_cast<int*>(ntl) + 1;
    S->plan.tile_expert = reinterpret_cast<int*>(te);
    S->plan.tile_row0 = reinterpret_cast<int*>(tr0);
    S->plan.tile_rows = reinterpret_cast<int*>(trn);
    S->plan.inv = reinterpret_cast<int*>(inv);
    S->row_w = roww; S->xs = xs; S->h = h; S->ys = ys; S->hs = hs; S->yss = yss; S->xh = xh;
    S->max_tiles = max_tiles;
  }
  return off;
}

void fill_stacked(GemmParams& P, int m, const gemq_stacked_t& W) {
  P.wq[m] = reinterpret_cast<const uint32_t*>(W.wq);
  P.scales[m] = static_cast<const __half*>(W.scales);
  P.zeros[m] = static_cast<const __half*>(W.zeros);
}

void fill_single(GemmParams& P, int m, const gemq_single_t& W) {
  P.wq[m] = reinterpret_cast<const uint32_t*>(W.wq);
  P.scales[m] = static_cast<const __half*>(W.scales);
  P.zeros[m] = static_cast<const __half*>(W.zeros);
}

}  // namespace

extern "C" int gemq_dequant_gemm_tc(const void* x, const int64_t* expert, const int32_t* wq, const void* scales,
                                    const void* zeros, const int32_t* nbits, const int32_t* wq_strides,
                                    const int32_t* zs_strides, int fixed_bits, void* y, int M, int N, int K,
                                    int group_size, int x_is_bf16, int32_t* err, gemq_stream_t stream) {
  if (!x || !wq || !scales || !zeros || !y || !err || M <= 0 || N <= 0 || K <= 0 || group_size <= 0)
    return GEMQ_ERR_BAD_ARG;
  if (!nbits && (fixed_bits < 1 || fixed_bits > 4)) return GEMQ_ERR_BAD_ARG;
  if (!gemm_shape_ok(N, K, group_size)) return GEMQ_ERR_BAD_SHAPE;
  if (!aligned16(x) || !aligned16(y)) return GEMQ_ERR_ALIGN;
  GemmParams P = {};
  if (!tensor_map_2d(&P.a_map, x, 2, K, M, kGemmBK, kGemmBM, true)) return GEMQ_ERR_LAUNCH;
  P.wq[0] = reinterpret_cast<const uint32_t*>(wq);
  P.scales[0] = static_cast<const __half*>(scales);
  P.zeros[0] = static_cast<const __half*>(zeros);
  P.nbits = nbits; P.wq_strides = wq_strides; P.zs_strides = zs_strides; P.fixed_bits = fixed_bits;
  P.single_expert = reinterpret_cast<const long long*>(expert);
  P.rows_single = M;
  P.N = N; P.K = K; P.G = group_size;
  P.out = y;
  P.err = err;
  return launch_gemm(P, false, x_is_bf16 != 0, cdiv(M, kGemmBM), static_cast<cudaStream_t>(stream));
}

extern "C" size_t gemq_moe_prefill_scratch_bytes(const gemq_moe_layer_t* L, int tokens) {
  if (!L || tokens <= 0 || L->top_k <= 0 || L->n_experts <= 0) return 0;
  return prefill_bytes(L, tokens, nullptr, nullptr);
}

extern "C" int gemq_moe_prefill(const gemq_moe_layer_t* L, const void* x, void* out, int64_t* idx, void* w,
                                float* logits, int tokens, int do_route, int route_mode, int x_is_bf16,
                                void* scratch, size_t scratch_bytes, gemq_stream_t stream) {
  if (!L || !x || !out || !idx || !w || !scratch || tokens <= 0) return GEMQ_ERR_BAD_ARG;
  const int D = L->hidden, F = L->ffn, A = L->top_k, E = L->n_experts, SF = L->shared_ffn, G = L->group_size;
  if (A > kMaxSlots || E > 256) return GEMQ_ERR_BAD_SHAPE;
  if (!gemm_shape_ok(F, D, G) || !gemm_shape_ok(D, F, G) || D % 8) return GEMQ_ERR_BAD_SHAPE;
  if (SF && (!gemm_shape_ok(SF, D, G) || !gemm_shape_ok(D, SF, G))) return GEMQ_ERR_BAD_SHAPE;
  if (!aligned16(scratch) || !aligned16(x) || !aligned16(out)) return GEMQ_ERR_ALIGN;
  PrefillScratch S;
  if (prefill_bytes(L, tokens, &S, static_cast<char*>(scratch)) > scratch_bytes) return GEMQ_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool bf = x_is_bf16 != 0;
  const int R = tokens * A;

  if (do_route) {
    const void* gate = L->gate;
    const int rc = gemq_moe_route(x, gate, tokens, D, E, A, route_mode, L->renorm, x_is_bf16, idx, w, logits, stream);
    if (rc) return rc;
  }
  prefill_zero_kernel<<<cdiv(E + 2, 256), 256, 0, st>>>(S.plan, E);
  cudaMemsetAsync(S.err, 0, sizeof(int), st);
  prefill_count_kernel<<<cdiv(R, 256), 256, 0, st>>>(S.plan, reinterpret_cast<const long long*>(idx), R, E, S.err);
  prefill_plan_kernel<<<1, 32, 0, st>>>(S.plan, E, S.max_tiles);
  if (bf)
    prefill_scatter_kernel<__nv_bfloat16><<<cdiv(R, 8), 256, 0, st>>>(
        S.plan, reinterpret_cast<const long long*>(idx), static_cast<const __nv_bfloat16*>(w),
        static_cast<const __nv_bfloat16*>(x), static_cast<__half*>(S.xs), static_cast<__half*>(S.row_w), R, A, D, E);
  else
    prefill_scatter_kernel<__half><<<cdiv(R, 8), 256, 0, st>>>(
        S.plan, reinterpret_cast<const long long*>(idx), static_cast<const __half*>(w), static_cast<const __half*>(x),
        static_cast<__half*>(S.xs), static_cast<__half*>(S.row_w), R, A, D, E);
  if (int rc = launch_status()) return rc;

  // gate/up GEMMs with the SiLU*mul epilogue
  GemmParams U = {};
  if (!tensor_map_2d(&U.a_map, S.xs, 2, D, R, kGemmBK, kGemmBM, true)) return GEMQ_ERR_LAUNCH;
  fill_stacked(U, 0, L->w1);
  fill_stacked(U, 1, L->w3);
  U.nbits = L->w1.nbits; U.wq_strides = L->w1.wq_strides; U.zs_strides = L->w1.zs_strides;
  U.tile_expert = S.plan.tile_expert; U.tile_row0 = S.plan.tile_row0; U.tile_rows = S.plan.tile_rows;
  U.n_tiles = S.plan.n_tiles;
  U.N = F; U.K = D; U.G = G;
  U.out = S.h;
  U.err = S.err;
  if (int rc = launch_gemm(U, true, false, S.max_tiles, st)) return rc;

  // down GEMM, scaled by the routing weight
  GemmParams Dn = {};
  if (!tensor_map_2d(&Dn.a_map, S.h, 2, F, R, kGemmBK, kGemmBM, true)) return GEMQ_ERR_LAUNCH;
  fill_stacked(Dn, 0, L->w2);
  Dn.nbits = L->w2.nbits; Dn.wq_strides = L->w2.wq_strides; Dn.zs_strides = L->w2.zs_strides;
  Dn.tile_expert = S.plan.tile_expert; Dn.tile_row0 = S.plan.tile_row0; Dn.tile_rows = S.plan.tile_rows;
  Dn.n_tiles = S.plan.n_tiles;
  Dn.N = D; Dn.K = F; Dn.G = G;
  Dn.out = S.ys;
  Dn.row_weight = S.row_w;
  Dn.err = S.err;
  if (int rc = launch_gemm(Dn, false, false, S.max_tiles, st)) return rc;

  if (SF) {  // shared experts on all tokens (moe_block.py:419-430)
    const void* xsh = x;
    if (bf) {
      const size_t n8 = static_cast<size_t>(tokens) * D / 8;
      to_half_kernel<__nv_bfloat16><<<static_cast<unsigned>((n8 + 255) / 256), 256, 0, st>>>(
          static_cast<const __nv_bfloat16*>(x), static_cast<__half*>(S.xh), n8);
      xsh = S.xh;
    }
    GemmParams SU = {};
    if (!tensor_map_2d(&SU.a_map, xsh, 2, D, tokens, kGemmBK, kGemmBM, true)) return GEMQ_ERR_LAUNCH;
    fill_single(SU, 0, L->s1);
    fill_single(SU, 1, L->s3);
    SU.fixed_bits = L->s1.nbits;
    SU.rows_single = tokens;
    SU.N = SF; SU.K = D; SU.G = L->s1.group_size;
    SU.out = S.hs;
    SU.err = S.err;
    if (int rc = launch_gemm(SU, true, false, cdiv(tokens, kGemmBM), st)) return rc;
    GemmParams SD = {};
    if (!tensor_map_2d(&SD.a_map, S.hs, 2, SF, tokens, kGemmBK, kGemmBM, true)) return GEMQ_ERR_LAUNCH;
    fill_single(SD, 0, L->s2);
    SD.fixed_bits = L->s2.nbits;
    SD.rows_single = tokens;
    SD.N = D; SD.K = SF; SD.G = L->s2.group_size;
    SD.out = S.yss;
    SD.err = S.err;
    if (int rc = launch_gemm(SD, false, false, cdiv(tokens, kGemmBM), st)) return rc;
  }
  if (bf)
    prefill_combine_kernel<__nv_bfloat16><<<tokens, 128, 0, st>>>(
        S.plan.inv, reinterpret_cast<const long long*>(idx), static_cast<const __half*>(S.ys),
        SF ? static_cast<const __half*>(S.yss) : nullptr, static_cast<__nv_bfloat16*>(out), tokens, A, D);
  else
    prefill_combine_kernel<__half><<<tokens, 128, 0, st>>>(
        S.plan.inv, reinterpret_cast<const long long*>(idx), static_cast<const __half*>(S.ys),
        SF ? static_cast<const __half*>(S.yss) : nullptr, static_cast<__half*>(out), tokens, A, D);
  return launch_status();
}

// Error word of the last gemq_moe_prefill on this scratch (0 = no wait expired); device pointer.
extern "C" const int32_t* gemq_moe_prefill_error_word(const gemq_moe_layer_t* L, int tokens, void* scratch) {
  if (!L || !scratch || tokens <= 0) return nullptr;
  PrefillScratch S;
  prefill_bytes(L, tokens, &S, static_cast<char*>(scratch));
  return S.err;
}

