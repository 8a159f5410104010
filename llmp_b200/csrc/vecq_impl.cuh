// llmp.vecq on B200: quantized matrix-vector products over Q8_1 activations
// (dense rows, grouped matrices, routed experts; optional fused GLU of a gate
// and an up projection).  Interface and semantics follow the reference's
// src/kernels/ggml/vecq.h:23-49 and vecq.cu:457-665; the design does not.
//
// The product is a pure HBM stream of weight blocks, so the kernel is built
// around bytes in flight rather than around GGML's MMVQ loop:
//   * a "unit" is the smallest piece of a weight row a lane decodes alone and
//     that starts on a vector-load boundary: for Q4_K one 32-byte nibble chunk
//     (two 32-value sub-blocks) plus the super-block's 16-byte header; for
//     Q8_0 four blocks (136 bytes, 8-byte aligned) or one block (2-byte
//     aligned fallback);
//   * a team of LPR lanes walks one weight row, unit u = it * LPR + lane; a
//     lane issues the loads of U units x R rows (x 2 matrices with a GLU)
//     before it decodes any of them, all as 128/64-bit streaming loads that
//     bypass L1;
//   * the pass's activation rows are staged once a CTA into shared memory in
//     a 16-byte aligned split form (int8 values; per block d and d * sum q),
//     so a unit's activations are four 128-bit shared loads per token;
//   * int8 products are dp4a into int32 per 32-value block, scaled in F32; the
//     team's partial sums meet in a fixed-order xor-shuffle tree (no atomics),
//     so a (token, row) sum does not depend on what else the launch computes;
//   * dense launches fetch their first units BEFORE waiting on the kernel in
//     front (programmatic dependent launch): weights depend on no kernel.
#ifndef LLMP_B200_CSRC_VECQ_IMPL_CUH_
#define LLMP_B200_CSRC_VECQ_IMPL_CUH_

#include <algorithm>

#include "common.cuh"

namespace llmp_b200 {
namespace vecq {

// Routed (token, slot) pairs a launch.  The reference's operator stops at 128 pairs of 16
// tokens (llmp_ops.cc:2932, 2950); this kernel's pair lists take eight times that, so a
// routed block of up to 128 tokens reads every named expert's weights once.
constexpr int kMaxPairs = 1024;
constexpr int kMaxRoutedTokens = 128;
constexpr int kMaxThreads = 256;

using Desc = llmp_b200_vecq_desc;

// ------------------------------------------------------------------ units
// Q4_K super-block: FP16 d, FP16 dmin, 12 bytes of 6-bit scales/minima, 128
// bytes of nibbles (tests/unit/dsv4_fast_test.cc:167-194).
struct Q4KUnit {
  static constexpr int kType = LLMP_B200_TYPE_Q4_K;
  static constexpr int kBlockBytes = 144;
  static constexpr int kBlockElems = 256;
  static constexpr int kUnitElems = 64;  // two sub-blocks
  uint4 head;                            // d, dmin, scales[12]
  uint4 q[2];                            // 32 bytes of nibbles

  static __device__ __forceinline__ int UnitsPerRow(int k) { return k / kUnitElems; }
  __device__ __forceinline__ void Zero() {
    head = make_uint4(0, 0, 0, 0);
    q[0] = q[1] = make_uint4(0, 0, 0, 0);
  }
  // `row` points at the row's first block; 16-byte aligned by the host check.
  __device__ __forceinline__ void Load(const std::uint8_t* row, int u) {
    const std::uint8_t* sb = row + (static_cast<std::size_t>(u >> 2) * kBlockBytes);
    head = LoadStream16(sb);
    const std::uint8_t* chunk = sb + 16 + ((u & 3) * 32);
    q[0] = LoadStream16(chunk);
    q[1] = LoadStream16(chunk + 16);
  }
  // The same unit out of a row staged in shared memory (16-byte aligned).
  __device__ __forceinline__ void LoadShared(const std::uint8_t* row, int u) {
    const std::uint8_t* sb = row + (static_cast<std::size_t>(u >> 2) * kBlockBytes);
    head = *reinterpret_cast<const uint4*>(sb);
    const std::uint8_t* chunk = sb + 16 + ((u & 3) * 32);
    q[0] = *reinterpret_cast<const uint4*>(chunk);
    q[1] = *reinterpret_cast<const uint4*>(chunk + 16);
  }
};

// The 6-bit scale and minimum of sub-blocks 2c and 2c+1 of a super-block whose
// 12 scale bytes are the words s0 s1 s2: byte pairs, low byte the even one.
__device__ __forceinline__ void Q4KScalePair(std::uint32_t s0, std::uint32_t s1, std::uint32_t s2,
                                             int c, std::uint32_t* sc, std::uint32_t* mn) {
  const int shift = (c & 1) * 16;
  const std::uint32_t a0 = (s0 >> shift) & 0xffffu;
  const std::uint32_t a1 = (s1 >> shift) & 0xffffu;
  const std::uint32_t a2 = (s2 >> shift) & 0xffffu;
  if (c < 2) {
    *sc = a0 & 0x3f3fu;
    *mn = a1 & 0x3f3fu;
  } else {
    *sc = (a2 & 0x0f0fu) | ((a0 >> 2) & 0x3030u);
    *mn = ((a2 >> 4) & 0x0f0fu) | ((a1 >> 2) & 0x3030u);
  }
}

// Decoded for the dot products: nibbles split into the two sub-blocks.
struct Q4KDecoded {
  int lo[8];
  int hi[8];
  float dsc0, dsc1, dmn0, dmn1;  // d * sc, dmin * m of the two sub-blocks
  __device__ __forceinline__ void From(const Q4KUnit& r, int u) {
    const std::uint32_t w[8] = {r.q[0].x, r.q[0].y, r.q[0].z, r.q[0].w,
                                r.q[1].x, r.q[1].y, r.q[1].z, r.q[1].w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      lo[i] = static_cast<int>(w[i] & 0x0f0f0f0fu);
      hi[i] = static_cast<int>((w[i] >> 4) & 0x0f0f0f0fu);
    }
    std::uint32_t sc, mn;
    Q4KScalePair(r.head.y, r.head.z, r.head.w, u & 3, &sc, &mn);
    const float d = HalfBitsToFloat(r.head.x & 0xffffu);
    const float dmin = HalfBitsToFloat(r.head.x >> 16);
    dsc0 = d * static_cast<float>(sc & 0xffu);
    dsc1 = d * static_cast<float>(sc >> 8);
    dmn0 = dmin * static_cast<float>(mn & 0xffu);
    dmn1 = dmin * static_cast<float>(mn >> 8);
  }
};

// The two sub-blocks' int32 sums against a token's 64 staged activations.
__device__ __forceinline__ void Q4KDots(const Q4KDecoded& w, const uint4* a, int* dot0, int* dot1) {
  int s0 = 0, s1 = 0;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint4 x = a[i];
    s0 = Dp4a(w.lo[4 * i + 0], static_cast<int>(x.x), s0);
    s0 = Dp4a(w.lo[4 * i + 1], static_cast<int>(x.y), s0);
    s0 = Dp4a(w.lo[4 * i + 2], static_cast<int>(x.z), s0);
    s0 = Dp4a(w.lo[4 * i + 3], static_cast<int>(x.w), s0);
    const uint4 y = a[2 + i];
    s1 = Dp4a(w.hi[4 * i + 0], static_cast<int>(y.x), s1);
    s1 = Dp4a(w.hi[4 * i + 1], static_cast<int>(y.y), s1);
    s1 = Dp4a(w.hi[4 * i + 2], static_cast<int>(y.z), s1);
    s1 = Dp4a(w.hi[4 * i + 3], static_cast<int>(y.w), s1);
  }
  *dot0 = s0;
  *dot1 = s1;
}

// Q8_0: FP16 d then 32 int8 (src/kernels/decode/decoders.cuh:106-125), 34
// bytes, so a block starts on a 2-byte boundary only.  kBlocks = 4: a unit is
// 136 bytes fetched as 17 8-byte loads (rows 8-byte aligned); kBlocks = 1: 17
// 2-byte loads.
template <int kBlocks>
struct Q8_0Unit {
  static constexpr int kType = LLMP_B200_TYPE_Q8_0;
  static constexpr int kBlockBytes = 34;
  static constexpr int kBlockElems = 32;
  static constexpr int kUnitElems = 32 * kBlocks;
  static constexpr int kWords = kBlocks == 4 ? 34 : 9;
  std::uint32_t w[kWords];

  static __device__ __forceinline__ int UnitsPerRow(int k) { return k / kUnitElems; }
  __device__ __forceinline__ void Zero() {
#pragma unroll
    for (int i = 0; i < kWords; ++i) w[i] = 0;
  }
  __device__ __forceinline__ void Load(const std::uint8_t* row, int u) {
    const std::uint8_t* p = row + (static_cast<std::size_t>(u) * kBlockBytes * kBlocks);
    if constexpr (kBlocks == 4) {
#pragma unroll
      for (int i = 0; i < 17; ++i) {
        const uint2 v = LoadStream8(p + (8 * i));
        w[2 * i] = v.x;
        w[2 * i + 1] = v.y;
      }
    } else {
      const auto* h = reinterpret_cast<const unsigned short*>(p);
      // word 0: d in the low half; words 1..8: the 32 values.
      w[0] = __ldg(h);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        w[1 + i] = static_cast<std::uint32_t>(__ldg(h + 1 + (2 * i))) |
                   (static_cast<std::uint32_t>(__ldg(h + 2 + (2 * i))) << 16);
      }
    }
  }
  // Four-block units out of a row staged in shared memory (8-byte aligned).
  __device__ __forceinline__ void LoadShared(const std::uint8_t* row, int u) {
    static_assert(kBlocks == 4 || kBlocks == 1, "unit sizes");
    const std::uint8_t* p = row + (static_cast<std::size_t>(u) * kBlockBytes * kBlocks);
    if constexpr (kBlocks == 4) {
#pragma unroll
      for (int i = 0; i < 17; ++i) {
        const uint2 v = *reinterpret_cast<const uint2*>(p + (8 * i));
        w[2 * i] = v.x;
        w[2 * i + 1] = v.y;
      }
    } else {
      Load(row, u);
    }
  }
  // Block j's scale and its int `i` (4 values) out of the unit's words.
  __device__ __forceinline__ float Scale(int j) const {
    if constexpr (kBlocks == 4) {
      const int at = 34 * j;  // byte offset, even
      const std::uint32_t word = w[at / 4];
      return HalfBitsToFloat((at % 4) == 0 ? (word & 0xffffu) : (word >> 16));
    } else {
      return HalfBitsToFloat(w[0] & 0xffffu);
    }
  }
  __device__ __forceinline__ int Int(int j, int i) const {
    if constexpr (kBlocks == 4) {
      const int at = (34 * j) + 2 + (4 * i);
      if ((at % 4) == 0) return static_cast<int>(w[at / 4]);
      return static_cast<int>(__byte_perm(w[at / 4], w[(at / 4) + 1], 0x5432));
    } else {
      return static_cast<int>(w[1 + i]);
    }
  }
};

// ------------------------------------------------------------------ staging
// Shared memory a pass holds: for each of its P tokens, the k int8 values (16-byte aligned),
// then k / 32 float2 (d, d * sum q).  Every 64 values are followed by 16 bytes of padding: the
// lanes of a team read consecutive units at once, and at a pitch of 64 or 128 bytes their
// 128-bit loads would meet on two bank groups, or one; at 80 they spread over all eight.
__host__ __device__ inline int StagedAt(int value) { return value + ((value >> 6) << 4); }
__host__ __device__ inline std::size_t StageBytes(int k, int tokens) {
  const std::size_t one =
      (static_cast<std::size_t>(StagedAt(k)) + 16 + (static_cast<std::size_t>(k / 32) * 8) + 15) / 16 * 16;
  return static_cast<std::size_t>(tokens) * one;
}
// Where a token's scales start (16-byte aligned: the float4 reads of the Q4_K path).
__host__ __device__ inline int StagedScales(int k) { return (StagedAt(k) + 15) / 16 * 16; }

// One Q8_1 block (36 bytes, 4-byte aligned) a thread.
__device__ __forceinline__ void StageRow(const std::uint8_t* __restrict__ y, int k,
                                         std::uint8_t* __restrict__ qs,
                                         float2* __restrict__ scales, int tid, int threads) {
  for (int b = tid; b < k / 32; b += threads) {
    const auto* src = reinterpret_cast<const std::uint32_t*>(y + (static_cast<std::size_t>(b) * 36));
    const std::uint32_t ds = src[0];
    std::uint32_t v[8];
    int isum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i] = src[1 + i];
      isum = Dp4a(0x01010101, static_cast<int>(v[i]), isum);
    }
    auto* dst = reinterpret_cast<uint4*>(qs + StagedAt(b * 32));
    dst[0] = make_uint4(v[0], v[1], v[2], v[3]);
    dst[1] = make_uint4(v[4], v[5], v[6], v[7]);
    const float d = HalfBitsToFloat(ds & 0xffffu);
    scales[b] = make_float2(d, d * static_cast<float>(isum));
  }
}

// ------------------------------------------------------------------ kernel
// Unit: Q4KUnit or Q8_0Unit<>.  P tokens a pass, LPR lanes a row, R rows a
// team at once, U units a lane in flight per row, kGlu: gate and up together.
template <typename Unit, int P, int LPR, int R, int U, bool kGlu>
__global__ void __launch_bounds__(kMaxThreads)
VecQKernel(const Desc a) {
  constexpr int kMats = kGlu ? 2 : 1;
  constexpr int kTeams = 32 / LPR;
  extern __shared__ __align__(16) unsigned char stage[];
  __shared__ int pairs[kMaxPairs];  // token << 8 | slot
  __shared__ int count;

  const int tid = static_cast<int>(threadIdx.x);
  const int threads = static_cast<int>(blockDim.x);
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int team = lane / LPR;
  const int lt = lane % LPR;
  const int rows_per_cta = (threads >> 5) * kTeams * R;
  const int row0 = (static_cast<int>(blockIdx.x) * rows_per_cta) + (((warp * kTeams) + team) * R);
  const int k = a.ncols_x;
  const int units = Unit::UnitsPerRow(k);
  const bool routed = a.ids != nullptr;

  GridLaunchDependents();

  Unit raw[U][R][kMats];
  const std::uint8_t* rowp[R][kMats];
  auto set_rows = [&](int expert) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = min(row0 + r, a.nrows - 1);
      const std::size_t at = (static_cast<std::size_t>(expert) * a.stride_expert +
                              static_cast<std::size_t>(row) * a.stride_row) *
                             Unit::kBlockBytes;
      rowp[r][0] = static_cast<const std::uint8_t*>(a.w) + at;
      if constexpr (kGlu) rowp[r][1] = static_cast<const std::uint8_t*>(a.g) + at;
    }
  };
  auto load_chunk = [&](int chunk) {
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const int u = (((chunk * U) + i) * LPR) + lt;
#pragma unroll
      for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int m = 0; m < kMats; ++m) {
          if (u < units) {
            raw[i][r][m].Load(rowp[r][m], u);
          } else {
            raw[i][r][m].Zero();
          }
        }
      }
    }
  };

  int expert = 0;
  if (!routed) {
    // Dense (one slot), or grouped: grid row y names the matrix.
    expert = static_cast<int>(blockIdx.y);
    set_rows(expert);
    load_chunk(0);  // before the wait: weights depend on no earlier kernel
    if (tid < a.tokens) pairs[tid] = (tid << 8) | expert;
    if (tid == 0) count = a.tokens;
  }
  GridDependencyWait();
  if (routed) {
    // One CTA row per distinct expert (the ownership rule of vecq.cu:514-546): grid
    // row y is a (token, slot) pair, and the CTA whose pair is the FIRST to name an
    // expert computes every pair that names it, in pair order; the others leave.
    // The list is built by the whole CTA: a thread takes a contiguous run of
    // pairs and counts its matches, the counts are scanned across the CTA, and
    // each thread drops its matches at its offset.
    const int s = static_cast<int>(blockIdx.y);
    expert = a.ids[((s / a.used) * a.ids_stride) + (s % a.used)];
    const int total = a.tokens * a.used;
    const int run = (total + threads - 1) / threads;
    const int lo = min(tid * run, total), hi = min(lo + run, total);
    int mine = 0;
    for (int q = lo; q < hi; ++q) {
      mine += a.ids[((q / a.used) * a.ids_stride) + (q % a.used)] == expert ? 1 : 0;
    }
    // exclusive scan of `mine` over the CTA (at most eight warps)
    __shared__ int warp_total[kMaxThreads / 32];
    int before = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, before, d);
      if (lane >= d) before += up;
    }
    if (lane == 31) warp_total[warp] = before;
    __syncthreads();
    int earlier = 0;
    for (int w = 0; w < warp; ++w) earlier += warp_total[w];
    before += earlier - mine;
    // The pair in front of every other match decides the ownership; exactly one
    // thread holds it (this CTA's own pair matches, so there is one).
    if (mine > 0 && before == 0) {
      int q = lo;
      while (a.ids[((q / a.used) * a.ids_stride) + (q % a.used)] != expert) ++q;
      int all = 0;
      for (int w = 0; w < (threads >> 5); ++w) all += warp_total[w];
      count = q == s ? all : 0;
    }
    __syncthreads();
    if (count != 0) {
      for (int q = lo; q < hi; ++q) {
        const int t = q / a.used, j = q % a.used;
        if (a.ids[(t * a.ids_stride) + j] == expert) pairs[before++] = (t << 8) | j;
      }
    }
    set_rows(expert);
  }
  __syncthreads();
  const int n = count;
  if (n == 0) return;
  if (routed) load_chunk(0);

  const int chunks = (units + (U * LPR) - 1) / (U * LPR);
  const std::size_t token_bytes = StageBytes(k, 1);

  for (int p = 0; p < n; p += P) {
    const int m_live = min(P, n - p);
    // Stage the pass's activation rows.
    for (int j = 0; j < m_live; ++j) {
      const int pr = pairs[p + j];
      const std::uint8_t* y = static_cast<const std::uint8_t*>(a.y) +
                              ((static_cast<std::size_t>(pr >> 8) * a.y_token +
                                static_cast<std::size_t>(pr & 0xff) * a.y_slot) * 36);
      std::uint8_t* qs = stage + (j * token_bytes);
      StageRow(y, k, qs, reinterpret_cast<float2*>(qs + StagedScales(k)), tid, threads);
    }
    __syncthreads();

    float acc[P][R][kMats];
#pragma unroll
    for (int j = 0; j < P; ++j)
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < kMats; ++m) acc[j][r][m] = 0.0f;

    for (int chunk = 0; chunk < chunks; ++chunk) {
      if (p != 0 || chunk != 0) load_chunk(chunk);
#pragma unroll
      for (int i = 0; i < U; ++i) {
        const int u = min((((chunk * U) + i) * LPR) + lt, units - 1);  // zeros past the row
        if constexpr (Unit::kType == LLMP_B200_TYPE_Q4_K) {
          Q4KDecoded dec[R][kMats];
#pragma unroll
          for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < kMats; ++m) dec[r][m].From(raw[i][r][m], u);
#pragma unroll
          for (int j = 0; j < P; ++j) {
            if (j < m_live) {
              const std::uint8_t* qs = stage + (j * token_bytes);
              const uint4* av = reinterpret_cast<const uint4*>(qs + (u * 80));
              const uint4 a4[4] = {av[0], av[1], av[2], av[3]};
              const float4 s4 = *reinterpret_cast<const float4*>(qs + StagedScales(k) + (u * 16));
#pragma unroll
              for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < kMats; ++m) {
                  int d0, d1;
                  Q4KDots(dec[r][m], a4, &d0, &d1);
                  // d8 * (d * sc) * dot - (d8 * sum q) * (dmin * m), per sub-block
                  float v = (s4.x * dec[r][m].dsc0) * static_cast<float>(d0);
                  v = fmaf(s4.z * dec[r][m].dsc1, static_cast<float>(d1), v);
                  v = fmaf(-s4.y, dec[r][m].dmn0, v);
                  v = fmaf(-s4.w, dec[r][m].dmn1, v);
                  acc[j][r][m] += v;
                }
            }
          }
        } else {
          constexpr int kB = Unit::kUnitElems / 32;
#pragma unroll
          for (int j = 0; j < P; ++j) {
            if (j < m_live) {
              const std::uint8_t* qs = stage + (j * token_bytes);
              const float2* sv = reinterpret_cast<const float2*>(qs + StagedScales(k)) + (u * kB);
#pragma unroll
              for (int b = 0; b < kB; ++b) {
                const uint4* av =
                    reinterpret_cast<const uint4*>(qs + StagedAt((u * Unit::kUnitElems) + (32 * b)));
                const uint4 x0 = av[0], x1 = av[1];
                const float d8 = sv[b].x;
                const int xs[8] = {static_cast<int>(x0.x), static_cast<int>(x0.y),
                                   static_cast<int>(x0.z), static_cast<int>(x0.w),
                                   static_cast<int>(x1.x), static_cast<int>(x1.y),
                                   static_cast<int>(x1.z), static_cast<int>(x1.w)};
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                  for (int m = 0; m < kMats; ++m) {
                    if constexpr (Unit::kType == LLMP_B200_TYPE_Q8_0) {
                      int sumi = 0;
#pragma unroll
                      for (int q = 0; q < 8; ++q) sumi = Dp4a(raw[i][r][m].Int(b, q), xs[q], sumi);
                      // d8_0 * d8_1 * sumi (vecq.cu:398-418)
                      acc[j][r][m] += raw[i][r][m].Scale(b) * d8 * static_cast<float>(sumi);
                    } else {
                      // the other block types (vecq_more.cuh) know their own sub-block product
                      acc[j][r][m] += raw[i][r][m].Dot(b, xs, d8, sv[b].y);
                    }
                  }
              }
            }
          }
        }
      }
    }

    // The team's partial sums: fixed xor tree, then one lane writes.
#pragma unroll
    for (int j = 0; j < P; ++j) {
      if (j >= m_live) continue;
      const int pr = pairs[p + j];
      float* dst = a.dst + (static_cast<std::size_t>(pr >> 8) * a.dst_token) +
                   (static_cast<std::size_t>(pr & 0xff) * a.dst_slot);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float v[kMats];
#pragma unroll
        for (int m = 0; m < kMats; ++m) {
          v[m] = acc[j][r][m];
#pragma unroll
          for (int offset = LPR / 2; offset > 0; offset >>= 1) {
            v[m] += __shfl_xor_sync(0xffffffffu, v[m], offset);
          }
        }
        if (lt == 0 && row0 + r < a.nrows) {
          if constexpr (kGlu) {
            dst[row0 + r] = Glu(a.glu, v[1], v[0], a.limit);
          } else {
            dst[row0 + r] = v[0];
          }
        }
      }
    }
    __syncthreads();  // before the next pass restages
  }
}

// ------------------------------------------------------------------ launch table
struct Variant {
  const char* name;
  int lpr, r, u, warps;
};
// Index = the `variant` argument.  Each exists for every type, P and GLU.
constexpr Variant kVariants[] = {
    {"l4r1u2w4", 4, 1, 2, 4},   {"l8r1u2w4", 8, 1, 2, 4},   {"l16r1u2w4", 16, 1, 2, 4},
    {"l32r1u2w4", 32, 1, 2, 4}, {"l4r2u2w4", 4, 2, 2, 4},   {"l8r2u2w4", 8, 2, 2, 4},
    {"l16r2u2w4", 16, 2, 2, 4}, {"l32r2u2w4", 32, 2, 2, 4}, {"l4r1u2w8", 4, 1, 2, 8},
    {"l8r1u2w8", 8, 1, 2, 8},   {"l16r1u2w8", 16, 1, 2, 8}, {"l32r1u2w8", 32, 1, 2, 8},
    {"l4r2u2w8", 4, 2, 2, 8},   {"l8r2u2w8", 8, 2, 2, 8},   {"l16r2u2w8", 16, 2, 2, 8},
    {"l32r2u2w8", 32, 2, 2, 8}, {"l8r1u4w4", 8, 1, 4, 4},   {"l16r1u4w4", 16, 1, 4, 4},
    {"l32r1u4w4", 32, 1, 4, 4}, {"l8r1u4w8", 8, 1, 4, 8},   {"l16r1u4w8", 16, 1, 4, 8},
    {"l32r1u4w8", 32, 1, 4, 8},
    // The persistent TMA-fed stream kernel (vecq_stream.cuh); dense products only.
    {"stream", 0, 0, 0, 0},
    // One lane per weight row over warp-private TMA rings (vecq_rowlane.cuh);
    // dense Q4_K products of up to 8 tokens.
    {"rowlane", 0, 0, 0, 0},
    // The same with the rows a warp forced (r field), for measurement.
    {"rowlane.r1", 0, 1, 0, 0},
    {"rowlane.r2", 0, 2, 0, 0},
    {"rowlane.r4", 0, 4, 0, 0},
    {"rowlane.r8", 0, 8, 0, 0},
    {"rowlane.r16", 0, 16, 0, 0},
    {"rowlane.r32", 0, 32, 0, 0},
    // Half an SM a CTA (u field = 1), so consecutive kernels overlap.
    {"rowlane.half", 0, 0, 1, 0},
    // The int8 products on mma.sync tiles of 16 rows (vecq_rowmma.cuh); dense Q4_K
    // products of up to 8 tokens.
    {"rowmma", 0, 0, 0, 0},
    // ... with 2, 3 or 4 smaller CTAs an SM (u field), so that consecutive kernels overlap.
    {"rowmma.c2", 0, 0, 2, 0},
    {"rowmma.c3", 0, 0, 3, 0},
    {"rowmma.c4", 0, 0, 4, 0},
    // The MMA's columns are the tokens (r field = 8): eight MMAs a super-block for up to eight
    // tokens; 2 to 8 tokens.
    {"rowmma.t8", 0, 8, 0, 0},
    {"rowmma.t8c2", 0, 8, 2, 0},
};
constexpr int kVariantCount = static_cast<int>(sizeof(kVariants) / sizeof(kVariants[0]));
constexpr int kStreamVariant = kVariantCount - 15;
constexpr int kRowLaneVariant = kVariantCount - 14;  // and its seven forced forms after it
constexpr int kRowMmaVariant = kVariantCount - 6;    // its three split forms and the two token-column forms after it

template <typename Unit, int P, int LPR, int R, int U, bool kGlu>
cudaError_t LaunchOne(const Desc& d, int warps, cudaStream_t stream) {
  auto* kernel = VecQKernel<Unit, P, LPR, R, U, kGlu>;
  const std::size_t smem = StageBytes(d.ncols_x, P);
  if (smem > 48 * 1024) {
    // Idempotent and cheap; not an allocation.
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
    if (e != cudaSuccess) return e;
  }
  const int rows_per_cta = warps * (32 / LPR) * R;
  const bool routed = d.ids != nullptr;
  const dim3 grid(static_cast<unsigned>((d.nrows + rows_per_cta - 1) / rows_per_cta),
                  static_cast<unsigned>(routed ? d.used * d.tokens : d.used));
  return LaunchPdl(kernel, grid, dim3(static_cast<unsigned>(warps * 32)), smem, stream, d);
}

template <typename Unit, int P, bool kGlu>
cudaError_t LaunchShape(const Desc& d, const Variant& v, cudaStream_t stream) {
  if constexpr (Unit::kType == LLMP_B200_TYPE_Q8_0 && Unit::kUnitElems == 32) {
    // The 2-byte aligned fallback keeps one configuration.
    return LaunchOne<Unit, P, 8, 1, 2, kGlu>(d, 4, stream);
  } else {
    // A Q8_0 unit is 34 registers against Q4_K's 12: fewer in flight a lane.
    constexpr bool kWide = Unit::kType == LLMP_B200_TYPE_Q8_0;
#define LLMP_CASE(L, RR, UU)                                                            \
  if (v.lpr == L && v.r == RR && v.u == UU) {                                           \
    constexpr int kU = kWide ? ((UU == 4 && RR == 1 && !kGlu) ? 2 : 1) : UU;            \
    return LaunchOne<Unit, P, L, RR, kU, kGlu>(d, v.warps, stream);                     \
  }
    LLMP_CASE(4, 1, 2) LLMP_CASE(8, 1, 2) LLMP_CASE(16, 1, 2) LLMP_CASE(32, 1, 2)
    LLMP_CASE(4, 2, 2) LLMP_CASE(8, 2, 2) LLMP_CASE(16, 2, 2) LLMP_CASE(32, 2, 2)
    LLMP_CASE(8, 1, 4) LLMP_CASE(16, 1, 4) LLMP_CASE(32, 1, 4)
#undef LLMP_CASE
    return cudaErrorInvalidValue;
  }
}

template <typename Unit>
cudaError_t LaunchType(const Desc& d, int p, const Variant& v, cudaStream_t stream) {
  const bool glu = d.glu != LLMP_B200_GLU_NONE;
#define LLMP_P(PP) \
  if (p == PP) return glu ? LaunchShape<Unit, PP, true>(d, v, stream) : LaunchShape<Unit, PP, false>(d, v, stream);
  LLMP_P(1) LLMP_P(2) LLMP_P(4) LLMP_P(8)
#undef LLMP_P
  return cudaErrorInvalidValue;
}

inline int UnitsOf(int type, const Desc& d, bool q8_fast) {
  return type == LLMP_B200_TYPE_Q4_K ? d.ncols_x / 64 : (q8_fast ? d.ncols_x / 128 : d.ncols_x / 32);
}

// The launch configuration a shape takes when the caller names none: lanes a
// row so that a lane walks about four units, two rows a team when the grid
// still covers the machine twice over.
inline int DefaultVariant(int units, int nrows, int slots, bool glu, int p, int sms) {
  int lpr = 32;
  while (lpr > 4 && units < lpr * 4) lpr /= 2;
  if (units % lpr != 0) {
    for (int c = 32; c >= 4; c /= 2) {
      if (units % c == 0 && units / c >= 2) { lpr = c; break; }
    }
  }
  const int warps = 4;
  int r = 1;
  if (!glu && p <= 2) {
    const long ctas = static_cast<long>((nrows + (warps * (32 / lpr) * 2) - 1) /
                                        (warps * (32 / lpr) * 2)) * slots;
    if (ctas >= 2L * sms * 4) r = 2;
  }
  for (int i = 0; i < kVariantCount; ++i) {
    const Variant& v = kVariants[i];
    if (v.lpr == lpr && v.r == r && v.u == 2 && v.warps == warps) return i;
  }
  return 1;
}

}  // namespace vecq
}  // namespace llmp_b200

#endif  // LLMP_B200_CSRC_VECQ_IMPL_CUH_
