// Dense Q4_K llmp.vecq for 1..8 tokens with the int8 products on the tensor
// cores (mma.sync m16n8k32, u8 x s8 -> s32): the same exact per-sub-block int32
// sums and the same F32 scale fold as the dp4a kernels (vecq_rowlane.cuh), at
// about half their instructions and a third of their shared-memory traffic per
// super-block.  Interface and sums' contract are the reference's
// (src/kernels/ggml/vecq.h:23-49, vecq.cu:457-665); the structure is B200's.
//
//   * One persistent CTA per SM owns a contiguous, evenly divided range of
//     output rows, staged WHOLE in shared memory by the bulk-copy engine: one
//     cp.async.bulk per 16-row tile and matrix when rows follow one another in
//     memory at a pitch that spreads the tile's rows over the banks, else one per
//     row at a padded pitch.  A tile completes on its own mbarrier, so warps
//     start on the first tile while the rest stream in; the copies are requested
//     before the programmatic-dependency wait (weights depend on no kernel).
//   * A warp-step multiplies 16 rows x one 256-value super-block column.  The
//     A fragments are the rows' 4-bit codes straight out of the staged blocks:
//     lane (g, t) reads bytes 8t..8t+7 of a 32-byte chunk of rows g and g + 8
//     (one 64-bit load each), masks the low nibbles for the chunk's even
//     sub-block and the high nibbles, left in place as 16 x code, for the odd
//     one.  The MMA's k slots are a free permutation of the sub-block's 32
//     values as long as A and B agree, which is what lets a lane take eight
//     CONSECUTIVE bytes.
//   * The B fragment routes sub-blocks to columns: for sub-block s the token's
//     32 activations sit in column s and every other column is zero, and the
//     eight MMAs of a super-block accumulate into ONE C fragment.  Column s of
//     C is then the exact sum of sub-block s alone, and the fragment layout
//     hands lane (g, t) the sums of sub-blocks 2t and 2t + 1 for rows g and
//     g + 8: the scale fold runs on all 32 lanes with no shuffle.
//   * Each lane folds its two sub-blocks, d8 * (sc * sum) and (d8 * sum q) * m,
//     multiplies by the super-block's d and dmin and adds to its row's running
//     F32 sum; the four lanes of a row meet in a fixed xor tree once a tile.
//   * Warps form a grid (column groups x tile groups) over the CTA's share; the
//     column groups' partial sums of a row meet through shared memory in column
//     order.  Tokens are processed one after another with the same arithmetic, so
//     a (token, row) result does not depend on the other tokens of the launch.
//   * Every mbarrier wait is bounded and reports through the fault counter.
#ifndef LLMP_B200_CSRC_VECQ_ROWMMA_CUH_
#define LLMP_B200_CSRC_VECQ_ROWMMA_CUH_

#include "peer.cuh"
#include "vecq_stream.cuh"

namespace llmp_b200 {
namespace vecq {

constexpr int kRowMmaMaxWarps = 24;
constexpr int kRowMmaMaxTiles = 16;       // 16-row tiles a pass (one mbarrier each)
constexpr int kRowMmaMaxColGroups = 12;   // so that every token count runs the same column split
// Warps a CTA by tokens a pass: 85 registers a thread for one token, 128 for two, 168 beyond.
__host__ __device__ constexpr int RowMmaWarpLimit(int p) { return p == 1 ? 24 : p == 2 ? 16 : 12; }

struct RowMmaPlan {
  int grid;
  int warps;          // WC * WT
  int col_groups;     // WC: warps that split a row's super-block columns
  int tile_groups;    // WT: warps that split a pass's row tiles
  int columns;        // UR = k / 256
  int pass_rows;      // rows a pass stages (a multiple of 16, or the CTA's whole share)
  int pass_pad;       // pass_rows rounded up to whole tiles: the partial sums' row count
  int pitch;          // bytes between staged rows
  int packed;         // one bulk copy a tile and matrix (pitch == a row's bytes)
  int acts_bytes;     // one token's staged activations: k int8, then k / 32 x (d, d * sum q)
  int partial_floats; // col_groups * pass_rows(16-padded) * P * mats
  int smem_bytes;
  unsigned int* faults;
  PeerFan fan;  // world > 0: token 0's results also go, tagged, into every rank's vector (peer.cuh)
};

__device__ __forceinline__ void MmaU8S8(int (&c)[4], std::uint32_t a0, std::uint32_t a1,
                                        std::uint32_t a2, std::uint32_t a3, std::uint32_t b0,
                                        std::uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// kTokenColumns (P == 8): the MMA's eight columns are the TOKENS, not the sub-blocks.  One MMA
// a sub-block takes all (up to eight) tokens at once - eight MMAs a super-block whatever the
// token count, against eight a token - and the fragment hands lane (g, t) the sums of rows g
// and g + 8 for tokens 2t and 2t + 1: it folds all eight sub-blocks itself, in order, and no
// lanes have to meet.  (A token's F32 bits then differ from the one-token kernels': the order
// of the sub-blocks' terms is another.)
template <int P, bool kGlu, bool kTokenColumns = false>
__global__ void __launch_bounds__(RowMmaWarpLimit(P) * 32, 1)
VecQRowMmaKernel(const Desc a, const RowMmaPlan plan) {
  static_assert(!kTokenColumns || P == 8, "token columns: eight tokens a pass");
  constexpr int kMats = kGlu ? 2 : 1;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) std::uint64_t full[kRowMmaMaxTiles];

  const int tid = static_cast<int>(threadIdx.x);
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int g = lane >> 2;  // the fragment's group: rows g and g + 8, column g of B
  const int t = lane & 3;
  const int UR = plan.columns;
  const int wc = warp % plan.col_groups;
  const int wt = warp / plan.col_groups;

  const int cta_begin = static_cast<int>((static_cast<long>(blockIdx.x) * a.nrows) / gridDim.x);
  const int cta_end = static_cast<int>((static_cast<long>(blockIdx.x + 1) * a.nrows) / gridDim.x);

  // smem: [P tokens' activations][the staged rows, matrix after matrix][partial sums]
  unsigned char* acts = smem;
  unsigned char* rows_at = smem + (static_cast<std::size_t>(P) * plan.acts_bytes);
  float* partial = reinterpret_cast<float*>(
      rows_at + (static_cast<std::size_t>(kMats) * plan.pass_rows * plan.pitch));

  const std::uint8_t* mats[kMats];
  mats[0] = static_cast<const std::uint8_t*>(a.w);
  if constexpr (kGlu) mats[1] = static_cast<const std::uint8_t*>(a.g);
  const std::uint32_t row_bytes = static_cast<std::uint32_t>(UR) * 144u;

  if (tid == 0) {
    for (int i = 0; i < kRowMmaMaxTiles; ++i) MbarInit(&full[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // Warp 0 requests a pass: rows [first, first + count) of the CTA's share.
  auto request_pass = [&](int first, int count) {
    const int tiles = (count + 15) >> 4;
    for (int i = 0; i < tiles; ++i) {
      const int r0 = i * 16;
      const int n = min(16, count - r0);
      if (lane == 0) MbarExpectTx(&full[i], static_cast<std::uint32_t>(n) * row_bytes * kMats);
      __syncwarp();
      if (plan.packed) {
        if (lane < kMats) {
          BulkLoad(rows_at + ((static_cast<std::size_t>(lane) * plan.pass_rows + r0) * plan.pitch),
                   mats[lane] + (static_cast<std::size_t>(first + r0) * a.stride_row * 144),
                   static_cast<std::uint32_t>(n) * row_bytes, &full[i]);
        }
      } else {
        for (int c = lane; c < n * kMats; c += 32) {
          const int m = c / n, r = c % n;
          BulkLoad(rows_at + ((static_cast<std::size_t>(m) * plan.pass_rows + r0 + r) * plan.pitch),
                   mats[m] + (static_cast<std::size_t>(first + r0 + r) * a.stride_row * 144),
                   row_bytes, &full[i]);
        }
      }
    }
  };

  GridLaunchDependents();
  if (warp == 0 && cta_end > cta_begin) {
    request_pass(cta_begin, min(plan.pass_rows, cta_end - cta_begin));
  }
  GridDependencyWait();

  // Stage the tokens' activations, one Q8_1 block a thread: the int8 values as they
  // are (32 a block), then per block (d, d * sum q).
  {
    const int blocks = UR * 8;
    for (int p = 0; p < P; ++p) {
      const int token = min(p, a.tokens - 1);
      unsigned char* q = acts + (static_cast<std::size_t>(p) * plan.acts_bytes);
      float2* sc = reinterpret_cast<float2*>(q + (static_cast<std::size_t>(UR) * 256));
      for (int b = tid; b < blocks; b += static_cast<int>(blockDim.x)) {
        const auto* src = reinterpret_cast<const std::uint32_t*>(
            static_cast<const std::uint8_t*>(a.y) +
            ((static_cast<std::size_t>(token) * a.y_token + b) * 36));
        std::uint32_t v[8];
        int isum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          v[i] = src[1 + i];
          isum = Dp4a(0x01010101, static_cast<int>(v[i]), isum);
        }
        const float d = HalfBitsToFloat(src[0] & 0xffffu);
        auto* dst = reinterpret_cast<uint4*>(q + (static_cast<std::size_t>(b) * 32));
        dst[0] = make_uint4(v[0], v[1], v[2], v[3]);
        dst[1] = make_uint4(v[4], v[5], v[6], v[7]);
        sc[b] = make_float2(d, d * static_cast<float>(isum));
      }
    }
  }
  __syncthreads();

  bool healthy = true;
  std::uint32_t parity = 0;
  for (int first = cta_begin; first < cta_end; first += plan.pass_rows) {
    const int count = min(plan.pass_rows, cta_end - first);
    const int tiles = (count + 15) >> 4;
    if (first != cta_begin) {
      if (warp == 0) {
        FenceProxyAsync();
        request_pass(first, count);
      }
    }
    for (int tile = wt; tile < tiles; tile += plan.tile_groups) {
      if (healthy && lane == 0 && !MbarWait(&full[tile], parity)) {
        healthy = false;
        atomicAdd(plan.faults, 1u);
      }
      healthy = __shfl_sync(0xffffffffu, healthy ? 1 : 0, 0) != 0;
      if (!healthy) break;
      // rows g and g + 8 of the tile, clamped into the pass (the last tile may be short)
      const int r_lo = min((tile * 16) + g, count - 1);
      const int r_hi = min((tile * 16) + g + 8, count - 1);
      float acc[kMats][2][P];
#pragma unroll
      for (int m = 0; m < kMats; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int p = 0; p < P; ++p) acc[m][h][p] = 0.0f;

      if constexpr (kTokenColumns) {
        // lane (g, t): column g of B is token g; its results are tokens 2t and 2t + 1
        const unsigned char* b_tok =
            acts + (static_cast<std::size_t>(min(g, a.tokens - 1)) * plan.acts_bytes);
        const float2* sc_a = reinterpret_cast<const float2*>(
            acts + (static_cast<std::size_t>(min(2 * t, a.tokens - 1)) * plan.acts_bytes) +
            (static_cast<std::size_t>(UR) * 256));
        const float2* sc_b = reinterpret_cast<const float2*>(
            acts + (static_cast<std::size_t>(min((2 * t) + 1, a.tokens - 1)) * plan.acts_bytes) +
            (static_cast<std::size_t>(UR) * 256));
        float sums[kMats][2][2];  // [matrix][row g / g + 8][token 2t / 2t + 1]
#pragma unroll
        for (int m = 0; m < kMats; ++m)
#pragma unroll
          for (int h = 0; h < 2; ++h) sums[m][h][0] = sums[m][h][1] = 0.0f;
        for (int c = wc; c < UR; c += plan.col_groups) {
          uint2 bq[8];
#pragma unroll
          for (int sb = 0; sb < 8; ++sb) {
            bq[sb] = *reinterpret_cast<const uint2*>(b_tok + (((c * 8) + sb) * 32) + (8 * t));
          }
#pragma unroll
          for (int m = 0; m < kMats; ++m) {
            const unsigned char* lo_row =
                rows_at + ((static_cast<std::size_t>(m) * plan.pass_rows + r_lo) * plan.pitch) + (c * 144);
            const unsigned char* hi_row =
                rows_at + ((static_cast<std::size_t>(m) * plan.pass_rows + r_hi) * plan.pitch) + (c * 144);
            const uint4 h0 = *reinterpret_cast<const uint4*>(lo_row);
            const uint4 h1 = *reinterpret_cast<const uint4*>(hi_row);
            float pr[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}}, mr[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              const uint2 x = *reinterpret_cast<const uint2*>(lo_row + 16 + (cc * 32) + (8 * t));
              const uint2 y = *reinterpret_cast<const uint2*>(hi_row + 16 + (cc * 32) + (8 * t));
              int even[4] = {0, 0, 0, 0}, odd[4] = {0, 0, 0, 0};
              MmaU8S8(even, x.x & 0x0f0f0f0fu, y.x & 0x0f0f0f0fu, x.y & 0x0f0f0f0fu, y.y & 0x0f0f0f0fu,
                      bq[2 * cc].x, bq[2 * cc].y);
              MmaU8S8(odd, x.x & 0xf0f0f0f0u, y.x & 0xf0f0f0f0u, x.y & 0xf0f0f0f0u, y.y & 0xf0f0f0f0u,
                      bq[(2 * cc) + 1].x, bq[(2 * cc) + 1].y);
              std::uint32_t sc0, mn0, sc1, mn1;
              Q4KScalePair(h0.y, h0.z, h0.w, cc, &sc0, &mn0);
              Q4KScalePair(h1.y, h1.z, h1.w, cc, &sc1, &mn1);
              const int scale[2][2] = {{static_cast<int>(sc0 & 0xffu), static_cast<int>(sc0 >> 8)},
                                       {static_cast<int>(sc1 & 0xffu), static_cast<int>(sc1 >> 8)}};
              const float minimum[2][2] = {{static_cast<float>(mn0 & 0xffu), static_cast<float>(mn0 >> 8)},
                                           {static_cast<float>(mn1 & 0xffu), static_cast<float>(mn1 >> 8)}};
              // sub-blocks 2cc and 2cc + 1, in that order: d8 * (sc * dot) and (d8 * sum q) * m
#pragma unroll
              for (int o = 0; o < 2; ++o) {
                const float2 ta = sc_a[(c * 8) + (2 * cc) + o], tb = sc_b[(c * 8) + (2 * cc) + o];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  const int da = o == 0 ? even[2 * h] : (odd[2 * h] >> 4);
                  const int db = o == 0 ? even[(2 * h) + 1] : (odd[(2 * h) + 1] >> 4);
                  pr[h][0] = fmaf(ta.x, static_cast<float>(da * scale[h][o]), pr[h][0]);
                  pr[h][1] = fmaf(tb.x, static_cast<float>(db * scale[h][o]), pr[h][1]);
                  mr[h][0] = fmaf(ta.y, minimum[h][o], mr[h][0]);
                  mr[h][1] = fmaf(tb.y, minimum[h][o], mr[h][1]);
                }
              }
            }
            const float d0 = HalfBitsToFloat(h0.x & 0xffffu), dm0 = HalfBitsToFloat(h0.x >> 16);
            const float d1 = HalfBitsToFloat(h1.x & 0xffffu), dm1 = HalfBitsToFloat(h1.x >> 16);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              sums[m][0][j] += (d0 * pr[0][j]) - (dm0 * mr[0][j]);
              sums[m][1][j] += (d1 * pr[1][j]) - (dm1 * mr[1][j]);
            }
          }
        }
        // a lane's sums are whole: rows g, g + 8 x tokens 2t, 2t + 1 of this column group
#pragma unroll
        for (int m = 0; m < kMats; ++m)
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const int r = (tile * 16) + g + (8 * h);
              partial[(((static_cast<std::size_t>(wc) * plan.pass_pad + r) * P + (2 * t) + j) * kMats) + m] =
                  sums[m][h][j];
            }
      } else {
      for (int c = wc; c < UR; c += plan.col_groups) {
        // The token's B fragments for this column when there is one token: built
        // once, used for both matrices.
        std::uint32_t bq[P == 1 ? 2 : 1];
        float2 bs[P == 1 ? 2 : 1];
        if constexpr (P == 1) {
          const uint2 w2 = *reinterpret_cast<const uint2*>(acts + (((c * 8) + g) * 32) + (8 * t));
          bq[0] = w2.x;
          bq[1] = w2.y;
          const float2* sc = reinterpret_cast<const float2*>(acts + (static_cast<std::size_t>(UR) * 256));
          bs[0] = sc[(c * 8) + (2 * t)];
          bs[1] = sc[(c * 8) + (2 * t) + 1];
        }
#pragma unroll
        for (int m = 0; m < kMats; ++m) {
          const unsigned char* lo_row =
              rows_at + ((static_cast<std::size_t>(m) * plan.pass_rows + r_lo) * plan.pitch) + (c * 144);
          const unsigned char* hi_row =
              rows_at + ((static_cast<std::size_t>(m) * plan.pass_rows + r_hi) * plan.pitch) + (c * 144);
          // A fragments of the four chunks: low nibbles (even sub-block), high nibbles
          // in place (odd sub-block, 16 x code).
          std::uint32_t alo[4][4], ahi[4][4];
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            const uint2 x = *reinterpret_cast<const uint2*>(lo_row + 16 + (cc * 32) + (8 * t));
            const uint2 y = *reinterpret_cast<const uint2*>(hi_row + 16 + (cc * 32) + (8 * t));
            alo[cc][0] = x.x & 0x0f0f0f0fu; ahi[cc][0] = x.x & 0xf0f0f0f0u;
            alo[cc][1] = y.x & 0x0f0f0f0fu; ahi[cc][1] = y.x & 0xf0f0f0f0u;
            alo[cc][2] = x.y & 0x0f0f0f0fu; ahi[cc][2] = x.y & 0xf0f0f0f0u;
            alo[cc][3] = y.y & 0x0f0f0f0fu; ahi[cc][3] = y.y & 0xf0f0f0f0u;
          }
          // The two rows' headers: d, dmin and the scales / minima of sub-blocks 2t, 2t+1.
          const uint4 h0 = *reinterpret_cast<const uint4*>(lo_row);
          const uint4 h1 = *reinterpret_cast<const uint4*>(hi_row);
          std::uint32_t sc0, mn0, sc1, mn1;
          Q4KScalePair(h0.y, h0.z, h0.w, t, &sc0, &mn0);
          Q4KScalePair(h1.y, h1.z, h1.w, t, &sc1, &mn1);
          const float d0 = HalfBitsToFloat(h0.x & 0xffffu), dm0 = HalfBitsToFloat(h0.x >> 16);
          const float d1 = HalfBitsToFloat(h1.x & 0xffffu), dm1 = HalfBitsToFloat(h1.x >> 16);
#pragma unroll
          for (int p = 0; p < P; ++p) {
            std::uint32_t q0, q1;
            float2 s0, s1;
            if constexpr (P == 1) {
              q0 = bq[0]; q1 = bq[1]; s0 = bs[0]; s1 = bs[1];
            } else {
              const unsigned char* ap = acts + (static_cast<std::size_t>(p) * plan.acts_bytes);
              const uint2 w2 = *reinterpret_cast<const uint2*>(ap + (((c * 8) + g) * 32) + (8 * t));
              q0 = w2.x;
              q1 = w2.y;
              const float2* sc = reinterpret_cast<const float2*>(ap + (static_cast<std::size_t>(UR) * 256));
              s0 = sc[(c * 8) + (2 * t)];
              s1 = sc[(c * 8) + (2 * t) + 1];
            }
            int dots[4] = {0, 0, 0, 0};
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              // sub-block 2cc in column 2cc, sub-block 2cc + 1 in column 2cc + 1
              const bool even = g == (2 * cc), odd = g == (2 * cc) + 1;
              MmaU8S8(dots, alo[cc][0], alo[cc][1], alo[cc][2], alo[cc][3], even ? q0 : 0u,
                      even ? q1 : 0u);
              MmaU8S8(dots, ahi[cc][0], ahi[cc][1], ahi[cc][2], ahi[cc][3], odd ? q0 : 0u,
                      odd ? q1 : 0u);
            }
            // dots: {row g, sub-block 2t}, {row g, 2t+1 (x16)}, {row g+8, 2t}, {row g+8, 2t+1 (x16)}
            // d * sum_s d8_s * (sc_s * dot_s)  -  dmin * sum_s (d8_s * sum q_s) * m_s
            const float p0 = fmaf(s1.x, static_cast<float>((dots[1] >> 4) * static_cast<int>(sc0 >> 8)),
                                  s0.x * static_cast<float>(dots[0] * static_cast<int>(sc0 & 0xffu)));
            const float m0 = fmaf(s1.y, static_cast<float>(mn0 >> 8), s0.y * static_cast<float>(mn0 & 0xffu));
            const float p1 = fmaf(s1.x, static_cast<float>((dots[3] >> 4) * static_cast<int>(sc1 >> 8)),
                                  s0.x * static_cast<float>(dots[2] * static_cast<int>(sc1 & 0xffu)));
            const float m1 = fmaf(s1.y, static_cast<float>(mn1 >> 8), s0.y * static_cast<float>(mn1 & 0xffu));
            acc[m][0][p] += (d0 * p0) - (dm0 * m0);
            acc[m][1][p] += (d1 * p1) - (dm1 * m1);
          }
        }
      }
      // The four lanes of a row meet (fixed tree); lane t == 0 leaves the column
      // group's partial sum of rows g and g + 8.
#pragma unroll
      for (int m = 0; m < kMats; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int p = 0; p < P; ++p) {
            float v = acc[m][h][p];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if (t == 0) {
              const int r = (tile * 16) + g + (8 * h);
              partial[(((static_cast<std::size_t>(wc) * plan.pass_pad + r) * P + p) * kMats) + m] = v;
            }
          }
    }
      }
    // every column group's partial sums of the pass are written; a wait that ran out
    // anywhere in the CTA ends it for all: nothing of an incomplete pass is stored
    if (__syncthreads_or(healthy ? 0 : 1) != 0) return;
    // Row sums in column-group order, the GLU, the store.
    for (int i = tid; i < count * P; i += static_cast<int>(blockDim.x)) {
      const int r = i / P, p = i % P;
      if (p >= a.tokens) continue;
      float v[kMats];
#pragma unroll
      for (int m = 0; m < kMats; ++m) {
        float s = 0.0f;
        for (int w = 0; w < plan.col_groups; ++w) {
          s += partial[(((static_cast<std::size_t>(w) * plan.pass_pad + r) * P + p) * kMats) + m];
        }
        v[m] = s;
      }
      float* dst = a.dst + (static_cast<std::size_t>(p) * a.dst_token) + first + r;
      float result;
      if constexpr (kGlu) {
        result = Glu(a.glu, v[1], v[0], a.limit);
      } else {
        result = v[0];
      }
      *dst = result;
      if (plan.fan.world > 0 && p == 0) FanStore(plan.fan, FanTag(plan.fan), first + r, result);
    }
    __syncthreads();  // before the next pass overwrites rows and partial sums
    parity ^= 1u;
  }
}

// Host: the geometry, or false if the product does not fit (k too long for one
// 16-row tile a pass).
inline bool PlanRowMma(const Desc& d, int p, int sms, RowMmaPlan* plan, int ctas_per_sm = 1,
                       bool token_columns = false) {
  const int mats = d.glu != LLMP_B200_GLU_NONE ? 2 : 1;
  const int ur = d.ncols_x / 256;
  if (ur < 1) return false;
  // Several smaller CTAs an SM leave room for the NEXT kernel's CTAs (programmatic
  // dependents) to become resident and fetch their weights while this one drains.
  const int grid = std::max(1, std::min(sms * ctas_per_sm, (d.nrows + 15) / 16));
  const int warp_cap = std::max(1, RowMmaWarpLimit(p) / ctas_per_sm);
  const int cta_rows = (d.nrows + grid - 1) / grid;
  const int row_bytes = ur * 144;
  const bool contiguous = d.stride_row == ur;
  // A pitch that spreads rows g = 0..7 over the banks for 64-bit loads: 32 or 96 mod 128.
  const bool good = (row_bytes % 128 == 32) || (row_bytes % 128 == 96);
  const int pitch = (contiguous && good) ? row_bytes : ((row_bytes + 127) / 128 * 128) + 32;
  // (token columns: lanes of eight different tokens read at once; a token pitch of 32 bytes
  // mod 128 keeps their 64-bit loads on different banks)
  const int acts_bytes = token_columns ? ((((ur * 256) + (ur * 8 * 8)) + 127) / 128 * 128) + 32
                                       : (ur * 256) + (ur * 8 * 8);
  const int budget = (218 * 1024 / ctas_per_sm) - (p * acts_bytes) - 2048;
  if (budget <= 0) return false;
  // Warps: column groups x tile groups.  The column split fixes the order a row's
  // sums are added in, so it is chosen from k and the CTA's share alone (the same for
  // every token count); the tile split takes what the token count's warp limit leaves.
  const int tiles_cta = (cta_rows + 15) / 16;
  int wc = 1;
  {
    long best_load = 1L << 60;
    int best_warps = 0;
    for (int c = 1; c <= std::min({ur, kRowMmaMaxColGroups, warp_cap}); ++c) {
      const int wt = std::max(1, std::min(tiles_cta, (kRowMmaMaxWarps / ctas_per_sm) / c));
      const long load = static_cast<long>((ur + c - 1) / c) * ((tiles_cta + wt - 1) / wt);
      if (load < best_load || (load == best_load && c * wt > best_warps)) {
        best_load = load;
        best_warps = c * wt;
        wc = c;
      }
    }
  }
  int rows = cta_rows;
  for (;;) {
    const int padded = (rows + 15) / 16 * 16;
    const long need = static_cast<long>(mats) * rows * pitch + static_cast<long>(wc) * padded * p * mats * 4;
    if (need <= budget && padded / 16 <= kRowMmaMaxTiles) {
      const int wt = std::max(1, std::min(padded / 16, warp_cap / wc));
      plan->grid = grid;
      plan->warps = wc * wt;
      plan->col_groups = wc;
      plan->tile_groups = wt;
      plan->columns = ur;
      plan->pass_rows = rows;
      plan->pass_pad = padded;
      plan->pitch = pitch;
      plan->packed = (contiguous && good) ? 1 : 0;
      plan->acts_bytes = acts_bytes;
      plan->partial_floats = wc * padded * p * mats;
      plan->smem_bytes = (p * acts_bytes) + (mats * rows * pitch) + (plan->partial_floats * 4);
      break;
    }
    if (rows <= 16) return false;
    rows = std::max(16, ((rows / 2) + 15) / 16 * 16);  // more passes of fewer rows
  }
  plan->faults = FaultCounter();
  plan->fan = PeerFan{};
  return plan->faults != nullptr;
}

template <int P, bool kGlu>
cudaError_t LaunchRowMmaOne(const Desc& d, const RowMmaPlan& plan, cudaStream_t stream) {
  auto* kernel = VecQRowMmaKernel<P, kGlu>;
  static thread_local int configured_device = -1;
  int device = -1;
  cudaGetDevice(&device);
  if (configured_device != device) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               220 * 1024);
    if (e != cudaSuccess) return e;
    configured_device = device;
  }
  return LaunchPdl(kernel, dim3(static_cast<unsigned>(plan.grid)),
                   dim3(static_cast<unsigned>(plan.warps * 32)),
                   static_cast<std::size_t>(plan.smem_bytes), stream, d, plan);
}

template <bool kGlu>
cudaError_t LaunchRowMmaTokensOne(const Desc& d, const RowMmaPlan& plan, cudaStream_t stream) {
  auto* kernel = VecQRowMmaKernel<8, kGlu, true>;
  static thread_local int configured_device = -1;
  int device = -1;
  cudaGetDevice(&device);
  if (configured_device != device) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               220 * 1024);
    if (e != cudaSuccess) return e;
    configured_device = device;
  }
  return LaunchPdl(kernel, dim3(static_cast<unsigned>(plan.grid)),
                   dim3(static_cast<unsigned>(plan.warps * 32)),
                   static_cast<std::size_t>(plan.smem_bytes), stream, d, plan);
}

cudaError_t LaunchRowMma(const Desc& d, int p, const RowMmaPlan& plan, cudaStream_t stream);
cudaError_t LaunchRowMmaTokens(const Desc& d, const RowMmaPlan& plan, cudaStream_t stream);

}  // namespace vecq
}  // namespace llmp_b200

#endif  // LLMP_B200_CSRC_VECQ_ROWMMA_CUH_
