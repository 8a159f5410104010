// Dense Q4_K llmp.vecq for 1..8 tokens as a persistent HBM stream with one
// lane per weight row.  Interface and sums' contract are the reference's
// (src/kernels/ggml/vecq.h:23-49, vecq.cu:457-665); the structure is B200's.
//
//   * One CTA per SM owns a contiguous, evenly divided range of output rows;
//     its W warps split that range, R rows a warp.
//   * A lane is (row r, phase ph), R * PH <= 32 (6 x 5 for k = 2560: ten
//     super-blocks a row in two steps of five).  The warp sweeps the
//     row's super-blocks ("columns") PH at a time; lane (r, ph) decodes column
//     j * PH + ph of row r.  A lane therefore accumulates its row's whole dot
//     product in registers; the PH phases meet in phase order at the end.  No atomics, no cross-warp traffic, and a (token, row) sum does
//     not depend on the other tokens of the launch.
//   * Weights reach shared memory through the TMA bulk-copy engine: for every
//     column step each row's PH consecutive super-blocks (PH * 144 bytes) are
//     one cp.async.bulk into the warp's PRIVATE ring of stages, completing on
//     that stage's mbarrier.  Warps never synchronize with each other in the
//     main loop.  The ring holds most of the CTA's bytes, so nearly the whole
//     matrix is requested in the first microsecond: that, not arithmetic, is
//     what bounds a 15-30 MB product.
//   * The first stages are requested BEFORE the programmatic-dependency wait
//     (weights depend on no earlier kernel); activations are staged after it.
//   * Row pieces sit at a pitch chosen so that the eight lanes of a quarter
//     warp read distinct bank groups (128-bit shared loads, no conflicts).
//   * Activations are staged once a CTA, interleaved by column so that the
//     lanes of different phases read adjacent 16-byte chunks and lanes of the
//     same phase broadcast.
//   * Every mbarrier wait is bounded and reports through the fault counter.
#ifndef LLMP_B200_CSRC_VECQ_ROWLANE_CUH_
#define LLMP_B200_CSRC_VECQ_ROWLANE_CUH_

#include "peer.cuh"
#include "vecq_stream.cuh"

namespace llmp_b200 {
namespace vecq {

constexpr int kRowLaneMaxWarps = 12;      // a CTA that owns its SM
constexpr int kRowLaneHalfWarps = 9;      // a CTA that shares its SM with the next kernel's
constexpr int kRowLaneMaxStages = 8;

struct RowLanePlan {
  int warps;         // W
  int rows;          // R rows a warp
  int phases;        // PH phases, R * PH <= 32
  int columns;       // UR = k / 256
  int steps;         // J = ceil(UR / PH)
  int stages;        // S_w, ring depth a warp
  int pitch;         // bytes between a stage's rows
  int stage_bytes;   // R * pitch * mats
  int acts_bytes;    // one token's staged activations
  int smem_bytes;
  int grid;
  int half;          // the kHalf instantiation
  double score;      // the planner's figure of merit (lane use x warps x ring depth)
  int f32_input;     // activations are F32: quantize to Q8_1 while staging
  int q8_row_blocks; // Q8_1 blocks between tokens' rows in q8_out
  std::uint8_t* q8_out;  // optional: the Q8_1 blocks, written by CTA 0
  // Optional: the OUTPUT's Q8_1 blocks (what the next product reads).  The warp
  // that completes a 32-row block of a token's output quantizes it.
  std::uint8_t* q8_dst;
  unsigned int* q8_rows_done;  // [tokens][nrows / 32] counters, zero between launches
  unsigned int* faults;
  PeerFan fan;  // world > 0: token 0's results also go, tagged, into every rank's vector (peer.cuh)
  RowSplit split;        // the rows of a CTA and of its warps (at most R a warp)
  int phase_reciprocal;  // ceil(65536 / R): lane / R without a division
};

// kHalf: at most half an SM's registers and shared memory, so that the kernel
// after this one (launched as a programmatic dependent) becomes resident and
// requests its weights while this one still computes.
template <int P, bool kGlu, bool kHalf>
__global__ void __launch_bounds__(kHalf ? kRowLaneHalfWarps * 32 : kRowLaneMaxWarps * 32,
                                  kHalf ? 2 : 1)
VecQRowLaneKernel(const Desc a, const RowLanePlan plan) {
  constexpr int kMats = kGlu ? 2 : 1;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) std::uint64_t full[kRowLaneMaxWarps][kRowLaneMaxStages];

  const int tid = static_cast<int>(threadIdx.x);
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int R = plan.rows;
  const int PH = plan.phases;
  const int UR = plan.columns;
  const int J = plan.steps;
  const int S = plan.stages;
  // Lanes R * PH and up (when R * PH < 32) idle through the column steps.
  const int ph = (lane * plan.phase_reciprocal) >> 16;  // lane / R
  const int r = lane - (ph * R);

  // This CTA's rows, then this warp's share of them (at most R).
  int row_begin, my_rows;
  WarpRows(plan.split, static_cast<int>(blockIdx.x), warp, &row_begin, &my_rows);
  const int row_end = row_begin + my_rows;

  unsigned char* acts = smem;
  unsigned char* ring = smem + (static_cast<std::size_t>(P) * plan.acts_bytes) +
                        (static_cast<std::size_t>(warp) * S * plan.stage_bytes);

  if (lane < S) {
    MbarInit(&full[warp][lane], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  // Requests the next column step of this warp's rows into its stage (steps are
  // requested in order): a copy a row and matrix, issued by one elected lane with
  // the warp converged, their operands uniform.  (An SM's copy engine takes these
  // 720-byte copies at about one every 20 cycles, as fast as their bytes arrive;
  // whole rows a copy, half as many, measured slower: a step's sums could then not
  // start before the other step's columns had landed.  No pointer array indexed by
  // a variable: it would live in local memory.)
  int next = 0, next_stage = 0;
  auto request = [&]() __attribute__((always_inline)) {
    const int cols = min(PH, UR - (next * PH));
    const std::uint32_t piece = static_cast<std::uint32_t>(cols) * 144u;
    unsigned char* base = ring + (static_cast<std::size_t>(next_stage) * plan.stage_bytes);
    if (ElectOne()) {
      MbarExpectTx(&full[warp][next_stage], piece * static_cast<std::uint32_t>(my_rows * kMats));
#pragma unroll
      for (int m = 0; m < kMats; ++m) {
        const std::uint8_t* src =
            static_cast<const std::uint8_t*>(kGlu && m != 0 ? a.g : a.w) +
            ((static_cast<std::size_t>(row_begin) * a.stride_row + static_cast<std::size_t>(next) * PH) * 144);
        unsigned char* dst = base + (static_cast<std::size_t>(m) * R * plan.pitch);
        for (int row = 0; row < my_rows; ++row) {
          BulkLoad(dst, src, piece, &full[warp][next_stage]);
          src += static_cast<std::size_t>(a.stride_row) * 144;
          dst += plan.pitch;
        }
      }
    }
    __syncwarp();
    ++next;
    if (++next_stage == S) next_stage = 0;
  };

  GridLaunchDependents();
  // Only the first column step is requested now, the next one each time a step has
  // landed (below): the copy engine serves the copies it holds side by side, so with
  // every step requested at once they all complete together, at the end of the
  // transfer, and no step's sums overlap it.
  if (my_rows > 0) request();
  GridDependencyWait();

  // Stage the tokens' activations: one Q8_1 block a thread.  Column c's i-th
  // 16-byte chunk is chunk (i * UR + c); its scales follow in four float4
  // planes: d[0..3], d[4..7], d * sum q [0..3], [4..7].  With plan.f32_input the
  // activations are F32 and every CTA quantizes them itself, with the
  // arithmetic of the Q8_1 quantizer (q8_1.cu: d = amax / 127 rounded to FP16,
  // q = roundf(x / d), the sum a butterfly over indices 16, 8, 4, 2, 1 apart),
  // so the staged values are the blocks' values bit for bit; CTA 0 also writes
  // the blocks out when the caller wants them.
  {
    const int blocks = UR * 8;
    for (int t = 0; t < P; ++t) {
      const int token = min(t, a.tokens - 1);
      uint4* q = reinterpret_cast<uint4*>(acts + (static_cast<std::size_t>(t) * plan.acts_bytes));
      float* sc = reinterpret_cast<float*>(q + (16 * UR));
      for (int b = tid; b < blocks; b += static_cast<int>(blockDim.x)) {
        std::uint32_t v[8];
        int isum = 0;
        float d;
        if (plan.f32_input) {
          const float4* src = reinterpret_cast<const float4*>(
              static_cast<const float*>(a.y) + (static_cast<std::size_t>(token) * a.y_token) +
              (static_cast<std::size_t>(b) * 32));
          float x[32], sum[32];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 f = src[i];
            x[4 * i] = f.x; x[4 * i + 1] = f.y; x[4 * i + 2] = f.z; x[4 * i + 3] = f.w;
          }
          float amax = 0.0f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            amax = fmaxf(amax, fabsf(x[i]));
            sum[i] = x[i];
          }
#pragma unroll
          for (int offset = 16; offset > 0; offset >>= 1) {
#pragma unroll
            for (int i = 0; i < offset; ++i) sum[i] = sum[i] + sum[i + offset];
          }
          const float df = amax / 127.0f;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            std::uint32_t packed = 0;
            if (amax != 0.0f) {
#pragma unroll
              for (int c4 = 0; c4 < 4; ++c4) {
                const int qi = static_cast<int>(roundf(x[(4 * i) + c4] / df));
                packed |= (static_cast<std::uint32_t>(qi) & 0xffu) << (8 * c4);
              }
            }
            v[i] = packed;
            isum = Dp4a(0x01010101, static_cast<int>(packed), isum);
          }
          const __half dh = __float2half_rn(df);
          d = __half2float(dh);
          if (plan.q8_out != nullptr && blockIdx.x == 0 && t < a.tokens) {
            auto* out = reinterpret_cast<std::uint32_t*>(
                plan.q8_out + ((static_cast<std::size_t>(t) * plan.q8_row_blocks + b) * 36));
            out[0] = static_cast<std::uint32_t>(__half_as_ushort(dh)) |
                     (static_cast<std::uint32_t>(__half_as_ushort(__float2half_rn(sum[0]))) << 16);
#pragma unroll
            for (int i = 0; i < 8; ++i) out[1 + i] = v[i];
          }
        } else {
          const auto* src = reinterpret_cast<const std::uint32_t*>(
              static_cast<const std::uint8_t*>(a.y) +
              ((static_cast<std::size_t>(token) * a.y_token + b) * 36));
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            v[i] = src[1 + i];
            isum = Dp4a(0x01010101, static_cast<int>(v[i]), isum);
          }
          d = HalfBitsToFloat(src[0] & 0xffffu);
        }
        const int c = b >> 3, g = b & 7;
        q[((2 * g) * UR) + c] = make_uint4(v[0], v[1], v[2], v[3]);
        q[((2 * g + 1) * UR) + c] = make_uint4(v[4], v[5], v[6], v[7]);
        sc[((((g >> 2)) * UR + c) * 4) + (g & 3)] = d;
        sc[((((2 + (g >> 2))) * UR + c) * 4) + (g & 3)] = d * static_cast<float>(isum);
      }
    }
  }
  __syncthreads();
  if (my_rows == 0) return;

  float acc[P][kMats];
#pragma unroll
  for (int t = 0; t < P; ++t)
#pragma unroll
    for (int m = 0; m < kMats; ++m) acc[t][m] = 0.0f;

  bool healthy = true;
  int s = 0;
  std::uint32_t parity = 0;
  for (int j = 0; j < J; ++j) {
    if (healthy && !WarpAwait(&full[warp][s], parity, lane)) {
      healthy = false;
      if (lane == 0) atomicAdd(plan.faults, 1u);
    }
    // The next step travels while this one is summed (its stage was read a step ago).
    if (S > 1 && next < J) {
      FenceProxyAsync();
      request();
    }
    const int c = (j * PH) + ph;
    if (ph < PH && c < UR && r < my_rows) {
      const unsigned char* base = ring + (static_cast<std::size_t>(s) * plan.stage_bytes);
      const uint4* act_q[P];  // this column's first chunk, per token
#pragma unroll
      for (int t = 0; t < P; ++t) {
        act_q[t] = reinterpret_cast<const uint4*>(acts + (static_cast<std::size_t>(t) * plan.acts_bytes)) + c;
      }
#pragma unroll
      for (int m = 0; m < kMats; ++m) {
        Q4KBlockUnit raw;
        raw.LoadShared(base + ((static_cast<std::size_t>(m) * R + r) * plan.pitch), ph);
        int sc[8], mn[8];
        Q4KBlockScales(raw, sc, mn);
        float fmn[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) fmn[g] = static_cast<float>(mn[g]);
        float sumd[P], summ[P];
        int dots[P][8];
#pragma unroll
        for (int t = 0; t < P; ++t) sumd[t] = summ[t] = 0.0f;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const std::uint32_t words[8] = {raw.q[2 * cc].x,     raw.q[2 * cc].y,
                                          raw.q[2 * cc].z,     raw.q[2 * cc].w,
                                          raw.q[2 * cc + 1].x, raw.q[2 * cc + 1].y,
                                          raw.q[2 * cc + 1].z, raw.q[2 * cc + 1].w};
          std::uint32_t lo[8], hi[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            lo[i] = words[i] & 0x0f0f0f0fu;
            hi[i] = words[i] & 0xf0f0f0f0u;  // 16 * code: the factor is shifted out below
          }
#pragma unroll
          for (int t = 0; t < P; ++t) {
            const uint4* q = act_q[t] + ((4 * cc) * UR);
            const uint4 a0 = q[0], a1 = q[UR];
            const uint4 a2 = q[2 * UR], a3 = q[3 * UR];
            // Two short chains per sub-block instead of one of eight: integer
            // sums, so the grouping changes no bit.
            int d0 = 0, e0 = 0, d1 = 0, e1 = 0;
            d0 = Dp4aU8S8(lo[0], static_cast<int>(a0.x), d0);
            e0 = Dp4aU8S8(lo[4], static_cast<int>(a1.x), e0);
            d1 = Dp4aU8S8(hi[0], static_cast<int>(a2.x), d1);
            e1 = Dp4aU8S8(hi[4], static_cast<int>(a3.x), e1);
            d0 = Dp4aU8S8(lo[1], static_cast<int>(a0.y), d0);
            e0 = Dp4aU8S8(lo[5], static_cast<int>(a1.y), e0);
            d1 = Dp4aU8S8(hi[1], static_cast<int>(a2.y), d1);
            e1 = Dp4aU8S8(hi[5], static_cast<int>(a3.y), e1);
            d0 = Dp4aU8S8(lo[2], static_cast<int>(a0.z), d0);
            e0 = Dp4aU8S8(lo[6], static_cast<int>(a1.z), e0);
            d1 = Dp4aU8S8(hi[2], static_cast<int>(a2.z), d1);
            e1 = Dp4aU8S8(hi[6], static_cast<int>(a3.z), e1);
            d0 = Dp4aU8S8(lo[3], static_cast<int>(a0.w), d0);
            e0 = Dp4aU8S8(lo[7], static_cast<int>(a1.w), e0);
            d1 = Dp4aU8S8(hi[3], static_cast<int>(a2.w), d1);
            e1 = Dp4aU8S8(hi[7], static_cast<int>(a3.w), e1);
            dots[t][2 * cc] = d0 + e0;
            dots[t][(2 * cc) + 1] = (d1 + e1) >> 4;
          }
        }
        // d * sum_g d8_g * (sc_g * dot_g)  -  dmin * sum_g (d8_g * sum q_g) * m_g
#pragma unroll
        for (int t = 0; t < P; ++t) {
          const float4* scl = reinterpret_cast<const float4*>(act_q[t] + (16 * UR));
          const float4 dA = scl[0], dB = scl[UR], fA = scl[2 * UR], fB = scl[3 * UR];
          const float dd[8] = {dA.x, dA.y, dA.z, dA.w, dB.x, dB.y, dB.z, dB.w};
          const float ff[8] = {fA.x, fA.y, fA.z, fA.w, fB.x, fB.y, fB.z, fB.w};
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            sumd[t] = fmaf(dd[g], static_cast<float>(dots[t][g] * sc[g]), sumd[t]);
            summ[t] = fmaf(ff[g], fmn[g], summ[t]);
          }
        }
        const float d = HalfBitsToFloat(raw.head.x & 0xffffu);
        const float dmin = HalfBitsToFloat(raw.head.x >> 16);
#pragma unroll
        for (int t = 0; t < P; ++t) acc[t][m] += (d * sumd[t]) - (dmin * summ[t]);
      }
    }
    __syncwarp();
    if (S == 1 && next < J) {  // a one-stage ring: the stage just read takes the next step
      FenceProxyAsync();
      request();
    }
    if (++s == S) {
      s = 0;
      parity ^= 1u;
    }
  }

  // A stage that never arrived: nothing of this warp's rows is stored.
  if (!healthy) return;

  // The phases of a row meet in phase order: lane r adds lanes r + R, r + 2R, ...
#pragma unroll
  for (int t = 0; t < P; ++t) {
    float v[kMats];
#pragma unroll
    for (int m = 0; m < kMats; ++m) {
      v[m] = acc[t][m];
      for (int k = 1; k < PH; ++k) {
        v[m] += __shfl_sync(0xffffffffu, acc[t][m], (r + (k * R)) & 31);
      }
    }
    if (ph == 0 && r < my_rows && t < a.tokens) {
      float* dst = a.dst + (static_cast<std::size_t>(t) * a.dst_token) + row_begin + r;
      float result;
      if constexpr (kGlu) {
        result = Glu(a.glu, v[1], v[0], a.limit);
      } else {
        result = v[0];
      }
      *dst = result;
      if (plan.fan.world > 0 && t == 0) FanStore(plan.fan, FanTag(plan.fan), row_begin + r, result);
    }
  }

  // The output as Q8_1 blocks too: every warp counts its rows into the 32-row
  // blocks they fall in (at most two: R <= 32); the warp whose count completes a
  // block reads the block's 32 values back from L2 and quantizes them with the
  // Q8_1 quantizer's arithmetic (d = amax / 127 as FP16, q = roundf(x / d), the sum
  // a butterfly over indices 16, 8, 4, 2, 1 apart), so the blocks are the ones the
  // separate quantizer writes, bit for bit.  nrows is a multiple of 512 here, so
  // a token's row of blocks has no padding.
  if (plan.q8_dst != nullptr) {
    __threadfence();  // this warp's rows are visible before they are counted
    __syncwarp();
    const int row_blocks = a.nrows >> 5;
    const int b0 = row_begin >> 5, b1 = (row_end - 1) >> 5;
    const int t = lane >> 1;
    const int blk = (lane & 1) ? b1 : b0;
    bool mine = false;
    if (t < a.tokens && ((lane & 1) == 0 || b1 != b0)) {
      const int lo = max(row_begin, blk << 5), hi = min(row_end, (blk << 5) + 32);
      const unsigned int count = static_cast<unsigned int>(hi - lo);
      unsigned int* counter = plan.q8_rows_done + (static_cast<std::size_t>(t) * row_blocks) + blk;
      mine = atomicAdd(counter, count) + count == 32u;
      if (mine) *counter = 0u;  // as the next launch expects it
    }
    unsigned int done = __ballot_sync(0xffffffffu, mine);
    if (done != 0u) __threadfence();
    while (done != 0u) {
      const int src = __ffs(static_cast<int>(done)) - 1;
      done &= done - 1u;
      const int tt = src >> 1;
      const int bb = (src & 1) ? b1 : b0;
      const float x = __ldcg(a.dst + (static_cast<std::size_t>(tt) * a.dst_token) + (bb << 5) + lane);
      float amax = fabsf(x), sum = x;
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
        sum = sum + __shfl_xor_sync(0xffffffffu, sum, offset);
      }
      const float df = amax / 127.0f;
      const int q = amax != 0.0f ? static_cast<int>(roundf(x / df)) : 0;
      std::uint8_t* out = plan.q8_dst + ((static_cast<std::size_t>(tt) * row_blocks + bb) * 36);
      reinterpret_cast<signed char*>(out + 4)[lane] = static_cast<signed char>(q);
      if (lane == 0) {
        *reinterpret_cast<std::uint32_t*>(out) =
            static_cast<std::uint32_t>(__half_as_ushort(__float2half_rn(df))) |
            (static_cast<std::uint32_t>(__half_as_ushort(__float2half_rn(sum))) << 16);
      }
    }
  }
}

// Host: the geometry for a dense Q4_K product, or false if it does not fit.
inline bool PlanRowLane(const Desc& d, int p, int sms, int force_rows, bool half,
                        RowLanePlan* plan, int force_phases = 0) {
  const int mats = d.glu != LLMP_B200_GLU_NONE ? 2 : 1;
  const int ur = d.ncols_x / 256;
  if (ur < 1) return false;
  const int grid = std::max(1, std::min(sms, d.nrows));
  const int cta_rows = (d.nrows + grid - 1) / grid;
  const int acts_bytes = (ur * 256) + (ur * 64);
  const int budget = (half ? 110 : 220) * 1024 - (p * acts_bytes) - 1024;
  const int max_warps = half ? kRowLaneHalfWarps : kRowLaneMaxWarps;
  if (budget <= 0) return false;
  double best_score = -1.0;
  RowLanePlan best{};
  for (int rows = 1; rows <= 32; ++rows) {
    if (force_rows > 0 && rows != force_rows) continue;
    const int warps = (cta_rows + rows - 1) / rows;
    if (warps < 1 || warps > max_warps) continue;
    for (int phases = 1; phases <= 32 / rows; ++phases) {
    if (force_phases > 0 && phases != force_phases) continue;
    const int steps = (ur + phases - 1) / phases;
    // The pitch between a stage's rows: the pad (in 16-byte units) that leaves the
    // fewest quarter-warp bank-group collisions for 128-bit loads, lane (r, ph)
    // reading at r * pitch + ph * 144.
    int pitch16 = phases * 9;
    {
      int best_pad = 0, best_hits = 1 << 30;
      for (int pad = 0; pad < 8; ++pad) {
        int hits = 0;
        for (int q = 0; q < 4; ++q) {
          int seen[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int l = 8 * q; l < (8 * q) + 8; ++l) {
            if (l >= rows * phases) continue;
            const int bank = ((l % rows) * (pitch16 + pad) + (l / rows) * 9) % 8;
            hits += seen[bank]++;
          }
        }
        if (hits < best_hits) {
          best_hits = hits;
          best_pad = pad;
        }
      }
      pitch16 += best_pad;
    }
    const int pitch = pitch16 * 16;
    const int stage_bytes = rows * pitch * mats;
    int stages = std::min({steps, kRowLaneMaxStages, budget / (warps * stage_bytes)});
    if (stages < 1) continue;
    // (a forced geometry may run on a one-stage ring: slower, but the sums keep their order)
    if (stages < steps && stages < 2 && force_phases == 0) continue;
    // Lane utilization, with a preference for more warps and for a ring that
    // holds the whole range.
    // (all 32 lanes of every warp count: lanes past R * PH idle)
    const double lanes = static_cast<double>(cta_rows) * ur /
                         (static_cast<double>(warps) * 32 * steps);
    const double score = lanes * (0.6 + 0.4 * std::min(1.0, warps / 8.0)) *
                         (0.7 + 0.3 * static_cast<double>(stages) / steps);
    if (score > best_score) {
      best_score = score;
      best.warps = warps;
      best.rows = rows;
      best.phases = phases;
      best.columns = ur;
      best.steps = steps;
      best.stages = stages;
      best.pitch = pitch;
      best.stage_bytes = stage_bytes;
      best.acts_bytes = acts_bytes;
      best.smem_bytes = (p * acts_bytes) + (warps * stages * stage_bytes);
      best.grid = grid;
      best.half = half ? 1 : 0;
      best.score = score;
      best.f32_input = 0;
      best.q8_row_blocks = 0;
      best.q8_out = nullptr;
      best.q8_dst = nullptr;
      best.q8_rows_done = nullptr;
    }
    }
  }
  if (best_score < 0.0) return false;
  best.faults = FaultCounter();
  if (best.faults == nullptr) return false;
  best.split = MakeRowSplit(d.nrows, best.grid, best.warps);
  best.phase_reciprocal = (65536 + best.rows - 1) / best.rows;
  *plan = best;
  return true;
}

template <int P, bool kGlu, bool kHalf>
cudaError_t LaunchRowLaneOne(const Desc& d, const RowLanePlan& plan, cudaStream_t stream) {
  auto* kernel = VecQRowLaneKernel<P, kGlu, kHalf>;
  // Once a device (and host thread): the most any plan asks for.
  static thread_local int configured_device = -1;
  int device = -1;
  cudaGetDevice(&device);
  if (configured_device != device) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (kHalf ? 110 : 220) * 1024);
    if (e != cudaSuccess) return e;
    configured_device = device;
  }
  return LaunchPdl(kernel, dim3(static_cast<unsigned>(plan.grid)),
                   dim3(static_cast<unsigned>(plan.warps * 32)),
                   static_cast<std::size_t>(plan.smem_bytes), stream, d, plan);
}

cudaError_t LaunchRowLane(const Desc& d, int p, const RowLanePlan& plan, cudaStream_t stream);

}  // namespace vecq
}  // namespace llmp_b200

#endif  // LLMP_B200_CSRC_VECQ_ROWLANE_CUH_
