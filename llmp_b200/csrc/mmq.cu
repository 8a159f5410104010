// MMQ on B200: the prefill product of Q4_K weights with Q8_1-MMQ activations,
// dense or per routed expert.  Semantics follow the reference's use of GGML's
// mul_mat_q (src/kernels/ggml/mul_mat_q.cu:67-130, 453-462, 551-737; the tile
// loop's shape in-tree at mul_mat_q_glu.cu:93-135; the activation block's
// writer at mul_mat_q_glu.cu:170-218): per 32-value group an exact int32
// product C = sum code * q, then in F32
//     sum += (d * sc)_half * d8 * C;   sum += (-dmin * m)_half * s8
// with d8, s8 the group's FP16 scale and stored input sum.
//
// The int8 contraction runs on tcgen05 (kind::i8, int32 accumulators in TMEM).
// Q4_K's per-group scales forbid accumulating across groups in the tensor
// core, so every 128x128x32 MMA lands in its own TMEM buffer (three of them, so
// the tensor core runs ahead) and a wide epilogue (16 warps) folds each group's
// int32 tile into F32 register accumulators: acc += ((d*sc) * C) * d8.  That
// fold is CUDA-core work per output element per group, fed by one shared-memory
// word (d8) per element, and bounds the kernel.  The min terms need no integer
// product: sum over groups of (-dmin*m)_half * s8_half is a plain FP16
// contraction over K = k / 32, which the tensor core takes (kind::f16, F32
// accumulate, a fourth TMEM buffer) from two small K-major FP16 tiles that the
// decode warps fill; the epilogue adds that buffer once at the end.
//
//   warp 0       TMA: per k-step the activation int8 tile (128 tokens x 128 K
//                bytes) straight out of the [k/128][col] block array through a
//                3-D tensor map (row pitch 144 B, origin past the 16-byte block
//                header) into the 128-byte-swizzled layout the MMA reads; per
//                super-block column (two k-steps) the 128 weight rows' raw
//                Q4_K blocks and the tokens' block headers into a raw stage;
//   warps 1-2    decode, two weight rows a thread, from the raw stage: unpack
//                the k-step's 128 nibbles to int8 into the swizzled K-major
//                tile, the four groups' d*sc as F32 and -dmin*m as FP16, the
//                tokens' d8 (F32) and s8 (FP16);
//   warp 3       allocates TMEM and issues the MMAs;
//   warps 4-19   epilogue: thread = (weight row, a quarter of the token
//                columns): loads its 32 columns, hands the buffer back to the
//                tensor core at once, then folds.
// Rows past the matrix and tokens past the batch are TMA's zero fill.
// Measured on M 4096, K 4096, N 14336 (TOP/s): min terms folded on CUDA cores
// and the decode warps fetching weights with uncoalesced global loads 122-173;
// min terms on the tensor core and TMA-fed decode 229; every lane polling its
// barrier (no shuffle) 245; 16 epilogue warps of 32 columns 267; the fold in
// packed F32x2 arithmetic 270.  With the
// epilogue only handing buffers back the kernel runs at 425, with the tensor
// core free-running at 555: one tcgen05.commit per 32-value group costs about
// 335 cycles of tensor-pipe time whatever else happens.  Replacing the
// integer-to-float conversion by an integer add onto a magic exponent measured slower (242).
// Every wait is bounded; a wait that runs out raises the device fault counter.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "mmq.cuh"
#include "tc.cuh"

namespace llmp_b200 {
namespace {

using Desc = llmp_b200_mmq_desc;

// ------------------------------------------------------------------ quantizer
// block_q8_1_mmq, DS4 layout: 4 x (FP16 d, FP16 sum of the inputs), 128 int8.
// Blocks ordered [k / 128][col].  Eight lanes a 32-value group, four values a
// lane; the sum is taken four-per-lane then over the lanes 4, 2, 1 apart.
template <bool kBf16>
__global__ void __launch_bounds__(256)
QuantizeMmqKernel(const void* __restrict__ x, std::int64_t row_stride, int k, std::int64_t cols,
                  const std::int32_t* __restrict__ ids_src, std::uint8_t* __restrict__ out,
                  std::int64_t lanes_total) {
  GridLaunchDependents();
  GridDependencyWait();
  const std::int64_t i = (static_cast<std::int64_t>(blockIdx.x) * 256) + threadIdx.x;
  const bool live = i < lanes_total;
  const std::int64_t group = (live ? i : 0) / 8;  // (col, k / 32)
  const int part = static_cast<int>(i % 8);
  const int groups = k / 32;
  const std::int64_t col = group / groups;
  const int g = static_cast<int>(group % groups);
  float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (live) {
    const std::int64_t src_row = ids_src != nullptr ? ids_src[col] : col;
    const std::int64_t at = (src_row * row_stride) + (g * 32) + (part * 4);
    if constexpr (kBf16) {
      const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(x) + at);
      v[0] = __uint_as_float(raw.x << 16);
      v[1] = __uint_as_float(raw.x & 0xffff0000u);
      v[2] = __uint_as_float(raw.y << 16);
      v[3] = __uint_as_float(raw.y & 0xffff0000u);
    } else {
      const float4 f = *reinterpret_cast<const float4*>(static_cast<const float*>(x) + at);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    }
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  float sum = ((v[0] + v[1]) + v[2]) + v[3];
#pragma unroll
  for (int offset = 4; offset > 0; offset >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
    sum = sum + __shfl_xor_sync(0xffffffffu, sum, offset);
  }
  if (!live) return;
  std::uint32_t packed = 0;
  float d = 0.0f;
  if (amax > 0.0f) {
    const float d_inv = 127.0f / amax;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int q = static_cast<int>(roundf(v[c] * d_inv));
      packed |= (static_cast<std::uint32_t>(q) & 0xffu) << (8 * c);
    }
    d = 1.0f / d_inv;
  }
  std::uint8_t* block = out + ((static_cast<std::int64_t>(g / 4) * cols + col) * 144);
  *reinterpret_cast<std::uint32_t*>(block + 16 + ((g % 4) * 32) + (part * 4)) = packed;
  if (part == 0) {
    const std::uint32_t ds = static_cast<std::uint32_t>(__half_as_ushort(__float2half_rn(d))) |
                             (static_cast<std::uint32_t>(__half_as_ushort(__float2half_rn(sum)))
                              << 16);
    *reinterpret_cast<std::uint32_t*>(block + ((g % 4) * 4)) = ds;
  }
}

// ------------------------------------------------------------------ GEMM
constexpr int kTileRows = 128;  // weight rows: the MMA's M, one TMEM lane each
constexpr int kTileCols = 128;  // tokens: the MMA's N
constexpr int kBK = 128;        // K bytes a stage: four 32-value groups
constexpr int kStages = 3;
constexpr int kBuffers = 3;     // TMEM group-result buffers of kTileCols columns
constexpr int kMinColumn = kBuffers * kTileCols;  // TMEM: the F32 sum of the min terms
constexpr int kWBytes = kTileRows * kBK, kYBytes = kTileCols * kBK;
constexpr int kScaleBytes = 4 * 128 * 4;  // [group][row or col] F32
constexpr int kStageBytes = kWBytes + kYBytes + (2 * kScaleBytes);
// The min terms' operands: FP16 [128 rows][64 groups] K-major, 128-byte swizzled
// like the int8 tiles; one tile holds 16 k-steps, two tiles alternate.
constexpr int kMinTileBytes = 128 * 128;
constexpr int kMinSteps = 16;  // k-steps a tile of min operands covers
// Raw stages: what TMA brings for one super-block column (two k-steps): the 128
// weight rows' Q4_K blocks, then the 128 tokens' block headers of both k-steps.
constexpr int kRawStages = 2;
constexpr int kRawWBytes = 128 * 144;
constexpr int kRawHBytes = 128 * 16;
constexpr int kRawBytes = kRawWBytes + (2 * kRawHBytes);
constexpr int kEpilogueWarps = 16;
constexpr int kDecodeWarps = 2;  // warps 1 .. kDecodeWarps
constexpr int kMmaWarp = kDecodeWarps + 1;
constexpr int kFirstEpilogueWarp = kDecodeWarps + 2;  // a multiple of 4: warp % 4 is its TMEM quadrant
constexpr int kThreads = (kFirstEpilogueWarp + kEpilogueWarps) * 32;
static_assert(kFirstEpilogueWarp % 4 == 0, "epilogue warp e must sit in TMEM quadrant e % 4");
constexpr int kEpilogueCols = kTileCols / (kEpilogueWarps / 4);  // columns a thread
constexpr int kChunk = 32;                                       // columns a TMEM load
constexpr int kChunks = kEpilogueCols / kChunk;
constexpr int kSmem =
    (kStages * kStageBytes) + (4 * kMinTileBytes) + (kRawStages * kRawBytes) + 1024 + 512;

// Two F32 lanes in one 64-bit register: sm_100's packed F32 arithmetic does two
// roundings-to-nearest per instruction, the same results as two scalar ones.
__device__ __forceinline__ std::uint64_t Pack2(float lo, float hi) {
  std::uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void Unpack2(std::uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ std::uint64_t Mul2(std::uint64_t a, std::uint64_t b) {
  std::uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ std::uint64_t Fma2(std::uint64_t a, std::uint64_t b, std::uint64_t c) {
  std::uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

struct Shared {
  std::uint64_t y_full[kStages];
  std::uint64_t w_full[kStages];
  std::uint64_t empty[kStages];
  std::uint64_t tmem_full[kBuffers];
  std::uint64_t tmem_empty[kBuffers];
  std::uint64_t raw_full[kRawStages];
  std::uint64_t raw_empty[kRawStages];
  std::uint64_t min_free[2];  // the tensor core has read a tile of min operands
  std::uint64_t min_full;     // the min terms' sum is complete in tensor memory
  std::uint32_t tmem_base;
  std::uint32_t abort;
};

__global__ void __launch_bounds__(kThreads, 1)
MmqQ4KKernel(const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_w,
             const __grid_constant__ CUtensorMap map_h, const Desc a,
             const std::int32_t* __restrict__ worklist, unsigned int* faults) {
  extern __shared__ unsigned char raw_smem[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<std::uintptr_t>(raw_smem) + 1023) & ~static_cast<std::uintptr_t>(1023));
  unsigned char* w_tiles = smem;
  unsigned char* y_tiles = w_tiles + (kStages * kWBytes);
  unsigned char* min_w = y_tiles + (kStages * kYBytes);  // [2] tiles: (-dmin * m) per weight row
  unsigned char* min_y = min_w + (2 * kMinTileBytes);    // [2] tiles: s8 per token
  unsigned char* raw = min_y + (2 * kMinTileBytes);      // [kRawStages] raw stages
  float* scales = reinterpret_cast<float*>(raw + (kRawStages * kRawBytes));
  Shared* sh = reinterpret_cast<Shared*>(reinterpret_cast<unsigned char*>(scales) +
                                         (kStages * 2 * kScaleBytes));
  // scales of stage s: ax[4][128] (weight rows, d * sc), bx[4][128] (tokens, d8)
  auto stage_scales = [&](int s) { return scales + (static_cast<std::size_t>(s) * 2 * 512); };

  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int ksteps = a.k / kBK;

  // The tile: weight rows [row0, row0 + 128) of expert e against sorted
  // columns [col0, col0 + 128) of that expert's range [c_begin, c_end).
  // With a worklist (built on the device from the expert bounds) grid row y
  // names entry y: {expert, first column}; entry 0 holds the entry count.
  int expert = static_cast<int>(blockIdx.z);
  int col0;
  if (worklist != nullptr) {
    if (static_cast<int>(blockIdx.y) >= worklist[0]) return;
    expert = worklist[1 + (2 * blockIdx.y)];
    col0 = worklist[2 + (2 * blockIdx.y)];
  } else {
    const int c_begin = a.expert_bounds != nullptr ? a.expert_bounds[expert] : 0;
    col0 = c_begin + (static_cast<int>(blockIdx.y) * kTileCols);
  }
  const int c_end = a.expert_bounds != nullptr ? a.expert_bounds[expert + 1] : a.ncols;
  const int row0 = static_cast<int>(blockIdx.x) * kTileRows;
  if (col0 >= c_end) return;  // uniform for the CTA, before any barrier

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::MbarInit(&sh->y_full[s], 1);
      tc::MbarInit(&sh->w_full[s], kDecodeWarps);
      tc::MbarInit(&sh->empty[s], kEpilogueWarps);
    }
    for (int b = 0; b < kBuffers; ++b) {
      tc::MbarInit(&sh->tmem_full[b], 1);
      tc::MbarInit(&sh->tmem_empty[b], kEpilogueWarps);
    }
    for (int r = 0; r < kRawStages; ++r) {
      tc::MbarInit(&sh->raw_full[r], 1);
      tc::MbarInit(&sh->raw_empty[r], kDecodeWarps);
    }
    tc::MbarInit(&sh->min_free[0], 1);
    tc::MbarInit(&sh->min_free[1], 1);
    tc::MbarInit(&sh->min_full, 1);
    sh->abort = 0;
    tc::MbarInitFence();
  }
  if (warp == kMmaWarp) {
    tc::TmemAlloc(&sh->tmem_base, 512);
    tc::TmemRelinquish();
  }
  tc::TcFenceBefore();
  __syncthreads();
  tc::TcFenceAfter();
  const std::uint32_t tmem = sh->tmem_base;
  volatile std::uint32_t* abort_flag = &sh->abort;
  auto give_up = [&]() {
    *abort_flag = 1;
    atomicAdd(faults, 1u);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tc::PrefetchMap(&map_y);
      tc::PrefetchMap(&map_w);
      tc::PrefetchMap(&map_h);
      for (int ks = 0; ks < ksteps && !*abort_flag; ++ks) {
        if ((ks & 1) == 0) {
          // One super-block column (k-steps ks, ks + 1): the weight rows' blocks and
          // the tokens' block headers, for the decode warps.
          const int column = ks >> 1;
          const int rs = column % kRawStages;
          if (!tc::MbarWaitSleep(&sh->raw_empty[rs], ((column / kRawStages) & 1) ^ 1, 128)) {
            give_up();
            break;
          }
          unsigned char* stage = raw + (rs * kRawBytes);
          tc::MbarExpectTx(&sh->raw_full[rs], kRawBytes);
          asm volatile(
              "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
              " [%0], [%1, {%3, %4, %5}], [%2];"
              ::"r"(tc::Smem(stage)), "l"(&map_w), "r"(tc::Smem(&sh->raw_full[rs])),
                "r"(column * 144), "r"(row0), "r"(expert)
              : "memory");
          asm volatile(
              "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
              " [%0], [%1, {%3, %4, %5}], [%2];"
              ::"r"(tc::Smem(stage + kRawWBytes)), "l"(&map_h), "r"(tc::Smem(&sh->raw_full[rs])),
                "r"(0), "r"(col0), "r"(ks)
              : "memory");
        }
        const int s = ks % kStages;
        if (!tc::MbarWaitSleep(&sh->empty[s], ((ks / kStages) & 1) ^ 1, 256)) {
          give_up();
          break;
        }
        tc::MbarExpectTx(&sh->y_full[s], kYBytes);
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(tc::Smem(y_tiles + (s * kYBytes))), "l"(&map_y), "r"(tc::Smem(&sh->y_full[s])),
              "r"(0), "r"(col0), "r"(ks)
            : "memory");
      }
    }
  } else if (warp >= 1 && warp <= kDecodeWarps) {
    // ------------------------------------------------------------ decode
    const int t0 = (static_cast<int>(threadIdx.x) - 32);  // first weight row / token of this thread
    // Rows past the matrix and tokens past the batch arrive as zero blocks (TMA's
    // fill): zero scales, zero codes, nothing stored for them.
    for (int ks = 0; ks < ksteps && !*abort_flag; ++ks) {
      const int s = ks % kStages;
      const int half = ks & 1;
      const int column = ks >> 1;
      const int rs = column % kRawStages;
      const int mt = (ks / kMinSteps) & 1;  // the tile of min operands this k-step writes into
      bool ok = true;
      if (lane == 0) {
        if (half == 0) ok = tc::MbarWait(&sh->raw_full[rs], (column / kRawStages) & 1);
        ok = ok && tc::MbarWaitSleep(&sh->empty[s], ((ks / kStages) & 1) ^ 1, 64);
        // ... and the tensor core is done with the min tile's contents of 32 k-steps ago
        if (ks >= 2 * kMinSteps && ks % kMinSteps == 0) {
          ok = ok && tc::MbarWait(&sh->min_free[mt], ((ks / (2 * kMinSteps)) - 1) & 1);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) {
        if (lane == 0) give_up();
        break;
      }
      const unsigned char* stage = raw + (rs * kRawBytes);
      float* sc = stage_scales(s);
#pragma unroll  // the rows of a thread are independent: their latencies overlap
      for (int t = t0; t < kTileRows; t += kDecodeWarps * 32) {
        const unsigned char* sb = stage + (t * 144);
        const uint4 head = *reinterpret_cast<const uint4*>(sb);
        uint4 q[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          q[i] = *reinterpret_cast<const uint4*>(sb + 16 + (half * 64) + (i * 16));
        }
        const uint4 ds =
            *reinterpret_cast<const uint4*>(stage + kRawWBytes + (half * kRawHBytes) + (t * 16));
        // int8 codes into the swizzled K-major tile: row t, 16-byte chunk j at j ^ (t % 8)
        unsigned char* wt = w_tiles + (s * kWBytes) + ((t >> 3) * 1024) + ((t & 7) * 128);
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const uint4 lo0 = make_uint4(q[2 * cc].x & 0x0f0f0f0fu, q[2 * cc].y & 0x0f0f0f0fu,
                                       q[2 * cc].z & 0x0f0f0f0fu, q[2 * cc].w & 0x0f0f0f0fu);
          const uint4 lo1 = make_uint4(q[2 * cc + 1].x & 0x0f0f0f0fu, q[2 * cc + 1].y & 0x0f0f0f0fu,
                                       q[2 * cc + 1].z & 0x0f0f0f0fu, q[2 * cc + 1].w & 0x0f0f0f0fu);
          const uint4 hi0 = make_uint4((q[2 * cc].x >> 4) & 0x0f0f0f0fu, (q[2 * cc].y >> 4) & 0x0f0f0f0fu,
                                       (q[2 * cc].z >> 4) & 0x0f0f0f0fu, (q[2 * cc].w >> 4) & 0x0f0f0f0fu);
          const uint4 hi1 = make_uint4((q[2 * cc + 1].x >> 4) & 0x0f0f0f0fu, (q[2 * cc + 1].y >> 4) & 0x0f0f0f0fu,
                                       (q[2 * cc + 1].z >> 4) & 0x0f0f0f0fu, (q[2 * cc + 1].w >> 4) & 0x0f0f0f0fu);
          const int j = cc * 4;  // groups 2cc (chunks j, j+1) and 2cc+1 (chunks j+2, j+3)
          *reinterpret_cast<uint4*>(wt + (((j + 0) ^ (t & 7)) * 16)) = lo0;
          *reinterpret_cast<uint4*>(wt + (((j + 1) ^ (t & 7)) * 16)) = lo1;
          *reinterpret_cast<uint4*>(wt + (((j + 2) ^ (t & 7)) * 16)) = hi0;
          *reinterpret_cast<uint4*>(wt + (((j + 3) ^ (t & 7)) * 16)) = hi1;
        }
        // The four groups' half products (d * sc, -dmin * m): GGML's tile loader
        // multiplies in half precision.
        const std::uint32_t s0 = head.y, s1 = head.z, s2 = head.w;
        const __half d = __ushort_as_half(static_cast<unsigned short>(head.x & 0xffffu));
        const __half dmin = __hneg(__ushort_as_half(static_cast<unsigned short>(head.x >> 16)));
        std::uint32_t mins[4];
#pragma unroll
        for (int gl = 0; gl < 4; ++gl) {
          int scv, mnv;
          if (half == 0) {
            scv = static_cast<int>((s0 >> (8 * gl)) & 63u);
            mnv = static_cast<int>((s1 >> (8 * gl)) & 63u);
          } else {
            scv = static_cast<int>(((s2 >> (8 * gl)) & 15u) | (((s0 >> ((8 * gl) + 6)) & 3u) << 4));
            mnv = static_cast<int>(((s2 >> ((8 * gl) + 4)) & 15u) | (((s1 >> ((8 * gl) + 6)) & 3u) << 4));
          }
          sc[(gl * 128) + t] = __half2float(__hmul(d, __int2half_rn(scv)));
          mins[gl] = __half_as_ushort(__hmul(dmin, __int2half_rn(mnv)));
        }
        const std::uint32_t dsw[4] = {ds.x, ds.y, ds.z, ds.w};
#pragma unroll
        for (int gl = 0; gl < 4; ++gl) sc[512 + (gl * 128) + t] = HalfBitsToFloat(dsw[gl] & 0xffffu);
        // Row t of both min tiles, the four halves of this k-step: byte (ks % 16) * 8
        // of the 128-byte row, 16-byte chunks swizzled like the int8 tiles.
        const int kk = ks % kMinSteps;
        const int at = ((t >> 3) * 1024) + ((t & 7) * 128) + ((((kk >> 1) ^ (t & 7))) * 16) +
                       ((kk & 1) * 8);
        *reinterpret_cast<uint2*>(min_w + (mt * kMinTileBytes) + at) =
            make_uint2(mins[0] | (mins[1] << 16), mins[2] | (mins[3] << 16));
        *reinterpret_cast<uint2*>(min_y + (mt * kMinTileBytes) + at) =
            make_uint2((dsw[0] >> 16) | (dsw[1] & 0xffff0000u), (dsw[2] >> 16) | (dsw[3] & 0xffff0000u));
        // The last FP16 MMA reads 16 groups: zero what the k range leaves unwritten.
        if (ks == ksteps - 1) {
          for (int pad = ks + 1; pad % 4 != 0; ++pad) {
            const int pk = pad % kMinSteps;
            const int pat = ((t >> 3) * 1024) + ((t & 7) * 128) + ((((pk >> 1) ^ (t & 7))) * 16) +
                            ((pk & 1) * 8);
            *reinterpret_cast<uint2*>(min_w + (mt * kMinTileBytes) + pat) = make_uint2(0u, 0u);
            *reinterpret_cast<uint2*>(min_y + (mt * kMinTileBytes) + pat) = make_uint2(0u, 0u);
          }
        }
      }
      tc::FenceProxyAsync();  // generic-proxy writes, read by the tensor core's proxy
      __syncwarp();
      if (lane == 0) {
        if (half == 1) tc::MbarArrive(&sh->raw_empty[rs]);  // all of the raw stage is read
        tc::MbarArrive(&sh->w_full[s]);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const std::uint32_t idesc = tc::IdescI8(kTileRows, kTileCols, false, true);
      std::uint32_t group = 0;
      for (int ks = 0; ks < ksteps && !*abort_flag; ++ks) {
        const int s = ks % kStages;
        {
          const bool w_ok = tc::MbarWait(&sh->w_full[s], (ks / kStages) & 1);
          if (!w_ok) {
            give_up();
            break;
          }
        }
        {
          const bool y_ok = tc::MbarWait(&sh->y_full[s], (ks / kStages) & 1);
          if (!y_ok) {
            give_up();
            break;
          }
        }
        tc::TcFenceAfter();
        const std::uint64_t wdesc = tc::SmemDesc(w_tiles + (s * kWBytes), true, 1024);
        const std::uint64_t ydesc = tc::SmemDesc(y_tiles + (s * kYBytes), true, 1024);
        for (int gl = 0; gl < 4; ++gl, ++group) {
          const int b = static_cast<int>(group % kBuffers);
          if (!tc::MbarWait(&sh->tmem_empty[b], ((group / kBuffers) & 1u) ^ 1u)) {
            give_up();
            break;
          }
          tc::TcFenceAfter();
          tc::MmaI8(tmem + (b * kTileCols), wdesc + (gl * 2), ydesc + (gl * 2), idesc, false);
          tc::TcCommit(&sh->tmem_full[b]);
        }
        // Every fourth k-step completes 16 groups of min operands: one FP16 MMA
        // (K 16) adds their products to the F32 sum.
        if (ks % 4 == 3 || ks == ksteps - 1) {
          const int mt = (ks / kMinSteps) & 1;
          const int q = (ks % kMinSteps) / 4;  // 32 bytes along the swizzled row each
          tc::MmaF16(tmem + kMinColumn, tc::SmemDesc(min_w + (mt * kMinTileBytes), true, 1024) + (q * 2),
                     tc::SmemDesc(min_y + (mt * kMinTileBytes), true, 1024) + (q * 2),
                     tc::IdescF16(kTileRows, kTileCols), ks >= 4);
          if (ks % kMinSteps == kMinSteps - 1) tc::TcCommit(&sh->min_free[mt]);
          if (ks == ksteps - 1) tc::TcCommit(&sh->min_full);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int ew = warp - kFirstEpilogueWarp;
    const int quadrant = warp & 3;          // TMEM lanes this warp may touch
    const int colgroup = ew >> 2;           // which kEpilogueCols columns
    const int rt = (quadrant * 32) + lane;  // weight row of the tile
    const std::uint32_t lane_base = static_cast<std::uint32_t>(quadrant * 32) << 16;
    std::uint64_t acc2[kEpilogueCols / 2];  // columns 2i, 2i + 1
#pragma unroll
    for (int i = 0; i < kEpilogueCols / 2; ++i) acc2[i] = 0ull;
    bool ok = true;
    int bb = 0;                  // the group's TMEM buffer and its use's parity
    std::uint32_t parity = 0;
    for (int ks = 0; ks < ksteps && ok && !*abort_flag; ++ks) {
      const int s = ks % kStages;
      const float* sc = stage_scales(s);
#pragma unroll
      for (int gl = 0; gl < 4; ++gl) {
        if (!ok) break;
        ok = tc::MbarWait(&sh->tmem_full[bb], parity);  // every lane polls: no shuffle after
        if (!__all_sync(0xffffffffu, ok)) {
          if (lane == 0) give_up();
          ok = false;
          break;
        }
        tc::TcFenceAfter();
        const std::uint32_t at = tmem + lane_base + (bb * kTileCols) + (colgroup * kEpilogueCols);
        // All of the thread's columns at once, then the buffer goes straight back to
        // the tensor core: the fold below overlaps the next groups' MMAs.
        std::uint32_t r[kChunks][kChunk];
#pragma unroll
        for (int c = 0; c < kChunks; ++c) tc::TmemLoad32(at + (c * kChunk), r[c]);
        const float ax = sc[(gl * 128) + rt];
        const float* bx = sc + 512 + (gl * 128) + (colgroup * kEpilogueCols);
        tc::TmemLoadWait();
        tc::TcFenceBefore();
        __syncwarp();
        if (lane == 0) tc::MbarArrive(&sh->tmem_empty[bb]);
        const std::uint64_t ax2 = Pack2(ax, ax);
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
#pragma unroll
          for (int v = 0; v < kChunk / 4; ++v) {
            const float4 x4 = *reinterpret_cast<const float4*>(bx + (c * kChunk) + (v * 4));
            const float xs[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
              const int i = ((c * kChunk) + (v * 4) + j) / 2;
              // (ax * C) rounded, times d8, added: as the scalar sequence, two columns at once
              std::uint64_t u2;
              u2 = Mul2(Pack2(static_cast<float>(static_cast<int>(r[c][(v * 4) + j])),
                              static_cast<float>(static_cast<int>(r[c][(v * 4) + j + 1]))),
                        ax2);
              acc2[i] = Fma2(u2, Pack2(xs[j], xs[j + 1]), acc2[i]);
            }
          }
        }
        if (++bb == kBuffers) {
          bb = 0;
          parity ^= 1u;
        }
      }
      __syncwarp();
      if (lane == 0 && ok) tc::MbarArrive(&sh->empty[s]);  // the stage's scales are consumed
    }
    // The min terms: sum over the groups of (-dmin * m) * s8, taken by the tensor core.
    if (ok) {
      if (lane == 0) ok = tc::MbarWait(&sh->min_full, 0);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok && lane == 0) give_up();
    }
    float acc[kEpilogueCols];  // the min terms first, then plus the folded groups
    if (ok) {
      tc::TcFenceAfter();
      const std::uint32_t at = tmem + lane_base + kMinColumn + (colgroup * kEpilogueCols);
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        std::uint32_t r[kChunk];
        tc::TmemLoad32(at + (c * kChunk), r);
        tc::TmemLoadWait();
#pragma unroll
        for (int j = 0; j < kChunk; ++j) acc[(c * kChunk) + j] = __uint_as_float(r[j]);
      }
    }
#pragma unroll
    for (int i = 0; i < kEpilogueCols / 2; ++i) {
      float lo, hi;
      Unpack2(acc2[i], lo, hi);
      acc[2 * i] += lo;
      acc[(2 * i) + 1] += hi;
    }
    if (ok && row0 + rt < a.nrows) {
#pragma unroll  // fully: a dynamic index would put acc[] in local memory
      for (int i = 0; i < kEpilogueCols; ++i) {
        const int c = col0 + (colgroup * kEpilogueCols) + i;
        if (c < c_end) {
          const int dst_col = a.ids_dst != nullptr ? a.ids_dst[c] : c;
          a.dst[(static_cast<std::size_t>(dst_col) * a.dst_col_stride) + row0 + rt] = acc[i];
        }
      }
    }
  }

  tc::TcFenceBefore();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc::TcFenceAfter();
    tc::TmemDealloc(tmem, 512);
  }
}

int CheckDesc(const Desc& d) {
  if (d.type != LLMP_B200_TYPE_Q4_K) {
    return Reject("mmq: weight type %d is not one this build computes (Q4_K)", d.type);
  }
  if (d.w == nullptr || d.y == nullptr || d.dst == nullptr || d.k < 256 || d.k % 256 != 0 ||
      d.nrows < 1 || d.ncols < 1) {
    return Reject("mmq: Q4_K weights [k, n], Q8_1-MMQ activations of ncols columns, an F32 output; "
                  "k a positive multiple of 256");
  }
  if (d.stride_row < d.k / 256 || d.stride_expert < 0 || d.dst_col_stride < d.nrows) {
    return Reject("mmq: strides must cover a row");
  }
  if (!Aligned(d.w, 16) || !Aligned(d.y, 16) || !Aligned(d.dst, 4)) {
    return Reject("mmq: weights and activation blocks 16-byte aligned");
  }
  if (d.expert_bounds == nullptr && d.experts > 1) {
    return Reject("mmq: expert bounds exactly with experts");
  }
  if (d.expert_bounds != nullptr && (d.experts < 1 || d.experts > 65535)) {
    return Reject("mmq: 1 to 65535 experts");
  }
  return 0;
}

}  // namespace

int LaunchMmq(const llmp_b200_mmq_desc& d, const std::int32_t* worklist, int max_tiles,
              void* stream) {
  if (const int status = CheckDesc(d); status != 0) return status;
  if (const int status = DeviceStatus(); status != 0) return status;
  const tc::EncodeTiledFn encode = tc::EncodeTiled();
  if (encode == nullptr) return Reject("mmq: the driver has no tensor-map encoder");
  CUtensorMap map_y;
  {
    const cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(d.ncols),
                                static_cast<cuuint64_t>(d.k / 128)};
    const cuuint64_t strides[2] = {144, static_cast<cuuint64_t>(d.ncols) * 144};
    const cuuint32_t box[3] = {128, kTileCols, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    void* base = const_cast<std::uint8_t*>(static_cast<const std::uint8_t*>(d.y) + 16);
    if (encode(&map_y, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, base, dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      return Reject("mmq: the driver refused a tensor map for the activation blocks");
    }
  }
  // The weights as bytes [expert][row][k / 256 * 144]: a box is one block of 128 rows.
  CUtensorMap map_w;
  {
    const int experts = d.expert_bounds != nullptr ? d.experts : 1;
    const cuuint64_t row_pitch = static_cast<cuuint64_t>(d.stride_row) * 144;
    const cuuint64_t expert_pitch =
        experts > 1 ? static_cast<cuuint64_t>(d.stride_expert) * 144
                    : row_pitch * static_cast<cuuint64_t>(d.nrows);
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(d.k / 256) * 144,
                                static_cast<cuuint64_t>(d.nrows), static_cast<cuuint64_t>(experts)};
    const cuuint64_t strides[2] = {row_pitch, expert_pitch};
    const cuuint32_t box[3] = {144, kTileRows, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    if (encode(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(d.w), dims, strides,
               box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      return Reject("mmq: the driver refused a tensor map for the weight blocks");
    }
  }
  // The activation blocks' 16-byte headers [k / 128][col]: a box is 128 tokens, two k-steps.
  CUtensorMap map_h;
  {
    const cuuint64_t dims[3] = {16, static_cast<cuuint64_t>(d.ncols),
                                static_cast<cuuint64_t>(d.k / 128)};
    const cuuint64_t strides[2] = {144, static_cast<cuuint64_t>(d.ncols) * 144};
    const cuuint32_t box[3] = {16, kTileCols, 2};
    const cuuint32_t elem[3] = {1, 1, 1};
    if (encode(&map_h, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(d.y), dims, strides,
               box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_NONE,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      return Reject("mmq: the driver refused a tensor map for the activation headers");
    }
  }
  unsigned int* faults = FaultCounter();
  if (faults == nullptr) return Reject("mmq: no fault counter on this device");
  static thread_local int configured_device = -1;
  int device = -1;
  cudaGetDevice(&device);
  if (configured_device != device) {
    const cudaError_t e =
        cudaFuncSetAttribute(MmqQ4KKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return Failed(e, "mmq attribute");
    configured_device = device;
  }
  dim3 grid(static_cast<unsigned>((d.nrows + kTileRows - 1) / kTileRows), 1, 1);
  if (worklist != nullptr) {
    if (max_tiles < 1) return Reject("mmq: a worklist needs its capacity");
    grid.y = static_cast<unsigned>(max_tiles);
  } else {
    const int experts = d.expert_bounds != nullptr ? d.experts : 1;
    const int max_cols = d.expert_bounds != nullptr ? d.max_cols_per_expert : d.ncols;
    if (max_cols < 1) return Reject("mmq: max_cols_per_expert >= 1 with experts");
    grid.y = static_cast<unsigned>((max_cols + kTileCols - 1) / kTileCols);
    grid.z = static_cast<unsigned>(experts);
  }
  if (grid.y > 65535u) return Reject("mmq: more column tiles than a grid holds");
  MmqQ4KKernel<<<grid, kThreads, kSmem, static_cast<cudaStream_t>(stream)>>>(map_y, map_w, map_h, d,
                                                                             worklist, faults);
  const cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return Failed(cudaGetLastError(), "mmq launch");
  return 0;
}

}  // namespace llmp_b200

extern "C" {

int64_t llmp_b200_mmq_q8_1_bytes(int64_t k, int64_t cols) { return (k / 128) * cols * 144; }

int llmp_b200_mmq_quantize(const void* x, int is_bf16, int64_t row_stride, int64_t k, int64_t cols,
                           const int32_t* ids_src, void* out, void* stream) {
  using namespace llmp_b200;
  if (x == nullptr || out == nullptr || k < 128 || k % 128 != 0 || cols < 1 || row_stride < k) {
    return Reject("mmq.quantize: [k, rows] input with k a positive multiple of 128, cols >= 1");
  }
  const int elem = is_bf16 ? 2 : 4;
  if (!Aligned(x, 16) || (row_stride * elem) % 16 != 0 || !Aligned(out, 16)) {
    return Reject("mmq.quantize: input rows and output 16-byte aligned");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  const std::int64_t lanes = cols * (k / 32) * 8;
  const std::int64_t grid = (lanes + 255) / 256;
  if (grid > 0x7fffffffLL) return Reject("mmq.quantize: more blocks than a grid holds");
  auto* s = static_cast<cudaStream_t>(stream);
  const cudaError_t e =
      is_bf16 ? LaunchPdl(QuantizeMmqKernel<true>, dim3(static_cast<unsigned>(grid)), dim3(256), 0,
                          s, x, row_stride, static_cast<int>(k), cols, ids_src,
                          static_cast<std::uint8_t*>(out), lanes)
              : LaunchPdl(QuantizeMmqKernel<false>, dim3(static_cast<unsigned>(grid)), dim3(256), 0,
                          s, x, row_stride, static_cast<int>(k), cols, ids_src,
                          static_cast<std::uint8_t*>(out), lanes);
  if (e != cudaSuccess) return Failed(e, "mmq.quantize launch");
  return 0;
}

size_t llmp_b200_mmq_scratch(const llmp_b200_mmq_desc* desc, int sms) {
  (void)desc;
  (void)sms;
  return 0;  // group results live in tensor memory; no stream-k fixup pass
}

int llmp_b200_mmq(const llmp_b200_mmq_desc* desc, int sms, void* stream) {
  (void)sms;
  if (desc == nullptr) return llmp_b200::Reject("mmq: null descriptor");
  return llmp_b200::LaunchMmq(*desc, nullptr, 0, stream);
}

}  // extern "C"
