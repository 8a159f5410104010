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
// core, so every 128 x 128 x 32 MMA lands in its own TMEM buffer (three of them,
// so the tensor core runs ahead) and a wide epilogue (16 warps) folds each
// group's int32 tile into F32 register accumulators: acc += ((d*sc) * C) * d8.
// The MMA's M side (the TMEM lanes) is the TOKENS and its N side (the TMEM
// columns) the weight rows: an epilogue thread is one token with 32 weight rows
// in registers, so the activation scale d8 is one scalar a thread and group,
// the weight scales d*sc are one broadcast 128-bit shared load per four
// elements, and a thread's results are 128 contiguous bytes of the output.
// The min terms need no integer product: sum over groups of (-dmin*m)_half *
// s8_half is a plain FP16 contraction over K = k / 32, which the tensor core
// takes (kind::f16, F32 accumulate, a fourth TMEM buffer) from two small K-major
// FP16 tiles; the epilogue adds that buffer once at the end.
//
// Weights reach the MMA in one of two ways.
//   * SLAB (llmp_b200_q4k_relayout once at load time, or per call into caller
//     scratch): the Q4_K blocks unpacked to what the tensor core reads, int8
//     codes K-major, (d*sc)_half as F32 in [k-step][group][row] tiles, (-dmin*m)
//     as FP16 K-major.  The producer warp brings all of it by TMA straight into
//     the swizzled tiles; nothing is decoded in the GEMM's critical path.
//   * RAW (no slab, no scratch): two decode warps unpack the Q4_K blocks of a
//     TMA-fed raw stage into the same tiles, k-step by k-step.
//
//   warp 0       TMA producer: per k-step the activation int8 tile (128 tokens x
//                128 K bytes) straight out of the [k/128][col] block array through
//                a 3-D tensor map (row pitch 144 B, origin past the 16-byte block
//                header) and, with a slab, the weight tile and its scales; per
//                two k-steps the tokens' block headers (and, raw, the weight
//                rows' Q4_K blocks) into a raw stage;
//   warps 1-2    the activation headers into d8 (F32) and s8 (FP16, the min
//                tile); raw mode: also the weight blocks into the int8 tile, the
//                four groups' d*sc and -dmin*m;
//   warp 3       allocates TMEM and issues the MMAs;
//   warps 4-19   epilogue: thread = (token, a quarter of the weight rows): loads
//                its 32 columns, hands the buffer back to the tensor core at
//                once, then folds.
// Rows past the matrix and tokens past the batch are TMA's zero fill.
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
  // (the index arithmetic runs beside the tail of the kernel before, not after it)
  const std::int64_t i = (static_cast<std::int64_t>(blockIdx.x) * 256) + threadIdx.x;
  const bool live = i < lanes_total;
  const std::int64_t group = (live ? i : 0) / 8;  // (col, k / 32)
  const int part = static_cast<int>(i % 8);
  const int groups = k / 32;
  const std::int64_t col = group / groups;
  const int g = static_cast<int>(group - (col * groups));
  GridDependencyWait();
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

// ------------------------------------------------------------------ slab
// The weights unpacked for the tensor core (llmp_b200_q4k_relayout).  Per expert:
//   codes  int8  [n][k]                      K-major rows, the MMA's B operand
//   ax     F32   [n / 128 up][k / 128][4][128]   (d * sc)_half of a tile's rows, a
//                                            k-step's four groups: 2 KB contiguous
//   mw     FP16  [n][G]                      (-dmin * m)_half, K-major; G = k / 32
//                                            rounded up to 64 (zero padding)
struct Slab {
  std::size_t codes, ax, mw, total;
  int row_tiles, ksteps, gpad;
};
Slab SlabOf(int n, int k, int experts) {
  Slab s;
  s.row_tiles = (n + 127) / 128;
  s.ksteps = k / 128;
  s.gpad = ((k / 32) + 63) / 64 * 64;
  const auto up = [](std::size_t v) { return (v + 255) / 256 * 256; };
  s.codes = 0;
  s.ax = up(static_cast<std::size_t>(experts) * n * k);
  s.mw = s.ax + up(static_cast<std::size_t>(experts) * s.row_tiles * s.ksteps * 512 * 4);
  s.total = s.mw + up(static_cast<std::size_t>(experts) * n * s.gpad * 2);
  return s;
}

__device__ __forceinline__ void ScaleAndMin(std::uint32_t s0, std::uint32_t s1, std::uint32_t s2,
                                            int g, int* sc, int* mn) {
  // 6-bit fields: groups 0..3 in the low six bits of bytes 0..3 (scales) and 4..7
  // (minima); groups 4..7 as the nibbles of bytes 8..11 with their top two bits in
  // bits 6..7 of bytes 0..3 / 4..7.
  const int gl = g & 3;
  if (g < 4) {
    *sc = static_cast<int>((s0 >> (8 * gl)) & 63u);
    *mn = static_cast<int>((s1 >> (8 * gl)) & 63u);
  } else {
    *sc = static_cast<int>(((s2 >> (8 * gl)) & 15u) | (((s0 >> ((8 * gl) + 6)) & 3u) << 4));
    *mn = static_cast<int>(((s2 >> ((8 * gl) + 4)) & 15u) | (((s1 >> ((8 * gl) + 6)) & 3u) << 4));
  }
}

// A warp takes 32 consecutive rows of one super-block column: lane = row, so the
// scale tiles are written 128 bytes a warp.
__global__ void __launch_bounds__(256)
RelayoutQ4KKernel(const std::uint8_t* __restrict__ w, int n, int k, std::int64_t stride_row,
                  std::int64_t stride_expert, int experts, std::uint8_t* __restrict__ slab,
                  const Slab layout, int glu_inter) {
  GridLaunchDependents();
  GridDependencyWait();  // the slab may still be read by the product queued before
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int sbs = k / 256;
  const int row_groups = layout.row_tiles * 4;  // 32-row groups an expert, padding included
  const std::int64_t item = (static_cast<std::int64_t>(blockIdx.x) * 8) + (threadIdx.x >> 5);
  if (item >= static_cast<std::int64_t>(experts) * row_groups * sbs) return;
  const int sb = static_cast<int>(item % sbs);
  const int rg = static_cast<int>((item / sbs) % row_groups);
  const int e = static_cast<int>(item / (static_cast<std::int64_t>(sbs) * row_groups));
  const int row = (rg * 32) + lane;
  const bool live = row < n;
  uint4 head = make_uint4(0, 0, 0, 0), q[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) q[i] = make_uint4(0, 0, 0, 0);
  // For the GLU write-back the slab's rows interleave the gate and up rows (the source holds
  // glu_inter gate rows, then as many up rows): slab rows 32g .. 32g + 15 are gate rows
  // 16g .. 16g + 15 and slab rows 32g + 16 .. 32g + 31 the up rows of the same outputs, so an
  // epilogue thread's 32 rows are 16 (gate, up) pairs.
  int from = row;
  if (glu_inter > 0) from = (lane < 16 ? 0 : glu_inter) + (rg * 16) + (lane & 15);
  if (live) {
    const auto* src = reinterpret_cast<const uint4*>(
        w + ((static_cast<std::int64_t>(e) * stride_expert + static_cast<std::int64_t>(from) * stride_row + sb) * 144));
    head = LoadStream16(src);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = LoadStream16(src + 1 + i);
  }
  const __half d = __ushort_as_half(static_cast<unsigned short>(head.x & 0xffffu));
  const __half dmin = __hneg(__ushort_as_half(static_cast<unsigned short>(head.x >> 16)));
  float* ax = reinterpret_cast<float*>(slab + layout.ax) +
              ((static_cast<std::int64_t>(e) * layout.row_tiles + (row >> 7)) * layout.ksteps * 512);
  std::uint32_t mins[4];
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    int scv, mnv;
    ScaleAndMin(head.y, head.z, head.w, g, &scv, &mnv);
    // the half-precision products of GGML's tile loader
    ax[((((2 * sb) + (g >> 2)) * 4 + (g & 3)) * 128) + (row & 127)] =
        live ? __half2float(__hmul(d, __int2half_rn(scv))) : 0.0f;
    const std::uint32_t bits = live ? __half_as_ushort(__hmul(dmin, __int2half_rn(mnv))) : 0u;
    if ((g & 1) == 0) {
      mins[g >> 1] = bits;
    } else {
      mins[g >> 1] |= bits << 16;
    }
  }
  if (!live) return;
  auto* codes = reinterpret_cast<uint4*>(
      slab + layout.codes + ((static_cast<std::int64_t>(e) * n + row) * k) + (static_cast<std::int64_t>(sb) * 256));
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint4 a = q[2 * c], b = q[(2 * c) + 1];
    codes[(4 * c) + 0] = make_uint4(a.x & 0x0f0f0f0fu, a.y & 0x0f0f0f0fu, a.z & 0x0f0f0f0fu, a.w & 0x0f0f0f0fu);
    codes[(4 * c) + 1] = make_uint4(b.x & 0x0f0f0f0fu, b.y & 0x0f0f0f0fu, b.z & 0x0f0f0f0fu, b.w & 0x0f0f0f0fu);
    codes[(4 * c) + 2] = make_uint4((a.x >> 4) & 0x0f0f0f0fu, (a.y >> 4) & 0x0f0f0f0fu,
                                    (a.z >> 4) & 0x0f0f0f0fu, (a.w >> 4) & 0x0f0f0f0fu);
    codes[(4 * c) + 3] = make_uint4((b.x >> 4) & 0x0f0f0f0fu, (b.y >> 4) & 0x0f0f0f0fu,
                                    (b.z >> 4) & 0x0f0f0f0fu, (b.w >> 4) & 0x0f0f0f0fu);
  }
  auto* mw = reinterpret_cast<uint4*>(slab + layout.mw +
                                      ((static_cast<std::int64_t>(e) * n + row) * layout.gpad * 2));
  mw[sb] = make_uint4(mins[0], mins[1], mins[2], mins[3]);
  if (sb == sbs - 1) {
    for (int pad = sbs; pad < layout.gpad / 8; ++pad) mw[pad] = make_uint4(0, 0, 0, 0);
  }
}

// ------------------------------------------------------------------ GEMM
constexpr int kTileCols = 128;  // tokens: the MMA's M, one TMEM lane each
constexpr int kTileRows = 128;  // weight rows: the MMA's N, one TMEM column each
constexpr int kBK = 128;        // K bytes a stage: four 32-value groups
constexpr int kStages = 3;
constexpr int kBuffers = 3;     // TMEM group-result buffers of kTileRows columns
constexpr int kMinColumn = kBuffers * kTileRows;  // TMEM: the F32 sum of the min terms
constexpr int kWBytes = kTileRows * kBK, kYBytes = kTileCols * kBK;
constexpr int kScaleBytes = 4 * 128 * 4;  // [group][row or token] F32
constexpr int kStageBytes = kWBytes + kYBytes + (2 * kScaleBytes);
// The min terms' operands: FP16 [128 rows or tokens][64 groups] K-major, 128-byte
// swizzled like the int8 tiles; one tile holds 16 k-steps, two tiles alternate.
constexpr int kMinTileBytes = 128 * 128;
constexpr int kMinSteps = 16;  // k-steps a tile of min operands covers
// Raw stages: what TMA brings for one super-block column (two k-steps): the 128
// weight rows' Q4_K blocks (raw mode only), then the 128 tokens' block headers of
// both k-steps.
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
constexpr int kEpilogueRows = kTileRows / (kEpilogueWarps / 4);  // weight rows a thread
static_assert(kEpilogueRows == 32, "one 32-column TMEM load a group");
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
  std::uint64_t y_full[kStages];   // the stage's TMA bytes have landed
  std::uint64_t w_full[kStages];   // the decode warps have written their part
  std::uint64_t empty[kStages];
  std::uint64_t tmem_full[kBuffers];
  std::uint64_t tmem_empty[kBuffers];
  std::uint64_t raw_full[kRawStages];
  std::uint64_t raw_empty[kRawStages];
  std::uint64_t minw_full[2];  // slab mode: a tile of weight min operands has landed
  std::uint64_t min_free[2];   // the tensor core has read a tile of min operands
  std::uint64_t min_full;      // the min terms' sum is complete in tensor memory
  std::uint32_t tmem_base;
  std::uint32_t abort;
};

struct Params {
  Desc a;
  const std::int32_t* worklist;
  unsigned int* faults;
  const float* ax;       // slab: the scale tiles
  int ax_ksteps;         // k-steps a row tile's scales span
  int ax_row_tiles;
  std::int32_t* sums;    // verification: the int32 group sums [col][row][k / 32], or null
  // GLU write-back (slab with interleaved gate / up rows): the GLU of every (gate, up) pair,
  // requantized to Q8_1-MMQ blocks [nrows / 2 / 128][ncols], instead of the F32 output.
  std::uint8_t* glu_out;
  int glu;
  float limit;
};

template <bool kSlab>
__global__ void __launch_bounds__(kThreads, 1)
MmqQ4KKernel(const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_w,
             const __grid_constant__ CUtensorMap map_h, const __grid_constant__ CUtensorMap map_mw,
             const Params p) {
  const Desc& a = p.a;
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
  if (p.worklist != nullptr) {
    if (static_cast<int>(blockIdx.y) >= p.worklist[0]) return;
    expert = p.worklist[1 + (2 * blockIdx.y)];
    col0 = p.worklist[2 + (2 * blockIdx.y)];
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
    for (int t = 0; t < 2; ++t) {
      tc::MbarInit(&sh->minw_full[t], 1);
      tc::MbarInit(&sh->min_free[t], 1);
    }
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
    atomicAdd(p.faults, 1u);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tc::PrefetchMap(&map_y);
      tc::PrefetchMap(&map_w);
      tc::PrefetchMap(&map_h);
      if constexpr (kSlab) tc::PrefetchMap(&map_mw);
      for (int ks = 0; ks < ksteps && !*abort_flag; ++ks) {
        if ((ks & 1) == 0) {
          // One super-block column (k-steps ks, ks + 1): the tokens' block headers
          // and, raw, the weight rows' blocks, for the decode warps.
          const int column = ks >> 1;
          const int rs = column % kRawStages;
          if (!tc::MbarWaitSleep(&sh->raw_empty[rs], ((column / kRawStages) & 1) ^ 1, 128)) {
            give_up();
            break;
          }
          unsigned char* stage = raw + (rs * kRawBytes);
          tc::MbarExpectTx(&sh->raw_full[rs], kSlab ? 2 * kRawHBytes : kRawBytes);
          if constexpr (!kSlab) {
            asm volatile(
                "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                " [%0], [%1, {%3, %4, %5}], [%2];"
                ::"r"(tc::Smem(stage)), "l"(&map_w), "r"(tc::Smem(&sh->raw_full[rs])),
                  "r"(column * 144), "r"(row0), "r"(expert)
                : "memory");
          }
          asm volatile(
              "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
              " [%0], [%1, {%3, %4, %5}], [%2];"
              ::"r"(tc::Smem(stage + kRawWBytes)), "l"(&map_h), "r"(tc::Smem(&sh->raw_full[rs])),
                "r"(0), "r"(col0), "r"(ks)
              : "memory");
        }
        if constexpr (kSlab) {
          // Every 16 k-steps a tile of the weight rows' min operands.
          if (ks % kMinSteps == 0) {
            const int mt = (ks / kMinSteps) & 1;
            if (ks >= 2 * kMinSteps &&
                !tc::MbarWaitSleep(&sh->min_free[mt], ((ks / (2 * kMinSteps)) - 1) & 1, 128)) {
              give_up();
              break;
            }
            tc::MbarExpectTx(&sh->minw_full[mt], kMinTileBytes);
            asm volatile(
                "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                " [%0], [%1, {%3, %4, %5}], [%2];"
                ::"r"(tc::Smem(min_w + (mt * kMinTileBytes))), "l"(&map_mw),
                  "r"(tc::Smem(&sh->minw_full[mt])), "r"((ks / kMinSteps) * 128), "r"(row0),
                  "r"(expert)
                : "memory");
          }
        }
        const int s = ks % kStages;
        if (!tc::MbarWaitSleep(&sh->empty[s], ((ks / kStages) & 1) ^ 1, 256)) {
          give_up();
          break;
        }
        tc::MbarExpectTx(&sh->y_full[s], kSlab ? kYBytes + kWBytes + kScaleBytes : kYBytes);
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(tc::Smem(y_tiles + (s * kYBytes))), "l"(&map_y), "r"(tc::Smem(&sh->y_full[s])),
              "r"(0), "r"(col0), "r"(ks)
            : "memory");
        if constexpr (kSlab) {
          asm volatile(
              "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
              " [%0], [%1, {%3, %4, %5}], [%2];"
              ::"r"(tc::Smem(w_tiles + (s * kWBytes))), "l"(&map_w), "r"(tc::Smem(&sh->y_full[s])),
                "r"(ks * kBK), "r"(row0), "r"(expert)
              : "memory");
          const float* src = p.ax + ((((static_cast<std::int64_t>(expert) * p.ax_row_tiles) +
                                       blockIdx.x) * p.ax_ksteps + ks) * 512);
          tc::BulkLoad(stage_scales(s), src, kScaleBytes, &sh->y_full[s]);
        }
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
      const int kk = ks % kMinSteps;
#pragma unroll  // the rows of a thread are independent: their latencies overlap
      for (int t = t0; t < kTileRows; t += kDecodeWarps * 32) {
        // Row t of a min tile, the four halves of this k-step: byte (ks % 16) * 8 of
        // the 128-byte row, 16-byte chunks swizzled like the int8 tiles.
        const int at = ((t >> 3) * 1024) + ((t & 7) * 128) + ((((kk >> 1) ^ (t & 7))) * 16) +
                       ((kk & 1) * 8);
        if constexpr (!kSlab) {
          const unsigned char* sb = stage + (t * 144);
          const uint4 head = *reinterpret_cast<const uint4*>(sb);
          uint4 q[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            q[i] = *reinterpret_cast<const uint4*>(sb + 16 + (half * 64) + (i * 16));
          }
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
          const __half d = __ushort_as_half(static_cast<unsigned short>(head.x & 0xffffu));
          const __half dmin = __hneg(__ushort_as_half(static_cast<unsigned short>(head.x >> 16)));
          std::uint32_t mins[4];
#pragma unroll
          for (int gl = 0; gl < 4; ++gl) {
            int scv, mnv;
            ScaleAndMin(head.y, head.z, head.w, (half * 4) + gl, &scv, &mnv);
            sc[(gl * 128) + t] = __half2float(__hmul(d, __int2half_rn(scv)));
            mins[gl] = __half_as_ushort(__hmul(dmin, __int2half_rn(mnv)));
          }
          *reinterpret_cast<uint2*>(min_w + (mt * kMinTileBytes) + at) =
              make_uint2(mins[0] | (mins[1] << 16), mins[2] | (mins[3] << 16));
        }
        // The token's header of this k-step: four (d8, s8) pairs.
        const uint4 ds =
            *reinterpret_cast<const uint4*>(stage + kRawWBytes + (half * kRawHBytes) + (t * 16));
        const std::uint32_t dsw[4] = {ds.x, ds.y, ds.z, ds.w};
#pragma unroll
        for (int gl = 0; gl < 4; ++gl) sc[512 + (gl * 128) + t] = HalfBitsToFloat(dsw[gl] & 0xffffu);
        *reinterpret_cast<uint2*>(min_y + (mt * kMinTileBytes) + at) =
            make_uint2((dsw[0] >> 16) | (dsw[1] & 0xffff0000u), (dsw[2] >> 16) | (dsw[3] & 0xffff0000u));
        // The last FP16 MMA reads 16 groups: zero what the k range leaves unwritten.
        if (ks == ksteps - 1) {
          for (int pad = ks + 1; pad % 4 != 0; ++pad) {
            const int pk = pad % kMinSteps;
            const int pat = ((t >> 3) * 1024) + ((t & 7) * 128) + ((((pk >> 1) ^ (t & 7))) * 16) +
                            ((pk & 1) * 8);
            if constexpr (!kSlab) {
              *reinterpret_cast<uint2*>(min_w + (mt * kMinTileBytes) + pat) = make_uint2(0u, 0u);
            }
            *reinterpret_cast<uint2*>(min_y + (mt * kMinTileBytes) + pat) = make_uint2(0u, 0u);
          }
        }
      }
      tc::FenceProxyAsync();  // generic-proxy writes, read by the tensor core's proxy
      __syncwarp();
      if (lane == 0) {
        if (half == 1 || ks == ksteps - 1) tc::MbarArrive(&sh->raw_empty[rs]);  // the raw stage is read
        tc::MbarArrive(&sh->w_full[s]);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // A (M, the TMEM lanes): tokens, signed int8.  B (N, the TMEM columns): weight
      // rows, unsigned codes.
      const std::uint32_t idesc = tc::IdescI8(kTileCols, kTileRows, true, false);
      std::uint32_t group = 0;
      for (int ks = 0; ks < ksteps && !*abort_flag; ++ks) {
        const int s = ks % kStages;
        if (!tc::MbarWait(&sh->w_full[s], (ks / kStages) & 1) ||
            !tc::MbarWait(&sh->y_full[s], (ks / kStages) & 1)) {
          give_up();
          break;
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
          tc::MmaI8(tmem + (b * kTileRows), ydesc + (gl * 2), wdesc + (gl * 2), idesc, false);
          tc::TcCommit(&sh->tmem_full[b]);
        }
        // Every fourth k-step completes 16 groups of min operands: one FP16 MMA
        // (K 16) adds their products to the F32 sum.
        if (ks % 4 == 3 || ks == ksteps - 1) {
          const int mt = (ks / kMinSteps) & 1;
          const int q = (ks % kMinSteps) / 4;  // 32 bytes along the swizzled row each
          if constexpr (kSlab) {
            if (q == 0 && !tc::MbarWait(&sh->minw_full[mt], (ks / (2 * kMinSteps)) & 1)) {
              give_up();
              break;
            }
            tc::TcFenceAfter();
          }
          tc::MmaF16(tmem + kMinColumn, tc::SmemDesc(min_y + (mt * kMinTileBytes), true, 1024) + (q * 2),
                     tc::SmemDesc(min_w + (mt * kMinTileBytes), true, 1024) + (q * 2),
                     tc::IdescF16(kTileCols, kTileRows), ks >= 4);
          if (ks % kMinSteps == kMinSteps - 1) tc::TcCommit(&sh->min_free[mt]);
          if (ks == ksteps - 1) tc::TcCommit(&sh->min_full);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int ew = warp - kFirstEpilogueWarp;
    const int quadrant = warp & 3;          // TMEM lanes this warp may touch
    const int rowgroup = ew >> 2;           // which kEpilogueRows weight rows
    const int tt = (quadrant * 32) + lane;  // token of the tile
    const std::uint32_t lane_base = static_cast<std::uint32_t>(quadrant * 32) << 16;
    std::uint64_t acc2[kEpilogueRows / 2];  // rows 2i, 2i + 1
#pragma unroll
    for (int i = 0; i < kEpilogueRows / 2; ++i) acc2[i] = 0ull;
    const int col = col0 + tt;  // this thread's sorted column
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
        const std::uint32_t at = tmem + lane_base + (bb * kTileRows) + (rowgroup * kEpilogueRows);
        // The thread's 32 rows at once, then the buffer goes straight back to the
        // tensor core: the fold below overlaps the next groups' MMAs.
        std::uint32_t r[32];
        tc::TmemLoad32(at, r);
        const float bx = sc[512 + (gl * 128) + tt];
        const float4* ax4 = reinterpret_cast<const float4*>(sc + (gl * 128) + (rowgroup * kEpilogueRows));
        tc::TmemLoadWait();
        tc::TcFenceBefore();
        __syncwarp();
        if (lane == 0) tc::MbarArrive(&sh->tmem_empty[bb]);
        if (p.sums != nullptr) {
          // verification: the exact group sums, before any float touches them
          if (col < c_end) {
            const int groups = a.k / 32;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int row = row0 + (rowgroup * kEpilogueRows) + j;
              if (row < a.nrows) {
                p.sums[((static_cast<std::size_t>(col) * a.nrows + row) * groups) + (ks * 4) + gl] =
                    static_cast<std::int32_t>(r[j]);
              }
            }
          }
        }
        const std::uint64_t bx2 = Pack2(bx, bx);
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          const float4 x4 = ax4[v];  // the same address in every lane: a broadcast
          // (ax * C) rounded, times d8, added: as the scalar sequence, two rows at once
          const std::uint64_t u01 =
              Mul2(Pack2(static_cast<float>(static_cast<int>(r[(4 * v)])),
                         static_cast<float>(static_cast<int>(r[(4 * v) + 1]))),
                   Pack2(x4.x, x4.y));
          const std::uint64_t u23 =
              Mul2(Pack2(static_cast<float>(static_cast<int>(r[(4 * v) + 2])),
                         static_cast<float>(static_cast<int>(r[(4 * v) + 3]))),
                   Pack2(x4.z, x4.w));
          acc2[2 * v] = Fma2(u01, bx2, acc2[2 * v]);
          acc2[(2 * v) + 1] = Fma2(u23, bx2, acc2[(2 * v) + 1]);
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
    float acc[kEpilogueRows];  // the min terms first, then plus the folded groups
    if (ok) {
      tc::TcFenceAfter();
      std::uint32_t r[32];
      tc::TmemLoad32(tmem + lane_base + kMinColumn + (rowgroup * kEpilogueRows), r);
      tc::TmemLoadWait();
#pragma unroll
      for (int j = 0; j < 32; ++j) acc[j] = __uint_as_float(r[j]);
    }
#pragma unroll
    for (int i = 0; i < kEpilogueRows / 2; ++i) {
      float lo, hi;
      Unpack2(acc2[i], lo, hi);
      acc[2 * i] += lo;
      acc[(2 * i) + 1] += hi;
    }
    if (p.glu_out != nullptr) {
      // The thread's 32 rows are 16 gate rows then the 16 up rows of the same outputs.  A
      // Q8_1-MMQ group is 32 outputs: this thread's 16 and those of the thread of the same
      // token one row group over (another warp), so the two trade their maxima and their
      // four-value partial sums through shared memory (the first weight stage: every MMA has
      // retired) and each forms the group's scale and sum exactly as the quantizer kernel
      // does (eight lanes of four values, xor tree 4, 2, 1).  Every epilogue warp reaches the
      // barrier, also one whose wait ran out: it stores nothing.
      float h[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) h[j] = Glu(p.glu, acc[j], acc[16 + j], p.limit);
      float part[4], amax = 0.0f;
#pragma unroll
      for (int l = 0; l < 4; ++l) {
        part[l] = ((h[4 * l] + h[(4 * l) + 1]) + h[(4 * l) + 2]) + h[(4 * l) + 3];
#pragma unroll
        for (int c = 0; c < 4; ++c) amax = fmaxf(amax, fabsf(h[(4 * l) + c]));
      }
      float* trade = reinterpret_cast<float*>(w_tiles);  // [4 row groups][128 tokens][8]
      float* mine = trade + (((rowgroup * kTileCols) + tt) * 8);
      mine[0] = amax;
      mine[1] = ok ? 1.0f : 0.0f;
      *reinterpret_cast<float4*>(mine + 4) = make_float4(part[0], part[1], part[2], part[3]);
      asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueWarps * 32) : "memory");
      const float* other = trade + ((((rowgroup ^ 1) * kTileCols) + tt) * 8);
      const float4 theirs = *reinterpret_cast<const float4*>(other + 4);
      const bool both = ok && other[1] != 0.0f;
      amax = fmaxf(amax, other[0]);
      // lanes 0..3 of the quantizer hold the lower row group's values, 4..7 the upper's
      const bool low = (rowgroup & 1) == 0;
      const float p0 = low ? part[0] : theirs.x, p1 = low ? part[1] : theirs.y;
      const float p2 = low ? part[2] : theirs.z, p3 = low ? part[3] : theirs.w;
      const float p4 = low ? theirs.x : part[0], p5 = low ? theirs.y : part[1];
      const float p6 = low ? theirs.z : part[2], p7 = low ? theirs.w : part[3];
      const float sum = ((p0 + p4) + (p2 + p6)) + ((p1 + p5) + (p3 + p7));
      const int out_first = (row0 / 2) + (rowgroup * 16);  // this thread's first GLU output
      if (both && col < c_end && row0 + (rowgroup * kEpilogueRows) < a.nrows) {
        std::uint32_t packed[4] = {0, 0, 0, 0};
        float d = 0.0f;
        if (amax > 0.0f) {
          const float d_inv = 127.0f / amax;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int q = static_cast<int>(roundf(h[j] * d_inv));
            packed[j >> 2] |= (static_cast<std::uint32_t>(q) & 0xffu) << (8 * (j & 3));
          }
          d = 1.0f / d_inv;
        }
        std::uint8_t* block = p.glu_out + (((static_cast<std::size_t>(out_first >> 7) * a.ncols) + col) * 144);
        const int at = out_first & 127;
        *reinterpret_cast<uint4*>(block + 16 + at) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        if (low) {
          *reinterpret_cast<std::uint32_t*>(block + ((at >> 5) * 4)) =
              static_cast<std::uint32_t>(__half_as_ushort(__float2half_rn(d))) |
              (static_cast<std::uint32_t>(__half_as_ushort(__float2half_rn(sum))) << 16);
        }
      }
    } else if (ok && col < c_end) {
      const int dst_col = a.ids_dst != nullptr ? a.ids_dst[col] : col;
      const int first = row0 + (rowgroup * kEpilogueRows);
      float* out = a.dst + (static_cast<std::size_t>(dst_col) * a.dst_col_stride) + first;
      // 128 contiguous bytes a thread: 128-bit stores when the output allows them
      const bool vector = (a.dst_col_stride % 4 == 0) &&
                          (reinterpret_cast<std::uintptr_t>(a.dst) % 16 == 0) && first + 32 <= a.nrows;
      if (vector) {
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          reinterpret_cast<float4*>(out)[v] =
              make_float4(acc[4 * v], acc[(4 * v) + 1], acc[(4 * v) + 2], acc[(4 * v) + 3]);
        }
      } else {
#pragma unroll  // fully: a dynamic index would put acc[] in local memory
        for (int j = 0; j < 32; ++j) {
          if (first + j < a.nrows) out[j] = acc[j];
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

int CheckDesc(const Desc& d, bool no_f32_output) {
  if (d.type != LLMP_B200_TYPE_Q4_K) {
    return Reject("mmq: weight type %d is not one this build computes (Q4_K)", d.type);
  }
  if ((d.w == nullptr && d.w_slab == nullptr) || d.y == nullptr ||
      (d.dst == nullptr && !no_f32_output) || d.k < 256 ||
      d.k % 256 != 0 || d.nrows < 1 || d.ncols < 1) {
    return Reject("mmq: Q4_K weights [k, n] (blocks or slab), Q8_1-MMQ activations of ncols columns, "
                  "an F32 output; k a positive multiple of 256");
  }
  if (d.stride_row < d.k / 256 || d.stride_expert < 0 ||
      (d.dst_col_stride < d.nrows && !no_f32_output)) {
    return Reject("mmq: strides must cover a row");
  }
  if ((d.w != nullptr && !Aligned(d.w, 16)) || !Aligned(d.y, 16) || !Aligned(d.dst, 4) ||
      (d.w_slab != nullptr && !Aligned(d.w_slab, 256)) ||
      (d.scratch != nullptr && !Aligned(d.scratch, 256))) {
    return Reject("mmq: weights and activation blocks 16-byte aligned; slab and scratch 256");
  }
  if (d.expert_bounds == nullptr && d.experts > 1) {
    return Reject("mmq: expert bounds exactly with experts");
  }
  if (d.expert_bounds != nullptr && (d.experts < 1 || d.experts > 65535)) {
    return Reject("mmq: 1 to 65535 experts");
  }
  return 0;
}

template <typename Fn>
bool Encode3D(CUtensorMap* map, Fn encode, const void* base, cuuint64_t d0, cuuint64_t d1,
              cuuint64_t d2, cuuint64_t s1, cuuint64_t s2, cuuint32_t b0, cuuint32_t b1,
              cuuint32_t b2, bool swizzle, CUtensorMapL2promotion promotion) {
  const cuuint64_t dims[3] = {d0, d1, d2};
  const cuuint64_t strides[2] = {s1, s2};
  const cuuint32_t box[3] = {b0, b1, b2};
  const cuuint32_t elem[3] = {1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box,
                elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, promotion,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int Relayout(const void* w, int n, int k, std::int64_t stride_row, std::int64_t stride_expert,
             int experts, void* slab, void* stream, int glu_inter = 0) {
  const Slab layout = SlabOf(n, k, experts);
  const std::int64_t items = static_cast<std::int64_t>(experts) * layout.row_tiles * 4 * (k / 256);
  const std::int64_t grid = (items + 7) / 8;
  if (grid > 0x7fffffffLL) return Reject("q4k_relayout: more blocks than a grid holds");
  const cudaError_t e = LaunchPdl(RelayoutQ4KKernel, dim3(static_cast<unsigned>(grid)), dim3(256), 0,
                                  static_cast<cudaStream_t>(stream),
                                  static_cast<const std::uint8_t*>(w), n, k, stride_row, stride_expert,
                                  experts, static_cast<std::uint8_t*>(slab), layout, glu_inter);
  if (e != cudaSuccess) return Failed(e, "q4k_relayout launch");
  return 0;
}

}  // namespace

int LaunchMmq(const llmp_b200_mmq_desc& d, const std::int32_t* worklist, int max_tiles,
              void* stream, std::int32_t* sums, const MmqGlu* glu) {
  if (const int status = CheckDesc(d, glu != nullptr); status != 0) return status;
  if (glu != nullptr) {
    if (d.w_slab == nullptr || glu->blocks == nullptr || d.nrows % 64 != 0 || d.ids_dst != nullptr ||
        sums != nullptr || !Aligned(glu->blocks, 16) || glu->glu < LLMP_B200_GLU_SWIGLU ||
        glu->glu > LLMP_B200_GLU_GEGLU || (glu->glu == LLMP_B200_GLU_GEGLU && glu->limit != 0.0f)) {
      return Reject("mmq_glu: a slab of interleaved gate / up rows (llmp_b200_q4k_relayout_glu), rows a "
                    "multiple of 64, no output scatter, 16-byte aligned output blocks, a GLU");
    }
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  const tc::EncodeTiledFn encode = tc::EncodeTiled();
  if (encode == nullptr) return Reject("mmq: the driver has no tensor-map encoder");
  const int experts = d.expert_bounds != nullptr ? d.experts : 1;
  // The weights' slab: the caller's (relayout at load time), or built now in the
  // caller's scratch; without either the kernel decodes the raw blocks itself.
  const std::uint8_t* slab = static_cast<const std::uint8_t*>(d.w_slab);
  bool queued = false;
  if (slab == nullptr && d.scratch != nullptr) {
    const int status = Relayout(d.w, d.nrows, d.k, d.stride_row,
                                experts > 1 ? d.stride_expert
                                            : static_cast<std::int64_t>(d.stride_row) * d.nrows,
                                experts, d.scratch, stream);
    if (status != 0) return status;
    slab = static_cast<const std::uint8_t*>(d.scratch);
    queued = true;
  }
  const auto fail = [&](int status) { return (queued && status > 0) ? -status : status; };
  const Slab layout = SlabOf(d.nrows, d.k, experts);
  CUtensorMap map_y, map_w, map_h, map_mw;
  if (!Encode3D(&map_y, encode, static_cast<const std::uint8_t*>(d.y) + 16, 128,
                static_cast<cuuint64_t>(d.ncols), static_cast<cuuint64_t>(d.k / 128), 144,
                static_cast<cuuint64_t>(d.ncols) * 144, 128, kTileCols, 1, true,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) {
    return fail(Reject("mmq: the driver refused a tensor map for the activation blocks"));
  }
  // The activation blocks' 16-byte headers [k / 128][col]: a box is 128 tokens, two k-steps.
  if (!Encode3D(&map_h, encode, d.y, 16, static_cast<cuuint64_t>(d.ncols),
                static_cast<cuuint64_t>(d.k / 128), 144, static_cast<cuuint64_t>(d.ncols) * 144, 16,
                kTileCols, 2, false, CU_TENSOR_MAP_L2_PROMOTION_NONE)) {
    return fail(Reject("mmq: the driver refused a tensor map for the activation headers"));
  }
  if (slab != nullptr) {
    // int8 codes [expert][row][k]: a box is 128 rows of one k-step, swizzled for the MMA.
    if (!Encode3D(&map_w, encode, slab + layout.codes, static_cast<cuuint64_t>(d.k),
                  static_cast<cuuint64_t>(d.nrows), static_cast<cuuint64_t>(experts),
                  static_cast<cuuint64_t>(d.k), static_cast<cuuint64_t>(d.k) * d.nrows, kBK,
                  kTileRows, 1, true, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) ||
        !Encode3D(&map_mw, encode, slab + layout.mw, static_cast<cuuint64_t>(layout.gpad) * 2,
                  static_cast<cuuint64_t>(d.nrows), static_cast<cuuint64_t>(experts),
                  static_cast<cuuint64_t>(layout.gpad) * 2,
                  static_cast<cuuint64_t>(layout.gpad) * 2 * d.nrows, 128, kTileRows, 1, true,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) {
      return fail(Reject("mmq: the driver refused a tensor map for the weight slab"));
    }
  } else {
    // The weights as bytes [expert][row][k / 256 * 144]: a box is one block of 128 rows.
    const cuuint64_t row_pitch = static_cast<cuuint64_t>(d.stride_row) * 144;
    const cuuint64_t expert_pitch = experts > 1 ? static_cast<cuuint64_t>(d.stride_expert) * 144
                                                : row_pitch * static_cast<cuuint64_t>(d.nrows);
    if (!Encode3D(&map_w, encode, d.w, static_cast<cuuint64_t>(d.k / 256) * 144,
                  static_cast<cuuint64_t>(d.nrows), static_cast<cuuint64_t>(experts), row_pitch,
                  expert_pitch, 144, kTileRows, 1, false, CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) {
      return fail(Reject("mmq: the driver refused a tensor map for the weight blocks"));
    }
    map_mw = map_w;  // unused
  }
  Params p{};
  p.a = d;
  p.worklist = worklist;
  p.faults = FaultCounter();
  if (p.faults == nullptr) return fail(Reject("mmq: no fault counter on this device"));
  p.ax = slab != nullptr ? reinterpret_cast<const float*>(slab + layout.ax) : nullptr;
  p.ax_ksteps = layout.ksteps;
  p.ax_row_tiles = layout.row_tiles;
  p.sums = sums;
  if (glu != nullptr) {
    p.glu_out = static_cast<std::uint8_t*>(glu->blocks);
    p.glu = glu->glu;
    p.limit = glu->limit;
  }
  static thread_local int configured_device = -1;
  int device = -1;
  cudaGetDevice(&device);
  if (configured_device != device) {
    cudaError_t e = cudaFuncSetAttribute(MmqQ4KKernel<false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e == cudaSuccess) {
      e = cudaFuncSetAttribute(MmqQ4KKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    }
    if (e != cudaSuccess) return fail(Failed(e, "mmq attribute"));
    configured_device = device;
  }
  dim3 grid(static_cast<unsigned>((d.nrows + kTileRows - 1) / kTileRows), 1, 1);
  if (worklist != nullptr) {
    if (max_tiles < 1) return fail(Reject("mmq: a worklist needs its capacity"));
    grid.y = static_cast<unsigned>(max_tiles);
  } else {
    const int max_cols = d.expert_bounds != nullptr ? d.max_cols_per_expert : d.ncols;
    if (max_cols < 1) return fail(Reject("mmq: max_cols_per_expert >= 1 with experts"));
    grid.y = static_cast<unsigned>((max_cols + kTileCols - 1) / kTileCols);
    grid.z = static_cast<unsigned>(experts);
  }
  if (grid.y > 65535u) return fail(Reject("mmq: more column tiles than a grid holds"));
  auto* s = static_cast<cudaStream_t>(stream);
  if (slab != nullptr) {
    MmqQ4KKernel<true><<<grid, kThreads, kSmem, s>>>(map_y, map_w, map_h, map_mw, p);
  } else {
    MmqQ4KKernel<false><<<grid, kThreads, kSmem, s>>>(map_y, map_w, map_h, map_mw, p);
  }
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

size_t llmp_b200_q4k_slab_bytes(int nrows, int k, int experts) {
  if (nrows < 1 || k < 256 || k % 256 != 0 || experts < 1) return 0;
  return llmp_b200::SlabOf(nrows, k, experts).total;
}

int llmp_b200_q4k_relayout(const void* w, int nrows, int k, int stride_row, int64_t stride_expert,
                           int experts, void* slab, void* stream) {
  using namespace llmp_b200;
  if (w == nullptr || slab == nullptr || nrows < 1 || k < 256 || k % 256 != 0 || experts < 1 ||
      stride_row < k / 256 || (experts > 1 && stride_expert < static_cast<int64_t>(stride_row) * nrows)) {
    return Reject("q4k_relayout: Q4_K blocks [experts][n][k / 256], k a positive multiple of 256, "
                  "strides that cover a row and an expert, and a slab");
  }
  if (!Aligned(w, 16) || !Aligned(slab, 256)) {
    return Reject("q4k_relayout: blocks 16-byte aligned, the slab 256");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  return Relayout(w, nrows, k, stride_row, stride_expert, experts, slab, stream);
}

size_t llmp_b200_mmq_scratch(const llmp_b200_mmq_desc* desc, int sms) {
  (void)sms;
  if (desc == nullptr || desc->w_slab != nullptr) return 0;
  const int experts = desc->expert_bounds != nullptr ? desc->experts : 1;
  return llmp_b200_q4k_slab_bytes(desc->nrows, desc->k, experts);
}

int llmp_b200_mmq(const llmp_b200_mmq_desc* desc, int sms, void* stream) {
  (void)sms;
  if (desc == nullptr) return llmp_b200::Reject("mmq: null descriptor");
  return llmp_b200::LaunchMmq(*desc, nullptr, 0, stream, nullptr);
}

int llmp_b200_q4k_relayout_glu(const void* w, int inter, int k, int stride_row, int64_t stride_expert,
                               int experts, void* slab, void* stream) {
  using namespace llmp_b200;
  if (w == nullptr || slab == nullptr || inter < 32 || inter % 32 != 0 || k < 256 || k % 256 != 0 ||
      experts < 1 || stride_row < k / 256 ||
      (experts > 1 && stride_expert < static_cast<int64_t>(stride_row) * 2 * inter)) {
    return Reject("q4k_relayout_glu: Q4_K blocks [experts][2 * inter][k / 256] (gate rows, then up "
                  "rows), inter a positive multiple of 32, k of 256, and a slab");
  }
  if (!Aligned(w, 16) || !Aligned(slab, 256)) {
    return Reject("q4k_relayout_glu: blocks 16-byte aligned, the slab 256");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  return Relayout(w, 2 * inter, k, stride_row, stride_expert, experts, slab, stream, inter);
}

int llmp_b200_mmq_glu(const llmp_b200_mmq_desc* desc, int glu, float limit, void* blocks,
                      void* stream) {
  using namespace llmp_b200;
  if (desc == nullptr) return Reject("mmq_glu: null descriptor");
  const MmqGlu g{blocks, glu, limit};
  return LaunchMmq(*desc, nullptr, 0, stream, nullptr, &g);
}

int llmp_b200_mmq_block_sums(const llmp_b200_mmq_desc* desc, int32_t* sums, void* stream) {
  using namespace llmp_b200;
  if (desc == nullptr || sums == nullptr) return Reject("mmq_block_sums: a descriptor and an output");
  if (desc->expert_bounds != nullptr || desc->ids_dst != nullptr) {
    return Reject("mmq_block_sums: the dense product only");
  }
  return LaunchMmq(*desc, nullptr, 0, stream, sums);
}

}  // extern "C"
