// MXFP8 (E4M3 codes, one E8M0 scale per 32 values along K) on B200:
//   llmp.mxfp8.quantize  activations -> codes + scales in 128x4 scale atoms
//   llmp.mxfp8.swizzle   row-major weight scales -> scale atoms
//   llmp.mxfp8.gemm      D[m,n] = A[m,k] . B[n,k]^T, F32 accumulate, F32/BF16 out
// Semantics follow src/kernels/ggml/mxfp8_quant.cuh:22-46, llmp_ops.cu:610-663
// and mxfp8_cutlass.h:30-79 (the reference runs a CUTLASS SM120 kernel; this is
// a hand-written sm_100a one).
//
// The GEMM is a persistent, warp-specialised tcgen05 kernel:
//   warp 0   TMA producer: A (128 x 128 B) and B (192 x 128 B) tiles through
//            128-byte-swizzled tensor maps, and the tiles' scale atoms (512 B
//            each, already in the layout tcgen05.cp wants) as bulk copies,
//            into a 5-stage shared-memory ring;
//   warp 1   allocates tensor memory and issues the MMAs: per stage it copies
//            the scale atoms to TMEM (tcgen05.cp 32x128b.warpx4) and issues
//            four tcgen05.mma.kind::mxf8f6f4.block_scale of 128x192x32 whose
//            scale-factor ids pick the stage's four K blocks; TWO accumulators
//            (128 lanes x 192 F32 columns each) live in TMEM, so the next
//            tile's main loop runs while the epilogue drains the last one;
//   warps 2-5 epilogue: tcgen05.ld the accumulator 32 columns at a time, convert
//            and store the rows.
// 128 x 192 tiles: two accumulators plus the scale columns fit the 512 TMEM
// columns, and the benchmark shape (2048 x 12288) makes 1,024 tiles = 6.9 waves
// of 148 CTAs.  A 192-row B tile starts on a scale-atom boundary or in the
// middle of an atom; the atom copies are offset by two TMEM columns for the
// latter.  Tiles are walked M-fastest so co-running CTAs share B tiles in L2.
// Every mbarrier wait is bounded; a wait that runs out raises the fault counter
// and the CTA drains and frees its tensor memory.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "tc.cuh"

namespace llmp_b200 {
namespace {

using Gemm = llmp_b200_mxfp8_gemm_desc;

__host__ __device__ constexpr std::uint64_t AtomOffset(std::uint64_t row, std::uint64_t block,
                                                       std::uint64_t blocks) {
  // src/format/layout.h:107-112 (== moe_cutlass.h:42-46 SfOffset)
  return ((((row / 128) * (blocks / 4)) + (block / 4)) * 512) + ((row % 32) * 16) +
         (((row % 128) / 32) * 4) + (block % 4);
}

// ------------------------------------------------------------------ quantize
// mxfp8_quant.cuh:22-46
__device__ __forceinline__ std::uint32_t ScaleCode(float amax) {
  const std::uint32_t bits = __float_as_uint(amax * (1.0f / 448.0f));
  std::uint32_t e = (bits >> 23) & 0xffu;
  if ((bits & 0x7fffffu) != 0u) ++e;
  return e > 253u ? 253u : e;
}
__device__ __forceinline__ std::uint32_t Pack4(float a, float b, float c, float d, float inverse) {
  const __nv_fp8x2_storage_t lo =
      __nv_cvt_float2_to_fp8x2(make_float2(a * inverse, b * inverse), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi =
      __nv_cvt_float2_to_fp8x2(make_float2(c * inverse, d * inverse), __NV_SATFINITE, __NV_E4M3);
  return static_cast<std::uint32_t>(lo) | (static_cast<std::uint32_t>(hi) << 16);
}

// Eight lanes a 32-value block, four values a lane: coalesced reads and
// 128-bit code stores; padding rows (up to the scale atoms) write zero scales.
template <bool kBf16>
__global__ void __launch_bounds__(256)
QuantizeKernel(const void* __restrict__ x, std::int64_t x_stride, std::uint8_t* __restrict__ codes,
               std::uint8_t* __restrict__ scales, int k, int rows, std::int64_t lanes_total) {
  GridLaunchDependents();
  // (the index arithmetic runs beside the tail of the kernel before, not after it)
  const std::int64_t i = (static_cast<std::int64_t>(blockIdx.x) * 256) + threadIdx.x;
  const bool live = i < lanes_total;
  const std::int64_t item = (live ? i : 0) / 8;
  const int part = static_cast<int>(i % 8);
  const int blocks = k / 32;
  const int r = static_cast<int>(item / blocks);
  const int b = static_cast<int>(item - (static_cast<std::int64_t>(r) * blocks));
  GridDependencyWait();
  float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (live && r < rows) {
    const std::int64_t at = (static_cast<std::int64_t>(r) * x_stride) + (b * 32) + (part * 4);
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
#pragma unroll
  for (int offset = 4; offset > 0; offset >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
  }
  if (!live) return;
  const std::uint64_t sat = AtomOffset(static_cast<std::uint64_t>(r), static_cast<std::uint64_t>(b),
                                       static_cast<std::uint64_t>(blocks));
  if (r >= rows) {
    if (part == 0) scales[sat] = 0;
    return;
  }
  const std::uint32_t e = ScaleCode(amax);
  const float inverse = __uint_as_float((254u - e) << 23);
  *reinterpret_cast<std::uint32_t*>(codes + (static_cast<std::int64_t>(r) * k) + (b * 32) +
                                    (part * 4)) = Pack4(v[0], v[1], v[2], v[3], inverse);
  if (part == 0) scales[sat] = static_cast<std::uint8_t>(e);
}

__global__ void SwizzleKernel(const std::uint8_t* __restrict__ in, std::uint8_t* __restrict__ out,
                              int n, int blocks, std::int64_t items) {
  const std::int64_t i = (static_cast<std::int64_t>(blockIdx.x) * blockDim.x) + threadIdx.x;
  if (i >= items) return;
  const int r = static_cast<int>(i / blocks);
  const int b = static_cast<int>(i % blocks);
  out[AtomOffset(static_cast<std::uint64_t>(r), static_cast<std::uint64_t>(b),
                 static_cast<std::uint64_t>(blocks))] = r < n ? in[i] : 0;
}

// ------------------------------------------------------------------ GEMM
constexpr int kBM = 128, kBN = 192, kBK = 128, kStages = 5, kUmmaK = 32;
constexpr int kABytes = kBM * kBK, kBBytes = kBN * kBK;
constexpr int kSfaBytes = 512, kSfbBytes = 1024;
constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
constexpr int kGemmThreads = 192;
constexpr int kTmemColumns = 512;
// Two accumulators of kBN columns, then per stage 16 scale columns: A's atom at
// +0..3, B's two atoms at +4..7 and +8..11; the tile's 192 rows' scales start at
// +4 (tile on an atom boundary) or +6 (tile starting in the middle of an atom).
constexpr int kAccColumns = kBN;
constexpr int kSfColumn = 2 * kBN;
constexpr int kSfStride = 16;
constexpr int kGemmSmem = (kStages * kStageBytes) + 1024 /* alignment */ + 256 /* barriers */;

struct GemmShared {
  std::uint64_t full[kStages];
  std::uint64_t empty[kStages];
  std::uint64_t tmem_full[2];
  std::uint64_t tmem_empty[2];
  std::uint32_t tmem_base;
  std::uint32_t abort;
};

// 32 consecutive columns of one output row, from the accumulator's registers.
__device__ __forceinline__ void StoreChunk(void* __restrict__ d, bool bf16, int row, int col, int m,
                                           int n, const std::uint32_t (&r)[32]) {
  if (row >= m || col >= n) return;
  if (bf16) {
    auto* out = static_cast<__nv_bfloat16*>(d) + (static_cast<std::size_t>(row) * n) + col;
    if (col + 32 <= n && (n % 8) == 0) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        std::uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(r[(8 * v) + (2 * j)]),
                                                         __uint_as_float(r[(8 * v) + (2 * j) + 1]));
          w[j] = *reinterpret_cast<const std::uint32_t*>(&p);
        }
        reinterpret_cast<uint4*>(out)[v] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
      // unrolled, so that r[] is only ever indexed by constants and stays in registers
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (col + j < n) out[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
      }
    }
  } else {
    auto* out = static_cast<float*>(d) + (static_cast<std::size_t>(row) * n) + col;
    if (col + 32 <= n && (n % 4) == 0) {
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        reinterpret_cast<uint4*>(out)[v] =
            make_uint4(r[4 * v], r[(4 * v) + 1], r[(4 * v) + 2], r[(4 * v) + 3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (col + j < n) out[j] = __uint_as_float(r[j]);
      }
    }
  }
}

// This warp's 32 accumulator rows x kBN columns out of tensor memory and into D: the next
// 32 columns are already on their way while the last 32 are converted and stored.
__device__ __forceinline__ void DrainAccumulator(std::uint32_t taddr, void* __restrict__ d, bool bf16,
                                                 int row, int col0, int m, int n) {
  std::uint32_t r0[32], r1[32];
  tc::TmemLoad32(taddr, r0);
#pragma unroll
  for (int c = 0; c < kBN / 32; c += 2) {
    tc::TmemLoadWait32(r0);
    tc::TmemLoad32(taddr + ((c + 1) * 32), r1);
    StoreChunk(d, bf16, row, col0 + (c * 32), m, n, r0);
    tc::TmemLoadWait32(r1);
    if (c + 2 < kBN / 32) tc::TmemLoad32(taddr + ((c + 2) * 32), r0);
    StoreChunk(d, bf16, row, col0 + ((c + 1) * 32), m, n, r1);
  }
}

__global__ void __launch_bounds__(kGemmThreads, 1)
Mxfp8GemmKernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const std::uint8_t* __restrict__ sfa, const std::uint8_t* __restrict__ sfb,
                void* __restrict__ d, int m, int n, int k, int bf16, int sfb_rows_padded,
                unsigned int* faults) {
  extern __shared__ unsigned char raw_smem[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<std::uintptr_t>(raw_smem) + 1023) & ~static_cast<std::uintptr_t>(1023));
  unsigned char* a_tiles = smem;
  unsigned char* b_tiles = a_tiles + (kStages * kABytes);
  unsigned char* sfa_tiles = b_tiles + (kStages * kBBytes);
  unsigned char* sfb_tiles = sfa_tiles + (kStages * kSfaBytes);
  GemmShared* sh = reinterpret_cast<GemmShared*>(sfb_tiles + (kStages * kSfbBytes));

  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int tiles_m = (m + kBM - 1) / kBM;
  const int tiles_n = (n + kBN - 1) / kBN;
  const int tiles = tiles_m * tiles_n;
  const int ksteps = k / kBK;
  const int kb = k / 32;  // scales a row

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::MbarInit(&sh->full[s], 1);
      tc::MbarInit(&sh->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::MbarInit(&sh->tmem_full[b], 1);
      tc::MbarInit(&sh->tmem_empty[b], 4);
    }
    sh->abort = 0;
    tc::MbarInitFence();
  }
  if (warp == 1) {
    tc::TmemAlloc(&sh->tmem_base, kTmemColumns);
    tc::TmemRelinquish();
  }
  tc::TcFenceBefore();
  __syncthreads();
  tc::TcFenceAfter();
  const std::uint32_t tmem = sh->tmem_base;
  volatile std::uint32_t* abort_flag = &sh->abort;

  if (warp == 0) {
    // ---------------------------------------------------------- TMA producer
    // The whole warp walks the loop and one elected lane issues: loop state that is the same in
    // every lane stays where copy and tcgen05 instructions take their operands from (issued
    // from inside a one-lane branch each such instruction held the thread 60 to 190 cycles,
    // which bounded the kernel).  The next stage's barrier is looked at without blocking
    // before this stage's copies go out: a blocking wait costs about 180 cycles even on a
    // phase that completed long ago.
    const bool elected = tc::ElectOne();
    if (elected) {
      tc::PrefetchMap(&map_a);
      tc::PrefetchMap(&map_b);
    }
    std::uint32_t it = 0;
    bool ready = false, ok = true;
    for (int t = static_cast<int>(blockIdx.x); t < tiles && !*abort_flag; t += gridDim.x) {
      const int mb = t % tiles_m, nb = t / tiles_m;
      // The tile's B rows [nb * 192, +192) touch two scale atoms (128 rows each).
      const int atom0 = (nb * kBN) / 128;
      const bool second = (atom0 + 1) * 128 < sfb_rows_padded;
      const std::uint8_t* sfa_at = sfa + (static_cast<std::size_t>(mb) * (kb / 4) * 512);
      const std::uint8_t* sfb_at = sfb + (static_cast<std::size_t>(atom0) * (kb / 4) * 512);
      const std::size_t sfb_next = static_cast<std::size_t>(kb / 4) * 512;
      for (int ks = 0; ks < ksteps; ++ks, ++it) {
        const int s = static_cast<int>(it % kStages);
        if (!ready) ok = tc::MbarWait(&sh->empty[s], ((it / kStages) & 1u) ^ 1u);
        if (!ok) break;
        const std::uint32_t next = it + 1;
        ready = tc::MbarTest(&sh->empty[next % kStages], ((next / kStages) & 1u) ^ 1u);
        if (elected) {
          tc::MbarExpectTx(&sh->full[s], kABytes + kBBytes + kSfaBytes + (second ? 1024u : 512u));
          tc::TmaLoad2D(a_tiles + (s * kABytes), &map_a, ks * kBK, mb * kBM, &sh->full[s]);
          tc::TmaLoad2D(b_tiles + (s * kBBytes), &map_b, ks * kBK, nb * kBN, &sh->full[s]);
          tc::BulkLoad(sfa_tiles + (s * kSfaBytes), sfa_at + (ks * 512), 512, &sh->full[s]);
          tc::BulkLoad(sfb_tiles + (s * kSfbBytes), sfb_at + (ks * 512), 512, &sh->full[s]);
          if (second) {
            tc::BulkLoad(sfb_tiles + (s * kSfbBytes) + 512, sfb_at + sfb_next + (ks * 512), 512,
                         &sh->full[s]);
          }
        }
        ready = __all_sync(0xffffffffu, ready);
      }
      if (!__all_sync(0xffffffffu, ok)) {
        if (elected) {
          *abort_flag = 1;
          atomicAdd(faults, 1u);
        }
        break;
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    const bool elected = tc::ElectOne();
    std::uint32_t it = 0, tile_it = 0;
    bool ready = false;
    for (int t = static_cast<int>(blockIdx.x); t < tiles && !*abort_flag; t += gridDim.x, ++tile_it) {
      const int nb = t / tiles_m;
      const int acc = static_cast<int>(tile_it & 1u);
      bool ok = tc::MbarWait(&sh->tmem_empty[acc], ((tile_it >> 1) & 1u) ^ 1u);
      if (!__all_sync(0xffffffffu, ok)) {
        if (elected) {
          *abort_flag = 1;
          atomicAdd(faults, 1u);
        }
        break;
      }
      const std::uint32_t tacc = tmem + (acc * kAccColumns);
      // The two atoms always land on 4-column boundaries (tcgen05.cp's unit); an
      // odd tile starts in the middle of its first atom, whose last two columns
      // (rows 64..127) are the tile's first two: the MMA reads from +2.
      const int shift = (nb & 1) ? 2 : 0;
      for (int ks = 0; ks < ksteps; ++ks, ++it) {
        const int s = static_cast<int>(it % kStages);
        if (!ready) ok = tc::MbarWait(&sh->full[s], (it / kStages) & 1u);
        if (!ok) break;
        tc::TcFenceAfter();
        const std::uint32_t next = it + 1;
        ready = tc::MbarTest(&sh->full[next % kStages], (next / kStages) & 1u);
        const std::uint32_t tsfa = tmem + kSfColumn + (s * kSfStride);
        const std::uint32_t tsfb = tsfa + 4 + shift;
        const std::uint64_t adesc = tc::SmemDesc(a_tiles + (s * kABytes), true, 1024);
        const std::uint64_t bdesc = tc::SmemDesc(b_tiles + (s * kBBytes), true, 1024);
        if (elected) {
          tc::TmemCopyScales(tsfa, tc::SmemDesc(sfa_tiles + (s * kSfaBytes), false, 128));
          tc::TmemCopyScales(tsfa + 4, tc::SmemDesc(sfb_tiles + (s * kSfbBytes), false, 128));
          tc::TmemCopyScales(tsfa + 8, tc::SmemDesc(sfb_tiles + (s * kSfbBytes) + 512, false, 128));
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            // 32 bytes along K inside the 128-byte swizzle row: +2 in 16-byte units
            tc::MmaMxf8(tacc, adesc + (kk * 2), bdesc + (kk * 2), tc::IdescMxf8(kBM, kBN, kk, kk),
                        ks > 0 || kk > 0, tsfa, tsfb);
          }
          tc::TcCommit(&sh->empty[s]);  // the stage's bytes are free once these MMAs retire
        }
        ready = __all_sync(0xffffffffu, ready);
      }
      if (!__all_sync(0xffffffffu, ok)) {
        if (elected) {
          *abort_flag = 1;
          atomicAdd(faults, 1u);
        }
        break;
      }
      if (elected) tc::TcCommit(&sh->tmem_full[acc]);
    }
  } else {
    // ---------------------------------------------------------- epilogue
    const int quadrant = warp & 3;  // the TMEM lanes this warp may read
    std::uint32_t tile_it = 0;
    for (int t = static_cast<int>(blockIdx.x); t < tiles; t += gridDim.x, ++tile_it) {
      const int mb = t % tiles_m, nb = t / tiles_m;
      const int acc = static_cast<int>(tile_it & 1u);
      bool ok = true;
      if (lane == 0) ok = tc::MbarWait(&sh->tmem_full[acc], (tile_it >> 1) & 1u);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok || *abort_flag) {
        if (lane == 0 && !ok) {
          *abort_flag = 1;
          atomicAdd(faults, 1u);
        }
        break;
      }
      tc::TcFenceAfter();
      const int row = (mb * kBM) + (quadrant * 32) + lane;
      DrainAccumulator(tmem + (static_cast<std::uint32_t>(quadrant * 32) << 16) + (acc * kAccColumns),
                       d, bf16 != 0, row, nb * kBN, m, n);
      tc::TcFenceBefore();
      __syncwarp();
      if (lane == 0) tc::MbarArrive(&sh->tmem_empty[acc]);
    }
  }

  // Teardown: everyone meets, then the allocating warp frees tensor memory.
  tc::TcFenceBefore();
  __syncthreads();
  if (warp == 1) {
    tc::TcFenceAfter();
    tc::TmemDealloc(tmem, kTmemColumns);
  }
}

// ------------------------------------------------------------------ GEMM on CTA pairs
// The same roles over a cluster of two CTAs (cta_group::2): one 256 x 192 tile a pair.  Each
// CTA fetches its own 128 rows of A and 96 of the tile's 192 rows of B - 28 KB a k-step into
// an SM instead of 40 KB, which is what bounds the single-CTA kernel - plus its rows' scale
// atom and the tile's B scale atoms (both CTAs need all 192 columns' scales).  The even CTA's
// MMA thread issues M 256 MMAs that read both halves and accumulate 128 lanes x 192 columns in
// each CTA's tensor memory; tcgen05.commit reaches the barriers of both CTAs.  The odd CTA's
// MMA warp only relays "my stage has landed" to the even CTA, and its epilogue warps release
// an accumulator by arriving on the even CTA's barrier.  Loads carry no multicast.  Waits on
// barriers the other CTA arrives at are the ordinary ones: a cluster-scope acquire on every
// wait measured 2.2 times the whole kernel's time, and what crosses the pair is read by the
// tensor core's own path (operands) or ordered by tcgen05 fences (accumulators), not by this
// thread's loads.
constexpr int kPairBM = 256, kPairHalfN = kBN / 2, kPairStages = 7;
constexpr int kPairBBytes = kPairHalfN * kBK;
constexpr int kPairStageBytes = kABytes + kPairBBytes + kSfaBytes + kSfbBytes;
constexpr int kPairSmem = (kPairStages * kPairStageBytes) + 1024 + 512;
static_assert(kSfColumn + (kPairStages * kSfStride) <= kTmemColumns, "scale columns fit");


struct PairShared {
  std::uint64_t full[kPairStages];
  std::uint64_t empty[kPairStages];
  std::uint64_t tmem_full[2];
  std::uint64_t tmem_empty[2];  // even CTA: the epilogue warps of both CTAs
  std::uint32_t tmem_base;
  std::uint32_t abort;
};

__global__ void __launch_bounds__(kGemmThreads, 1)
Mxfp8GemmPairKernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const std::uint8_t* __restrict__ sfa, const std::uint8_t* __restrict__ sfb,
                    void* __restrict__ d, int m, int n, int k, int bf16, int sfa_rows_padded,
                    int sfb_rows_padded, unsigned int* faults) {
  extern __shared__ unsigned char raw_smem[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<std::uintptr_t>(raw_smem) + 1023) & ~static_cast<std::uintptr_t>(1023));
  unsigned char* a_tiles = smem;
  unsigned char* b_tiles = a_tiles + (kPairStages * kABytes);
  unsigned char* sfa_tiles = b_tiles + (kPairStages * kPairBBytes);
  unsigned char* sfb_tiles = sfa_tiles + (kPairStages * kSfaBytes);
  PairShared* sh = reinterpret_cast<PairShared*>(sfb_tiles + (kPairStages * kSfbBytes));

  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int rank = static_cast<int>(tc::ClusterCtaRank());  // 0: issues the MMAs
  const int pair = static_cast<int>(blockIdx.x) >> 1;
  const int pairs = static_cast<int>(gridDim.x) >> 1;
  const int tiles_m = (m + kPairBM - 1) / kPairBM;
  const int tiles_n = (n + kBN - 1) / kBN;
  const int tiles = tiles_m * tiles_n;
  const int ksteps = k / kBK;
  const int kb = k / 32;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      // the even CTA's "full" also counts the odd CTA's relay: one wait covers both halves
      tc::MbarInit(&sh->full[s], rank == 0 ? 2 : 1);
      tc::MbarInit(&sh->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::MbarInit(&sh->tmem_full[b], 1);
      tc::MbarInit(&sh->tmem_empty[b], 8);
    }
    sh->abort = 0;
    tc::MbarInitFence();
  }
  __syncthreads();
  if (warp == 1) {
    tc::TmemAllocPair(&sh->tmem_base, kTmemColumns);
    tc::TmemRelinquishPair();
  }
  tc::TcFenceBefore();
  __syncthreads();
  tc::ClusterBarrier();  // both CTAs' barriers are initialised before either reaches across
  tc::TcFenceAfter();
  const std::uint32_t tmem = sh->tmem_base;
  volatile std::uint32_t* abort_flag = &sh->abort;
  const std::uint32_t peer_abort = tc::PeerSmem(&sh->abort, static_cast<std::uint32_t>(rank ^ 1));
  auto give_up = [&]() {
    *abort_flag = 1;
    tc::StorePeerU32(peer_abort, 1u);
    atomicAdd(faults, 1u);
  };

  if (warp == 0) {
    // ---------------------------------------------------------- TMA producer (both CTAs)
    // The whole warp walks the loop and one elected lane issues the copies (see the MMA warp).
    const bool elected = tc::ElectOne();
    if (elected) {
      tc::PrefetchMap(&map_a);
      tc::PrefetchMap(&map_b);
    }
    std::uint32_t it = 0;
    bool ready = false, ok = true;
    for (int t = pair; t < tiles && !*abort_flag; t += pairs) {
      const int mb = t % tiles_m, nb = t / tiles_m;
      // This CTA's rows of A; a half tile wholly below the matrix reads zeros and borrows
      // the last atom's scales (its rows are never stored).
      int a_atom = (mb * 2) + rank;
      if (a_atom * 128 >= sfa_rows_padded) a_atom = (sfa_rows_padded / 128) - 1;
      const int atom0 = (nb * kBN) / 128;
      const bool second = (atom0 + 1) * 128 < sfb_rows_padded;
      const std::uint8_t* sfa_at = sfa + (static_cast<std::size_t>(a_atom) * (kb / 4) * 512);
      const std::uint8_t* sfb_at = sfb + (static_cast<std::size_t>(atom0) * (kb / 4) * 512);
      const std::size_t sfb_next = static_cast<std::size_t>(kb / 4) * 512;
      const int a_row = (mb * kPairBM) + (rank * kBM);
      const int b_row = (nb * kBN) + (rank * kPairHalfN);
      for (int ks = 0; ks < ksteps; ++ks, ++it) {
        const int s = static_cast<int>(it % kPairStages);
        if (!ready) ok = tc::MbarWait(&sh->empty[s], ((it / kPairStages) & 1u) ^ 1u);
        if (!ok) break;
        const std::uint32_t next = it + 1;
        ready = tc::MbarTest(&sh->empty[next % kPairStages], ((next / kPairStages) & 1u) ^ 1u);
        if (elected) {
          tc::MbarExpectTx(&sh->full[s],
                           kABytes + kPairBBytes + kSfaBytes + (second ? 1024u : 512u));
          tc::TmaLoad2D(a_tiles + (s * kABytes), &map_a, ks * kBK, a_row, &sh->full[s]);
          tc::TmaLoad2D(b_tiles + (s * kPairBBytes), &map_b, ks * kBK, b_row, &sh->full[s]);
          tc::BulkLoad(sfa_tiles + (s * kSfaBytes), sfa_at + (ks * 512), 512, &sh->full[s]);
          tc::BulkLoad(sfb_tiles + (s * kSfbBytes), sfb_at + (ks * 512), 512, &sh->full[s]);
          if (second) {
            tc::BulkLoad(sfb_tiles + (s * kSfbBytes) + 512, sfb_at + sfb_next + (ks * 512), 512,
                         &sh->full[s]);
          }
        }
        ready = __all_sync(0xffffffffu, ready);
      }
      if (!__all_sync(0xffffffffu, ok)) {
        if (elected) give_up();
        break;
      }
    }
  } else if (warp == 1) {
    if (rank == 1) {
      // ---------------------------------------------------------- relay (odd CTA)
      if (lane == 0) {
        std::uint32_t it = 0;
        for (int t = pair; t < tiles && !*abort_flag; t += pairs) {
          for (int ks = 0; ks < ksteps; ++ks, ++it) {
            const int s = static_cast<int>(it % kPairStages);
            if (!tc::MbarWait(&sh->full[s], (it / kPairStages) & 1u)) {
              give_up();
              break;
            }
            tc::MbarArrivePeer(tc::PeerSmem(&sh->full[s], 0u));
          }
        }
      }
    } else {
      // ---------------------------------------------------------- MMA issuer (even CTA)
      // The whole warp walks the loop and one elected lane issues: the loop's state (stage,
      // descriptors, tensor-memory addresses) is then the same in every lane, which lets the
      // compiler keep it where tcgen05 instructions take their operands from.  The
      // instruction stream of this warp is what bounds the kernel, so the next stage's
      // barrier is looked at, without blocking, before this stage's MMAs are issued.
      const bool elected = tc::ElectOne();
      std::uint32_t it = 0, tile_it = 0;
      bool ready = false;
      for (int t = pair; t < tiles && !*abort_flag; t += pairs, ++tile_it) {
        const int nb = t / tiles_m;
        const int acc = static_cast<int>(tile_it & 1u);
        bool ok = tc::MbarWait(&sh->tmem_empty[acc], ((tile_it >> 1) & 1u) ^ 1u);
        if (!__all_sync(0xffffffffu, ok)) {
          if (elected) give_up();
          break;
        }
        const std::uint32_t tacc = tmem + (acc * kAccColumns);
        const int shift = (nb & 1) ? 2 : 0;
        for (int ks = 0; ks < ksteps; ++ks, ++it) {
          const int s = static_cast<int>(it % kPairStages);
          if (!ready) ok = tc::MbarWait(&sh->full[s], (it / kPairStages) & 1u);
          if (!ok) break;
          tc::TcFenceAfter();
          const std::uint32_t next = it + 1;
          ready = tc::MbarTest(&sh->full[next % kPairStages], (next / kPairStages) & 1u);
          const std::uint32_t tsfa = tmem + kSfColumn + (s * kSfStride);
          const std::uint32_t tsfb = tsfa + 4 + shift;
          const std::uint64_t adesc = tc::SmemDesc(a_tiles + (s * kABytes), true, 1024);
          const std::uint64_t bdesc = tc::SmemDesc(b_tiles + (s * kPairBBytes), true, 1024);
          if (elected) {
            tc::TmemCopyScalesPair(tsfa, tc::SmemDesc(sfa_tiles + (s * kSfaBytes), false, 128));
            tc::TmemCopyScalesPair(tsfa + 4, tc::SmemDesc(sfb_tiles + (s * kSfbBytes), false, 128));
            tc::TmemCopyScalesPair(tsfa + 8,
                                   tc::SmemDesc(sfb_tiles + (s * kSfbBytes) + 512, false, 128));
#pragma unroll
            for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
              tc::MmaMxf8Pair(tacc, adesc + (kk * 2), bdesc + (kk * 2),
                              tc::IdescMxf8(kPairBM, kBN, kk, kk), ks > 0 || kk > 0, tsfa, tsfb);
            }
            tc::TcCommitPair(&sh->empty[s], 3);  // both CTAs' stage is free once these retire
          }
          ready = __all_sync(0xffffffffu, ready);
        }
        if (!__all_sync(0xffffffffu, ok)) {
          if (elected) give_up();
          break;
        }
        if (elected) tc::TcCommitPair(&sh->tmem_full[acc], 3);
      }
    }
  } else {
    // ---------------------------------------------------------- epilogue (both CTAs)
    const int quadrant = warp & 3;
    std::uint32_t tile_it = 0;
    for (int t = pair; t < tiles; t += pairs, ++tile_it) {
      const int mb = t % tiles_m, nb = t / tiles_m;
      const int acc = static_cast<int>(tile_it & 1u);
      bool ok = true;
      if (lane == 0) ok = tc::MbarWait(&sh->tmem_full[acc], (tile_it >> 1) & 1u);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok || *abort_flag) {
        if (lane == 0 && !ok) give_up();
        break;
      }
      tc::TcFenceAfter();
      const int row = (mb * kPairBM) + (rank * kBM) + (quadrant * 32) + lane;
      DrainAccumulator(tmem + (static_cast<std::uint32_t>(quadrant * 32) << 16) + (acc * kAccColumns),
                       d, bf16 != 0, row, nb * kBN, m, n);
      tc::TcFenceBefore();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) {
          tc::MbarArrive(&sh->tmem_empty[acc]);
        } else {
          tc::MbarArrivePeer(tc::PeerSmem(&sh->tmem_empty[acc], 0u));
        }
      }
    }
  }

  // Teardown: both CTAs meet (no thread may still reach into the other's memory), then the
  // allocating warps free the pair's tensor memory.
  tc::TcFenceBefore();
  __syncthreads();
  tc::ClusterBarrier();
  if (warp == 1) {
    tc::TcFenceAfter();
    tc::TmemDeallocPair(tmem, kTmemColumns);
  }
}

}  // namespace
}  // namespace llmp_b200

extern "C" {

uint64_t llmp_b200_mxfp8_padded_rows(uint64_t rows) { return (rows + 127) / 128 * 128; }

uint64_t llmp_b200_mxfp8_scale_offset(uint64_t row, uint64_t block, uint64_t blocks) {
  return llmp_b200::AtomOffset(row, block, blocks);
}

int llmp_b200_mxfp8_quantize(const void* x, int is_bf16, int64_t row_stride, int k, int rows,
                             void* codes, void* scales, void* stream) {
  using namespace llmp_b200;
  if (x == nullptr || codes == nullptr || scales == nullptr || rows < 1 || k < 128 ||
      k % 128 != 0 || row_stride < k) {
    return Reject("mxfp8.quantize: [k, rows] input with k a positive multiple of 128");
  }
  const int elem = is_bf16 ? 2 : 4;
  if (!Aligned(x, 16) || (row_stride * elem) % 16 != 0 || !Aligned(codes, 16)) {
    return Reject("mxfp8.quantize: input rows and codes 16-byte aligned");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  const std::int64_t padded = static_cast<std::int64_t>(llmp_b200_mxfp8_padded_rows(rows));
  const std::int64_t lanes = padded * (k / 32) * 8;
  const std::int64_t grid = (lanes + 255) / 256;
  if (grid > 0x7fffffffLL) return Reject("mxfp8.quantize: more blocks than a grid holds");
  auto* s = static_cast<cudaStream_t>(stream);
  const cudaError_t e =
      is_bf16 ? LaunchPdl(QuantizeKernel<true>, dim3(static_cast<unsigned>(grid)), dim3(256), 0, s,
                          x, row_stride, static_cast<std::uint8_t*>(codes),
                          static_cast<std::uint8_t*>(scales), k, rows, lanes)
              : LaunchPdl(QuantizeKernel<false>, dim3(static_cast<unsigned>(grid)), dim3(256), 0, s,
                          x, row_stride, static_cast<std::uint8_t*>(codes),
                          static_cast<std::uint8_t*>(scales), k, rows, lanes);
  if (e != cudaSuccess) return Failed(e, "mxfp8.quantize launch");
  return 0;
}

int llmp_b200_mxfp8_swizzle(const void* in, void* out, int n, int blocks, void* stream) {
  using namespace llmp_b200;
  if (in == nullptr || out == nullptr || n < 1 || blocks < 4 || blocks % 4 != 0) {
    return Reject("mxfp8.swizzle: scales [k / 32, n] with k / 32 a positive multiple of 4");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  const std::int64_t items =
      static_cast<std::int64_t>(llmp_b200_mxfp8_padded_rows(n)) * blocks;
  SwizzleKernel<<<static_cast<unsigned>((items + 255) / 256), 256, 0,
                  static_cast<cudaStream_t>(stream)>>>(static_cast<const std::uint8_t*>(in),
                                                       static_cast<std::uint8_t*>(out), n, blocks,
                                                       items);
  return Launched("mxfp8.swizzle launch");
}

int llmp_b200_mxfp8_gemm_available(void) { return llmp_b200_available(); }

size_t llmp_b200_mxfp8_gemm_scratch(const llmp_b200_mxfp8_gemm_desc* gemm, int sms) {
  (void)gemm;
  (void)sms;
  return 0;  // accumulators live in tensor memory; no workspace
}

int llmp_b200_mxfp8_gemm_variant(const llmp_b200_mxfp8_gemm_desc* gemm, int sms, int variant,
                                 void* stream) {
  using namespace llmp_b200;
  if (gemm == nullptr) return Reject("mxfp8.gemm: null descriptor");
  const Gemm& g = *gemm;
  if (g.m < 1 || g.n < 1 || g.k < 128 || g.k % 128 != 0) {
    return Reject("mxfp8.gemm: m, n >= 1 and k a positive multiple of 128");
  }
  if (g.a == nullptr || g.b == nullptr || g.a_scales == nullptr || g.b_scales == nullptr ||
      g.d == nullptr) {
    return Reject("mxfp8.gemm: codes, swizzled scales and an output");
  }
  if (!Aligned(g.a, 16) || !Aligned(g.b, 16) || !Aligned(g.a_scales, 16) ||
      !Aligned(g.b_scales, 16) || !Aligned(g.d, 16)) {
    return Reject("mxfp8.gemm: operands 16-byte aligned");
  }
  if (variant < 0 || variant > 2) return Reject("mxfp8.gemm: variant 0 (rule), 1 (one CTA a tile) or 2 (CTA pairs)");
  if (const int status = DeviceStatus(); status != 0) return status;
  if (sms <= 0) sms = SmCount();
  unsigned int* faults = FaultCounter();
  if (faults == nullptr) return Reject("mxfp8.gemm: no fault counter on this device");
  // Once a device: shared-memory limits, and how many CTA pairs it holds at once.
  static thread_local int configured_device = -1;
  static thread_local int resident_pairs = 0;
  int device = -1;
  cudaGetDevice(&device);
  if (configured_device != device) {
    cudaError_t e = cudaFuncSetAttribute(Mxfp8GemmKernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kGemmSmem);
    if (e == cudaSuccess) {
      e = cudaFuncSetAttribute(Mxfp8GemmPairKernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kPairSmem);
    }
    if (e != cudaSuccess) return Failed(e, "mxfp8.gemm attribute");
    const int clusters = llmp_b200_mxfp8_gemm_resident_pairs();
    resident_pairs = clusters;
    configured_device = device;
  }
  // Pairs once the matrix has more than one 128-row tile of rows (a pair's second CTA would
  // otherwise multiply zeros), and only if the device holds pairs of this size at all.
  const bool pairs = variant == 2 || (variant == 0 && g.m > kBM && resident_pairs > 0);
  if (pairs && resident_pairs < 1) return Reject("mxfp8.gemm: this device holds no CTA pair of the kernel's size");
  CUtensorMap map_a, map_b;
  if (!tc::MakeMapBytes2D(&map_a, g.a, static_cast<std::uint64_t>(g.m), static_cast<std::uint64_t>(g.k),
                          static_cast<std::uint64_t>(g.k), kBM, kBK) ||
      !tc::MakeMapBytes2D(&map_b, g.b, static_cast<std::uint64_t>(g.n), static_cast<std::uint64_t>(g.k),
                          static_cast<std::uint64_t>(g.k), pairs ? kPairHalfN : kBN, kBK)) {
    return Reject("mxfp8.gemm: the driver refused a tensor map for these operands");
  }
  const auto* a_scales = static_cast<const std::uint8_t*>(g.a_scales);
  const auto* b_scales = static_cast<const std::uint8_t*>(g.b_scales);
  const int n_padded = static_cast<int>(llmp_b200_mxfp8_padded_rows(static_cast<uint64_t>(g.n)));
  if (pairs) {
    const int tiles = ((g.m + kPairBM - 1) / kPairBM) * ((g.n + kBN - 1) / kBN);
    int count = tiles < sms / 2 ? tiles : sms / 2;
    if (count > resident_pairs) count = resident_pairs;
    if (count < 1) count = 1;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2u * static_cast<unsigned>(count));
    config.blockDim = dim3(kGemmThreads);
    config.dynamicSmemBytes = kPairSmem;
    config.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute cluster[1];
    cluster[0].id = cudaLaunchAttributeClusterDimension;
    cluster[0].val.clusterDim.x = 2;
    cluster[0].val.clusterDim.y = 1;
    cluster[0].val.clusterDim.z = 1;
    config.attrs = cluster;
    config.numAttrs = 1;
    const int m_padded = static_cast<int>(llmp_b200_mxfp8_padded_rows(static_cast<uint64_t>(g.m)));
    const cudaError_t e = cudaLaunchKernelEx(&config, Mxfp8GemmPairKernel, map_a, map_b, a_scales,
                                             b_scales, g.d, g.m, g.n, g.k, g.bf16 ? 1 : 0, m_padded,
                                             n_padded, faults);
    if (e != cudaSuccess) return Failed(e, "mxfp8.gemm pair launch");
    return 0;
  }
  const int tiles = ((g.m + kBM - 1) / kBM) * ((g.n + kBN - 1) / kBN);
  const int grid = tiles < sms ? tiles : sms;
  Mxfp8GemmKernel<<<grid, kGemmThreads, kGemmSmem, static_cast<cudaStream_t>(stream)>>>(
      map_a, map_b, a_scales, b_scales, g.d, g.m, g.n, g.k, g.bf16 ? 1 : 0, n_padded, faults);
  const cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return Failed(cudaGetLastError(), "mxfp8.gemm launch");
  return 0;
}

int llmp_b200_mxfp8_gemm(const llmp_b200_mxfp8_gemm_desc* gemm, int sms, void* stream) {
  return llmp_b200_mxfp8_gemm_variant(gemm, sms, 0, stream);
}



int llmp_b200_mxfp8_gemm_resident_pairs(void) {
  using namespace llmp_b200;
  if (DeviceStatus() != 0) return 0;
  if (cudaFuncSetAttribute(Mxfp8GemmPairKernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kPairSmem) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaLaunchConfig_t probe = {};
  probe.gridDim = dim3(2u * static_cast<unsigned>(SmCount()));
  probe.blockDim = dim3(kGemmThreads);
  probe.dynamicSmemBytes = kPairSmem;
  cudaLaunchAttribute cluster[1];
  cluster[0].id = cudaLaunchAttributeClusterDimension;
  cluster[0].val.clusterDim.x = 2;
  cluster[0].val.clusterDim.y = 1;
  cluster[0].val.clusterDim.z = 1;
  probe.attrs = cluster;
  probe.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, Mxfp8GemmPairKernel, &probe) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return clusters;
}

}  // extern "C"
