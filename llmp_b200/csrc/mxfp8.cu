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
  GridDependencyWait();
  const std::int64_t i = (static_cast<std::int64_t>(blockIdx.x) * 256) + threadIdx.x;
  const bool live = i < lanes_total;
  const std::int64_t item = (live ? i : 0) / 8;
  const int part = static_cast<int>(i % 8);
  const int blocks = k / 32;
  const int r = static_cast<int>(item / blocks);
  const int b = static_cast<int>(item % blocks);
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
    if (lane == 0) {
      tc::PrefetchMap(&map_a);
      tc::PrefetchMap(&map_b);
      std::uint32_t it = 0;
      for (int t = static_cast<int>(blockIdx.x); t < tiles && !*abort_flag; t += gridDim.x) {
        const int mb = t % tiles_m, nb = t / tiles_m;
        for (int ks = 0; ks < ksteps; ++ks, ++it) {
          const int s = static_cast<int>(it % kStages);
          if (!tc::MbarWait(&sh->empty[s], ((it / kStages) & 1u) ^ 1u)) {
            *abort_flag = 1;
            atomicAdd(faults, 1u);
            break;
          }
          // The tile's B rows [nb * 192, +192) touch two scale atoms (128 rows each).
          const int atom0 = (nb * kBN) / 128;
          const bool second = (atom0 + 1) * 128 < sfb_rows_padded;
          tc::MbarExpectTx(&sh->full[s], kABytes + kBBytes + kSfaBytes + (second ? 1024u : 512u));
          tc::TmaLoad2D(a_tiles + (s * kABytes), &map_a, ks * kBK, mb * kBM, &sh->full[s]);
          tc::TmaLoad2D(b_tiles + (s * kBBytes), &map_b, ks * kBK, nb * kBN, &sh->full[s]);
          tc::BulkLoad(sfa_tiles + (s * kSfaBytes),
                       sfa + ((static_cast<std::size_t>(mb) * (kb / 4) + ks) * 512), 512,
                       &sh->full[s]);
          tc::BulkLoad(sfb_tiles + (s * kSfbBytes),
                       sfb + ((static_cast<std::size_t>(atom0) * (kb / 4) + ks) * 512), 512,
                       &sh->full[s]);
          if (second) {
            tc::BulkLoad(sfb_tiles + (s * kSfbBytes) + 512,
                         sfb + ((static_cast<std::size_t>(atom0 + 1) * (kb / 4) + ks) * 512), 512,
                         &sh->full[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      std::uint32_t it = 0, tile_it = 0;
      for (int t = static_cast<int>(blockIdx.x); t < tiles && !*abort_flag; t += gridDim.x, ++tile_it) {
        const int nb = t / tiles_m;
        const int acc = static_cast<int>(tile_it & 1u);
        if (!tc::MbarWait(&sh->tmem_empty[acc], ((tile_it >> 1) & 1u) ^ 1u)) {
          *abort_flag = 1;
          atomicAdd(faults, 1u);
          break;
        }
        tc::TcFenceAfter();
        const std::uint32_t tacc = tmem + (acc * kAccColumns);
        // The two atoms always land on 4-column boundaries (tcgen05.cp's unit); an
        // odd tile starts in the middle of its first atom, whose last two columns
        // (rows 64..127) are the tile's first two: the MMA reads from +2.
        const int shift = (nb & 1) ? 2 : 0;
        for (int ks = 0; ks < ksteps; ++ks, ++it) {
          const int s = static_cast<int>(it % kStages);
          if (!tc::MbarWait(&sh->full[s], (it / kStages) & 1u)) {
            *abort_flag = 1;
            atomicAdd(faults, 1u);
            break;
          }
          tc::TcFenceAfter();
          const std::uint32_t tsfa = tmem + kSfColumn + (s * kSfStride);
          const std::uint32_t tsfb = tsfa + 4 + shift;
          tc::TmemCopyScales(tsfa, tc::SmemDesc(sfa_tiles + (s * kSfaBytes), false, 128));
          tc::TmemCopyScales(tsfa + 4, tc::SmemDesc(sfb_tiles + (s * kSfbBytes), false, 128));
          tc::TmemCopyScales(tsfa + 8,
                             tc::SmemDesc(sfb_tiles + (s * kSfbBytes) + 512, false, 128));
          const std::uint64_t adesc = tc::SmemDesc(a_tiles + (s * kABytes), true, 1024);
          const std::uint64_t bdesc = tc::SmemDesc(b_tiles + (s * kBBytes), true, 1024);
#pragma unroll
          for (int kk = 0; kk < kBK / kUmmaK; ++kk) {
            // 32 bytes along K inside the 128-byte swizzle row: +2 in 16-byte units
            tc::MmaMxf8(tacc, adesc + (kk * 2), bdesc + (kk * 2), tc::IdescMxf8(kBM, kBN, kk, kk),
                        ks > 0 || kk > 0, tsfa, tsfb);
          }
          tc::TcCommit(&sh->empty[s]);  // the stage's bytes are free once these MMAs retire
        }
        tc::TcCommit(&sh->tmem_full[acc]);
      }
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
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        std::uint32_t r[32];
        tc::TmemLoad32(tmem + (static_cast<std::uint32_t>(quadrant * 32) << 16) +
                           (acc * kAccColumns) + (c * 32), r);
        tc::TmemLoadWait();
        const int col = (nb * kBN) + (c * 32);
        if (row < m && col < n) {
          if (bf16) {
            auto* out = static_cast<__nv_bfloat16*>(d) + (static_cast<std::size_t>(row) * n) + col;
            if (col + 32 <= n && (n % 8) == 0) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 q;
                std::uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(r[(8 * v) + (2 * j)]),
                                                                 __uint_as_float(r[(8 * v) + (2 * j) + 1]));
                  w[j] = *reinterpret_cast<const std::uint32_t*>(&p);
                }
                q = make_uint4(w[0], w[1], w[2], w[3]);
                reinterpret_cast<uint4*>(out)[v] = q;
              }
            } else {
              for (int j = 0; j < 32 && col + j < n; ++j) {
                out[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
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
              for (int j = 0; j < 32 && col + j < n; ++j) out[j] = __uint_as_float(r[j]);
            }
          }
        }
      }
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

int llmp_b200_mxfp8_gemm(const llmp_b200_mxfp8_gemm_desc* gemm, int sms, void* stream) {
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
  if (const int status = DeviceStatus(); status != 0) return status;
  if (sms <= 0) sms = SmCount();
  CUtensorMap map_a, map_b;
  if (!tc::MakeMapBytes2D(&map_a, g.a, static_cast<std::uint64_t>(g.m), static_cast<std::uint64_t>(g.k),
                          static_cast<std::uint64_t>(g.k), kBM, kBK) ||
      !tc::MakeMapBytes2D(&map_b, g.b, static_cast<std::uint64_t>(g.n), static_cast<std::uint64_t>(g.k),
                          static_cast<std::uint64_t>(g.k), kBN, kBK)) {
    return Reject("mxfp8.gemm: the driver refused a tensor map for these operands");
  }
  unsigned int* faults = FaultCounter();
  if (faults == nullptr) return Reject("mxfp8.gemm: no fault counter on this device");
  static thread_local int configured_device = -1;
  int device = -1;
  cudaGetDevice(&device);
  if (configured_device != device) {
    const cudaError_t e = cudaFuncSetAttribute(
        Mxfp8GemmKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem);
    if (e != cudaSuccess) return Failed(e, "mxfp8.gemm attribute");
    configured_device = device;
  }
  const int tiles = ((g.m + kBM - 1) / kBM) * ((g.n + kBN - 1) / kBN);
  const int grid = tiles < sms ? tiles : sms;
  Mxfp8GemmKernel<<<grid, kGemmThreads, kGemmSmem, static_cast<cudaStream_t>(stream)>>>(
      map_a, map_b, static_cast<const std::uint8_t*>(g.a_scales),
      static_cast<const std::uint8_t*>(g.b_scales), g.d, g.m, g.n, g.k, g.bf16 ? 1 : 0,
      static_cast<int>(llmp_b200_mxfp8_padded_rows(static_cast<uint64_t>(g.n))), faults);
  const cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return Failed(cudaGetLastError(), "mxfp8.gemm launch");
  return 0;
}

}  // extern "C"
