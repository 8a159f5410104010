// The decode module's matrix product on B200: y = W x for any number of F32
// activation rows, the weight decoded on the fly and both operands rounded to
// the decoder's 16-bit MMA element (FP16 for Q8_0 blocks, BF16 for MXFP8), F32
// accumulation.  Interface and numerics follow decode::RunMatrix with
// MatrixPath::kMma (src/kernels/decode/products.h:96-120; tile kernel
// templates.cuh:236-440, which decodes to D::Mma and runs mma.sync tiles); the
// structure is B200's: tcgen05.mma kind::f16 with the whole K accumulated in
// tensor memory, operands written by decode warps straight into the
// 128-byte-swizzled K-major tiles the MMA reads.
//
//   warp 0       allocates TMEM, issues four MMAs (128 x 128 x 16) a k-step of 64
//                values, commits each stage back to the writers;
//   warps 1-4    weights: a thread a weight row, 64 values a k-step decoded
//                (d * q, or e4m3 * 2^(e-127)), rounded to the MMA element;
//   warps 5-8    activations: a thread an activation row, 64 floats a k-step
//                rounded to the MMA element;
//   warps 9-12   epilogue: the tile out of tensor memory, times the row's tensor
//                scale, to y.
// Rows past the matrix or the batch are written as zeros.  Every wait is bounded.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "tc.cuh"

namespace llmp_b200 {
namespace {

using Operand = llmp_b200_decode_operand;

constexpr int kTile = 128;     // weight rows (TMEM lanes) and activation rows (columns) a tile
constexpr int kStepK = 64;     // values a k-step: one 128-byte swizzle row of 16-bit elements
constexpr int kStages = 4;
constexpr int kTileBytes = kTile * 128;
constexpr int kThreads = 13 * 32;
constexpr int kSmem = (kStages * 2 * kTileBytes) + 1024 + 256;

struct Shared {
  std::uint64_t full[kStages];   // eight writer warps have filled the stage
  std::uint64_t empty[kStages];  // the tensor core has read it
  std::uint64_t done;            // the tile's sum is complete
  std::uint32_t tmem_base;
  std::uint32_t abort;
};

struct Args {
  Operand w;
  std::uint32_t first, outputs, rows;
  const float* x;
  std::uint64_t x_stride;
  float* y;
  std::uint64_t y_stride;
  // Grouped (decode::RunGrouped): grid z names the expert; its pairs [offsets[e],
  // offsets[e + 1]) are the tile's activation rows, x rows pair_rows[p], y rows
  // pair_out[p] (or p).  `w` then carries the format's k, rows and decoder.
  const Operand* experts;
  const std::int32_t* offsets;
  const std::int32_t* pair_rows;
  const std::int32_t* pair_out;
  std::uint32_t pairs, x_rows, y_rows;
};

__device__ __forceinline__ float E8m0(std::uint32_t e) {
  return e == 0 ? __uint_as_float(0x00400000u) : e == 255 ? __uint_as_float(0x7fffffffu)
                                                           : __uint_as_float(e << 23);
}

template <bool kBf16>
__device__ __forceinline__ std::uint32_t Pack(float lo, float hi) {
  if constexpr (kBf16) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const std::uint32_t*>(&p);
  } else {
    const __half2 p = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const std::uint32_t*>(&p);
  }
}

// 64 values of row `row` from value k0 on, as 32 packed pairs.
template <int kDecoder>
__device__ __forceinline__ void DecodeRow(const Operand& p, std::uint32_t row, std::uint32_t k0,
                                          std::uint32_t (&out)[32]) {
  constexpr bool kBf16 = kDecoder != LLMP_B200_DECODER_Q8_0_BLOCKS;
  const auto* data = static_cast<const std::uint8_t*>(p.data);
#pragma unroll
  for (int b = 0; b < 2; ++b) {
    const std::uint32_t kb = k0 + (b * 32);
    if (kb >= p.k) {
#pragma unroll
      for (int i = 0; i < 16; ++i) out[(16 * b) + i] = 0u;
      continue;
    }
    if constexpr (kDecoder == LLMP_B200_DECODER_Q8_0_BLOCKS) {
      const std::uint8_t* block = data + (row * p.row_bytes) + (static_cast<std::uint64_t>(kb / 32) * 34);
      const auto* h = reinterpret_cast<const unsigned short*>(block);
      const float d = HalfBitsToFloat(__ldg(h));
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const std::uint32_t pair = __ldg(h + 1 + i);
        out[(16 * b) + i] = Pack<kBf16>(d * static_cast<float>(static_cast<std::int8_t>(pair & 0xffu)),
                                        d * static_cast<float>(static_cast<std::int8_t>(pair >> 8)));
      }
    } else {
      const auto* scales = static_cast<const std::uint8_t*>(p.scales);
      const std::uint32_t blocks = p.k / 32, block = kb / 32;
      const std::uint64_t at =
          kDecoder == LLMP_B200_DECODER_MXFP8_SPLIT
              ? (static_cast<std::uint64_t>(row) * blocks) + block
              : ((((static_cast<std::uint64_t>(row) / 128) * (blocks / 4)) + (block / 4)) * 512) +
                    ((row % 32) * 16) + (((row % 128) / 32) * 4) + (block % 4);
      const float s = E8m0(__ldg(scales + at));
      const auto* codes = reinterpret_cast<const uint4*>(data + (row * p.row_bytes) + kb);
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const uint4 c = __ldg(codes + q);
        const std::uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const __half2_raw hh = __nv_cvt_fp8x2_to_halfraw2(
              static_cast<__nv_fp8x2_storage_t>((w[i / 2] >> (16 * (i % 2))) & 0xffffu), __NV_E4M3);
          out[(16 * b) + (8 * q) + i] = Pack<kBf16>(__half2float(__ushort_as_half(hh.x)) * s,
                                                    __half2float(__ushort_as_half(hh.y)) * s);
        }
      }
    }
  }
}

// Row t's 128 bytes into the swizzled tile: 16-byte chunk j at j ^ (t % 8).
__device__ __forceinline__ void StoreRow(unsigned char* tile, int t, const std::uint32_t (&v)[32]) {
  unsigned char* row = tile + ((t >> 3) * 1024) + ((t & 7) * 128);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    *reinterpret_cast<uint4*>(row + ((j ^ (t & 7)) * 16)) =
        make_uint4(v[4 * j], v[(4 * j) + 1], v[(4 * j) + 2], v[(4 * j) + 3]);
  }
}

template <int kDecoder, bool kGrouped>
__global__ void __launch_bounds__(kThreads, 1) DecodeMatrixKernel(const Args a, unsigned int* faults) {
  constexpr bool kBf16 = kDecoder != LLMP_B200_DECODER_Q8_0_BLOCKS;
  // The tile's weight and its activation rows [begin + m0, end).
  Operand w = a.w;
  std::uint32_t begin = 0, end = a.rows;
  if constexpr (kGrouped) {
    // The worklist and the operand table may be the kernel before's output.
    GridDependencyWait();
    const std::uint32_t e = blockIdx.z;
    const std::int32_t lo = a.offsets[e], hi = a.offsets[e + 1];
    begin = lo < 0 ? 0u : min(static_cast<std::uint32_t>(lo), a.pairs);
    end = hi < 0 ? begin : max(begin, min(static_cast<std::uint32_t>(hi), a.pairs));
    if (begin + (blockIdx.y * kTile) >= end) return;  // uniform: before any barrier
    w = a.experts[e];
    if (w.k != a.w.k || w.rows != a.w.rows || w.decoder != a.w.decoder) return;  // not of the format
    // The host never sees these device-resident operands: an expert whose pointers
    // or pitch the loads below could not take is skipped and counted, not read.
    const bool q8 = kDecoder == LLMP_B200_DECODER_Q8_0_BLOCKS;
    const std::uintptr_t where = reinterpret_cast<std::uintptr_t>(w.data);
    const bool usable =
        w.data != nullptr &&
        (q8 ? ((where | w.row_bytes) % 2 == 0 && w.row_bytes >= (w.k / 32) * 34ull)
            : ((where | w.row_bytes) % 16 == 0 && w.row_bytes >= w.k && w.scales != nullptr)) &&
        (w.tensor_scale == nullptr || w.rows_per_scale >= 1);
    if (!usable) {
      if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) atomicAdd(faults, 1u);
      return;
    }
  }
  extern __shared__ unsigned char raw_smem[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<std::uintptr_t>(raw_smem) + 1023) & ~static_cast<std::uintptr_t>(1023));
  unsigned char* w_tiles = smem;
  unsigned char* x_tiles = smem + (kStages * kTileBytes);
  Shared* sh = reinterpret_cast<Shared*>(x_tiles + (kStages * kTileBytes));

  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const std::uint32_t n0 = blockIdx.x * kTile;  // first output (weight row first + n0)
  const std::uint32_t m0 = begin + (blockIdx.y * kTile);  // first activation row (pair)
  const int ksteps = static_cast<int>((w.k + kStepK - 1) / kStepK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::MbarInit(&sh->full[s], 8);
      tc::MbarInit(&sh->empty[s], 1);
    }
    tc::MbarInit(&sh->done, 1);
    sh->abort = 0;
    tc::MbarInitFence();
  }
  if (warp == 0) {
    tc::TmemAlloc(&sh->tmem_base, 128);
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

  GridDependencyWait();  // the activations may be the kernel before's output
  if (warp == 0) {
    if (lane == 0) {
      const std::uint32_t idesc = tc::IdescF16(kTile, kTile, kBf16);
      for (int ks = 0; ks < ksteps && !*abort_flag; ++ks) {
        const int s = ks % kStages;
        if (!tc::MbarWait(&sh->full[s], (ks / kStages) & 1)) {
          give_up();
          break;
        }
        tc::TcFenceAfter();
        const std::uint64_t wdesc = tc::SmemDesc(w_tiles + (s * kTileBytes), true, 1024);
        const std::uint64_t xdesc = tc::SmemDesc(x_tiles + (s * kTileBytes), true, 1024);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {  // 16 values = 32 bytes along the swizzled row
          tc::MmaF16(tmem, wdesc + (kk * 2), xdesc + (kk * 2), idesc, ks > 0 || kk > 0);
        }
        tc::TcCommit(&sh->empty[s]);
      }
      tc::TcCommit(&sh->done);
    }
  } else if (warp <= 8) {
    const bool weights = warp <= 4;
    const int t = (static_cast<int>(threadIdx.x) - (weights ? 32 : 160));  // 0..127
    // The activation row this thread converts (grouped: the pair's x row; a pair naming a
    // row past x is computed as zeros and never stored).
    std::uint32_t x_row = m0 + t;
    bool x_live = m0 + t < end;
    if constexpr (kGrouped) {
      if (!weights && x_live) {
        const std::int32_t pr = __ldg(a.pair_rows + m0 + t);
        x_live = pr >= 0 && static_cast<std::uint32_t>(pr) < a.x_rows;
        x_row = static_cast<std::uint32_t>(pr);
      }
    }
    for (int ks = 0; ks < ksteps && !*abort_flag; ++ks) {
      const int s = ks % kStages;
      std::uint32_t v[32];
      if (weights) {
        if (n0 + t < a.outputs) {
          DecodeRow<kDecoder>(w, a.first + n0 + t, static_cast<std::uint32_t>(ks) * kStepK, v);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
      } else {
        const std::uint32_t k0 = static_cast<std::uint32_t>(ks) * kStepK;
        if (x_live) {
          const auto* xp = reinterpret_cast<const float4*>(a.x + (static_cast<std::uint64_t>(x_row) * a.x_stride) + k0);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float4 f = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (k0 + (4 * i) < w.k) f = __ldg(xp + i);   // k is a multiple of 32: whole float4s
            v[2 * i] = Pack<kBf16>(f.x, f.y);
            v[(2 * i) + 1] = Pack<kBf16>(f.z, f.w);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
      }
      bool ok = true;
      if (lane == 0) ok = tc::MbarWait(&sh->empty[s], ((ks / kStages) & 1) ^ 1);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) {
        if (lane == 0) give_up();
        break;
      }
      StoreRow((weights ? w_tiles : x_tiles) + (s * kTileBytes), t, v);
      tc::FenceProxyAsync();  // generic-proxy writes, read by the tensor core's proxy
      __syncwarp();
      if (lane == 0) tc::MbarArrive(&sh->full[s]);
    }
  } else {
    const int quadrant = warp & 3;  // the TMEM lanes this warp may read
    bool ok = true;
    if (lane == 0) ok = tc::MbarWait(&sh->done, 0);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok) {
      if (lane == 0) give_up();
    } else {
      tc::TcFenceAfter();
      const std::uint32_t n = n0 + (quadrant * 32) + lane;  // this thread's output
      const float scale = (n < a.outputs && w.tensor_scale != nullptr)
                              ? __ldg(w.tensor_scale + ((a.first + n) / w.rows_per_scale))
                              : 1.0f;
#pragma unroll 1
      for (int c = 0; c < kTile / 32; ++c) {
        std::uint32_t r[32];
        tc::TmemLoad32(tmem + (static_cast<std::uint32_t>(quadrant * 32) << 16) + (c * 32), r);
        tc::TmemLoadWait();
        if (n < a.outputs) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const std::uint32_t m = m0 + (c * 32) + j;
            if (m >= end) continue;
            std::uint32_t out = m;
            if constexpr (kGrouped) {
              const std::int32_t pr = __ldg(a.pair_rows + m);
              if (pr < 0 || static_cast<std::uint32_t>(pr) >= a.x_rows) continue;
              if (a.pair_out != nullptr) {
                const std::int32_t po = __ldg(a.pair_out + m);
                if (po < 0) continue;
                out = static_cast<std::uint32_t>(po);
              }
              if (out >= a.y_rows) continue;
            }
            a.y[(static_cast<std::uint64_t>(out) * a.y_stride) + n] = __uint_as_float(r[j]) * scale;
          }
        }
      }
    }
  }

  tc::TcFenceBefore();
  __syncthreads();
  if (warp == 0) {
    tc::TcFenceAfter();
    tc::TmemDealloc(tmem, 128);
  }
}

template <int kDecoder, bool kGrouped>
cudaError_t Launch(const Args& a, unsigned int groups, unsigned int* faults, cudaStream_t s) {
  static thread_local int configured_device = -1;
  int device = -1;
  cudaGetDevice(&device);
  if (configured_device != device) {
    const cudaError_t e = cudaFuncSetAttribute(DecodeMatrixKernel<kDecoder, kGrouped>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return e;
    configured_device = device;
  }
  // Grouped: every expert gets the row tiles its pairs could need at most; a CTA whose
  // tile lies past the expert's pairs leaves at once.
  const std::uint32_t rows = kGrouped ? a.pairs : a.rows;
  const dim3 grid((a.outputs + kTile - 1) / kTile, (rows + kTile - 1) / kTile, groups);
  return LaunchPdl(DecodeMatrixKernel<kDecoder, kGrouped>, grid, dim3(kThreads),
                   static_cast<std::size_t>(kSmem), s, a, faults);
}

int CheckFormat(const Operand& w, const char* what) {
  if (w.decoder > LLMP_B200_DECODER_MXFP8_ATOMS) {
    return Reject("%s: decoder %u is not one this build has (Q8_0 blocks, MXFP8)", what, w.decoder);
  }
  if (w.k < 32 || w.k % 32 != 0 || w.rows < 1 ||
      (w.decoder == LLMP_B200_DECODER_MXFP8_ATOMS && w.k % 128 != 0)) {
    return Reject("%s: k a positive multiple of 32 (128 with scale atoms), at least one row", what);
  }
  return 0;
}

template <bool kGrouped>
cudaError_t LaunchDecoder(const Args& a, unsigned int groups, unsigned int* faults, cudaStream_t s) {
  return a.w.decoder == LLMP_B200_DECODER_Q8_0_BLOCKS
             ? Launch<LLMP_B200_DECODER_Q8_0_BLOCKS, kGrouped>(a, groups, faults, s)
         : a.w.decoder == LLMP_B200_DECODER_MXFP8_SPLIT
             ? Launch<LLMP_B200_DECODER_MXFP8_SPLIT, kGrouped>(a, groups, faults, s)
             : Launch<LLMP_B200_DECODER_MXFP8_ATOMS, kGrouped>(a, groups, faults, s);
}

}  // namespace
}  // namespace llmp_b200

extern "C" {

int llmp_b200_decode_matrix(const llmp_b200_decode_product* product, void* stream) {
  using namespace llmp_b200;
  if (product == nullptr) return Reject("decode.matrix: null product");
  const Operand& w = product->w;
  if (w.decoder > LLMP_B200_DECODER_MXFP8_ATOMS) {
    return Reject("decode.matrix: decoder %u is not one this build has (Q8_0 blocks, MXFP8)", w.decoder);
  }
  const bool q8 = w.decoder == LLMP_B200_DECODER_Q8_0_BLOCKS;
  if (w.data == nullptr || w.k < 32 || w.k % 32 != 0 || w.rows < 1 ||
      w.row_bytes < (q8 ? (w.k / 32) * 34ull : w.k) ||
      (q8 ? (!Aligned(w.data, 2) || w.row_bytes % 2 != 0)
          : (!Aligned(w.data, 16) || w.row_bytes % 16 != 0 || w.scales == nullptr)) ||
      (w.decoder == LLMP_B200_DECODER_MXFP8_ATOMS && w.k % 128 != 0) ||
      (w.tensor_scale != nullptr && w.rows_per_scale < 1)) {
    return Reject("decode.matrix: a Q8_0 (2-byte aligned) or MXFP8 (16-byte aligned, with scales) weight "
                  "of k a positive multiple of 32");
  }
  if (product->outputs < 1 || product->rows < 1 || product->x == nullptr || product->y == nullptr ||
      product->first + product->outputs > w.rows || product->rows > 0x7fffff80ull ||
      product->outputs > 0x7fffff80ull) {
    return Reject("decode.matrix: at least one activation row and output, rows inside the matrix");
  }
  if (product->x_stride < w.k || product->y_stride < product->outputs || !Aligned(product->x, 16) ||
      product->x_stride % 4 != 0 || !Aligned(product->y, 4)) {
    return Reject("decode.matrix: activation rows of k floats, 16-byte aligned; output rows of "
                  "`outputs` floats");
  }
  if ((product->rows + 127) / 128 > 65535) return Reject("decode.matrix: more row tiles than a grid holds");
  if (const int status = DeviceStatus(); status != 0) return status;
  unsigned int* faults = FaultCounter();
  if (faults == nullptr) return Reject("decode.matrix: no fault counter on this device");
  Args a{};
  a.w = w;
  a.first = static_cast<std::uint32_t>(product->first);
  a.outputs = static_cast<std::uint32_t>(product->outputs);
  a.rows = static_cast<std::uint32_t>(product->rows);
  a.x = product->x;
  a.x_stride = product->x_stride;
  a.y = product->y;
  a.y_stride = product->y_stride;
  const cudaError_t e = LaunchDecoder<false>(a, 1, faults, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return Failed(e, "decode.matrix launch");
  return 0;
}

int llmp_b200_decode_grouped(const llmp_b200_decode_grouped_product* g, void* stream) {
  using namespace llmp_b200;
  if (g == nullptr) return Reject("decode.grouped: null product");
  if (const int status = CheckFormat(g->format, "decode.grouped"); status != 0) return status;
  if (g->experts == nullptr || g->experts_count < 1 || g->experts_count > 65535 ||
      g->offsets == nullptr || g->pair_rows == nullptr || g->x == nullptr || g->y == nullptr) {
    return Reject("decode.grouped: 1 to 65535 expert operands, offsets, pair rows, x and y");
  }
  if (g->outputs < 1 || g->first + g->outputs > g->format.rows || g->pairs < 1 ||
      g->pairs > 0x7fffff80ull || (g->pairs + 127) / 128 > 65535 || g->x_rows < 1 || g->y_rows < 1) {
    return Reject("decode.grouped: outputs inside the matrices; 1 .. 8,388,480 pairs");
  }
  if (g->x_stride < g->format.k || g->y_stride < g->outputs || !Aligned(g->x, 16) ||
      g->x_stride % 4 != 0 || !Aligned(g->y, 4) || !Aligned(g->experts, 8)) {
    return Reject("decode.grouped: activation rows of k floats, 16-byte aligned; output rows of "
                  "`outputs` floats");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  unsigned int* faults = FaultCounter();
  if (faults == nullptr) return Reject("decode.grouped: no fault counter on this device");
  Args a{};
  a.w = g->format;
  a.first = static_cast<std::uint32_t>(g->first);
  a.outputs = static_cast<std::uint32_t>(g->outputs);
  a.rows = 0;
  a.x = g->x;
  a.x_stride = g->x_stride;
  a.y = g->y;
  a.y_stride = g->y_stride;
  a.experts = g->experts;
  a.offsets = g->offsets;
  a.pair_rows = g->pair_rows;
  a.pair_out = g->pair_out;
  a.pairs = static_cast<std::uint32_t>(g->pairs);
  a.x_rows = static_cast<std::uint32_t>(g->x_rows);
  a.y_rows = static_cast<std::uint32_t>(g->y_rows);
  const cudaError_t e = LaunchDecoder<true>(a, static_cast<unsigned int>(g->experts_count), faults,
                                            static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return Failed(e, "decode.grouped launch");
  return 0;
}

}  // extern "C"
