// The decode module's vector products and row lookups: y = W x with F32
// activations and the weight decoded on the fly, 1 to 16 activation rows, plain
// or as the GLU of a gate and an up product (decode::RunVector / RunVectorGlu,
// src/kernels/decode/products.h:96-147), and the decoded rows themselves
// (decode::RunRows, products.h:170-186).
//
// What is kept from the reference is the ARITHMETIC, because its results are the
// contract (templates.cuh:95-145): a weight row's sum is formed by 32 partial
// sums, partial l over the 16-value segments l, l + 32, ... with one fused
// multiply-add a value in index order; the partials meet in a butterfly 16, 8,
// 4, 2, 1 apart; the sum is scaled by the row's tensor scale.  The kernel
// around that order is this build's:
//
//   * persistent CTAs, one an SM, each owning a contiguous run of output rows
//     that its warps split; a warp walks its rows one at a time;
//   * a row's bytes (both matrices' with a GLU) arrive in the warp's PRIVATE
//     ring of shared-memory stages by the bulk-copy engine (cp.async.bulk
//     completing on the stage's mbarrier), several rows ahead of the one being
//     summed, and the first of them are requested before the programmatic-
//     dependency wait: weights depend on no earlier kernel.  Warps never
//     synchronize with each other after the activations are staged;
//   * a lane reads its segment out of the staged row with the widest aligned
//     shared load the encoding allows (Q8_0's 34-byte blocks put a segment on a
//     2-byte boundary: five aligned words and a funnel shift);
//   * the activation rows are staged once a CTA when they fit, else read
//     through L1;
//   * rows that are not 16-byte aligned (Q8_0 only promises 2), or too long for
//     the ring, are read in place with the loads their alignment allows.
// Every mbarrier wait is bounded; a wait that runs out raises the device fault
// counter and the warp stores nothing more.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <algorithm>

#include "common.cuh"
#include "tc.cuh"

namespace llmp_b200 {
namespace {

using Operand = llmp_b200_decode_operand;

constexpr int kMaxWarps = 16;
constexpr int kMaxStages = 4;
constexpr int kRingBudget = 144 * 1024;
constexpr int kActsBudget = 64 * 1024;

struct Args {
  Operand w, w2;
  std::uint32_t first, first2, outputs, rows;
  const float* x;
  std::uint64_t x_stride;
  float* y;
  std::uint64_t y_stride;
  int glu;  // -1: plain product
  float limit;
};

struct Plan {
  int grid, warps, stages;
  std::uint32_t copy_bytes;   // a row's bytes as the bulk copy moves them (0: rows are read in place)
  std::uint32_t stage_bytes;  // one stage: copy_bytes x matrices, 16-byte multiples
  std::uint32_t acts_bytes;   // the staged activations (0: read through L1)
  unsigned int* faults;
};

// ---------------------------------------------------------------- elements
__device__ __forceinline__ float E8m0(std::uint32_t e) {
  // 2^(e - 127); e = 0 is the subnormal 2^-127, e = 255 NaN
  return e == 0 ? __uint_as_float(0x00400000u) : e == 255 ? __uint_as_float(0x7fffffffu)
                                                           : __uint_as_float(e << 23);
}
// E2M1 (sign, two exponent bits, one mantissa bit; bias 1; e = 0 is subnormal):
// +-{0, 0.5, 1, 1.5, 2, 3, 4, 6}, assembled as F32 bits.
__device__ __forceinline__ float E2m1(std::uint32_t code) {
  const std::uint32_t e = (code >> 1) & 3u, m = code & 1u;
  const std::uint32_t magnitude = e != 0 ? ((e + 126u) << 23) | (m << 22) : m * 0x3F000000u;
  return __uint_as_float(magnitude | ((code & 8u) << 28));
}
// One E4M3 byte (OCP: bias 7, subnormals, 0x7F / 0xFF NaN) through the hardware conversion.
__device__ __forceinline__ float E4m3(std::uint32_t byte) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
  return __half2float(__ushort_as_half(h.x));
}
// NVFP4's block scale: E4M3's value for 0x00-0x7E, NaN from 0x7F up.
__device__ __forceinline__ float Ue4m3(std::uint32_t byte) {
  return byte >= 0x7Fu ? __uint_as_float(0x7fffffffu) : E4m3(byte);
}
__host__ __device__ constexpr std::uint64_t AtomAt(std::uint64_t row, std::uint64_t block,
                                                   std::uint64_t blocks) {
  return ((((row / 128) * (blocks / 4)) + (block / 4)) * 512) + ((row % 32) * 16) +
         (((row % 128) / 32) * 4) + (block % 4);
}

// ---------------------------------------------------------------- decoders
// Bytes of a row's codes that hold one 16-value segment, per decoder.
__host__ __device__ constexpr int SegmentBytesX2(int decoder) {  // twice the bytes (Q8_0: 17)
  return decoder == LLMP_B200_DECODER_Q8_0_BLOCKS                                             ? 34
         : (decoder == LLMP_B200_DECODER_MXFP8_SPLIT || decoder == LLMP_B200_DECODER_MXFP8_ATOMS) ? 32
         : (decoder == LLMP_B200_DECODER_BF16_DENSE || decoder == LLMP_B200_DECODER_F16_DENSE)    ? 64
                                                                                                   : 16;
}

// Segment `seg` of a row whose code bytes start at `codes` (shared memory when
// `staged`, 16-byte aligned there; else global memory with the alignment the
// entry point checked) into v[16], each value decoded exactly as the reference's
// decoder does (decoders.cuh: code times block scale, exact in F32).
template <int kDecoder>
__device__ __forceinline__ void LoadSegment(const Operand& p, const std::uint8_t* codes, bool staged,
                                            std::uint32_t row, std::uint32_t seg, float (&v)[16]) {
  if constexpr (kDecoder == LLMP_B200_DECODER_Q8_0_BLOCKS) {
    // Half a 34-byte block: d at byte 34 b, the segment's 16 int8 at 34 b + 2 + 16 h.
    const std::uint32_t at = ((seg >> 1) * 34u) + 2u + ((seg & 1u) * 16u);
    std::uint32_t q[4];
    float d;
    if (staged) {
      // five aligned words cover the 16 bytes; they start two bytes in when at % 4 == 2
      const auto* words = reinterpret_cast<const std::uint32_t*>(codes + (at & ~3u));
      const std::uint32_t w0 = words[0], w1 = words[1], w2 = words[2], w3 = words[3];
      const std::uint32_t shift = (at & 2u) * 8u;
      const std::uint32_t w4 = shift != 0 ? words[4] : 0u;
      q[0] = __funnelshift_r(w0, w1, shift);
      q[1] = __funnelshift_r(w1, w2, shift);
      q[2] = __funnelshift_r(w2, w3, shift);
      q[3] = __funnelshift_r(w3, w4, shift);
      d = HalfBitsToFloat(*reinterpret_cast<const unsigned short*>(codes + ((seg >> 1) * 34u)));
    } else {
      const auto* h = reinterpret_cast<const unsigned short*>(codes + at);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        q[i] = static_cast<std::uint32_t>(__ldg(h + (2 * i))) |
               (static_cast<std::uint32_t>(__ldg(h + (2 * i) + 1)) << 16);
      }
      d = HalfBitsToFloat(__ldg(reinterpret_cast<const unsigned short*>(codes + ((seg >> 1) * 34u))));
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      v[i] = d * static_cast<float>(static_cast<std::int8_t>((q[i / 4] >> (8 * (i % 4))) & 0xffu));
    }
  } else if constexpr (kDecoder == LLMP_B200_DECODER_MXFP8_SPLIT ||
                       kDecoder == LLMP_B200_DECODER_MXFP8_ATOMS) {
    const auto* scales = static_cast<const std::uint8_t*>(p.scales);
    const std::uint32_t blocks = p.k / 32;
    const float s = E8m0(__ldg(scales + (kDecoder == LLMP_B200_DECODER_MXFP8_SPLIT
                                             ? (static_cast<std::uint64_t>(row) * blocks) + (seg >> 1)
                                             : AtomAt(row, seg >> 1, blocks))));
    const auto* src = reinterpret_cast<const uint4*>(codes + (seg * 16u));
    const uint4 c = staged ? *src : __ldg(src);
    const std::uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // two E4M3 bytes to two halves (exact), then to F32
      const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(
          static_cast<__nv_fp8x2_storage_t>((w[i / 2] >> (16 * (i % 2))) & 0xffffu), __NV_E4M3);
      v[2 * i] = __half2float(__ushort_as_half(h.x)) * s;
      v[(2 * i) + 1] = __half2float(__ushort_as_half(h.y)) * s;
    }
  } else if constexpr (kDecoder == LLMP_B200_DECODER_BF16_DENSE ||
                       kDecoder == LLMP_B200_DECODER_F16_DENSE) {
    const auto* src = reinterpret_cast<const uint4*>(codes + (seg * 32u));
    const uint4 c0 = staged ? src[0] : __ldg(src);
    const uint4 c1 = staged ? src[1] : __ldg(src + 1);
    const std::uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if constexpr (kDecoder == LLMP_B200_DECODER_BF16_DENSE) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[(2 * i) + 1] = __uint_as_float(w[i] & 0xffff0000u);
      } else {
        v[2 * i] = HalfBitsToFloat(w[i] & 0xffffu);
        v[(2 * i) + 1] = HalfBitsToFloat(w[i] >> 16);
      }
    }
  } else {
    // E2M1 codes, value 2 i in byte i's low nibble: NVFP4 (a UE4M3 scale a segment)
    // or MXFP4 (an E8M0 scale two segments), scales row-major or in scale atoms.
    const auto* scales = static_cast<const std::uint8_t*>(p.scales);
    constexpr bool kNv = kDecoder == LLMP_B200_DECODER_NVFP4_SPLIT ||
                         kDecoder == LLMP_B200_DECODER_NVFP4_ATOMS;
    constexpr bool kAtoms = kDecoder == LLMP_B200_DECODER_NVFP4_ATOMS ||
                            kDecoder == LLMP_B200_DECODER_MXFP4_ATOMS;
    const std::uint32_t blocks = kNv ? p.k / 16 : p.k / 32;
    const std::uint32_t block = kNv ? seg : seg >> 1;
    const std::uint32_t code = __ldg(scales + (kAtoms ? AtomAt(row, block, blocks)
                                                      : (static_cast<std::uint64_t>(row) * blocks) + block));
    const float s = kNv ? Ue4m3(code) : E8m0(code);
    const auto* src = reinterpret_cast<const uint2*>(codes + (seg * 8u));
    const uint2 c = staged ? *src : __ldg(src);
    const std::uint32_t w[2] = {c.x, c.y};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const std::uint32_t b = (w[i / 4] >> (8 * (i % 4))) & 0xffu;
      v[2 * i] = E2m1(b & 15u) * s;
      v[(2 * i) + 1] = E2m1(b >> 4) * s;
    }
  }
}

// acc[t] += v . x[t, 16 seg ..), one fused multiply-add a value in index order.
template <int kCols>
__device__ __forceinline__ void Accumulate(const float* xs, std::uint64_t xs_stride, bool xs_shared,
                                           std::uint32_t rows, std::uint32_t seg, const float (&w)[16],
                                           float (&acc)[kCols]) {
#pragma unroll
  for (int t = 0; t < kCols; ++t) {
    if (static_cast<std::uint32_t>(t) < rows) {
      const auto* xp = reinterpret_cast<const float4*>(xs + (static_cast<std::uint64_t>(t) * xs_stride) +
                                                       (seg * 16u));
      float s = acc[t];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 x = xs_shared ? xp[q] : __ldg(xp + q);
        s = fmaf(w[4 * q], x.x, s);
        s = fmaf(w[(4 * q) + 1], x.y, s);
        s = fmaf(w[(4 * q) + 2], x.z, s);
        s = fmaf(w[(4 * q) + 3], x.w, s);
      }
      acc[t] = s;
    }
  }
}

__device__ __forceinline__ float Butterfly(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 16);
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v;
}

__device__ __forceinline__ float TensorScale(const Operand& p, std::uint32_t row) {
  return p.tensor_scale != nullptr ? __ldg(p.tensor_scale + (row / p.rows_per_scale)) : 1.0f;
}

template <int kDecoder, int kCols, bool kGlu>
__global__ void __launch_bounds__(kMaxWarps * 32, 1)
DecodeVectorKernel(const Args a, const Plan plan) {
  constexpr int kMats = kGlu ? 2 : 1;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) std::uint64_t full[kMaxWarps][kMaxStages];

  const int tid = static_cast<int>(threadIdx.x);
  const int warp = tid >> 5;
  const std::uint32_t lane = static_cast<std::uint32_t>(tid) & 31u;
  const bool staged = plan.copy_bytes != 0;
  const int S = plan.stages;

  // This CTA's outputs, then this warp's share of them.
  const std::uint32_t cta_begin =
      static_cast<std::uint32_t>((static_cast<std::uint64_t>(blockIdx.x) * a.outputs) / gridDim.x);
  const std::uint32_t cta_end =
      static_cast<std::uint32_t>((static_cast<std::uint64_t>(blockIdx.x + 1) * a.outputs) / gridDim.x);
  const std::uint32_t span = cta_end - cta_begin;
  const std::uint32_t begin = cta_begin + ((static_cast<std::uint32_t>(warp) * span) / plan.warps);
  const std::uint32_t end = cta_begin + ((static_cast<std::uint32_t>(warp + 1) * span) / plan.warps);
  const int mine = static_cast<int>(end - begin);

  unsigned char* ring = smem + plan.acts_bytes + (static_cast<std::size_t>(warp) * S * plan.stage_bytes);
  const auto* w_data = static_cast<const std::uint8_t*>(a.w.data);
  const auto* w2_data = static_cast<const std::uint8_t*>(a.w2.data);

  // Row j of this warp's run into its stage: one bulk copy a matrix.
  auto request = [&](int j) {
    const int s = j % S;
    if (lane == 0) tc::MbarExpectTx(&full[warp][s], plan.copy_bytes * kMats);
    __syncwarp();
    if (lane < kMats) {
      const std::uint8_t* src =
          lane == 0 ? w_data + (static_cast<std::uint64_t>(a.first + begin + j) * a.w.row_bytes)
                    : w2_data + (static_cast<std::uint64_t>(a.first2 + begin + j) * a.w2.row_bytes);
      tc::BulkLoad(ring + (static_cast<std::size_t>(s) * plan.stage_bytes) + (lane * plan.copy_bytes),
                   src, plan.copy_bytes, &full[warp][s]);
    }
  };

  if (staged) {
    if (lane == 0) {
      for (int s = 0; s < S; ++s) tc::MbarInit(&full[warp][s], 1);
      tc::MbarInitFence();
    }
    __syncwarp();
  }
  GridLaunchDependents();
  if (staged) {
    for (int j = 0; j < min(S, mine); ++j) request(j);
  }
  GridDependencyWait();

  // The activation rows, once a CTA, when they fit.
  const bool xs_shared = plan.acts_bytes != 0;
  const float* xs = a.x;
  std::uint64_t xs_stride = a.x_stride;
  if (xs_shared) {
    auto* dst = reinterpret_cast<float4*>(smem);
    const std::uint32_t quads = a.w.k / 4;
    for (std::uint32_t t = 0; t < a.rows; ++t) {
      const auto* src = reinterpret_cast<const float4*>(a.x + (static_cast<std::uint64_t>(t) * a.x_stride));
      for (std::uint32_t i = static_cast<std::uint32_t>(tid); i < quads; i += blockDim.x) {
        dst[(static_cast<std::size_t>(t) * quads) + i] = __ldg(src + i);
      }
    }
    xs = reinterpret_cast<const float*>(smem);
    xs_stride = a.w.k;
    __syncthreads();
  }

  const std::uint32_t segs = a.w.k / 16;
  for (int j = 0; j < mine; ++j) {
    const std::uint32_t n = begin + static_cast<std::uint32_t>(j);
    const std::uint32_t row = a.first + n, row2 = a.first2 + n;
    const std::uint8_t* codes = w_data + (static_cast<std::uint64_t>(row) * a.w.row_bytes);
    const std::uint8_t* codes2 = w2_data + (static_cast<std::uint64_t>(row2) * a.w2.row_bytes);
    if (staged) {
      const int s = j % S;
      bool ok = true;
      if (lane == 0) ok = tc::MbarWait(&full[warp][s], static_cast<std::uint32_t>((j / S) & 1));
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) {
        if (lane == 0) atomicAdd(plan.faults, 1u);
        return;  // nothing of an incomplete stage is summed or stored
      }
      codes = ring + (static_cast<std::size_t>(s) * plan.stage_bytes);
      codes2 = codes + plan.copy_bytes;
    }
    float g[kCols], u[kGlu ? kCols : 1];
#pragma unroll
    for (int t = 0; t < kCols; ++t) g[t] = 0.0f;
    if constexpr (kGlu) {
#pragma unroll
      for (int t = 0; t < kCols; ++t) u[t] = 0.0f;
    }
    for (std::uint32_t seg = lane; seg < segs; seg += 32u) {
      float v[16];
      LoadSegment<kDecoder>(a.w, codes, staged, row, seg, v);
      Accumulate<kCols>(xs, xs_stride, xs_shared, a.rows, seg, v, g);
      if constexpr (kGlu) {
        LoadSegment<kDecoder>(a.w2, codes2, staged, row2, seg, v);
        Accumulate<kCols>(xs, xs_stride, xs_shared, a.rows, seg, v, u);
      }
    }
    if (staged) {
      __syncwarp();  // every lane has read the stage
      if (j + S < mine) {
        tc::FenceProxyAsync();
        request(j + S);
      }
    }
    const float scale = TensorScale(a.w, row);
    const float scale2 = kGlu ? TensorScale(a.w2, row2) : 1.0f;
#pragma unroll
    for (int t = 0; t < kCols; ++t) {
      if (static_cast<std::uint32_t>(t) < a.rows) {
        float out = Butterfly(g[t]) * scale;
        if constexpr (kGlu) out = Glu(a.glu, out, Butterfly(u[t]) * scale2, a.limit);
        if (lane == 0) a.y[(static_cast<std::uint64_t>(t) * a.y_stride) + n] = out;
      }
    }
  }
}

// decode::RunRows (templates.cuh:441-466): y[i, :] = the decoded row ids[i] times
// its tensor scale; an id outside the matrix gives a zero row and raises *bad.
// A warp a row here, a lane a segment at a time.
template <int kDecoder>
__global__ void __launch_bounds__(256)
DecodeRowsKernel(const Operand w, const std::int32_t* __restrict__ ids, std::uint32_t count,
                 float* __restrict__ y, std::uint64_t y_stride, int* bad) {
  GridLaunchDependents();
  GridDependencyWait();
  const std::uint32_t lane = threadIdx.x & 31u;
  const std::uint32_t i = (blockIdx.x * (blockDim.x >> 5)) + (threadIdx.x >> 5);
  if (i >= count) return;
  const std::int32_t id = ids[i];
  float4* out = reinterpret_cast<float4*>(y + (static_cast<std::uint64_t>(i) * y_stride));
  const std::uint32_t segs = w.k / 16;
  if (id < 0 || static_cast<std::uint32_t>(id) >= w.rows) {
    for (std::uint32_t seg = lane; seg < segs; seg += 32u) {
#pragma unroll
      for (int q = 0; q < 4; ++q) out[(seg * 4u) + q] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    if (lane == 0 && bad != nullptr) *bad = 1;
    return;
  }
  const std::uint32_t row = static_cast<std::uint32_t>(id);
  const float scale = TensorScale(w, row);
  const std::uint8_t* codes = static_cast<const std::uint8_t*>(w.data) + (static_cast<std::uint64_t>(row) * w.row_bytes);
  for (std::uint32_t seg = lane; seg < segs; seg += 32u) {
    float v[16];
    LoadSegment<kDecoder>(w, codes, false, row, seg, v);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      out[(seg * 4u) + q] = make_float4(v[4 * q] * scale, v[(4 * q) + 1] * scale, v[(4 * q) + 2] * scale,
                                        v[(4 * q) + 3] * scale);
    }
  }
}

// ---------------------------------------------------------------- host
int CheckOperand(const Operand& p, const char* what) {
  if (p.decoder > LLMP_B200_DECODER_MXFP4_ATOMS) {
    return Reject("decode: %s: decoder %u is not one this build has", what, p.decoder);
  }
  const int d = static_cast<int>(p.decoder);
  const bool q8 = d == LLMP_B200_DECODER_Q8_0_BLOCKS;
  const bool dense = d == LLMP_B200_DECODER_BF16_DENSE || d == LLMP_B200_DECODER_F16_DENSE;
  if (p.data == nullptr || p.k < 32 || p.k % 32 != 0 || p.rows < 1 ||
      p.row_bytes < (static_cast<std::uint64_t>(p.k / 16) * SegmentBytesX2(d)) / 2) {
    return Reject("decode: %s: codes, k a positive multiple of 32, rows that hold k values", what);
  }
  if (q8 ? (!Aligned(p.data, 2) || p.row_bytes % 2 != 0)
         : (!Aligned(p.data, 16) || p.row_bytes % 16 != 0 || (!dense && p.scales == nullptr))) {
    return Reject("decode: %s: Q8_0 rows 2-byte aligned; other rows 16-byte aligned, block scales "
                  "with the block-scaled encodings", what);
  }
  const bool atoms8 = d == LLMP_B200_DECODER_MXFP8_ATOMS || d == LLMP_B200_DECODER_MXFP4_ATOMS;
  if ((atoms8 && p.k % 128 != 0) || (d == LLMP_B200_DECODER_NVFP4_ATOMS && p.k % 64 != 0)) {
    return Reject("decode: %s: scale atoms hold four blocks a row", what);
  }
  if (p.tensor_scale != nullptr && p.rows_per_scale < 1) {
    return Reject("decode: %s: tensor scales need rows_per_scale", what);
  }
  return 0;
}

// The geometry: warps and ring depth from the row's bytes, activations staged when they fit.
bool MakePlan(const Args& a, int mats, Plan* plan) {
  const int sms = SmCount();
  if (sms < 1) return false;
  plan->faults = FaultCounter();
  if (plan->faults == nullptr) return false;
  const int d = static_cast<int>(a.w.decoder);
  const std::uint64_t row = (static_cast<std::uint64_t>(a.w.k / 16) * SegmentBytesX2(d)) / 2;
  const auto bulk_ok = [&](const Operand& p) {
    return Aligned(p.data, 16) && p.row_bytes % 16 == 0 && row % 16 == 0;
  };
  const std::uint64_t acts = static_cast<std::uint64_t>(a.rows) * a.w.k * 4;
  plan->acts_bytes = acts <= kActsBudget ? static_cast<std::uint32_t>(acts) : 0u;
  plan->grid = static_cast<int>(std::min<std::uint64_t>(static_cast<std::uint64_t>(sms), a.outputs));
  const std::uint64_t per_cta = (a.outputs + plan->grid - 1) / plan->grid;
  int warps = static_cast<int>(std::min<std::uint64_t>(kMaxWarps, per_cta));
  plan->copy_bytes = 0;
  plan->stage_bytes = 0;
  plan->stages = 1;
  if (bulk_ok(a.w) && (mats == 1 || bulk_ok(a.w2)) && row * mats * 2 <= kRingBudget) {
    // at least two stages a warp; fewer warps when rows are long
    while (warps > 1 && row * mats * 2 * warps > kRingBudget) --warps;
    const std::uint64_t rows_a_warp = (per_cta + warps - 1) / warps;
    std::uint64_t stages = kRingBudget / (row * mats * warps);
    stages = std::min<std::uint64_t>(stages, static_cast<std::uint64_t>(kMaxStages));
    stages = std::min<std::uint64_t>(stages, std::max<std::uint64_t>(rows_a_warp, 1));
    plan->stages = static_cast<int>(stages);
    plan->copy_bytes = static_cast<std::uint32_t>(row);
    plan->stage_bytes = static_cast<std::uint32_t>(row * mats);
  }
  plan->warps = warps;
  return true;
}

template <int kDecoder, int kCols, bool kGlu>
cudaError_t LaunchOne(const Args& a, const Plan& plan, cudaStream_t s) {
  auto* kernel = DecodeVectorKernel<kDecoder, kCols, kGlu>;
  const std::size_t smem = plan.acts_bytes +
                           (static_cast<std::size_t>(plan.warps) * plan.stages * plan.stage_bytes);
  static thread_local int configured_device = -1;
  int device = -1;
  cudaGetDevice(&device);
  if (configured_device != device) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               kRingBudget + kActsBudget);
    if (e != cudaSuccess) return e;
    configured_device = device;
  }
  return LaunchPdl(kernel, dim3(static_cast<unsigned>(plan.grid)),
                   dim3(static_cast<unsigned>(plan.warps * 32)), smem, s, a, plan);
}

template <int kDecoder, bool kGlu>
cudaError_t LaunchCols(const Args& a, const Plan& plan, cudaStream_t s) {
  if (a.rows <= 1) return LaunchOne<kDecoder, 1, kGlu>(a, plan, s);
  if (a.rows <= 2) return LaunchOne<kDecoder, 2, kGlu>(a, plan, s);
  if (a.rows <= 4) return LaunchOne<kDecoder, 4, kGlu>(a, plan, s);
  if (a.rows <= 8) return LaunchOne<kDecoder, 8, kGlu>(a, plan, s);
  return LaunchOne<kDecoder, 16, kGlu>(a, plan, s);
}

template <bool kGlu>
cudaError_t Launch(const Args& a, const Plan& plan, cudaStream_t s) {
  switch (a.w.decoder) {
#define LLMP_DECODER(ID) \
  case ID: return LaunchCols<ID, kGlu>(a, plan, s);
    LLMP_DECODER(LLMP_B200_DECODER_Q8_0_BLOCKS)
    LLMP_DECODER(LLMP_B200_DECODER_MXFP8_SPLIT)
    LLMP_DECODER(LLMP_B200_DECODER_MXFP8_ATOMS)
    LLMP_DECODER(LLMP_B200_DECODER_BF16_DENSE)
    LLMP_DECODER(LLMP_B200_DECODER_F16_DENSE)
    LLMP_DECODER(LLMP_B200_DECODER_NVFP4_SPLIT)
    LLMP_DECODER(LLMP_B200_DECODER_NVFP4_ATOMS)
    LLMP_DECODER(LLMP_B200_DECODER_MXFP4_SPLIT)
    LLMP_DECODER(LLMP_B200_DECODER_MXFP4_ATOMS)
#undef LLMP_DECODER
    default: return cudaErrorInvalidValue;
  }
}

int Run(const Args& a, void* stream) {
  if (a.outputs < 1 || a.rows < 1 || a.rows > 16 || a.x == nullptr || a.y == nullptr) {
    return Reject("decode.vector: 1 to 16 activation rows, at least one output, x and y");
  }
  if (a.x_stride < a.w.k || a.y_stride < a.outputs || !Aligned(a.x, 16) || a.x_stride % 4 != 0 ||
      !Aligned(a.y, 4)) {
    return Reject("decode.vector: activation rows of k floats, 16-byte aligned; output rows of "
                  "`outputs` floats");
  }
  if (static_cast<std::uint64_t>(a.first) + a.outputs > a.w.rows) {
    return Reject("decode.vector: rows first .. first + outputs lie inside the matrix");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  Plan plan{};
  if (!MakePlan(a, a.glu < 0 ? 1 : 2, &plan)) return Reject("decode.vector: no fault counter on this device");
  const cudaError_t e = a.glu < 0 ? Launch<false>(a, plan, static_cast<cudaStream_t>(stream))
                                  : Launch<true>(a, plan, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return Failed(e, "decode.vector launch");
  return 0;
}

}  // namespace
}  // namespace llmp_b200

extern "C" {

int llmp_b200_decode_vector(const llmp_b200_decode_product* product, void* stream) {
  using namespace llmp_b200;
  if (product == nullptr) return Reject("decode.vector: null product");
  if (const int status = CheckOperand(product->w, "weight"); status != 0) return status;
  if (product->first > 0xffffffffull || product->outputs > 0xffffffffull || product->rows > 16) {
    return Reject("decode.vector: first, outputs within 32 bits; 1 to 16 rows");
  }
  Args a{};
  a.w = product->w;
  a.w2 = product->w;
  a.first = static_cast<std::uint32_t>(product->first);
  a.first2 = a.first;
  a.outputs = static_cast<std::uint32_t>(product->outputs);
  a.rows = static_cast<std::uint32_t>(product->rows);
  a.x = product->x;
  a.x_stride = product->x_stride;
  a.y = product->y;
  a.y_stride = product->y_stride;
  a.glu = -1;
  return Run(a, stream);
}

int llmp_b200_decode_vector_glu(const llmp_b200_decode_glu_product* product, void* stream) {
  using namespace llmp_b200;
  if (product == nullptr) return Reject("decode.vector_glu: null product");
  if (const int status = CheckOperand(product->gate, "gate"); status != 0) return status;
  if (const int status = CheckOperand(product->up, "up"); status != 0) return status;
  if (product->gate.k != product->up.k || product->gate.decoder != product->up.decoder) {
    return Reject("decode.vector_glu: gate and up of one K and (in this build) one decoder");
  }
  if (product->glu < LLMP_B200_GLU_SWIGLU || product->glu > LLMP_B200_GLU_GEGLU ||
      (product->glu == LLMP_B200_GLU_GEGLU && product->limit != 0.0f)) {
    return Reject("decode.vector_glu: SwiGLU, clamped SwiGLU or GeGLU (tanh, no limit)");
  }
  if (product->gate_first > 0xffffffffull || product->up_first > 0xffffffffull ||
      product->outputs > 0xffffffffull || product->rows > 16 ||
      product->up_first + product->outputs > product->up.rows) {
    return Reject("decode.vector_glu: rows inside the matrices; 1 to 16 activation rows");
  }
  Args a{};
  a.w = product->gate;
  a.w2 = product->up;
  a.first = static_cast<std::uint32_t>(product->gate_first);
  a.first2 = static_cast<std::uint32_t>(product->up_first);
  a.outputs = static_cast<std::uint32_t>(product->outputs);
  a.rows = static_cast<std::uint32_t>(product->rows);
  a.x = product->x;
  a.x_stride = product->x_stride;
  a.y = product->y;
  a.y_stride = product->y_stride;
  a.glu = product->glu;
  a.limit = product->limit;
  return Run(a, stream);
}

int llmp_b200_decode_rows(const llmp_b200_decode_operand* weight, const int32_t* ids, uint64_t count,
                          float* y, uint64_t y_stride, int32_t* bad, void* stream) {
  using namespace llmp_b200;
  if (weight == nullptr || ids == nullptr || y == nullptr || count < 1 || count > 0x7fffffffull) {
    return Reject("decode.rows: a weight, row ids, an output and at least one row");
  }
  if (const int status = CheckOperand(*weight, "weight"); status != 0) return status;
  if (y_stride < weight->k || y_stride % 4 != 0 || !Aligned(y, 16) || !Aligned(ids, 4)) {
    return Reject("decode.rows: output rows of k floats, 16-byte aligned");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  const dim3 grid(static_cast<unsigned>((count + 7) / 8)), block(256);
  auto* s = static_cast<cudaStream_t>(stream);
  const auto n = static_cast<std::uint32_t>(count);
  cudaError_t e = cudaErrorInvalidValue;
  switch (weight->decoder) {
#define LLMP_DECODER(ID)                                                                      \
  case ID:                                                                                    \
    e = LaunchPdl(DecodeRowsKernel<ID>, grid, block, 0, s, *weight, ids, n, y, y_stride, bad); \
    break;
    LLMP_DECODER(LLMP_B200_DECODER_Q8_0_BLOCKS)
    LLMP_DECODER(LLMP_B200_DECODER_MXFP8_SPLIT)
    LLMP_DECODER(LLMP_B200_DECODER_MXFP8_ATOMS)
    LLMP_DECODER(LLMP_B200_DECODER_BF16_DENSE)
    LLMP_DECODER(LLMP_B200_DECODER_F16_DENSE)
    LLMP_DECODER(LLMP_B200_DECODER_NVFP4_SPLIT)
    LLMP_DECODER(LLMP_B200_DECODER_NVFP4_ATOMS)
    LLMP_DECODER(LLMP_B200_DECODER_MXFP4_SPLIT)
    LLMP_DECODER(LLMP_B200_DECODER_MXFP4_ATOMS)
#undef LLMP_DECODER
    default: break;
  }
  if (e != cudaSuccess) return Failed(e, "decode.rows launch");
  return 0;
}

}  // extern "C"
