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
//   * a row's bytes (both matrices' with a GLU; two rows at a time for up to
//     four activation rows) arrive chunk by chunk in the warp's PRIVATE ring of
//     shared-memory stages by the bulk-copy engine (cp.async.bulk completing on
//     the stage's mbarrier), several chunks ahead of the one being summed, and
//     the first of them are requested before the programmatic-dependency wait:
//     weights depend on no earlier kernel.  Warps never synchronize with each
//     other after the activations are staged;
//   * a lane reads its segment out of the staged row with the widest aligned
//     shared load the encoding allows (Q8_0's 34-byte blocks put a segment on a
//     2-byte boundary: five aligned words and a funnel shift);
//   * the activation rows are staged once a CTA when they fit, else read
//     through L1;
//   * rows that are not 16-byte aligned (Q8_0 only promises 2) are read in place
//     with the loads their alignment allows.
// Every mbarrier wait is bounded; a wait that runs out raises the device fault
// counter and the warp stores nothing more.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <type_traits>

#include "common.cuh"
#include "tc.cuh"

namespace llmp_b200 {
namespace {

using Operand = llmp_b200_decode_operand;

constexpr int kMaxWarps = 16;
constexpr int kMaxStages = 8;
constexpr int kRingBudget = 144 * 1024;
constexpr int kActsBudget = 80 * 1024;

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
  // The split of the outputs: CTA b owns rows_q + (b < rows_rem) of them, and a CTA
  // of span rows_q + e gives warp w warp_q[e] + (w < warp_rem[e]); no division runs
  // on the device.
  std::uint32_t rows_q, rows_rem, warp_q[2], warp_rem[2];
  int group;                  // weight rows summed together (a stage holds them all): 1 or 2
  std::uint32_t row_bytes;    // a row's code bytes
  std::uint32_t copy_bytes;   // a chunk: the bytes of chunk_segs segments of one row, as one bulk
                              // copy moves them (0: rows are read in place); the last may be shorter
  std::uint32_t chunk_segs;   // segments a chunk: a multiple of 32 (whole rounds of the lanes)
  std::uint32_t chunks;       // chunks a row
  std::uint32_t stage_bytes;  // one stage: copy_bytes x matrices x group, 16-byte multiples
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

// Loads from a shared-memory ADDRESS.  A pointer that is global memory on one
// path and shared memory on another compiles to generic loads, which queue with
// the global ones; the staged paths therefore carry 32-bit shared addresses.
__device__ __forceinline__ std::uint32_t SharedU16(std::uint32_t at) {
  std::uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(at));
  return v;
}
template <int kOffset = 0>
__device__ __forceinline__ std::uint32_t SharedU32(std::uint32_t at) {
  std::uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(at), "n"(kOffset));
  return v;
}
__device__ __forceinline__ uint2 SharedU64(std::uint32_t at) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(at));
  return v;
}
template <int kOffset = 0>
__device__ __forceinline__ uint4 SharedU128(std::uint32_t at) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(at), "n"(kOffset));
  return v;
}

// ---------------------------------------------------------------- decoders
// Bytes of a row's codes that hold one 16-value segment, per decoder.
__host__ __device__ constexpr int SegmentBytesX2(int decoder) {  // twice the bytes (Q8_0: 17)
  return decoder == LLMP_B200_DECODER_Q8_0_BLOCKS                                             ? 34
         : (decoder == LLMP_B200_DECODER_MXFP8_SPLIT || decoder == LLMP_B200_DECODER_MXFP8_ATOMS) ? 32
         : (decoder == LLMP_B200_DECODER_BF16_DENSE || decoder == LLMP_B200_DECODER_F16_DENSE)    ? 64
                                                                                                   : 16;
}

// One 16-value segment as it is stored: the code words and the block's scale.
struct Raw {
  std::uint32_t w[8];  // Q8_0: 4 words of int8; MXFP8: 4 of E4M3; dense: 8 of two 16-bit values; FP4: 2 of E2M1
  float scale;         // d, the E8M0 or the UE4M3 value; unused by the dense encodings
};

// Raw segment to v[16], each value decoded exactly as the reference's decoder does
// (decoders.cuh: code times block scale, exact in F32).  kSummed: the values only
// feed sums that start at +0, so a zero's sign is free.
template <int kDecoder, bool kSummed>
__device__ __forceinline__ void Expand(const Raw& raw, float (&v)[16]) {
  if constexpr (kDecoder == LLMP_B200_DECODER_Q8_0_BLOCKS) {
    const float d = raw.scale;
    // A half that is not finite (no real block has one) takes the two-step form, which
    // gives the reference's infinities and NaNs; so does the row lookup, always.
    const bool finite = (__float_as_uint(d) & 0x7f800000u) != 0x7f800000u;
    if (kSummed && finite) {
      // d b in one fused multiply-add a value, without the conversion unit: b + 128
      // goes into bits 8-15 of 1.0f, which reads 1 + (b + 128) 2^-15, and
      // (2^15 d) (1 + (b + 128) 2^-15) - (1 + 2^-8) (2^15 d) = d b.  Both constants
      // are exact (a half's 11 significant bits times 257 is 20 bits) and so is the
      // result (19 bits): the bits of d times float(b), but for b = 0 under a
      // negative d, which gives +0 here and -0 there; a sum that starts at +0 is the
      // same with either.
      const float ds = d * 32768.0f, offset = ds * -1.00390625f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const std::uint32_t bits =
            __byte_perm(raw.w[i / 4] ^ 0x80808080u, 0x3F800000u, 0x7604u | ((i % 4) << 4));
        v[i] = fmaf(__uint_as_float(bits), ds, offset);
      }
    } else {
      // b + 128 as the low mantissa byte of 2^23, minus (2^23 + 128), times d: exact
      // steps that keep the sign of a zero.
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const std::uint32_t bits = __byte_perm(raw.w[i / 4] ^ 0x80808080u, 0x4B000000u, 0x7440u | (i % 4));
        v[i] = d * (__uint_as_float(bits) - 8388736.0f);
      }
    }
  } else if constexpr (kDecoder == LLMP_B200_DECODER_MXFP8_SPLIT ||
                       kDecoder == LLMP_B200_DECODER_MXFP8_ATOMS) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // two E4M3 bytes to two halves (exact), then to F32
      const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(
          static_cast<__nv_fp8x2_storage_t>((raw.w[i / 2] >> (16 * (i % 2))) & 0xffffu), __NV_E4M3);
      v[2 * i] = __half2float(__ushort_as_half(h.x)) * raw.scale;
      v[(2 * i) + 1] = __half2float(__ushort_as_half(h.y)) * raw.scale;
    }
  } else if constexpr (kDecoder == LLMP_B200_DECODER_BF16_DENSE ||
                       kDecoder == LLMP_B200_DECODER_F16_DENSE) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if constexpr (kDecoder == LLMP_B200_DECODER_BF16_DENSE) {
        v[2 * i] = __uint_as_float(raw.w[i] << 16);
        v[(2 * i) + 1] = __uint_as_float(raw.w[i] & 0xffff0000u);
      } else {
        v[2 * i] = HalfBitsToFloat(raw.w[i] & 0xffffu);
        v[(2 * i) + 1] = HalfBitsToFloat(raw.w[i] >> 16);
      }
    }
  } else {
    // E2M1 codes, value 2 i in byte i's low nibble
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const std::uint32_t b = (raw.w[i / 4] >> (8 * (i % 4))) & 0xffu;
      v[2 * i] = E2m1(b & 15u) * raw.scale;
      v[(2 * i) + 1] = E2m1(b >> 4) * raw.scale;
    }
  }
}

// The block scale of segment `seg` of row `row` for the block-scaled encodings
// (scales row-major or in scale atoms; NVFP4 a UE4M3 a segment, the MX encodings
// an E8M0 two segments).
template <int kDecoder>
__device__ __forceinline__ float BlockScale(const Operand& p, std::uint32_t row, std::uint32_t seg) {
  constexpr bool kNv = kDecoder == LLMP_B200_DECODER_NVFP4_SPLIT || kDecoder == LLMP_B200_DECODER_NVFP4_ATOMS;
  constexpr bool kAtoms = kDecoder == LLMP_B200_DECODER_MXFP8_ATOMS ||
                          kDecoder == LLMP_B200_DECODER_NVFP4_ATOMS ||
                          kDecoder == LLMP_B200_DECODER_MXFP4_ATOMS;
  const auto* scales = static_cast<const std::uint8_t*>(p.scales);
  const std::uint32_t blocks = kNv ? p.k / 16 : p.k / 32;
  const std::uint32_t block = kNv ? seg : seg >> 1;
  const std::uint32_t code = __ldg(scales + (kAtoms ? AtomAt(row, block, blocks)
                                                    : (static_cast<std::uint64_t>(row) * blocks) + block));
  return kNv ? Ue4m3(code) : E8m0(code);
}

__host__ __device__ constexpr bool BlockScaled(int decoder) {
  return decoder != LLMP_B200_DECODER_Q8_0_BLOCKS && decoder != LLMP_B200_DECODER_BF16_DENSE &&
         decoder != LLMP_B200_DECODER_F16_DENSE;
}

// Segment `seg` of a row whose code bytes start at `codes` in global memory, with
// the alignment the entry point checked (Q8_0 rows only promise two bytes).
template <int kDecoder>
__device__ __forceinline__ void FetchGlobal(const Operand& p, const std::uint8_t* codes, std::uint32_t row,
                                            std::uint32_t seg, Raw& raw) {
  if constexpr (kDecoder == LLMP_B200_DECODER_Q8_0_BLOCKS) {
    // Half a 34-byte block: d at byte 34 b, the segment's 16 int8 at 34 b + 2 + 16 h.
    const std::uint32_t at = ((seg >> 1) * 34u) + 2u + ((seg & 1u) * 16u);
    const auto* h = reinterpret_cast<const unsigned short*>(codes + at);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      raw.w[i] = static_cast<std::uint32_t>(__ldg(h + (2 * i))) |
                 (static_cast<std::uint32_t>(__ldg(h + (2 * i) + 1)) << 16);
    }
    raw.scale = HalfBitsToFloat(__ldg(reinterpret_cast<const unsigned short*>(codes + ((seg >> 1) * 34u))));
  } else {
    constexpr int kBytes = SegmentBytesX2(kDecoder) / 2;  // 16, 32 or 8
    if constexpr (kBytes == 8) {
      const uint2 c = __ldg(reinterpret_cast<const uint2*>(codes + (seg * 8u)));
      raw.w[0] = c.x, raw.w[1] = c.y;
    } else {
#pragma unroll
      for (int i = 0; i < kBytes / 16; ++i) {
        const uint4 c = __ldg(reinterpret_cast<const uint4*>(codes + (seg * kBytes)) + i);
        raw.w[4 * i] = c.x, raw.w[(4 * i) + 1] = c.y, raw.w[(4 * i) + 2] = c.z, raw.w[(4 * i) + 3] = c.w;
      }
    }
    if constexpr (BlockScaled(kDecoder)) raw.scale = BlockScale<kDecoder>(p, row, seg);
  }
}

// What a lane needs to find its segments lane, lane + 32, ... in a staged row; they
// are a round's bytes apart (Q8_0: 544, a multiple of 4), so all of this is the
// lane's own and the loop only moves the round's shared address.
template <int kDecoder>
struct StagedLane {
  std::uint32_t words;  // from the round's address to the segment's first aligned word
  std::uint32_t last;   // Q8_0: to the fifth word when the codes start two bytes in, else the fourth again
  std::uint32_t scale;  // Q8_0: to the block's d
  std::uint32_t shift;  // Q8_0: 16 when the codes start two bytes into their first word
  __device__ __forceinline__ explicit StagedLane(std::uint32_t lane) {
    if constexpr (kDecoder == LLMP_B200_DECODER_Q8_0_BLOCKS) {
      const std::uint32_t odd = lane & 1u;
      const std::uint32_t at = (17u * lane) + 2u - odd;  // 34 (lane / 2) + 2 + 16 (lane % 2)
      shift = (at & 2u) * 8u;
      words = at & ~3u;
      last = words + (shift != 0 ? 16u : 12u);  // nothing past the segment is touched
      scale = 17u * (lane - odd);
    } else {
      words = lane * (SegmentBytesX2(kDecoder) / 2);
      last = 0, scale = 0, shift = 0;
    }
  }
};
__host__ __device__ constexpr std::uint32_t RoundBytes(int decoder) { return 16u * SegmentBytesX2(decoder); }

// The lane's segment of the round staged at shared address `round` (16-byte
// aligned): the widest aligned shared loads the encoding allows (Q8_0's 34-byte
// blocks put a segment on a 2-byte boundary: five aligned words and a funnel shift).
template <int kDecoder>
__device__ __forceinline__ void FetchStaged(const Operand& p, std::uint32_t round, const StagedLane<kDecoder>& at,
                                            std::uint32_t row, std::uint32_t seg, Raw& raw) {
  if constexpr (kDecoder == LLMP_B200_DECODER_Q8_0_BLOCKS) {
    const std::uint32_t words = round + at.words;
    const std::uint32_t w0 = SharedU32<0>(words), w1 = SharedU32<4>(words), w2 = SharedU32<8>(words),
                        w3 = SharedU32<12>(words), w4 = SharedU32<0>(round + at.last);
    raw.w[0] = __funnelshift_r(w0, w1, at.shift);
    raw.w[1] = __funnelshift_r(w1, w2, at.shift);
    raw.w[2] = __funnelshift_r(w2, w3, at.shift);
    raw.w[3] = __funnelshift_r(w3, w4, at.shift);
    raw.scale = HalfBitsToFloat(static_cast<unsigned short>(SharedU16(round + at.scale)));
  } else {
    constexpr int kBytes = SegmentBytesX2(kDecoder) / 2;
    const std::uint32_t words = round + at.words;
    if constexpr (kBytes == 8) {
      const uint2 c = SharedU64(words);
      raw.w[0] = c.x, raw.w[1] = c.y;
    } else {
      const uint4 c = SharedU128<0>(words);
      raw.w[0] = c.x, raw.w[1] = c.y, raw.w[2] = c.z, raw.w[3] = c.w;
      if constexpr (kBytes == 32) {
        const uint4 c1 = SharedU128<16>(words);
        raw.w[4] = c1.x, raw.w[5] = c1.y, raw.w[6] = c1.z, raw.w[7] = c1.w;
      }
    }
    if constexpr (BlockScaled(kDecoder)) raw.scale = BlockScale<kDecoder>(p, row, seg);
  }
}

// The staged activations: a segment's 64 bytes every 80.  The lanes of a quarter
// warp read the same quad of eight consecutive segments at once; 64 bytes apart
// those meet on two 16-byte bank groups, 80 apart they take all eight.
constexpr std::uint32_t kSegmentPitch = 80;
__host__ __device__ constexpr std::uint64_t StagedRowBytes(std::uint64_t k) { return (k / 16) * kSegmentPitch; }

// acc[r][t] += w[r] . x[t, 16 seg ..) for the kG weight rows of a group, one fused
// multiply-add a value in index order; an activation value is read once a group.
// Quad q (four activations) of row t comes from `quad(t, q)`.
template <int kCols, int kG, typename Quad>
__device__ __forceinline__ void Accumulate(std::uint32_t rows, const float (&w)[kG][16],
                                           float (&acc)[kG][kCols], Quad quad) {
#pragma unroll
  for (int t = 0; t < kCols; ++t) {
    if (static_cast<std::uint32_t>(t) < rows) {
      float s[kG];
#pragma unroll
      for (int r = 0; r < kG; ++r) s[r] = acc[r][t];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 x = quad(t, q);
#pragma unroll
        for (int r = 0; r < kG; ++r) {
          s[r] = fmaf(w[r][4 * q], x.x, s[r]);
          s[r] = fmaf(w[r][(4 * q) + 1], x.y, s[r]);
          s[r] = fmaf(w[r][(4 * q) + 2], x.z, s[r]);
          s[r] = fmaf(w[r][(4 * q) + 3], x.w, s[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < kG; ++r) acc[r][t] = s[r];
    }
  }
}
// Quad q of the segment staged at shared address `at` (q a constant after unrolling).
__device__ __forceinline__ float4 StagedQuad(std::uint32_t at, int q) {
  const uint4 bits = q == 0 ? SharedU128<0>(at) : q == 1 ? SharedU128<16>(at)
                     : q == 2 ? SharedU128<32>(at) : SharedU128<48>(at);
  return make_float4(__uint_as_float(bits.x), __uint_as_float(bits.y), __uint_as_float(bits.z),
                     __uint_as_float(bits.w));
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

template <int kDecoder, int kCols, bool kGlu, int kG>
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

  // This CTA's outputs, then this warp's share of them, walked kG rows (a group) at a time.
  const std::uint32_t cta = blockIdx.x, extra = cta < plan.rows_rem ? 1u : 0u;
  const std::uint32_t cta_begin = (cta * plan.rows_q) + min(cta, plan.rows_rem);
  const std::uint32_t uwarp = static_cast<std::uint32_t>(warp);
  // (a parameter array indexed by a variable would be copied to local memory)
  const std::uint32_t warp_q = extra != 0 ? plan.warp_q[1] : plan.warp_q[0];
  const std::uint32_t warp_rem = extra != 0 ? plan.warp_rem[1] : plan.warp_rem[0];
  const std::uint32_t begin = cta_begin + (uwarp * warp_q) + min(uwarp, warp_rem);
  const int mine = static_cast<int>(warp_q + (uwarp < warp_rem ? 1u : 0u));
  const int groups = (mine + kG - 1) / kG;

  unsigned char* ring = smem + plan.acts_bytes + (static_cast<std::size_t>(warp) * S * plan.stage_bytes);
  const std::uint32_t ring_at = tc::Smem(ring);
  const auto* w_data = static_cast<const std::uint8_t*>(a.w.data);
  const auto* w2_data = static_cast<const std::uint8_t*>(a.w2.data);

  // Item i of this warp's run is chunk i % C of group i / C and goes to stage i % S:
  // one bulk copy a row and matrix (row r of the group, matrix m at
  // (r kMats + m) copy_bytes).  Chunks let the sums start when the first part of
  // a row has landed instead of the whole of it.
  const int C = static_cast<int>(plan.chunks);
  const int items = groups * C;
  int next = 0, next_group = 0, next_chunk = 0, next_stage = 0;  // the next item to request
  auto request = [&]() __attribute__((always_inline)) {
    const std::uint32_t live = static_cast<std::uint32_t>(min(kG, mine - (next_group * kG)));
    const std::uint32_t offset = static_cast<std::uint32_t>(next_chunk) * plan.copy_bytes;
    const std::uint32_t bytes = min(plan.copy_bytes, plan.row_bytes - offset);
    // One elected lane issues the item (the whole warp walks here: instructions of
    // the copy engine issued from a one-lane branch cost several times as much).
    if (tc::ElectOne()) {
      tc::MbarExpectTx(&full[warp][next_stage], bytes * kMats * live);
      unsigned char* dst = ring + (static_cast<std::size_t>(next_stage) * plan.stage_bytes);
      const std::uint64_t n = begin + (static_cast<std::uint32_t>(next_group) * kG);
#pragma unroll
      for (std::uint32_t r = 0; r < static_cast<std::uint32_t>(kG); ++r) {
        if (r < live) {
          tc::BulkLoad(dst + (r * kMats * plan.copy_bytes),
                       w_data + ((a.first + n + r) * a.w.row_bytes) + offset, bytes, &full[warp][next_stage]);
          if constexpr (kGlu) {
            tc::BulkLoad(dst + (((r * kMats) + 1) * plan.copy_bytes),
                         w2_data + ((a.first2 + n + r) * a.w2.row_bytes) + offset, bytes,
                         &full[warp][next_stage]);
          }
        }
      }
    }
    __syncwarp();
    ++next;
    if (++next_chunk == C) {
      next_chunk = 0;
      ++next_group;
    }
    if (++next_stage == S) next_stage = 0;
  };

  if (staged) {
    if (lane < static_cast<std::uint32_t>(S)) {
      tc::MbarInit(&full[warp][lane], 1);
      tc::MbarInitFence();
    }
    __syncwarp();
  }
  GridLaunchDependents();
  // Two chunks in flight now, the next each time one has landed (below), never the whole
  // ring at once: the copy engine serves the copies it holds side by side, so a ring
  // requested at once lands at once, at the end of the transfer, and no chunk's sums
  // overlap it.
  if (staged) {
    while (next < min(min(S, 2), items)) request();
  }
  GridDependencyWait();

  // The activation rows, once a CTA, when they fit.
  const bool xs_shared = plan.acts_bytes != 0;
  const float* xs = a.x;
  std::uint64_t xs_stride = a.x_stride;
  if (xs_shared) {
    const std::uint32_t quads = a.w.k / 4;
    for (std::uint32_t t = 0; t < a.rows; ++t) {
      const auto* src = reinterpret_cast<const float4*>(a.x + (static_cast<std::uint64_t>(t) * a.x_stride));
      unsigned char* dst = smem + (static_cast<std::size_t>(t) * StagedRowBytes(a.w.k));
#pragma unroll 4
      for (std::uint32_t i = static_cast<std::uint32_t>(tid); i < quads; i += blockDim.x) {
        *reinterpret_cast<float4*>(dst + ((i >> 2) * kSegmentPitch) + ((i & 3u) * 16u)) = __ldg(src + i);
      }
    }
    __syncthreads();
  }
  const std::uint32_t xs_at = tc::Smem(smem);
  const std::uint32_t xs_row_bytes = static_cast<std::uint32_t>(StagedRowBytes(a.w.k));
  const StagedLane<kDecoder> in_round(lane);

  const std::uint32_t segs = a.w.k / 16, chunk_segs = plan.chunk_segs;
  int item = 0, stage = 0;
  std::uint32_t phase = 0;
  for (int j = 0; j < groups; ++j) {
    const std::uint32_t n0 = begin + (static_cast<std::uint32_t>(j) * kG);
    const int live = min(kG, mine - (j * kG));
    // Row r of the group; a group's missing rows repeat its first (summed, never stored).
    std::uint32_t row[kG], row2[kG];
    const std::uint8_t* codes[kG];
    const std::uint8_t* codes2[kG];
#pragma unroll
    for (int r = 0; r < kG; ++r) {
      const std::uint32_t n = n0 + static_cast<std::uint32_t>(r < live ? r : 0);
      row[r] = a.first + n;
      row2[r] = a.first2 + n;
      codes[r] = w_data + (static_cast<std::uint64_t>(row[r]) * a.w.row_bytes);
      codes2[r] = w2_data + (static_cast<std::uint64_t>(row2[r]) * a.w2.row_bytes);
    }
    float g[kG][kCols], u[kGlu ? kG : 1][kCols];
#pragma unroll
    for (int r = 0; r < kG; ++r) {
#pragma unroll
      for (int t = 0; t < kCols; ++t) {
        g[r][t] = 0.0f;
        if constexpr (kGlu) u[r][t] = 0.0f;
      }
    }
    for (int c = 0; c < C; ++c, ++item) {
      // Where the row would start in shared memory if all of it were staged as this chunk is.
      std::uint32_t scodes[kG] = {}, scodes2[kG] = {};
      if (staged) {
        // Every lane looks once without blocking (a chunk requested long ago has
        // usually landed, and a blocking wait costs a few hundred cycles even then);
        // only if some lane saw the phase open does lane 0 wait, with its bound.
        if (!__all_sync(0xffffffffu, tc::MbarTest(&full[warp][stage], phase) ? 1 : 0)) {
          bool ok = true;
          if (lane == 0) ok = tc::MbarWait(&full[warp][stage], phase);
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) {
            if (lane == 0) atomicAdd(plan.faults, 1u);
            return;  // nothing of an incomplete stage is summed or stored
          }
        }
        // this chunk has landed: the next ones travel while it is summed (their stages
        // were read S chunks ago)
        while (next < items && next - item < min(S, 3)) {
          tc::FenceProxyAsync();
          request();
        }
#pragma unroll
        for (int r = 0; r < kG; ++r) {
          const int at = r < live ? r : 0;
          scodes[r] = ring_at + (static_cast<std::uint32_t>(stage) * plan.stage_bytes) +
                      (static_cast<std::uint32_t>(at) * kMats * plan.copy_bytes) -
                      (static_cast<std::uint32_t>(c) * plan.copy_bytes);
          scodes2[r] = scodes[r] + plan.copy_bytes;
        }
      }
      const std::uint32_t seg_begin = static_cast<std::uint32_t>(c) * chunk_segs;
      const std::uint32_t seg_end = min(segs, seg_begin + chunk_segs);
      // The rounds of the chunk.  The usual case (rows staged, activations staged)
      // is compiled with both facts known: its loop holds no branch on them, no
      // global-memory addressing, and shared addresses that only advance.
      auto rounds = [&](auto usual) {
        constexpr bool kUsual = decltype(usual)::value;
        const bool st = kUsual ? true : staged;
        const bool xsh = kUsual ? true : xs_shared;
        std::uint32_t round[kG], round2[kG];  // the round's bytes of each row, in the stage
#pragma unroll
        for (int r = 0; r < kG; ++r) {
          round[r] = scodes[r] + ((seg_begin / 32u) * RoundBytes(kDecoder));
          round2[r] = scodes2[r] + ((seg_begin / 32u) * RoundBytes(kDecoder));
        }
        std::uint32_t xa = xs_at + ((seg_begin + lane) * kSegmentPitch);  // the lane's staged activations
        for (std::uint32_t seg = seg_begin + lane; seg < seg_end; seg += 32u) {
          const auto staged_quad = [&](int t, int q) {
            return StagedQuad(xa + (static_cast<std::uint32_t>(t) * xs_row_bytes), q);
          };
          const auto global_quad = [&](int t, int q) {
            return __ldg(reinterpret_cast<const float4*>(xs + (static_cast<std::uint64_t>(t) * xs_stride)) +
                         (seg * 4u) + static_cast<std::uint32_t>(q));
          };
          float v[kG][16];
#pragma unroll
          for (int r = 0; r < kG; ++r) {
            Raw raw;
            if (st) {
              FetchStaged<kDecoder>(a.w, round[r], in_round, row[r], seg, raw);
            } else {
              FetchGlobal<kDecoder>(a.w, codes[r], row[r], seg, raw);
            }
            Expand<kDecoder, true>(raw, v[r]);
            round[r] += RoundBytes(kDecoder);
          }
          if (xsh) {
            Accumulate<kCols, kG>(a.rows, v, g, staged_quad);
          } else {
            Accumulate<kCols, kG>(a.rows, v, g, global_quad);
          }
          if constexpr (kGlu) {
#pragma unroll
            for (int r = 0; r < kG; ++r) {
              Raw raw;
              if (st) {
                FetchStaged<kDecoder>(a.w2, round2[r], in_round, row2[r], seg, raw);
              } else {
                FetchGlobal<kDecoder>(a.w2, codes2[r], row2[r], seg, raw);
              }
              Expand<kDecoder, true>(raw, v[r]);
              round2[r] += RoundBytes(kDecoder);
            }
            if (xsh) {
              Accumulate<kCols, kG>(a.rows, v, u, staged_quad);
            } else {
              Accumulate<kCols, kG>(a.rows, v, u, global_quad);
            }
          }
          xa += 32u * kSegmentPitch;
        }
      };
      if (staged && xs_shared) {
        rounds(std::true_type{});
      } else {
        rounds(std::false_type{});
      }
      if (staged) {
        __syncwarp();  // every lane has read the stage
        if (S == 1 && next < items) {  // a one-stage ring: the stage just read takes the next item
          tc::FenceProxyAsync();
          request();
        }
        if (++stage == S) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kG; ++r) {
      if (r < live) {
        const float scale = TensorScale(a.w, row[r]);
        const float scale2 = kGlu ? TensorScale(a.w2, row2[r]) : 1.0f;
#pragma unroll
        for (int t = 0; t < kCols; ++t) {
          if (static_cast<std::uint32_t>(t) < a.rows) {
            float out = Butterfly(g[r][t]) * scale;
            if constexpr (kGlu) out = Glu(a.glu, out, Butterfly(u[r][t]) * scale2, a.limit);
            if (lane == 0) a.y[(static_cast<std::uint64_t>(t) * a.y_stride) + n0 + r] = out;
          }
        }
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
    Raw raw;
    FetchGlobal<kDecoder>(w, codes, row, seg, raw);
    Expand<kDecoder, false>(raw, v);
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
  const std::uint64_t acts = static_cast<std::uint64_t>(a.rows) * StagedRowBytes(a.w.k);
  plan->acts_bytes = acts <= kActsBudget ? static_cast<std::uint32_t>(acts) : 0u;
  plan->grid = static_cast<int>(std::min<std::uint64_t>(static_cast<std::uint64_t>(sms), a.outputs));
  const std::uint64_t per_cta = (a.outputs + plan->grid - 1) / plan->grid;
  const int warps = static_cast<int>(std::min<std::uint64_t>(kMaxWarps, per_cta));
  plan->rows_q = a.outputs / static_cast<std::uint32_t>(plan->grid);
  plan->rows_rem = a.outputs % static_cast<std::uint32_t>(plan->grid);
  for (std::uint32_t e = 0; e < 2; ++e) {
    plan->warp_q[e] = (plan->rows_q + e) / static_cast<std::uint32_t>(warps);
    plan->warp_rem[e] = (plan->rows_q + e) % static_cast<std::uint32_t>(warps);
  }
  plan->row_bytes = static_cast<std::uint32_t>(row);
  plan->copy_bytes = 0;
  plan->stage_bytes = 0;
  plan->stages = 1;
  plan->chunk_segs = a.w.k / 16;
  plan->chunks = 1;
  // A warp's part of the ring, the bytes of one round (32 segments, one a lane) of a row.
  const std::uint64_t per_warp = (static_cast<std::uint64_t>(kRingBudget) / warps) & ~std::uint64_t{15};
  const std::uint64_t round = static_cast<std::uint64_t>(16) * SegmentBytesX2(d);
  // Two rows a group for up to four activation rows (an activation value read from
  // shared memory serves both; more columns would spill), when some warp has two
  // rows to sum and two stages of one round each fit.
  plan->group = (a.rows <= 4 && per_cta > static_cast<std::uint64_t>(warps) &&
                 round * mats * 2 * 2 <= per_warp) ? 2 : 1;
  const std::uint64_t unit = round * mats * plan->group;
  if (bulk_ok(a.w) && (mats == 1 || bulk_ok(a.w2)) && row <= 0xffffffffull && unit * 2 <= per_warp) {
    // Chunks of whole rounds, about four stages of them in a warp's part.
    const std::uint64_t rounds = (static_cast<std::uint64_t>(a.w.k / 16) + 31) / 32;
    const std::uint64_t r = std::min(rounds, std::max<std::uint64_t>(1, per_warp / (4 * unit)));
    const std::uint64_t chunks = (rounds + r - 1) / r;
    const std::uint64_t stage = r * unit;
    const std::uint64_t groups_a_warp = (((per_cta + warps - 1) / warps) + plan->group - 1) / plan->group;
    std::uint64_t stages = per_warp / stage;
    stages = std::min<std::uint64_t>(stages, static_cast<std::uint64_t>(kMaxStages));
    stages = std::min<std::uint64_t>(stages, std::max<std::uint64_t>(groups_a_warp * chunks, 1));
    plan->stages = static_cast<int>(stages);
    plan->copy_bytes = static_cast<std::uint32_t>(r * round);
    plan->chunk_segs = static_cast<std::uint32_t>(r * 32);
    plan->chunks = static_cast<std::uint32_t>(chunks);
    plan->stage_bytes = static_cast<std::uint32_t>(stage);
  }
  plan->warps = warps;
  return true;
}

template <int kDecoder, int kCols, bool kGlu, int kG>
cudaError_t LaunchOne(const Args& a, const Plan& plan, cudaStream_t s) {
  auto* kernel = DecodeVectorKernel<kDecoder, kCols, kGlu, kG>;
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
  if (plan.group == 2) {
    if (a.rows <= 1) return LaunchOne<kDecoder, 1, kGlu, 2>(a, plan, s);
    if (a.rows <= 2) return LaunchOne<kDecoder, 2, kGlu, 2>(a, plan, s);
    return LaunchOne<kDecoder, 4, kGlu, 2>(a, plan, s);
  }
  if (a.rows <= 1) return LaunchOne<kDecoder, 1, kGlu, 1>(a, plan, s);
  if (a.rows <= 2) return LaunchOne<kDecoder, 2, kGlu, 1>(a, plan, s);
  if (a.rows <= 4) return LaunchOne<kDecoder, 4, kGlu, 1>(a, plan, s);
  if (a.rows <= 8) return LaunchOne<kDecoder, 8, kGlu, 1>(a, plan, s);
  return LaunchOne<kDecoder, 16, kGlu, 1>(a, plan, s);
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
