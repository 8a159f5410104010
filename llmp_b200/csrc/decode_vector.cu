// The decode module's vector products: y = W x with F32 activations and the
// weight decoded on the fly, 1 to 16 activation rows, plain or as the GLU of a
// gate and an up product.  Interface and arithmetic are the reference's
// (src/kernels/decode/products.h:96-147; templates.cuh:83-186; decoders
// decoders.cuh:106-125 for Q8_0 blocks, :193-220 for MXFP8 with row-major scales
// or scale atoms): a warp a weight row; lane l takes the 16-value segments l,
// l + 32, ... and adds value * x in one fused multiply-add a value, in order; the
// lanes meet in a butterfly over lanes 16, 8, 4, 2, 1 apart; the sum is scaled by
// the row's tensor scale.  That order is kept, so the F32 results are the
// reference's bit for bit; what is this build's is the memory side (128-bit code
// loads, the E4M3 bytes converted by the hardware's FP8 conversion, the launch as
// a programmatic dependent).
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace llmp_b200 {
namespace {

using Operand = llmp_b200_decode_operand;

constexpr int kWarps = 8;

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

__device__ __forceinline__ float E8m0(std::uint32_t e) {
  // 2^(e - 127); e = 0 is the subnormal 2^-127, e = 255 NaN
  return e == 0 ? __uint_as_float(0x00400000u) : e == 255 ? __uint_as_float(0x7fffffffu)
                                                           : __uint_as_float(e << 23);
}

template <int kDecoder>
__device__ __forceinline__ void LoadSegment(const Operand& p, std::uint32_t row, std::uint32_t seg,
                                            float (&v)[16]) {
  const auto* data = static_cast<const std::uint8_t*>(p.data);
  if constexpr (kDecoder == LLMP_B200_DECODER_Q8_0_BLOCKS) {
    // 34-byte blocks: only two-byte loads are aligned.  Half a block a segment.
    const std::uint8_t* block = data + (row * p.row_bytes) + (static_cast<std::uint64_t>(seg >> 1) * 34);
    const float d = HalfBitsToFloat(__ldg(reinterpret_cast<const unsigned short*>(block)));
    const auto* q = reinterpret_cast<const unsigned short*>(block + 2 + ((seg & 1u) * 16u));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const std::uint32_t pair = __ldg(q + i);
      v[2 * i] = d * static_cast<float>(static_cast<std::int8_t>(pair & 0xffu));
      v[(2 * i) + 1] = d * static_cast<float>(static_cast<std::int8_t>(pair >> 8));
    }
  } else {
    const auto* scales = static_cast<const std::uint8_t*>(p.scales);
    const std::uint32_t blocks = p.k / 32;
    const std::uint32_t block = seg >> 1;
    const std::uint64_t at =
        kDecoder == LLMP_B200_DECODER_MXFP8_SPLIT
            ? (static_cast<std::uint64_t>(row) * blocks) + block
            : ((((static_cast<std::uint64_t>(row) / 128) * (blocks / 4)) + (block / 4)) * 512) +
                  ((row % 32) * 16) + (((row % 128) / 32) * 4) + (block % 4);
    const float s = E8m0(__ldg(scales + at));
    const uint4 c = __ldg(reinterpret_cast<const uint4*>(data + (row * p.row_bytes) + (seg * 16u)));
    const std::uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // two E4M3 bytes to two halves (exact), then to F32
      const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(
          static_cast<__nv_fp8x2_storage_t>((w[i / 2] >> (16 * (i % 2))) & 0xffffu), __NV_E4M3);
      v[2 * i] = __half2float(__ushort_as_half(h.x)) * s;
      v[(2 * i) + 1] = __half2float(__ushort_as_half(h.y)) * s;
    }
  }
}

template <int kCols>
__device__ __forceinline__ void Accumulate(const Args& a, std::uint32_t seg, const float (&w)[16],
                                           float (&acc)[kCols]) {
#pragma unroll
  for (int t = 0; t < kCols; ++t) {
    if (static_cast<std::uint32_t>(t) < a.rows) {
      const auto* xp = reinterpret_cast<const float4*>(a.x + (static_cast<std::uint64_t>(t) * a.x_stride) +
                                                       (seg * 16u));
      float s = acc[t];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 x = __ldg(xp + q);
        s = fmaf(w[4 * q], x.x, s);
        s = fmaf(w[(4 * q) + 1], x.y, s);
        s = fmaf(w[(4 * q) + 2], x.z, s);
        s = fmaf(w[(4 * q) + 3], x.w, s);
      }
      acc[t] = s;
    }
  }
}

__device__ __forceinline__ float WarpSum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

__device__ __forceinline__ float RowScale(const Operand& p, std::uint32_t row) {
  return p.tensor_scale != nullptr ? __ldg(p.tensor_scale + (row / p.rows_per_scale)) : 1.0f;
}

template <int kDecoder, int kCols, bool kGlu>
__global__ void __launch_bounds__(kWarps * 32) DecodeVectorKernel(const Args a) {
  GridLaunchDependents();
  GridDependencyWait();
  const std::uint32_t lane = threadIdx.x & 31u;
  const std::uint32_t n = (blockIdx.x * kWarps) + (threadIdx.x >> 5);
  if (n >= a.outputs) return;
  const std::uint32_t row = a.first + n, row2 = a.first2 + n;
  const std::uint32_t segs = a.w.k / 16;
  float g[kCols], u[kGlu ? kCols : 1];
#pragma unroll
  for (int t = 0; t < kCols; ++t) g[t] = 0.0f;
  if constexpr (kGlu) {
#pragma unroll
    for (int t = 0; t < kCols; ++t) u[t] = 0.0f;
  }
  for (std::uint32_t seg = lane; seg < segs; seg += 32u) {
    float w[16];
    LoadSegment<kDecoder>(a.w, row, seg, w);
    Accumulate<kCols>(a, seg, w, g);
    if constexpr (kGlu) {
      LoadSegment<kDecoder>(a.w2, row2, seg, w);
      Accumulate<kCols>(a, seg, w, u);
    }
  }
  const float scale = RowScale(a.w, row);
  const float scale2 = kGlu ? RowScale(a.w2, row2) : 1.0f;
#pragma unroll
  for (int t = 0; t < kCols; ++t) {
    if (static_cast<std::uint32_t>(t) < a.rows) {
      const float gs = WarpSum(g[t]);
      float out = gs * scale;
      if constexpr (kGlu) {
        const float us = WarpSum(u[t]);
        out = Glu(a.glu, gs * scale, us * scale2, a.limit);
      }
      if (lane == 0) a.y[(static_cast<std::uint64_t>(t) * a.y_stride) + n] = out;
    }
  }
}

int CheckOperand(const Operand& p, const char* what) {
  if (p.decoder > LLMP_B200_DECODER_MXFP8_ATOMS) {
    return Reject("decode.vector: %s: decoder %u is not one this build has (Q8_0 blocks, MXFP8)",
                  what, p.decoder);
  }
  const bool q8 = p.decoder == LLMP_B200_DECODER_Q8_0_BLOCKS;
  if (p.data == nullptr || p.k < 32 || p.k % 32 != 0 || p.rows < 1 ||
      p.row_bytes < (q8 ? (p.k / 32) * 34ull : p.k)) {
    return Reject("decode.vector: %s: codes, k a positive multiple of 32, rows that hold k values", what);
  }
  if (q8 ? (!Aligned(p.data, 2) || p.row_bytes % 2 != 0)
         : (!Aligned(p.data, 16) || p.row_bytes % 16 != 0 || p.scales == nullptr)) {
    return Reject("decode.vector: %s: Q8_0 rows 2-byte aligned; MXFP8 rows 16-byte aligned with scales", what);
  }
  if (p.decoder == LLMP_B200_DECODER_MXFP8_ATOMS && p.k % 128 != 0) {
    return Reject("decode.vector: %s: scale atoms hold four blocks a row: k a multiple of 128", what);
  }
  if (p.tensor_scale != nullptr && p.rows_per_scale < 1) {
    return Reject("decode.vector: %s: tensor scales need rows_per_scale", what);
  }
  return 0;
}

template <int kDecoder, bool kGlu>
cudaError_t LaunchCols(const Args& a, cudaStream_t s) {
  const dim3 grid((a.outputs + kWarps - 1) / kWarps), block(kWarps * 32);
  if (a.rows <= 1) return LaunchPdl(DecodeVectorKernel<kDecoder, 1, kGlu>, grid, block, 0, s, a);
  if (a.rows <= 2) return LaunchPdl(DecodeVectorKernel<kDecoder, 2, kGlu>, grid, block, 0, s, a);
  if (a.rows <= 4) return LaunchPdl(DecodeVectorKernel<kDecoder, 4, kGlu>, grid, block, 0, s, a);
  if (a.rows <= 8) return LaunchPdl(DecodeVectorKernel<kDecoder, 8, kGlu>, grid, block, 0, s, a);
  return LaunchPdl(DecodeVectorKernel<kDecoder, 16, kGlu>, grid, block, 0, s, a);
}

template <bool kGlu>
cudaError_t Launch(const Args& a, cudaStream_t s) {
  switch (a.w.decoder) {
    case LLMP_B200_DECODER_Q8_0_BLOCKS: return LaunchCols<LLMP_B200_DECODER_Q8_0_BLOCKS, kGlu>(a, s);
    case LLMP_B200_DECODER_MXFP8_SPLIT: return LaunchCols<LLMP_B200_DECODER_MXFP8_SPLIT, kGlu>(a, s);
    default: return LaunchCols<LLMP_B200_DECODER_MXFP8_ATOMS, kGlu>(a, s);
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
  const cudaError_t e = a.glu < 0 ? Launch<false>(a, static_cast<cudaStream_t>(stream))
                                  : Launch<true>(a, static_cast<cudaStream_t>(stream));
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
  if (product->first > 0xffffffffull || product->outputs > 0xffffffffull || product->rows > 16) {
    return Reject("decode.vector: first, outputs within 32 bits; 1 to 16 rows");
  }
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

}  // extern "C"
