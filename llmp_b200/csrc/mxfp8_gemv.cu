// llmp.mxfp8.mul_mat_vec on B200: MXFP8 weights (E4M3 codes [n, k], E8M0 scales
// [n, k / 32] ROW-MAJOR, not atoms) times up to 16 F32 activation columns.
// Semantics follow src/kernels/ggml/llmp_ops.cu:145-215: a 16-code vector's dot
// product is scaled by its block's scale before it joins the lane's sum, then
// the warp sums; F32 throughout.
//
// A pure HBM stream (1 byte a weight).  One warp a row pair; lane l takes
// vectors l, l + 32, ... as 128-bit streaming loads, four in flight a row;
// activations come through L1 (they are shared by every row); the first
// vectors are requested before the programmatic-dependency wait.
#include <cuda_fp8.h>

#include "common.cuh"

namespace llmp_b200 {
namespace {

constexpr int kWarps = 8;
constexpr int kRows = 2;

__device__ __forceinline__ void Decode16(const uint4 q, float out[16]) {
  const std::uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(
        static_cast<__nv_fp8x2_storage_t>(w[i] & 0xffffu), __NV_E4M3);
    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(
        static_cast<__nv_fp8x2_storage_t>(w[i] >> 16), __NV_E4M3);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    out[4 * i + 0] = a.x;
    out[4 * i + 1] = a.y;
    out[4 * i + 2] = b.x;
    out[4 * i + 3] = b.y;
  }
}

template <int kColumns>
__global__ void __launch_bounds__(kWarps * 32)
Mxfp8GemvKernel(const std::uint8_t* __restrict__ codes, const std::uint8_t* __restrict__ scales,
                const float* x, float* y, int n, int k, std::int64_t x_stride,
                std::int64_t y_stride) {
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int row0 = ((static_cast<int>(blockIdx.x) * kWarps) + (static_cast<int>(threadIdx.x) >> 5)) * kRows;
  GridLaunchDependents();
  if (row0 >= n) return;
  const int rows = min(kRows, n - row0);
  const int vectors = k / 16;
  const std::uint8_t* wrow[kRows];
  const std::uint8_t* srow[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    const int row = row0 + min(r, rows - 1);
    wrow[r] = codes + (static_cast<std::int64_t>(row) * k);
    srow[r] = scales + (static_cast<std::int64_t>(row) * (k / 32));
  }
  // The first vectors, before anything the kernel in front wrote is read.
  uint4 first[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    first[r] = lane < vectors ? LoadStream16(wrow[r] + (static_cast<std::int64_t>(lane) * 16))
                              : make_uint4(0, 0, 0, 0);
  }
  GridDependencyWait();
  float sum[kRows][kColumns];
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int c = 0; c < kColumns; ++c) sum[r][c] = 0.0f;

  for (int v = lane; v < vectors; v += 32) {
    uint4 q[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      q[r] = v == lane ? first[r] : LoadStream16(wrow[r] + (static_cast<std::int64_t>(v) * 16));
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      float wf[16];
      Decode16(q[r], wf);
      const float scale = __uint_as_float(static_cast<std::uint32_t>(srow[r][v >> 1]) << 23);
#pragma unroll
      for (int c = 0; c < kColumns; ++c) {
        const float4* xv = reinterpret_cast<const float4*>(x + (c * x_stride) + (v * 16));
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 a = xv[i];
          dot = fmaf(wf[4 * i + 0], a.x, dot);
          dot = fmaf(wf[4 * i + 1], a.y, dot);
          dot = fmaf(wf[4 * i + 2], a.z, dot);
          dot = fmaf(wf[4 * i + 3], a.w, dot);
        }
        sum[r][c] = fmaf(dot, scale, sum[r][c]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
#pragma unroll
    for (int c = 0; c < kColumns; ++c) {
      float v = sum[r][c];
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
      if (lane == 0 && r < rows) y[(c * y_stride) + row0 + r] = v;
    }
  }
}

template <int kColumns>
cudaError_t Launch(const std::uint8_t* codes, const std::uint8_t* scales, const float* x, float* y,
                   int n, int k, std::int64_t x_stride, std::int64_t y_stride, cudaStream_t s) {
  const int grid = (n + (kWarps * kRows) - 1) / (kWarps * kRows);
  return LaunchPdl(Mxfp8GemvKernel<kColumns>, dim3(static_cast<unsigned>(grid)), dim3(kWarps * 32),
                   0, s, codes, scales, x, y, n, k, x_stride, y_stride);
}

}  // namespace
}  // namespace llmp_b200

extern "C" int llmp_b200_mxfp8_mul_mat_vec(const void* codes, const void* scales, const float* x,
                                           int64_t x_stride, float* y, int64_t y_stride, int n,
                                           int k, int columns, void* stream) {
  using namespace llmp_b200;
  if (codes == nullptr || scales == nullptr || x == nullptr || y == nullptr || n < 1 || k < 32 ||
      k % 32 != 0 || columns < 1 || columns > 16 || x_stride < k || y_stride < n) {
    return Reject("mxfp8.mul_mat_vec: codes [k, n], scales [k / 32, n], 1..16 F32 columns, "
                  "k a positive multiple of 32");
  }
  if (!Aligned(codes, 16) || !Aligned(x, 16) || x_stride % 4 != 0 || !Aligned(y, 4)) {
    return Reject("mxfp8.mul_mat_vec: codes and activations 16-byte aligned");
  }
  // E8M0 0xFF (NaN) is not a scale a quantizer writes; 2^(s-127) is formed by
  // placing s in the exponent field, exact for 1..254 (0 gives zero for 2^-127).
  if (const int status = DeviceStatus(); status != 0) return status;
  auto* s = static_cast<cudaStream_t>(stream);
  const auto* c8 = static_cast<const std::uint8_t*>(codes);
  const auto* s8 = static_cast<const std::uint8_t*>(scales);
  cudaError_t e = cudaErrorInvalidValue;
  switch (columns) {
#define LLMP_C(C) case C: e = Launch<C>(c8, s8, x, y, n, k, x_stride, y_stride, s); break;
    LLMP_C(1) LLMP_C(2) LLMP_C(3) LLMP_C(4) LLMP_C(5) LLMP_C(6) LLMP_C(7) LLMP_C(8)
    LLMP_C(9) LLMP_C(10) LLMP_C(11) LLMP_C(12) LLMP_C(13) LLMP_C(14) LLMP_C(15) LLMP_C(16)
#undef LLMP_C
  }
  if (e != cudaSuccess) return Failed(e, "mxfp8.mul_mat_vec launch");
  return 0;
}
