// Host side of the tensor-core kernels' shared plumbing: TMA tensor maps.
#include "tc.cuh"

namespace llmp_b200 {
namespace tc {

EncodeTiledFn EncodeTiled() {
  static EncodeTiledFn cached = [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &result) !=
            cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return static_cast<EncodeTiledFn>(nullptr);
    }
    return reinterpret_cast<EncodeTiledFn>(fn);
  }();
  return cached;
}

bool MakeMapBytes2D(CUtensorMap* map, const void* base, std::uint64_t rows, std::uint64_t cols,
                    std::uint64_t row_pitch_bytes, std::uint32_t box_rows, std::uint32_t box_cols) {
  const EncodeTiledFn encode = EncodeTiled();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_pitch_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
         CUDA_SUCCESS;
}

}  // namespace tc
}  // namespace llmp_b200
