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

namespace {
// One warp waits, with a host-chosen limit, on a barrier nothing arrives at: the
// give-up path every kernel of this library takes when a copy never lands.
__global__ void WaitSelfTestKernel(std::uint32_t polls, std::int32_t* status, unsigned int* faults) {
  __shared__ __align__(8) std::uint64_t never;
  if (threadIdx.x == 0) {
    tc::MbarInit(&never, 1);
    tc::MbarInitFence();
  }
  __syncwarp();
  bool ok = true;
  if (threadIdx.x == 0) ok = tc::MbarWait(&never, 0, polls);
  ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  if (!ok && threadIdx.x == 0) {
    atomicAdd(faults, 1u);
    *status = 1;  // gave up, as designed
  } else if (threadIdx.x == 0) {
    *status = 2;  // a barrier without an arrival completed: never expected
  }
}
}  // namespace
}  // namespace llmp_b200

extern "C" int llmp_b200_wait_selftest(int polls, int32_t* status, void* stream) {
  using namespace llmp_b200;
  if (status == nullptr || polls < 1 || polls > 4096) {
    return Reject("wait_selftest: a device status word and 1 to 4096 polls");
  }
  if (const int code = DeviceStatus(); code != 0) return code;
  unsigned int* faults = FaultCounter();
  if (faults == nullptr) return Reject("wait_selftest: no fault counter on this device");
  WaitSelfTestKernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<std::uint32_t>(polls), status, faults);
  return Launched("wait_selftest launch");
}
