// The exchange of the column-sharded decode step without a collective library: a rank's
// product writes its slice of an activation vector, llmp_b200_peer_publish stores that slice
// into EVERY rank's copy of the gathered vector with plain peer stores (memory of the other
// GPUs mapped through CUDA IPC; no multicast, no TMA) and then raises a flag word in each
// rank's memory; the consumer (the Q8_1 quantizer, q8_1.cu) begins by waiting, with a bound,
// until every source rank's flag carries the step's number.  The reference models this
// exchange as a kAllGather node after an N-column sharded projection
// (src/ir/op.h:246-250, src/planner/partition.h:39-56, src/components/ffn.cc:67-81).
//
// Flags carry the step number (a device word raised once a step by
// llmp_b200_peer_begin_step), so a captured graph replays without host-side sequence
// numbers.  One gathered buffer a vector suffices: a rank can only write the next layer's
// slice after it has consumed every rank's slice of this layer, which those ranks produce
// after they finished reading the buffer.  No kernel here spins without a bound, and no
// kernel of one GPU waits for another kernel of the same GPU.
#include "peer.cuh"

namespace llmp_b200 {
namespace {

__global__ void BeginStepKernel(std::int32_t* step) {
  GridDependencyWait();
  if (threadIdx.x == 0 && blockIdx.x == 0) *step = *step + 1;
}

__global__ void __launch_bounds__(256) PublishKernel(const PeerPublish publish) {
  GridLaunchDependents();
  GridDependencyWait();  // the slice is the kernel before's output
  PeerPublishSlice(publish);
}

__global__ void WaitKernel(const PeerWait wait) {
  GridLaunchDependents();
  GridDependencyWait();
  PeerWaitAll(wait);
}

int CheckSite(const llmp_b200_peer_site* site, const char* who) {
  if (site == nullptr || site->world < 1 || site->world > 32 || site->rank < 0 ||
      site->rank >= site->world || site->buffers == nullptr || site->flags == nullptr ||
      site->step == nullptr || site->site < 0) {
    return Reject("%s: a site of 1 to 32 ranks with device tables of buffers and flags and a step word",
                  who);
  }
  return 0;
}

}  // namespace

PeerPublish PeerPublishOf(const llmp_b200_peer_site& site, const void* slice, std::size_t offset,
                          std::size_t bytes) {
  PeerPublish p{};
  p.slice = static_cast<const unsigned char*>(slice);
  p.offset = offset;
  p.bytes = bytes;
  p.buffers = site.buffers;
  p.flags = site.flags;
  p.step = site.step;
  p.world = site.world;
  p.rank = site.rank;
  p.site = site.site;
  return p;
}

PeerWait PeerWaitOf(const llmp_b200_peer_site& site, const std::int32_t* local_flags, int polls,
                    std::int32_t* status) {
  PeerWait w{};
  w.flags = local_flags + (static_cast<std::size_t>(site.site) * site.world);
  w.step = site.step;
  w.world = site.world;
  w.polls = polls;
  w.status = status;
  w.faults = FaultCounter();
  return w;
}

}  // namespace llmp_b200

extern "C" {

int llmp_b200_peer_alloc(size_t bytes, void** ptr) {
  using namespace llmp_b200;
  if (ptr == nullptr || bytes == 0) return Reject("peer_alloc: a size and somewhere to put the pointer");
  if (const int status = DeviceStatus(); status != 0) return status;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return Failed(e, "peer_alloc");
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    return Failed(e, "peer_alloc clear");
  }
  *ptr = p;
  return 0;
}

int llmp_b200_peer_free(void* ptr) {
  using namespace llmp_b200;
  if (ptr == nullptr) return 0;
  const cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? 0 : Failed(e, "peer_free");
}

int llmp_b200_peer_export(const void* ptr, void* handle) {
  using namespace llmp_b200;
  static_assert(sizeof(cudaIpcMemHandle_t) == LLMP_B200_PEER_HANDLE_BYTES, "handle size");
  if (ptr == nullptr || handle == nullptr) return Reject("peer_export: a pointer of llmp_b200_peer_alloc and 64 bytes");
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(ptr));
  if (e != cudaSuccess) return Failed(e, "peer_export");
  memcpy(handle, &h, sizeof(h));
  return 0;
}

int llmp_b200_peer_import(const void* handle, void** ptr) {
  using namespace llmp_b200;
  if (ptr == nullptr || handle == nullptr) return Reject("peer_import: 64 bytes of handle and somewhere to put the pointer");
  if (const int status = DeviceStatus(); status != 0) return status;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return Failed(e, "peer_import");
  *ptr = p;
  return 0;
}

int llmp_b200_peer_close(void* ptr) {
  using namespace llmp_b200;
  if (ptr == nullptr) return 0;
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? 0 : Failed(e, "peer_close");
}

int llmp_b200_peer_begin_step(int32_t* step, void* stream) {
  using namespace llmp_b200;
  if (step == nullptr) return Reject("peer_begin_step: the device step word");
  if (const int status = DeviceStatus(); status != 0) return status;
  const cudaError_t e = LaunchPdl(BeginStepKernel, dim3(1), dim3(32), 0,
                                  static_cast<cudaStream_t>(stream), step);
  return e == cudaSuccess ? 0 : Failed(e, "peer_begin_step launch");
}

int llmp_b200_peer_publish(const llmp_b200_peer_site* site, const void* slice, size_t offset,
                           size_t bytes, void* stream) {
  using namespace llmp_b200;
  if (const int status = CheckSite(site, "peer_publish"); status != 0) return status;
  if (slice == nullptr || bytes == 0 || !Aligned(slice, 16) || offset % 16 != 0) {
    return Reject("peer_publish: a 16-byte aligned slice at a 16-byte aligned offset");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  const cudaError_t e =
      LaunchPdl(PublishKernel, dim3(static_cast<unsigned>(site->world)), dim3(256), 0,
                static_cast<cudaStream_t>(stream), PeerPublishOf(*site, slice, offset, bytes));
  return e == cudaSuccess ? 0 : Failed(e, "peer_publish launch");
}

int llmp_b200_peer_wait(const llmp_b200_peer_site* site, const int32_t* local_flags, int polls,
                        int32_t* status, void* stream) {
  using namespace llmp_b200;
  if (const int code = CheckSite(site, "peer_wait"); code != 0) return code;
  if (local_flags == nullptr || polls < 1) return Reject("peer_wait: this rank's flag words and a poll limit");
  if (const int code = DeviceStatus(); code != 0) return code;
  const PeerWait w = PeerWaitOf(*site, local_flags, polls, status);
  const cudaError_t e = LaunchPdl(WaitKernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), w);
  return e == cudaSuccess ? 0 : Failed(e, "peer_wait launch");
}

}  // extern "C"
