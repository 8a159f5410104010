// Flag waits of the peer-store exchange (peer.cu), shared with the kernels that begin by
// waiting for a gathered buffer (the Q8_1 quantizer).
#ifndef LLMP_B200_CSRC_PEER_CUH_
#define LLMP_B200_CSRC_PEER_CUH_

#include "common.cuh"

namespace llmp_b200 {

// What a consumer kernel needs to wait for one exchange: this rank's flag row of the site
// (one word a source rank), the step word, and where to report a wait that ran out.
struct PeerWait {
  const std::int32_t* flags;  // null: no wait
  const std::int32_t* step;
  int world;
  int polls;
  std::int32_t* status;
  unsigned int* faults;
};

// What a kernel that also publishes needs: the slice it owes every rank.
struct PeerPublish {
  const unsigned char* slice;  // null: nothing to publish
  std::size_t offset, bytes;
  void* const* buffers;        // device array [world]
  std::int32_t* const* flags;  // device array [world]
  const std::int32_t* step;
  int world, rank, site;
};

// The in-band form (no flag words, no fence): a value travels as one 8-byte word {F32 bits,
// tag}, tag = (step << 8) | the exchange's number within the step, stored by the PRODUCING
// kernel itself into every rank's vector; a reader polls the word until it carries the tag it
// expects.  An 8-byte aligned store lands whole, so a word is either the old one or the new.
struct PeerFan {
  unsigned long long* const* words;  // device array [world]: every rank's vector of words
  const std::int32_t* step;
  int world;  // 0: the product does not fan out
  int base;   // word index of this rank's first value
  int tag;    // 0..255
};
// What a reader needs to wait for `count` words of its own vector.
struct PeerWords {
  const unsigned long long* words;  // null: nothing to wait for
  const std::int32_t* step;
  int count;
  int tag;
  int polls;
  std::int32_t* status;
  unsigned int* faults;
};

#ifdef __CUDACC__
__device__ __forceinline__ std::uint32_t FanTag(const PeerFan& f) {
  return (static_cast<std::uint32_t>(*f.step) << 8) | static_cast<std::uint32_t>(f.tag);
}
// value -> word base + row of every rank's vector.
__device__ __forceinline__ void FanStore(const PeerFan& f, std::uint32_t tag, int row, float value) {
  for (int to = 0; to < f.world; ++to) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(f.words[to] + f.base + row),
                 "r"(__float_as_uint(value)), "r"(tag)
                 : "memory");
  }
}
// Polls one word until it carries `tag` (at most `polls` looks, about 0.1 us apart); its
// value, and whether it arrived.
__device__ __forceinline__ bool AwaitWord(const unsigned long long* word, std::uint32_t tag, int polls,
                                          float* value) {
  std::uint32_t lo = 0, hi = 0;
  for (int i = 0; i < polls; ++i) {
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "l"(word) : "memory");
    if (hi == tag) {
      *value = __uint_as_float(lo);
      return true;
    }
    __nanosleep(100);
  }
  *value = __uint_as_float(lo);
  return false;
}
__device__ __forceinline__ void ReportLateWords(const PeerWords& w) {
  if (w.status != nullptr) *w.status = 1;
  if (w.faults != nullptr) atomicAdd(w.faults, 1u);
}

__device__ __forceinline__ std::int32_t LoadAcquireSys(const std::int32_t* p) {
  std::int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void StoreReleaseSys(std::int32_t* p, std::int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Every thread of the CTA calls this.  CTA b stores the slice into ranks b, b + gridDim.x, ...
// and flags each, so any grid publishes to any world.
__device__ __forceinline__ void PeerPublishSlice(const PeerPublish& p) {
  if (p.slice == nullptr) return;
  for (int to = static_cast<int>(blockIdx.x); to < p.world; to += static_cast<int>(gridDim.x)) {
    unsigned char* dst = static_cast<unsigned char*>(p.buffers[to]) + p.offset;
    const std::size_t vectors = p.bytes / 16;
    const uint4* src4 = reinterpret_cast<const uint4*>(p.slice);
    uint4* dst4 = reinterpret_cast<uint4*>(dst);
    for (std::size_t i = threadIdx.x; i < vectors; i += blockDim.x) dst4[i] = src4[i];
    for (std::size_t i = (vectors * 16) + threadIdx.x; i < p.bytes; i += blockDim.x) dst[i] = p.slice[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      StoreReleaseSys(p.flags[to] + (static_cast<std::size_t>(p.site) * p.world) + p.rank, *p.step);
    }
  }
}

// Every thread of the CTA calls this.  Thread r < world polls source rank r's flag until it
// reaches the step's number, at most `polls` times (about 0.1 us apart); the CTA then meets.
// True when every flag arrived.  A wait that runs out is reported once (thread 0 of CTA 0
// writes 1 to *status and raises the fault counter) and the caller carries on, so that the
// stream, a captured graph included, always finishes.
__device__ __forceinline__ bool PeerWaitAll(const PeerWait& w) {
  if (w.flags == nullptr) return true;
  bool arrived = true;
  if (static_cast<int>(threadIdx.x) < w.world) {
    const std::int32_t want = *w.step;
    // After one wait of the step has run out, the later ones look once: a rank that is gone
    // costs a step one time limit, not one per exchange.
    const int polls = (w.status != nullptr && *w.status != 0) ? 1 : w.polls;
    arrived = false;
    for (int i = 0; i < polls; ++i) {
      if (LoadAcquireSys(w.flags + threadIdx.x) - want >= 0) {
        arrived = true;
        break;
      }
      __nanosleep(100);
    }
  }
  const bool all = __syncthreads_and(arrived ? 1 : 0) != 0;
  if (!all && threadIdx.x == 0 && blockIdx.x == 0) {
    if (w.status != nullptr) *w.status = 1;
    if (w.faults != nullptr) atomicAdd(w.faults, 1u);
  }
  return all;
}
#endif  // __CUDACC__

}  // namespace llmp_b200

#endif  // LLMP_B200_CSRC_PEER_CUH_
