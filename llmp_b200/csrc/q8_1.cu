// llmp.q8_1: F32 activations to Q8_1 blocks, the input every vecq product
// reads.  Restates the quantizer the reference calls at
// src/kernels/ggml/vecq.cu:1095-1111 (GGML quantize_row_q8_1_cuda): blocks of
// 32, d = amax / 127 and the sum of the original inputs as FP16, q =
// roundf(x / d), each row padded with zero blocks to a multiple of 512 values.
//
// Eight lanes share a block, four consecutive values a lane (one 16-byte
// load).  The 32-value sum is formed as a butterfly over value indices 16, 8,
// 4, 2, 1 apart, so the FP16 it rounds to does not depend on the lane layout.
#include "peer.cuh"

namespace llmp_b200 {
namespace {

constexpr int kThreads = 256;

template <bool kVec>
__global__ void __launch_bounds__(kThreads)
QuantizeQ8_1Kernel(const float* __restrict__ x, std::int64_t k, std::int64_t rows,
                   std::int64_t stride_row, std::int64_t stride_plane, std::int64_t row_blocks,
                   std::int64_t total_lanes, std::uint8_t* __restrict__ out, const PeerWait gathered,
                   const PeerPublish publish) {
  // The products after this one may start fetching their weights now.
  GridLaunchDependents();
  // Where this thread reads and writes, worked out BEFORE the wait for the kernel
  // before (whose output the input is): the divisions, 64-bit only when they have
  // to be, then run beside that kernel's tail instead of after it.
  const std::int64_t i = (static_cast<std::int64_t>(blockIdx.x) * kThreads) + threadIdx.x;
  const bool live = i < total_lanes;  // whole groups of 8 lanes are live or not
  const std::int64_t block = (live ? i : 0) / 8;
  const int lane8 = static_cast<int>(i % 8);
  std::int64_t row, b, plane, plane_row;  // row over rows * planes
  if (rows == 1 && row_blocks <= 0x7fffffff && block <= 0x7fffffff) {
    const std::uint32_t block32 = static_cast<std::uint32_t>(block), per = static_cast<std::uint32_t>(row_blocks);
    const std::uint32_t row32 = block32 / per;
    row = row32, b = block32 - (row32 * per), plane = row32, plane_row = 0;
  } else {
    row = block / row_blocks;
    b = block % row_blocks;
    plane = row / rows;
    plane_row = row % rows;
  }
  const std::int64_t at = (b * 32) + (lane8 * 4);
  const float* src = x + (plane * stride_plane) + (plane_row * stride_row) + at;
  std::uint8_t* o = out + (block * 36);
  GridDependencyWait();
  // ... or, in the column-sharded step, a vector every rank stores a slice of (peer.cu):
  // store this rank's slice everywhere first (when this kernel is given it), then wait, with a
  // bound, for all the slices.  The CTAs of this small grid are all resident, so the ones that
  // wait for this rank's own flag do not keep the one that sets it from running.
  PeerPublishSlice(publish);
  PeerWaitAll(gathered);
  float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (live) {
    if (kVec && at + 4 <= k) {
      const float4 f = *reinterpret_cast<const float4*>(src);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (at + c < k) v[c] = src[c];
      }
    }
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  float s[4] = {v[0], v[1], v[2], v[3]};
#pragma unroll
  for (int offset = 4; offset > 0; offset >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      s[c] = s[c] + __shfl_xor_sync(0xffffffffu, s[c], offset);
    }
  }
  const float sum = (s[0] + s[2]) + (s[1] + s[3]);
  const float d = amax / 127.0f;
  std::uint32_t packed = 0;
  if (amax != 0.0f) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int q = static_cast<int>(roundf(v[c] / d));
      packed |= (static_cast<std::uint32_t>(q) & 0xffu) << (8 * c);
    }
  }
  if (!live) return;
  *reinterpret_cast<std::uint32_t*>(o + 4 + (lane8 * 4)) = packed;
  if (lane8 == 0) {
    const std::uint32_t ds = static_cast<std::uint32_t>(__half_as_ushort(__float2half_rn(d))) |
                             (static_cast<std::uint32_t>(__half_as_ushort(__float2half_rn(sum)))
                              << 16);
    *reinterpret_cast<std::uint32_t*>(o) = ds;
  }
}

// The quantizer over a vector that arrives as tagged words (peer.cuh): a thread polls the four
// words it quantizes, with a bound, before it uses them.  `hold`, when given, is another
// vector of words whose arrival the kernel waits for without using its values (the layer
// before's output, in the sharded step: nobody may overwrite what this rank still reads).
// With `x` the values come from x and the words are only waited for.
__global__ void __launch_bounds__(kThreads)
QuantizeWordsKernel(const float* __restrict__ x, const PeerWords in, const PeerWords hold,
                    std::int64_t k, std::int64_t row_blocks, std::int64_t total_lanes,
                    std::uint8_t* __restrict__ out) {
  GridLaunchDependents();
  GridDependencyWait();
  const std::int64_t i = (static_cast<std::int64_t>(blockIdx.x) * kThreads) + threadIdx.x;
  bool late = false;
  float unused;
  if (hold.words != nullptr) {
    const std::uint32_t tag = (static_cast<std::uint32_t>(*hold.step) << 8) | static_cast<std::uint32_t>(hold.tag);
    int polls = (hold.status != nullptr && *hold.status != 0) ? 1 : hold.polls;
    for (std::int64_t w = i; w < hold.count; w += static_cast<std::int64_t>(gridDim.x) * kThreads) {
      if (!AwaitWord(hold.words + w, tag, polls, &unused)) {
        late = true;
        polls = 1;
      }
    }
  }
  const bool live = i < total_lanes;
  const std::int64_t b = (live ? i : 0) / 8;
  const int lane8 = static_cast<int>(i % 8);
  const std::int64_t at = (b * 32) + (lane8 * 4);
  float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (live) {
    if (x != nullptr) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (at + c < k) v[c] = x[at + c];
      }
    } else {
      const std::uint32_t tag = (static_cast<std::uint32_t>(*in.step) << 8) | static_cast<std::uint32_t>(in.tag);
      int polls = (in.status != nullptr && *in.status != 0) ? 1 : in.polls;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (at + c < k && !AwaitWord(in.words + at + c, tag, polls, &v[c])) {
          late = true;
          polls = 1;
        }
      }
    }
  }
  if (late) ReportLateWords(hold.words != nullptr ? hold : in);
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  float s[4] = {v[0], v[1], v[2], v[3]};
#pragma unroll
  for (int offset = 4; offset > 0; offset >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      s[c] = s[c] + __shfl_xor_sync(0xffffffffu, s[c], offset);
    }
  }
  const float sum = (s[0] + s[2]) + (s[1] + s[3]);
  const float d = amax / 127.0f;
  std::uint32_t packed = 0;
  if (amax != 0.0f) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int q = static_cast<int>(roundf(v[c] / d));
      packed |= (static_cast<std::uint32_t>(q) & 0xffu) << (8 * c);
    }
  }
  if (!live) return;
  std::uint8_t* o = out + (b * 36);
  *reinterpret_cast<std::uint32_t*>(o + 4 + (lane8 * 4)) = packed;
  if (lane8 == 0) {
    const std::uint32_t ds = static_cast<std::uint32_t>(__half_as_ushort(__float2half_rn(d))) |
                             (static_cast<std::uint32_t>(__half_as_ushort(__float2half_rn(sum)))
                              << 16);
    *reinterpret_cast<std::uint32_t*>(o) = ds;
  }
}

}  // namespace
}  // namespace llmp_b200

extern "C" int64_t llmp_b200_q8_1_row_blocks(int64_t k) { return (k + 511) / 512 * 512 / 32; }

namespace llmp_b200 {
PeerWait PeerWaitOf(const llmp_b200_peer_site& site, const std::int32_t* local_flags, int polls,
                    std::int32_t* status);
PeerPublish PeerPublishOf(const llmp_b200_peer_site& site, const void* slice, std::size_t offset,
                          std::size_t bytes);
namespace {
int Quantize(const float* x, int64_t k, int64_t rows, int64_t planes, int64_t stride_row,
             int64_t stride_plane, void* out, const PeerWait& gathered, const PeerPublish& publish,
             void* stream) {
  if (x == nullptr || out == nullptr || k < 1 || rows < 1 || planes < 1) {
    return Reject("q8_1: F32 input [k, rows, planes] and an output, all non-empty");
  }
  if (!Aligned(x, 4) || !Aligned(out, 4) || stride_row < k || stride_plane < 0) {
    return Reject("q8_1: 4-byte aligned operands, rows at least k floats apart");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  const std::int64_t row_blocks = llmp_b200_q8_1_row_blocks(k);
  const std::int64_t total = rows * planes * row_blocks * 8;
  if (total / kThreads + 1 > 0x7fffffffLL) return Reject("q8_1: more blocks than a grid holds");
  const bool vec = Aligned(x, 16) && stride_row % 4 == 0 && stride_plane % 4 == 0;
  const dim3 grid(static_cast<unsigned>((total + kThreads - 1) / kThreads));
  auto* o = static_cast<std::uint8_t*>(out);
  const cudaError_t e =
      vec ? LaunchPdl(QuantizeQ8_1Kernel<true>, grid, dim3(kThreads), 0,
                      static_cast<cudaStream_t>(stream), x, k, rows, stride_row, stride_plane,
                      row_blocks, total, o, gathered, publish)
          : LaunchPdl(QuantizeQ8_1Kernel<false>, grid, dim3(kThreads), 0,
                      static_cast<cudaStream_t>(stream), x, k, rows, stride_row, stride_plane,
                      row_blocks, total, o, gathered, publish);
  if (e != cudaSuccess) return Failed(e, "q8_1 launch");
  return 0;
}
}  // namespace
}  // namespace llmp_b200

extern "C" {

int llmp_b200_q8_1_quantize(const float* x, int64_t k, int64_t rows, int64_t planes,
                            int64_t stride_row, int64_t stride_plane, void* out, void* stream) {
  return llmp_b200::Quantize(x, k, rows, planes, stride_row, stride_plane, out, llmp_b200::PeerWait{},
                             llmp_b200::PeerPublish{}, stream);
}

int llmp_b200_q8_1_quantize_gathered(const float* x, int64_t k, int64_t rows, int64_t stride_row,
                                     void* out, const llmp_b200_peer_site* site,
                                     const int32_t* local_flags, int polls, int32_t* status,
                                     void* stream) {
  using namespace llmp_b200;
  if (site == nullptr || local_flags == nullptr || polls < 1 || site->world < 1 || site->world > 32 ||
      site->step == nullptr || site->site < 0) {
    return Reject("q8_1 gathered: a site, this rank's flag words and a poll limit");
  }
  return Quantize(x, k, rows, 1, stride_row, 0, out, PeerWaitOf(*site, local_flags, polls, status),
                  PeerPublish{}, stream);
}

int llmp_b200_q8_1_quantize_words(const float* x, const uint64_t* words, int tag, int64_t k,
                                  const uint64_t* hold, int64_t hold_count, int hold_tag,
                                  const int32_t* step, void* out, int polls, int32_t* status,
                                  void* stream) {
  using namespace llmp_b200;
  if ((x == nullptr) == (words == nullptr) || out == nullptr || step == nullptr || k < 1 || polls < 1 ||
      tag < 0 || tag > 255 || hold_tag < 0 || hold_tag > 255 || (hold != nullptr && hold_count < 1)) {
    return Reject("q8_1 words: either x or a vector of words, the step word, tags of 0 to 255");
  }
  if (!Aligned(words, 8) || !Aligned(hold, 8) || !Aligned(x, 4) || !Aligned(out, 4)) {
    return Reject("q8_1 words: 8-byte aligned words");
  }
  if (const int code = DeviceStatus(); code != 0) return code;
  PeerWords in{}, held{};
  in.words = reinterpret_cast<const unsigned long long*>(words);
  in.step = step;
  in.count = static_cast<int>(k);
  in.tag = tag;
  in.polls = polls;
  in.status = status;
  in.faults = FaultCounter();
  held = in;
  held.words = reinterpret_cast<const unsigned long long*>(hold);
  held.count = static_cast<int>(hold_count);
  held.tag = hold_tag;
  const std::int64_t row_blocks = llmp_b200_q8_1_row_blocks(k);
  const std::int64_t total = row_blocks * 8;
  const dim3 grid(static_cast<unsigned>((total + kThreads - 1) / kThreads));
  const cudaError_t e = LaunchPdl(QuantizeWordsKernel, grid, dim3(kThreads), 0,
                                  static_cast<cudaStream_t>(stream), x, in, held, k, row_blocks, total,
                                  static_cast<std::uint8_t*>(out));
  return e == cudaSuccess ? 0 : Failed(e, "q8_1 words launch");
}

int llmp_b200_q8_1_quantize_exchange(const float* x, int64_t k, void* out,
                                     const llmp_b200_peer_site* site, const int32_t* local_flags,
                                     const void* slice, size_t offset, size_t bytes, int polls,
                                     int32_t* status, void* stream) {
  using namespace llmp_b200;
  if (site == nullptr || local_flags == nullptr || polls < 1 || site->world < 1 || site->world > 32 ||
      site->step == nullptr || site->site < 0 || site->buffers == nullptr || site->flags == nullptr ||
      site->rank < 0 || site->rank >= site->world) {
    return Reject("q8_1 exchange: a site, this rank's flag words and a poll limit");
  }
  if (slice == nullptr || bytes == 0 || !Aligned(slice, 16) || offset % 16 != 0) {
    return Reject("q8_1 exchange: a 16-byte aligned slice at a 16-byte aligned offset");
  }
  return Quantize(x, k, 1, 1, k, 0, out, PeerWaitOf(*site, local_flags, polls, status),
                  PeerPublishOf(*site, slice, offset, bytes), stream);
}

}  // extern "C"
