// Dense llmp.vecq as a persistent HBM stream (the fast path for dense
// products whose rows start on 16-byte boundaries; everything else takes the
// kernel in vecq_impl.cuh).  Same interface and sums' contract as
// src/kernels/ggml/vecq.cu:457-665; the structure is B200's:
//
//   * one CTA per SM owns a contiguous, evenly divided range of output rows;
//   * weight rows arrive in shared memory through the TMA bulk-copy engine
//     (cp.async.bulk, one copy per matrix and stage when rows are packed) into
//     a ring of stages, each completing on an mbarrier; the ring is as deep as
//     shared memory allows (~160 KB in flight per SM), which is what keeps HBM
//     busy for a 15-30 MB matrix that lasts a few microseconds;
//   * the first stages are requested BEFORE the programmatic-dependency wait:
//     weights depend on no earlier kernel;
//   * thread t owns unit (t mod units-per-row) of every row it meets, so its
//     activations (one unit per token) stay in registers for the whole kernel;
//   * per-unit partial sums go through shared memory and are summed per row
//     in a fixed order (strided by lane, then an xor-shuffle tree): no atomics,
//     and a (token, row) sum never depends on the other tokens of the launch;
//   * every mbarrier wait is bounded; a wait that runs out raises a device
//     flag the host can read (llmp_b200_device_faults) and the kernel finishes.
#ifndef LLMP_B200_CSRC_VECQ_STREAM_CUH_
#define LLMP_B200_CSRC_VECQ_STREAM_CUH_

#include "vecq_impl.cuh"

namespace llmp_b200 {

namespace vecq {

constexpr int kStreamThreads = 256;
constexpr int kStreamInFlight = 2;  // stages requested ahead of the one being summed
constexpr int kStreamMaxStages = 16;
constexpr std::uint32_t kWaitLimit = 1u << 22;  // polls of ~20-50 ns

// How a product's rows are dealt to CTAs and a CTA's to its warps, worked out on
// the host so that no division runs on the device: CTA b owns rows_q + (b <
// rows_rem) rows, and a CTA of rows_q + e rows gives warp w warp_q[e] + (w <
// warp_rem[e]) of them.
struct RowSplit {
  int rows_q, rows_rem, warp_q0, warp_q1, warp_rem0, warp_rem1;
};
inline RowSplit MakeRowSplit(int nrows, int grid, int warps) {
  RowSplit s{};
  s.rows_q = nrows / grid;
  s.rows_rem = nrows % grid;
  s.warp_q0 = s.rows_q / warps;
  s.warp_rem0 = s.rows_q % warps;
  s.warp_q1 = (s.rows_q + 1) / warps;
  s.warp_rem1 = (s.rows_q + 1) % warps;
  return s;
}
struct StreamPlan {
  int units_per_row;   // UR
  int rows_per_step;   // RS = threads / UR
  int rows_per_stage;  // RG, a multiple of RS
  int stages;          // S
  int row_bytes;
  int stage_bytes;     // all matrices
  int partial_floats;  // one buffer: P * RG * UR * mats
  int smem_bytes;
  int grid;
  bool packed;         // rows contiguous: one copy per matrix and stage
  unsigned int* faults;  // device counter a wait that ran out increments
  RowSplit split;        // the rows of a CTA (the warp part is unused)
  int unit_reciprocal;   // ceil(2^20 / UR): tid / UR without a division (tid < 1024)
};

__device__ __forceinline__ std::uint32_t SmemAddr(const void* p) {
  return static_cast<std::uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void MbarInit(std::uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count));
}
__device__ __forceinline__ void MbarExpectTx(std::uint64_t* bar, std::uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)),
               "r"(bytes)
               : "memory");
}
// Bounded: false if the phase did not complete within the limit.
__device__ __forceinline__ bool MbarWait(std::uint64_t* bar, std::uint32_t parity) {
  const std::uint32_t addr = SmemAddr(bar);
  for (std::uint32_t i = 0; i < kWaitLimit; ++i) {
    std::uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (i > 4) __nanosleep(40);  // leave the issue slots to the warps that have data
  }
  return false;
}
// One lane of the (converged) warp: what it issues to the copy engine takes its
// operands from uniform registers at once.
__device__ __forceinline__ bool ElectOne() {
  std::uint32_t pred = 0;
  asm volatile(
      "{\n"
      ".reg .b32 rx;\n"
      ".reg .pred px;\n"
      "elect.sync rx|px, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, px;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}
// One look at the phase without blocking: a blocking wait costs a few hundred
// cycles even on a phase that completed long ago.
__device__ __forceinline__ bool MbarTest(std::uint64_t* bar, std::uint32_t parity) {
  std::uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(SmemAddr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// The warp's wait for a stage: every lane looks once; only if some lane saw the
// phase open does lane 0 wait, with its bound.  False (for all lanes) if it ran out.
__device__ __forceinline__ bool WarpAwait(std::uint64_t* bar, std::uint32_t parity, int lane) {
  if (__all_sync(0xffffffffu, MbarTest(bar, parity) ? 1 : 0)) return true;
  int ok = 1;
  if (lane == 0) ok = MbarWait(bar, parity) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__device__ __forceinline__ void CtaRows(const RowSplit& s, int cta, int* begin, int* count) {
  *begin = (cta * s.rows_q) + min(cta, s.rows_rem);
  *count = s.rows_q + (cta < s.rows_rem ? 1 : 0);
}
__device__ __forceinline__ void WarpRows(const RowSplit& s, int cta, int warp, int* begin, int* count) {
  int cta_begin, cta_count;
  CtaRows(s, cta, &cta_begin, &cta_count);
  const bool extra = cta < s.rows_rem;
  const int q = extra ? s.warp_q1 : s.warp_q0, rem = extra ? s.warp_rem1 : s.warp_rem0;
  *begin = cta_begin + (warp * q) + min(warp, rem);
  *count = q + (warp < rem ? 1 : 0);
}

// Global -> this CTA's shared memory, completing `bytes` on the mbarrier.
__device__ __forceinline__ void BulkLoad(void* smem, const void* gmem, std::uint32_t bytes,
                                         std::uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(SmemAddr(smem)), "l"(gmem), "r"(bytes), "r"(SmemAddr(bar))
      : "memory");
}
__device__ __forceinline__ void FenceProxyAsync() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// One whole Q4_K super-block a thread (144 bytes, nine 128-bit shared loads):
// the 6-bit scales are unpacked once for the eight sub-blocks.  The one-token
// stream uses this unit; its activations (256 values) fit a thread's registers.
struct Q4KBlockUnit {
  static constexpr int kType = LLMP_B200_TYPE_Q4_K;
  static constexpr int kBlockBytes = 144;
  static constexpr int kBlockElems = 256;
  static constexpr int kUnitElems = 256;
  uint4 head;
  uint4 q[8];
  __device__ __forceinline__ void LoadShared(const std::uint8_t* row, int u) {
    const auto* sb = reinterpret_cast<const uint4*>(row + (static_cast<std::size_t>(u) * 144));
    head = sb[0];
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = sb[1 + i];
  }
};

// u8 x s8 dot product of four bytes into an s32 sum.
__device__ __forceinline__ int Dp4aU8S8(std::uint32_t a, int b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// A thread's activations for its unit, one token.
template <typename Unit>
struct UnitActs;

template <>
struct UnitActs<Q4KBlockUnit> {
  int q[64];     // 256 int8
  float d8[8];   // per 32-value block: d
  float fs[8];   // d * sum q
  __device__ __forceinline__ void Load(const std::uint8_t* y, int u) {
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      const auto* src = reinterpret_cast<const std::uint32_t*>(
          y + (static_cast<std::size_t>((u * 8) + g) * 36));
      int isum = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        q[(8 * g) + i] = static_cast<int>(src[1 + i]);
        isum = Dp4a(0x01010101, q[(8 * g) + i], isum);
      }
      d8[g] = HalfBitsToFloat(src[0] & 0xffffu);
      fs[g] = d8[g] * static_cast<float>(isum);
    }
  }
};

// The eight per-sub-block int32 sums (sum code * q) of a super-block.  The
// high nibbles are multiplied in place (16 * code as an unsigned byte) and
// the exact factor 16 is shifted out of the sum.
__device__ __forceinline__ void Q4KBlockDots(const Q4KBlockUnit& w, const int* aq, int dots[8]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const std::uint32_t words[8] = {w.q[2 * c].x,     w.q[2 * c].y,     w.q[2 * c].z,
                                    w.q[2 * c].w,     w.q[2 * c + 1].x, w.q[2 * c + 1].y,
                                    w.q[2 * c + 1].z, w.q[2 * c + 1].w};
    int lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      lo = Dp4aU8S8(words[i] & 0x0f0f0f0fu, aq[(16 * c) + i], lo);
      hi = Dp4aU8S8(words[i] & 0xf0f0f0f0u, aq[(16 * c) + 8 + i], hi);
    }
    dots[2 * c] = lo;
    dots[(2 * c) + 1] = hi >> 4;
  }
}

__device__ __forceinline__ void Q4KBlockScales(const Q4KBlockUnit& w, int sc[8], int mn[8]) {
  // The twelve bytes hold 6-bit fields: scales 0..3 and minima 0..3 in the low six
  // bits of bytes 0..3 and 4..7; scales / minima 4..7 as the low / high nibbles of
  // bytes 8..11 with their top two bits in bits 6..7 of bytes 0..3 / 4..7.  Unpacked
  // four at a time as packed bytes, then one extract a value.
  const std::uint32_t s0 = w.head.y, s1 = w.head.z, s2 = w.head.w;
  const std::uint32_t sc_lo = s0 & 0x3f3f3f3fu;
  const std::uint32_t mn_lo = s1 & 0x3f3f3f3fu;
  const std::uint32_t sc_hi = (s2 & 0x0f0f0f0fu) | ((s0 >> 2) & 0x30303030u);
  const std::uint32_t mn_hi = ((s2 >> 4) & 0x0f0f0f0fu) | ((s1 >> 2) & 0x30303030u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    sc[i] = static_cast<int>((sc_lo >> (8 * i)) & 0xffu);
    mn[i] = static_cast<int>((mn_lo >> (8 * i)) & 0xffu);
    sc[4 + i] = static_cast<int>((sc_hi >> (8 * i)) & 0xffu);
    mn[4 + i] = static_cast<int>((mn_hi >> (8 * i)) & 0xffu);
  }
}

// d * sum_g d8_g * (sc_g * dot_g)  -  dmin * sum_g (d8_g * sum q_g) * m_g
__device__ __forceinline__ float UnitDot(const Q4KBlockUnit& w, const UnitActs<Q4KBlockUnit>& a) {
  int dots[8], sc[8], mn[8];
  Q4KBlockDots(w, a.q, dots);
  Q4KBlockScales(w, sc, mn);
  float sumd = 0.0f, summ = 0.0f;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    sumd = fmaf(a.d8[g], static_cast<float>(dots[g] * sc[g]), sumd);
    summ = fmaf(a.fs[g], static_cast<float>(mn[g]), summ);
  }
  const float d = HalfBitsToFloat(w.head.x & 0xffffu);
  const float dmin = HalfBitsToFloat(w.head.x >> 16);
  return (d * sumd) - (dmin * summ);
}

template <>
struct UnitActs<Q4KUnit> {
  uint4 q[4];  // 64 int8
  float4 s;    // d8_0, d8_0 * sum q_0, d8_1, d8_1 * sum q_1
  __device__ __forceinline__ void Load(const std::uint8_t* y, int u) {
    std::uint32_t v[16];
    float sc[4];
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      const auto* src = reinterpret_cast<const std::uint32_t*>(
          y + (static_cast<std::size_t>((u * 2) + g) * 36));
      const std::uint32_t ds = src[0];
      int isum = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[(8 * g) + i] = src[1 + i];
        isum = Dp4a(0x01010101, static_cast<int>(v[(8 * g) + i]), isum);
      }
      const float d = HalfBitsToFloat(ds & 0xffffu);
      sc[2 * g] = d;
      sc[(2 * g) + 1] = d * static_cast<float>(isum);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    s = make_float4(sc[0], sc[1], sc[2], sc[3]);
  }
};

template <>
struct UnitActs<Q8_0Unit<4>> {
  int q[32];
  float d[4];
  __device__ __forceinline__ void Load(const std::uint8_t* y, int u) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const auto* src = reinterpret_cast<const std::uint32_t*>(
          y + (static_cast<std::size_t>((u * 4) + b) * 36));
      d[b] = HalfBitsToFloat(src[0] & 0xffffu);
#pragma unroll
      for (int i = 0; i < 8; ++i) q[(8 * b) + i] = static_cast<int>(src[1 + i]);
    }
  }
};

// One unit's product with one token's activations.
__device__ __forceinline__ float UnitDot(const Q4KDecoded& w, const UnitActs<Q4KUnit>& a) {
  int d0, d1;
  Q4KDots(w, a.q, &d0, &d1);
  float v = (a.s.x * w.dsc0) * static_cast<float>(d0);
  v = fmaf(a.s.z * w.dsc1, static_cast<float>(d1), v);
  v = fmaf(-a.s.y, w.dmn0, v);
  v = fmaf(-a.s.w, w.dmn1, v);
  return v;
}
__device__ __forceinline__ float UnitDot(const Q8_0Unit<4>& w, const UnitActs<Q8_0Unit<4>>& a) {
  float v = 0.0f;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    int sumi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) sumi = Dp4a(w.Int(b, i), a.q[(8 * b) + i], sumi);
    v += w.Scale(b) * a.d[b] * static_cast<float>(sumi);
  }
  return v;
}

template <typename Unit, int P, bool kGlu>
__global__ void __launch_bounds__(kStreamThreads, 1)
VecQStreamKernel(const Desc a, const StreamPlan plan) {
  constexpr int kMats = kGlu ? 2 : 1;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) std::uint64_t full[kStreamMaxStages];

  const int tid = static_cast<int>(threadIdx.x);
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int UR = plan.units_per_row;
  const int RS = plan.rows_per_step;
  const int RG = plan.rows_per_stage;
  const int S = plan.stages;
  const int step_row = static_cast<int>((static_cast<unsigned>(tid) * static_cast<unsigned>(plan.unit_reciprocal)) >> 20);
  const int u = tid - (step_row * UR);
  const bool active = step_row < RS;
  float* partial = reinterpret_cast<float*>(smem + (static_cast<std::size_t>(S) * plan.stage_bytes));

  // This CTA's rows, evenly divided over the grid.
  int row_begin, my_rows;
  CtaRows(plan.split, static_cast<int>(blockIdx.x), &row_begin, &my_rows);
  const int row_end = row_begin + my_rows;
  const int iterations = (my_rows + RG - 1) / RG;

  // (no pointer array indexed by a variable: it would live in local memory)
  const auto matrix = [&](int m) {
    return static_cast<const std::uint8_t*>(kGlu && m != 0 ? a.g : a.w);
  };
  const std::size_t row_pitch = static_cast<std::size_t>(a.stride_row) * Unit::kBlockBytes;

  if (tid < S) {
    MbarInit(&full[tid], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // Requests the rows of the next iteration into its stage (warp 0, converged;
  // iterations are requested in order).
  int next = 0, next_stage = 0;
  auto request = [&]() __attribute__((always_inline)) {
    const int s = next_stage;
    const int r0 = row_begin + (next * RG);
    const int rows = min(RG, row_end - r0);
    unsigned char* base = smem + (static_cast<std::size_t>(s) * plan.stage_bytes);
    if (lane == 0) {
      MbarExpectTx(&full[s], static_cast<std::uint32_t>(rows) * plan.row_bytes * kMats);
    }
    __syncwarp();
    if (plan.packed) {
      if (lane < kMats) {
        BulkLoad(base + (static_cast<std::size_t>(lane) * RG * plan.row_bytes),
                 matrix(lane) + (static_cast<std::size_t>(r0) * row_pitch),
                 static_cast<std::uint32_t>(rows) * plan.row_bytes, &full[s]);
      }
    } else {
      for (int c = lane; c < rows * kMats; c += 32) {
        const int m = c >= rows ? 1 : 0;
        const int r = c - (m * rows);
        BulkLoad(base + ((static_cast<std::size_t>(m) * RG + r) * plan.row_bytes),
                 matrix(m) + (static_cast<std::size_t>(r0 + r) * row_pitch), plan.row_bytes,
                 &full[s]);
      }
    }
    ++next;
    if (++next_stage == S) next_stage = 0;
  };

  GridLaunchDependents();
  // Two iterations in flight, not the whole ring: the copy engine serves the copies it
  // holds side by side, so a ring requested at once lands at once, at the end of the
  // transfer, and no iteration's sums overlap it.
  if (warp == 0) {
    while (next < min(min(S, kStreamInFlight), iterations)) request();
  }
  GridDependencyWait();

  // The thread's activations: unit u of each token's Q8_1 row.
  UnitActs<Unit> acts[P];
#pragma unroll
  for (int j = 0; j < P; ++j) {
    const int t = min(j, a.tokens - 1);
    acts[j].Load(static_cast<const std::uint8_t*>(a.y) +
                     (static_cast<std::size_t>(t) * a.y_token * 36), u);
  }

  bool healthy = true;
  const int partial_stride = plan.partial_floats;  // floats in one buffer
  int s = 0;
  std::uint32_t parity = 0;
  for (int it = 0; it < iterations; ++it) {
    const int r0 = row_begin + (it * RG);
    const int rows = min(RG, row_end - r0);
    if (healthy && !WarpAwait(&full[s], parity, lane)) {
      healthy = false;
      if (lane == 0) atomicAdd(plan.faults, 1u);
    }
    const unsigned char* base = smem + (static_cast<std::size_t>(s) * plan.stage_bytes);
    float* part = partial + ((it & 1) * partial_stride);
    if (active) {
      for (int r = step_row; r < rows; r += RS) {
#pragma unroll
        for (int m = 0; m < kMats; ++m) {
          const std::uint8_t* rowp = base + ((static_cast<std::size_t>(m) * RG + r) * plan.row_bytes);
          Unit raw;
          raw.LoadShared(rowp, u);
          if constexpr (Unit::kUnitElems == 64) {
            Q4KDecoded dec;
            dec.From(raw, u);
#pragma unroll
            for (int j = 0; j < P; ++j) {
              part[(((j * kMats) + m) * RG + r) * UR + u] = UnitDot(dec, acts[j]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < P; ++j) {
              part[(((j * kMats) + m) * RG + r) * UR + u] = UnitDot(raw, acts[j]);
            }
          }
        }
      }
    }
    __syncthreads();  // partials written; the stage's bytes are consumed
    if (warp == 0 && next < iterations) {  // the stage just read takes the next iteration
      FenceProxyAsync();
      request();
    }
    // Row sums: warp w takes (row, token) items w, w + 8, ...
    const int items = rows * P;
    for (int item = warp; item < items; item += kStreamThreads / 32) {
      const int r = item / P;
      const int j = item % P;
      if (j >= a.tokens) continue;
      float v[kMats];
#pragma unroll
      for (int m = 0; m < kMats; ++m) {
        const float* src = part + ((((j * kMats) + m) * RG + r) * UR);
        float sum = 0.0f;
        for (int i = lane; i < UR; i += 32) sum += src[i];
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
          sum += __shfl_xor_sync(0xffffffffu, sum, offset);
        }
        v[m] = sum;
      }
      if (lane == 0) {
        float* dst = a.dst + (static_cast<std::size_t>(j) * a.dst_token) + r0 + r;
        if constexpr (kGlu) {
          *dst = Glu(a.glu, v[1], v[0], a.limit);
        } else {
          *dst = v[0];
        }
      }
    }
    if (++s == S) {
      s = 0;
      parity ^= 1u;
    }
  }
}

// Host: whether the shape takes the stream kernel, and its plan.
inline bool PlanStream(const Desc& d, int unit_elems, int block_bytes, int block_elems, int p,
                       int sms, StreamPlan* plan) {
  const int mats = d.glu != LLMP_B200_GLU_NONE ? 2 : 1;
  const int ur = d.ncols_x / unit_elems;
  if (ur < 1 || ur > kStreamThreads) return false;
  const int row_bytes = (d.ncols_x / block_elems) * block_bytes;
  const long pitch = static_cast<long>(d.stride_row) * block_bytes;
  if (row_bytes % 16 != 0 || pitch % 16 != 0) return false;
  const int rs = kStreamThreads / ur;
  // Stage: whole steps of rows, about 12 KB, but at least one step.
  int steps = (12 * 1024) / std::max(1, rs * row_bytes * mats);
  steps = std::max(1, std::min(steps, 8));
  const int rg = rs * steps;
  const int stage_bytes = rg * row_bytes * mats;
  const int partial_floats = p * rg * ur * mats;
  const int budget = 200 * 1024 - (2 * partial_floats * 4);
  int stages = budget / stage_bytes;
  if (stages < 2) return false;
  stages = std::min(stages, kStreamMaxStages);
  plan->units_per_row = ur;
  plan->rows_per_step = rs;
  plan->rows_per_stage = rg;
  plan->stages = stages;
  plan->row_bytes = row_bytes;
  plan->stage_bytes = stage_bytes;
  plan->partial_floats = partial_floats;
  plan->smem_bytes = (stages * stage_bytes) + (2 * partial_floats * 4);
  plan->grid = std::max(1, std::min(sms, d.nrows));
  plan->packed = d.stride_row == d.ncols_x / block_elems;
  plan->split = MakeRowSplit(d.nrows, plan->grid, 1);
  plan->unit_reciprocal = ((1 << 20) + ur - 1) / ur;
  plan->faults = FaultCounter();
  return plan->faults != nullptr;
}

template <typename Unit, int P, bool kGlu>
cudaError_t LaunchStreamOne(const Desc& d, const StreamPlan& plan, cudaStream_t stream) {
  auto* kernel = VecQStreamKernel<Unit, P, kGlu>;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             plan.smem_bytes);
  if (e != cudaSuccess) return e;
  return LaunchPdl(kernel, dim3(static_cast<unsigned>(plan.grid)), dim3(kStreamThreads),
                   static_cast<std::size_t>(plan.smem_bytes), stream, d, plan);
}

template <typename Unit>
cudaError_t LaunchStream(const Desc& d, int p, const StreamPlan& plan, cudaStream_t stream) {
  const bool glu = d.glu != LLMP_B200_GLU_NONE;
#define LLMP_P(PP)                                                            \
  if (p == PP)                                                                \
    return glu ? LaunchStreamOne<Unit, PP, true>(d, plan, stream)             \
               : LaunchStreamOne<Unit, PP, false>(d, plan, stream);
  LLMP_P(1)
  if constexpr (Unit::kUnitElems != 256) {  // the whole-super-block unit is one-token only
    LLMP_P(2) LLMP_P(4) LLMP_P(8)
  }
#undef LLMP_P
  return cudaErrorInvalidValue;
}

}  // namespace vecq
}  // namespace llmp_b200

#endif  // LLMP_B200_CSRC_VECQ_STREAM_CUH_
