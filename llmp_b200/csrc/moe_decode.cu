// The routed MoE block for a handful of tokens as ONE launch (decode): Q8_1 of the token,
// every named expert's gate|up product with the GLU, Q8_1 of that, the down product and the
// weighted sum over the token's experts, which the reference runs as separate nodes
// (llmp.q8_1, llmp.vecq with ids and a GLU, llmp.q8_1, llmp.vecq per slot, llmp.moe.combine:
// src/kernels/ggml/vecq.cu:457-665, llmp_moe.cu:393-435) and llmp_b200.moe_ffn as five
// launches.  At one token those launches, not the 21 MB of expert weights, are the time.
//
// One CTA of 16 warps an SM, launched cooperatively (all resident).  Phase A: a warp asks for
// the gate and up rows of its four (slot, row) items by bulk copies into its own buffer
// (completing on its own barrier) and, while they travel, the CTA quantizes the token itself
// (the Q8_1 quantizer's arithmetic, q8_1.cu) into shared memory; a lane is (item,
// super-block), decodes one 144-byte super-block of each row, and the lanes of an item meet in
// an xor tree; the GLU output goes to scratch.  (Streaming 16-byte loads a lane, 144 bytes
// apart, ran the load unit at one sector a cycle: 8 to 10 us for this phase alone.)  One grid barrier (an arrival counter, waited for with a
// bound) while the first down rows already travel.  Phase B: every CTA quantizes all of the
// token's GLU rows itself (a few KB), then a warp is an output row: lane (slot, super-block) of the down product, the slots' sums
// weighted and added in slot order with the combine kernel's arithmetic (a product rounded,
// then added), so the result does not depend on the launch geometry.
#include "common.cuh"
#include "vecq_stream.cuh"

namespace llmp_b200 {
namespace {

using vecq::Q4KBlockUnit;

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxHidden = 8192;       // the token's staged activations
constexpr int kMaxGluValues = 8 * 2048;

// A row's Q8_1 blocks as the dot products read them: the int8 codes, a super-block's 256 every
// kCodePitch bytes, then per 32-value block (d, d * sum of the codes) as F32, a super-block's
// eight pairs every kScalePitch bytes.  The pitches are odd multiples of 16 and 8 bytes: the
// eight lanes of a quarter warp read eight different super-blocks, which 256- and 64-byte
// pitches would put on the same banks (measured: the whole kernel ran at the speed of those
// conflicts).
constexpr int kCodePitch = 272, kScalePitch = 72;
__host__ __device__ constexpr int StagedBytes(int k) { return (k / 256) * (kCodePitch + kScalePitch); }

// 32-value blocks of src (F32) quantized as the Q8_1 quantizer does (q8_1.cu: eight lanes a
// block, d = amax / 127 rounded to FP16, q = roundf(x / d) with the unrounded d) straight into
// that staged form.  Every load of a batch is in flight before the first value is used.
__device__ __forceinline__ void QuantizeToShared(const float* __restrict__ src, int k,
                                                 std::uint8_t* __restrict__ out, bool other_sms) {
  const int lanes = (k / 32) * 8;
  std::uint8_t* scales = out + ((k / 256) * kCodePitch);
  constexpr int kPasses = 4;
  for (int batch = 0; batch < lanes; batch += kPasses * kThreads) {
    float4 f[kPasses];
#pragma unroll
    for (int q = 0; q < kPasses; ++q) {
      const int i = batch + (q * kThreads) + static_cast<int>(threadIdx.x);
      f[q] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (i < lanes) {
        const float4* p = reinterpret_cast<const float4*>(src + ((i / 8) * 32) + ((i % 8) * 4));
        f[q] = other_sms ? __ldcg(p) : *p;  // written by other SMs: not through L1
      }
    }
#pragma unroll
    for (int q = 0; q < kPasses; ++q) {
      if (batch + (q * kThreads) >= lanes) break;  // uniform: whole passes only
      const int i = batch + (q * kThreads) + static_cast<int>(threadIdx.x);
      const bool live = i < lanes;
      const int block = (live ? i : 0) / 8, lane8 = i % 8;
      const float v[4] = {f[q].x, f[q].y, f[q].z, f[q].w};
      float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
      for (int offset = 4; offset > 0; offset >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
      }
      const float d = amax / 127.0f;
      std::uint32_t packed = 0;
      if (amax != 0.0f) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int qv = static_cast<int>(roundf(v[c] / d));
          packed |= (static_cast<std::uint32_t>(qv) & 0xffu) << (8 * c);
        }
      }
      int isum = Dp4a(0x01010101, static_cast<int>(packed), 0);
#pragma unroll
      for (int offset = 4; offset > 0; offset >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, offset);
      if (live) {
        *reinterpret_cast<std::uint32_t*>(out + ((block >> 3) * kCodePitch) + ((block & 7) * 32) +
                                          (lane8 * 4)) = packed;
        if (lane8 == 0) {
          const float d8 = __half2float(__float2half_rn(d));  // what the block would store
          *reinterpret_cast<float2*>(scales + ((block >> 3) * kScalePitch) + ((block & 7) * 8)) =
              make_float2(d8, d8 * static_cast<float>(isum));
        }
      }
    }
  }
}

// A super-block's dot product with super-block u of a staged row: the arithmetic of
// vecq::UnitDot with the activations read from shared memory as they are used.
__device__ __forceinline__ float DotStaged(const Q4KBlockUnit& w, const std::uint8_t* staged, int k,
                                           int u) {
  const uint4* aq = reinterpret_cast<const uint4*>(staged + (u * kCodePitch));
  const float2* sc8 =
      reinterpret_cast<const float2*>(staged + ((k / 256) * kCodePitch) + (u * kScalePitch));
  int sc[8], mn[8];
  vecq::Q4KBlockScales(w, sc, mn);
  float sumd = 0.0f, summ = 0.0f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const std::uint32_t words[8] = {w.q[2 * c].x,     w.q[2 * c].y,     w.q[2 * c].z,
                                    w.q[2 * c].w,     w.q[2 * c + 1].x, w.q[2 * c + 1].y,
                                    w.q[2 * c + 1].z, w.q[2 * c + 1].w};
    const uint4 a0 = aq[4 * c], a1 = aq[(4 * c) + 1], b0 = aq[(4 * c) + 2], b1 = aq[(4 * c) + 3];
    const int lo_a[8] = {static_cast<int>(a0.x), static_cast<int>(a0.y), static_cast<int>(a0.z),
                         static_cast<int>(a0.w), static_cast<int>(a1.x), static_cast<int>(a1.y),
                         static_cast<int>(a1.z), static_cast<int>(a1.w)};
    const int hi_a[8] = {static_cast<int>(b0.x), static_cast<int>(b0.y), static_cast<int>(b0.z),
                         static_cast<int>(b0.w), static_cast<int>(b1.x), static_cast<int>(b1.y),
                         static_cast<int>(b1.z), static_cast<int>(b1.w)};
    int lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      lo = vecq::Dp4aU8S8(words[i] & 0x0f0f0f0fu, lo_a[i], lo);
      hi = vecq::Dp4aU8S8(words[i] & 0xf0f0f0f0u, hi_a[i], hi);
    }
    const float2 s0 = sc8[2 * c], s1 = sc8[(2 * c) + 1];
    sumd = fmaf(s0.x, static_cast<float>(lo * sc[2 * c]), sumd);
    summ = fmaf(s0.y, static_cast<float>(mn[2 * c]), summ);
    sumd = fmaf(s1.x, static_cast<float>((hi >> 4) * sc[(2 * c) + 1]), sumd);
    summ = fmaf(s1.y, static_cast<float>(mn[(2 * c) + 1]), summ);
  }
  const float d = HalfBitsToFloat(w.head.x & 0xffffu);
  const float dmin = HalfBitsToFloat(w.head.x >> 16);
  return (d * sumd) - (dmin * summ);
}

// Every CTA arrives; true once all have.  The counter only ever grows (a launch adds
// gridDim.x), so it needs zeroing once, not between launches.
// In two halves, so that work that needs nothing from the other CTAs (the first down
// rows' requests) runs while the arrivals travel.
__device__ __forceinline__ unsigned int GridArrive(unsigned int* counter) {
  __threadfence();
  __syncthreads();
  unsigned int target = 0;
  if (threadIdx.x == 0) {
    const unsigned int mine = atomicAdd(counter, 1u);
    target = ((mine / gridDim.x) + 1u) * gridDim.x;
  }
  return target;  // thread 0's: what the counter reads once every CTA has arrived
}
__device__ __forceinline__ bool GridAwait(unsigned int* counter, unsigned int target, int polls) {
  bool ok = true;
  if (threadIdx.x == 0) {
    ok = false;
    for (int i = 0; i < polls; ++i) {
      unsigned int now;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(now) : "l"(counter) : "memory");
      if (static_cast<int>(now - target) >= 0) {
        ok = true;
        break;
      }
      __nanosleep(40);
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// Shared memory: the staged token, the staged GLU rows, then a buffer a warp for the weight
// rows it works on (32 lanes x 2 super-blocks: four gate/up row pairs in phase A, the eight
// slots' down rows in phase B), filled by bulk copies that complete on the warp's own barrier.
constexpr int kWarpBuffer = 32 * 2 * 144;
__host__ __device__ constexpr int Round128(int v) { return (v + 127) / 128 * 128; }
__host__ __device__ constexpr int DecodeSmem(int hidden, int glu_values) {
  return Round128(StagedBytes(hidden)) + Round128(StagedBytes(glu_values)) + (kWarps * kWarpBuffer);
}

__global__ void __launch_bounds__(kThreads, 1)
MoeDecodeKernel(const llmp_b200_moe_decode_desc a, unsigned int* faults, int polls) {
  extern __shared__ __align__(128) std::uint8_t smem[];
  __shared__ __align__(8) std::uint64_t landed[kWarps];
  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const int ur_a = a.hidden / 256;  // super-blocks of a gate / up row: a power of two <= 32
  const int ur_b = a.inter / 256;   // of a down row
  int span_b = 1;                   // lanes a slot in phase B: ur_b rounded up to a power of two
  while (span_b < ur_b) span_b *= 2;
  std::uint8_t* xq = smem;
  std::uint8_t* hq = xq + Round128(StagedBytes(a.hidden));
  std::uint8_t* rows = hq + Round128(StagedBytes(a.used * a.inter)) + (warp * kWarpBuffer);
  auto* counter = static_cast<unsigned int*>(a.scratch);
  float* glu_rows = reinterpret_cast<float*>(static_cast<std::uint8_t*>(a.scratch) + 256);
  const auto* gate_up = static_cast<const std::uint8_t*>(a.gate_up);
  const auto* down = static_cast<const std::uint8_t*>(a.down);
  if (lane == 0) {
    vecq::MbarInit(&landed[warp], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  std::uint32_t uses = 0;  // of this warp's barrier: the parity of the next wait
  bool healthy = true;

  GridDependencyWait();  // x, ids and weights may be the kernel before's output

  // Lane l's copy of a request (a whole weight row) and whether it has one; lane 0 arms the
  // barrier with the bytes of all of them first.  The buffer's last readers were this warp's
  // own shared-memory loads.
  auto request = [&](bool mine, const std::uint8_t* src, std::uint32_t bytes, int slot) {
    __syncwarp();
    vecq::FenceProxyAsync();
    const unsigned int copies = __ballot_sync(0xffffffffu, mine);
    if (lane == 0 && copies != 0) {
      vecq::MbarExpectTx(&landed[warp], bytes * static_cast<std::uint32_t>(__popc(copies)));
    }
    __syncwarp();
    if (mine) vecq::BulkLoad(rows + (static_cast<std::size_t>(slot) * bytes), src, bytes, &landed[warp]);
    return copies != 0;
  };
  auto wait = [&](bool pending) {
    if (!pending) return;
    bool ok = true;
    if (lane == 0) ok = vecq::MbarWait(&landed[warp], uses & 1u);
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    ++uses;
    if (!ok) {
      if (lane == 0 && healthy) atomicAdd(faults, 1u);
      healthy = false;
    }
  };
  // Token t's expert ids, read once a phase (each read is a trip to L2 on the kernel's
  // critical path): lane j < used holds slot j's, the others get it by shuffle.
  int lane_id = -1;
  auto token_ids = [&](int t) {
    lane_id = lane < a.used ? a.ids[(static_cast<std::int64_t>(t) * a.ids_stride) + lane] : -1;
  };
  auto slot_id = [&](int j) { return __shfl_sync(0xffffffffu, lane_id, j); };
  // Phase A's request for the round starting at item `first` of token t: the round's items
  // are consecutive rows of ONE expert (a slot's items are a multiple of a round's), so their
  // gate rows are one run of bytes and their up rows another: lane 0 fetches the first, lane 1
  // the second.  (A copy a row, eight a warp, kept the SM's copy engine busy for 2 K cycles
  // before the last was accepted: it takes a copy about every 20 cycles whatever its size.)
  const int items = a.used * a.inter;
  const int items_a_warp = 32 / ur_a;
  const std::uint32_t bytes_a = static_cast<std::uint32_t>(ur_a) * 144u;
  auto round_items = [&](int first) { return min(items_a_warp, items - first); };
  auto request_a = [&](int t, int first) {
    const int n = round_items(first);
    const int j = n > 0 ? first / a.inter : 0, i = first - (j * a.inter);
    const int e = slot_id(j);
    const bool mine = lane < 2 && n > 0 && e >= 0 && e < a.experts;
    const std::uint8_t* src = gate_up;
    if (mine) src += (((static_cast<std::size_t>(e) * 2) + lane) * a.inter + i) * bytes_a;
    return request(mine, src, static_cast<std::uint32_t>(max(n, 0)) * bytes_a, lane);
  };
  // Phase B's: lane j < used fetches slot j's row r of the down tensor.
  const std::uint32_t bytes_b = static_cast<std::uint32_t>(ur_b) * 144u;
  auto request_b = [&](int t, int r) {
    bool mine = lane < a.used && r < a.hidden;
    const std::uint8_t* src = down;
    const int e = lane_id;  // lane j's own slot
    mine = mine && e >= 0 && e < a.experts;
    if (mine) src += ((static_cast<std::size_t>(e) * a.hidden) + r) * bytes_b;
    return request(mine, src, bytes_b, lane);
  };

  // ---- phase A: h[t][j][i] = glu(gate_e[i] . x_t, up_e[i] . x_t), e = ids[t][j]
  const int first_a = ((static_cast<int>(blockIdx.x) * kWarps) + warp) * items_a_warp;
  const int step_a = static_cast<int>(gridDim.x) * kWarps * items_a_warp;
  const int cta_items = kWarps * items_a_warp;  // items a CTA and round: consecutive
  const int cta_first = static_cast<int>(blockIdx.x) * cta_items;
  const bool at_source = cta_items % 32 == 0;   // ... and whole Q8_1 blocks
  float* exchange = reinterpret_cast<float*>(hq);  // phase A only: the staged GLU rows' place
  std::uint8_t* staged_rows = reinterpret_cast<std::uint8_t*>(glu_rows);  // in scratch, a token's
  const std::size_t staged_pitch = static_cast<std::size_t>(Round128(StagedBytes(items)));
  for (int t = 0; t < a.tokens; ++t) {
    // the first round's rows travel while the token is quantized
    token_ids(t);
    bool pending = request_a(t, first_a);
    __syncthreads();  // the token before's staged values are no longer read
    QuantizeToShared(a.x + (static_cast<std::int64_t>(t) * a.x_stride), a.hidden, xq, false);
    __syncthreads();
    // (a CTA's warps walk the same number of rounds: the rounds meet at CTA barriers below)
    for (int base = cta_first, first = first_a; base < items; base += step_a, first += step_a) {
      if (first != first_a) pending = request_a(t, first);
      wait(pending);
      const int item = first + (lane / ur_a), sb = lane % ur_a;
      const bool valid = item < items;
      const int j = valid ? item / a.inter : 0, i = valid ? item - (j * a.inter) : 0;
      const int e = slot_id(j);
      const bool named = e >= 0 && e < a.experts;
      float dg = 0.0f, du = 0.0f;
      if (valid && named && healthy) {
        Q4KBlockUnit g, u;
        // the round's gate rows, then its up rows
        g.LoadShared(rows + (static_cast<std::size_t>(lane / ur_a) * bytes_a), sb);
        u.LoadShared(rows + (static_cast<std::size_t>(round_items(first) + (lane / ur_a)) * bytes_a), sb);
        dg = DotStaged(g, xq, a.hidden, sb);
        du = DotStaged(u, xq, a.hidden, sb);
      }
      for (int offset = ur_a / 2; offset > 0; offset >>= 1) {
        dg += __shfl_xor_sync(0xffffffffu, dg, offset);
        du += __shfl_xor_sync(0xffffffffu, du, offset);
      }
      const float value = named ? Glu(a.glu, dg, du, a.limit) : __uint_as_float(0x7fc00000u);
      if (!at_source) {
        if (valid && sb == 0 && healthy) {
          glu_rows[((static_cast<std::size_t>(t) * a.used) + j) * a.inter + i] = value;
        }
        continue;
      }
      // The round's GLU rows are quantized where they are: the CTA's items of a round are
      // whole 32-value blocks, so its warps pass their values through shared memory and
      // warp w quantizes block w with QuantizeToShared's arithmetic (the same d, codes and
      // sum whatever the lanes' order), straight into the staged form, in scratch; phase B
      // then only copies the staged bytes instead of every CTA quantizing every row again.
      if (sb == 0) exchange[(warp * items_a_warp) + (lane / ur_a)] = valid ? value : 0.0f;
      __syncthreads();
      const int n0 = base + (warp * 32);  // the block's first value among the token's used * inter
      if (warp < cta_items / 32 && n0 < items && healthy) {
        const float v = exchange[(warp * 32) + lane];
        float amax = fabsf(v);
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
        }
        const float d = amax / 127.0f;
        int q = 0;
        if (amax != 0.0f) q = static_cast<int>(roundf(v / d));
        q = static_cast<int>(static_cast<signed char>(q & 0xff));
        int isum = q;
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, offset);
        std::uint8_t* staged = staged_rows + (static_cast<std::size_t>(t) * staged_pitch);
        const int block = n0 >> 5;
        staged[((block >> 3) * kCodePitch) + ((block & 7) * 32) + lane] = static_cast<std::uint8_t>(q & 0xff);
        if (lane == 0) {
          const float d8 = __half2float(__float2half_rn(d));
          *reinterpret_cast<float2*>(staged + ((items / 256) * kCodePitch) + ((block >> 3) * kScalePitch) +
                                     ((block & 7) * 8)) = make_float2(d8, d8 * static_cast<float>(isum));
        }
      }
      if (base + step_a < items) __syncthreads();  // before the next round's values take the exchange's place
    }
  }

  // The first down rows are requested while the CTAs meet: they depend on no GLU row.
  const int first_b = (static_cast<int>(blockIdx.x) * kWarps) + warp;
  const int step_b = static_cast<int>(gridDim.x) * kWarps;
  const unsigned int all_arrived = GridArrive(counter);
  token_ids(0);
  bool pending_b = request_b(0, first_b);
  if (!GridAwait(counter, all_arrived, polls)) {
    if (threadIdx.x == 0) atomicAdd(faults, 1u);
    wait(pending_b);  // nothing may still be writing this CTA's shared memory when it leaves
    return;           // nothing of phase B is stored
  }
  GridLaunchDependents();

  // ---- phase B: dst[t][r] = sum_j weight[t][j] * (down_e[r] . h[t][j])
  for (int t = 0; t < a.tokens; ++t) {
    __syncthreads();
    if (at_source) {
      const uint2* src = reinterpret_cast<const uint2*>(staged_rows + (static_cast<std::size_t>(t) * staged_pitch));
      uint2* dst = reinterpret_cast<uint2*>(hq);
      for (int i = static_cast<int>(threadIdx.x); i < StagedBytes(items) / 8; i += kThreads) {
        dst[i] = __ldcg(src + i);  // written by other SMs: not through L1
      }
    } else {
      QuantizeToShared(glu_rows + (static_cast<std::size_t>(t) * a.used * a.inter), a.used * a.inter, hq,
                       true);
    }
    __syncthreads();
    const int j = lane / span_b, sb = lane % span_b;
    const bool active = j < a.used && sb < ur_b;
    if (t != 0) token_ids(t);  // (token 0's were read before the first down rows' request)
    const int slot_e = slot_id(active ? j : 0);
    const int e = active ? slot_e : -1;
    const bool named = e >= 0 && e < a.experts;
    // slot j's row is values [j * inter, (j + 1) * inter) of the staged GLU rows
    const int hsb = active ? (j * ur_b) + sb : 0;
    const float weight = j < a.used ? a.weights[(static_cast<std::int64_t>(t) * a.used) + j] : 0.0f;
    for (int r = first_b; r < a.hidden; r += step_b) {
      if (t != 0 || r != first_b) pending_b = request_b(t, r);
      wait(pending_b);
      float dot = 0.0f;
      if (active && named && healthy) {
        Q4KBlockUnit w;
        w.LoadShared(rows + (static_cast<std::size_t>(j) * bytes_b), sb);
        dot = DotStaged(w, hq, a.used * a.inter, hsb);
      }
      for (int offset = span_b / 2; offset > 0; offset >>= 1) {
        dot += __shfl_xor_sync(0xffffffffu, dot, offset);
      }
      // slot j's sum sits in lane j * span_b; a slot outside the experts contributes NaN
      float term = __fmul_rn(named ? dot : __uint_as_float(0x7fc00000u), weight);
      float y = 0.0f;
      for (int s2 = 0; s2 < a.used; ++s2) {
        const float v = __shfl_sync(0xffffffffu, term, s2 * span_b);
        y = s2 == 0 ? v : y + v;
      }
      if (lane == 0 && healthy) a.dst[(static_cast<std::int64_t>(t) * a.dst_stride) + r] = y;
    }
    if (t == 0 && first_b >= a.hidden) wait(pending_b);  // (a warp without a row: nothing was requested)
  }
}

}  // namespace
}  // namespace llmp_b200

extern "C" {

size_t llmp_b200_moe_decode_scratch(int used, int tokens, int inter) {
  if (used < 1 || tokens < 1 || inter < 1) return 0;
  return 256 + (static_cast<size_t>(used) * tokens * inter * sizeof(float));
}

int llmp_b200_moe_decode(const llmp_b200_moe_decode_desc* desc, void* stream) {
  using namespace llmp_b200;
  if (desc == nullptr) return Reject("moe_decode: null descriptor");
  const llmp_b200_moe_decode_desc& a = *desc;
  if (a.x == nullptr || a.ids == nullptr || a.weights == nullptr || a.gate_up == nullptr ||
      a.down == nullptr || a.dst == nullptr || a.scratch == nullptr) {
    return Reject("moe_decode: activations, ids, weights, both expert tensors, an output and scratch");
  }
  int ur_a = a.hidden / 256, span_b = 1;
  while (span_b < a.inter / 256) span_b *= 2;
  if (a.hidden < 256 || a.hidden % 256 != 0 || a.hidden > kMaxHidden || (ur_a & (ur_a - 1)) != 0 ||
      ur_a > 32 || a.inter < 256 || a.inter % 256 != 0 || a.used < 1 || a.used * span_b > 32 ||
      a.used * a.inter > kMaxGluValues || a.tokens < 1 || a.tokens > 16 || a.experts < 1) {
    return Reject("moe_decode: hidden a power-of-two multiple of 256 up to 8192, inter a multiple of "
                  "256, used * ceil_pow2(inter / 256) <= 32, used * inter <= 16384, 1 to 16 tokens");
  }
  if (a.glu < LLMP_B200_GLU_SWIGLU || a.glu > LLMP_B200_GLU_GEGLU ||
      (a.glu == LLMP_B200_GLU_GEGLU && a.limit != 0.0f)) {
    return Reject("moe_decode: a GLU (GeGLU without a clamp limit)");
  }
  if (!Aligned(a.x, 16) || a.x_stride % 4 != 0 || a.x_stride < a.hidden || !Aligned(a.gate_up, 16) ||
      !Aligned(a.down, 16) || !Aligned(a.scratch, 256) || !Aligned(a.dst, 4) || !Aligned(a.ids, 4) ||
      a.ids_stride < a.used || a.dst_stride < a.hidden) {
    return Reject("moe_decode: 16-byte aligned activations and experts, 256-byte aligned scratch");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  unsigned int* faults = FaultCounter();
  if (faults == nullptr) return Reject("moe_decode: no fault counter on this device");
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(SmCount()));
  config.blockDim = dim3(kThreads);
  config.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeCooperative;  // every CTA resident: they meet once
  attribute[0].val.cooperative = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  const int polls = 1 << 22;  // x 40 ns: a barrier that never fills gives up after 0.2 s
  const int smem = DecodeSmem(a.hidden, a.used * a.inter);
  static thread_local int configured_device = -1;
  int device = -1;
  cudaGetDevice(&device);
  if (configured_device != device) {
    const cudaError_t set = cudaFuncSetAttribute(MoeDecodeKernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 DecodeSmem(kMaxHidden, kMaxGluValues));
    if (set != cudaSuccess) return Failed(set, "moe_decode attribute");
    configured_device = device;
  }
  config.dynamicSmemBytes = static_cast<size_t>(smem);
  const cudaError_t e = cudaLaunchKernelEx(&config, MoeDecodeKernel, a, faults, polls);
  return e == cudaSuccess ? 0 : Failed(e, "moe_decode launch");
}

}  // extern "C"
