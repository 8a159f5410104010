// llmp.vecq entry points: operand checks, launch choice, and the per-block
// int32 sums used to verify the product kernels.  The kernels themselves are
// in vecq_impl.cuh, instantiated per weight type in vecq_q4k.cu / vecq_q8_0.cu.
#include <cstring>

#include "vecq_ranks.h"
#include "vecq_rowlane.cuh"
#include "vecq_rowmma.cuh"

namespace llmp_b200 {
namespace vecq {
extern template cudaError_t LaunchType<Q4KUnit>(const Desc&, int, const Variant&, cudaStream_t);
extern template cudaError_t LaunchType<Q8_0Unit<4>>(const Desc&, int, const Variant&, cudaStream_t);
extern template cudaError_t LaunchType<Q8_0Unit<1>>(const Desc&, int, const Variant&, cudaStream_t);
cudaError_t LaunchMore(int type, const Desc& d, int p, cudaStream_t stream);  // vecq_more.cu
extern template cudaError_t LaunchStream<Q4KUnit>(const Desc&, int, const StreamPlan&, cudaStream_t);
extern template cudaError_t LaunchStream<Q4KBlockUnit>(const Desc&, int, const StreamPlan&,
                                                       cudaStream_t);
extern template cudaError_t LaunchStream<Q8_0Unit<4>>(const Desc&, int, const StreamPlan&,
                                                      cudaStream_t);
}  // namespace vecq

namespace {
using namespace vecq;

// The int32 sums a product kernel forms, one thread a (row, unit): the same
// decode and dp4a functions the product uses.
__global__ void BlockSumsQ4K(const std::uint8_t* __restrict__ w, const std::uint8_t* __restrict__ y,
                             int k, int nrows, int stride_row, std::int32_t* __restrict__ dots,
                             std::int32_t* __restrict__ qsums) {
  const int blocks = k / 256;
  const long i = (static_cast<long>(blockIdx.x) * blockDim.x) + threadIdx.x;
  if (i >= static_cast<long>(nrows) * blocks) return;
  const int row = static_cast<int>(i / blocks);
  const int u = static_cast<int>(i % blocks);
  // Both decodes the product kernels use must give the same integers.
  Q4KBlockUnit raw;
  raw.LoadShared(w + (static_cast<std::size_t>(row) * stride_row * 144), u);  // plain loads
  UnitActs<Q4KBlockUnit> acts;
  acts.Load(y, u);
  int whole[8];
  Q4KBlockDots(raw, acts.q, whole);
  const std::size_t at = (static_cast<std::size_t>(row) * (k / 32)) + (u * 8);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    Q4KUnit part;
    part.Load(w + (static_cast<std::size_t>(row) * stride_row * 144), (u * 4) + c);
    Q4KDecoded dec;
    dec.From(part, c);
    const uint4 a4[4] = {
        make_uint4(acts.q[16 * c + 0], acts.q[16 * c + 1], acts.q[16 * c + 2], acts.q[16 * c + 3]),
        make_uint4(acts.q[16 * c + 4], acts.q[16 * c + 5], acts.q[16 * c + 6], acts.q[16 * c + 7]),
        make_uint4(acts.q[16 * c + 8], acts.q[16 * c + 9], acts.q[16 * c + 10], acts.q[16 * c + 11]),
        make_uint4(acts.q[16 * c + 12], acts.q[16 * c + 13], acts.q[16 * c + 14],
                   acts.q[16 * c + 15])};
    int d0, d1;
    Q4KDots(dec, a4, &d0, &d1);
    // A disagreement between the two decodes is reported as an impossible sum.
    dots[at + (2 * c)] = d0 == whole[2 * c] ? d0 : 0x7fffffff;
    dots[at + (2 * c) + 1] = d1 == whole[(2 * c) + 1] ? d1 : 0x7fffffff;
  }
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    int s = 0;
#pragma unroll
    for (int q = 0; q < 8; ++q) s = Dp4a(0x01010101, acts.q[(8 * g) + q], s);
    qsums[at + g] = s;
  }
}

template <int kBlocks>
__global__ void BlockSumsQ8_0(const std::uint8_t* __restrict__ w, const std::uint8_t* __restrict__ y,
                              int k, int nrows, int stride_row, std::int32_t* __restrict__ dots) {
  using Unit = Q8_0Unit<kBlocks>;
  const int units = Unit::UnitsPerRow(k);
  const long i = (static_cast<long>(blockIdx.x) * blockDim.x) + threadIdx.x;
  if (i >= static_cast<long>(nrows) * units) return;
  const int row = static_cast<int>(i / units);
  const int u = static_cast<int>(i % units);
  Unit raw;
  raw.Load(w + (static_cast<std::size_t>(row) * stride_row * 34), u);
#pragma unroll
  for (int b = 0; b < kBlocks; ++b) {
    const auto* src = reinterpret_cast<const std::uint32_t*>(
        y + (static_cast<std::size_t>((u * kBlocks) + b) * 36));
    int sumi = 0;
#pragma unroll
    for (int q = 0; q < 8; ++q) sumi = Dp4a(raw.Int(b, q), static_cast<int>(src[1 + q]), sumi);
    dots[(static_cast<std::size_t>(row) * (k / 32)) + (u * kBlocks) + b] = sumi;
  }
}

// Operand checks: the part of CheckVecQ (src/kernels/ggml/llmp_ops.cc:2915-2982)
// that a raw descriptor can express.
// The other block types (vecq_more.cuh): bytes and values a block, alignment of a block.
bool MoreType(int type) {
  return type == LLMP_B200_TYPE_Q4_0 || type == LLMP_B200_TYPE_Q5_0 || type == LLMP_B200_TYPE_IQ4_NL ||
         type == LLMP_B200_TYPE_Q5_K || type == LLMP_B200_TYPE_Q6_K;
}
int BlockBytesOf(int type) {
  switch (type) {
    case LLMP_B200_TYPE_Q4_K: return 144;
    case LLMP_B200_TYPE_Q8_0: return 34;
    case LLMP_B200_TYPE_Q5_0: return 22;
    case LLMP_B200_TYPE_Q5_K: return 176;
    case LLMP_B200_TYPE_Q6_K: return 210;
    default: return 18;  // Q4_0, IQ4_NL
  }
}
int BlockElemsOf(int type) {
  return type == LLMP_B200_TYPE_Q4_K || type == LLMP_B200_TYPE_Q5_K || type == LLMP_B200_TYPE_Q6_K ? 256 : 32;
}

int Check(int type, const Desc& d, bool* q8_fast) {
  if (type != LLMP_B200_TYPE_Q8_0 && type != LLMP_B200_TYPE_Q4_K && !MoreType(type)) {
    return Reject("vecq: weight type %d is not one this build computes (Q8_0, Q4_K, Q4_0, Q5_0, "
                  "IQ4_NL, Q5_K, Q6_K)", type);
  }
  if (d.w == nullptr || d.y == nullptr || d.dst == nullptr) {
    return Reject("vecq: quantized weights, a llmp.q8_1 input and an F32 output");
  }
  if (d.tokens < 1 || d.tokens > (d.ids != nullptr ? kMaxRoutedTokens : 16) || d.glu < 0 ||
      d.glu > 3 || ((d.glu != 0) != (d.g != nullptr))) {
    return Reject("vecq: 1 to 16 tokens (128 routed), and gate weights exactly with a GLU");
  }
  if (d.glu == LLMP_B200_GLU_GEGLU && d.limit != 0.0f) {
    return Reject("vecq: GeGLU uses GELU-tanh without a clamp limit");
  }
  // (the 32-value types are taken four blocks a unit: k a multiple of 128 for them)
  const int elems = MoreType(type) && BlockElemsOf(type) == 32 ? 128 : BlockElemsOf(type);
  if (d.ncols_x < elems || d.ncols_x % elems != 0 || d.nrows < 1) {
    return Reject("vecq: k a positive multiple of %d values for this type, n >= 1", elems);
  }
  if (d.used < 1 || d.used > 256 || d.used * d.tokens > (d.ids != nullptr ? kMaxPairs : 256 * 16)) {
    return Reject("vecq: used * tokens <= 1024 routed; at most 256 groups");
  }
  if (d.ids == nullptr && d.tokens > kMaxPairs) return Reject("vecq: tokens");
  if (d.stride_row < d.ncols_x / BlockElemsOf(type) || d.stride_expert < 0 || d.y_token < 0 || d.y_slot < 0 ||
      d.dst_token < 0 || d.dst_slot < 0 || (d.ids != nullptr && d.ids_stride < d.used)) {
    return Reject("vecq: strides must cover a row and be non-negative");
  }
  if (!Aligned(d.dst, 4) || !Aligned(d.y, 4) || (d.ids != nullptr && !Aligned(d.ids, 4))) {
    return Reject("vecq: output, Q8_1 input and ids 4-byte aligned");
  }
  if (type == LLMP_B200_TYPE_Q4_K || type == LLMP_B200_TYPE_Q5_K) {
    // 144- and 176-byte super-blocks: any block offset keeps a 16-byte aligned base aligned.
    if (!Aligned(d.w, 16) || (d.g != nullptr && !Aligned(d.g, 16))) {
      return Reject("vecq: Q4_K / Q5_K weights 16-byte aligned");
    }
  } else if (MoreType(type)) {
    if (!Aligned(d.w, 2) || (d.g != nullptr && !Aligned(d.g, 2))) {
      return Reject("vecq: weights 2-byte aligned");
    }
    if (d.ids != nullptr) return Reject("vecq: routed products take Q8_0 and Q4_K only");
  } else {
    if (!Aligned(d.w, 2) || (d.g != nullptr && !Aligned(d.g, 2))) {
      return Reject("vecq: Q8_0 weights 2-byte aligned");
    }
    *q8_fast = Aligned(d.w, 8) && (d.g == nullptr || Aligned(d.g, 8)) && d.stride_row % 4 == 0 &&
               d.stride_expert % 4 == 0 && d.ncols_x % 128 == 0;
  }
  if (StageBytes(d.ncols_x, 1) > 200 * 1024) {
    return Reject("vecq: k = %d does not fit the activation staging", d.ncols_x);
  }
  const std::uint64_t out = static_cast<std::uint64_t>(d.nrows) * d.used * d.tokens;
  if (out > 0x7fffffffULL) return Reject("vecq: output beyond the kernel's int offsets");
  const auto disjoint = [](const void* a, std::uint64_t an, const void* b, std::uint64_t bn) {
    const auto x = reinterpret_cast<std::uintptr_t>(a), y = reinterpret_cast<std::uintptr_t>(b);
    return x + an <= y || y + bn <= x;
  };
  const std::uint64_t dst_bytes =
      (static_cast<std::uint64_t>(d.tokens - 1) * d.dst_token +
       static_cast<std::uint64_t>(d.used - 1) * d.dst_slot + d.nrows) * 4;
  const std::uint64_t w_bytes = (static_cast<std::uint64_t>(d.nrows - 1) * d.stride_row +
                                 d.ncols_x / BlockElemsOf(type)) * BlockBytesOf(type);
  if (!disjoint(d.dst, dst_bytes, d.w, w_bytes) ||
      (d.g != nullptr && !disjoint(d.dst, dst_bytes, d.g, w_bytes)) ||
      !disjoint(d.dst, dst_bytes, d.y, static_cast<std::uint64_t>(d.ncols_x / 32) * 36)) {
    return Reject("vecq: a packed output disjoint from its operands");
  }
  return 0;
}

}  // namespace
}  // namespace llmp_b200

extern "C" {

int llmp_b200_vecq_variants(void) { return llmp_b200::kVariantCount; }

const char* llmp_b200_vecq_variant_name(int variant) {
  if (variant < 0 || variant >= llmp_b200::kVariantCount) return "";
  return llmp_b200::kVariants[variant].name;
}

int llmp_b200_vecq_rank_count(void) { return llmp_b200::vecq::kMeasuredRankCount; }

const char* llmp_b200_vecq_rank(int row, int* k, int* n, int* glu, int* tokens, float* microseconds) {
  if (row < 0 || row >= llmp_b200::vecq::kMeasuredRankCount) return "";
  const llmp_b200::vecq::MeasuredRank& r = llmp_b200::vecq::kMeasuredRanks[row];
  if (k != nullptr) *k = r.k;
  if (n != nullptr) *n = r.n;
  if (glu != nullptr) *glu = r.glu;
  if (tokens != nullptr) *tokens = r.tokens;
  if (microseconds != nullptr) *microseconds = r.microseconds;
  return r.variant;
}

namespace llmp_b200 {
namespace {
int LaunchVecQ(int type, const llmp_b200_vecq_desc* desc, int variant, bool f32_input, void* q8_out,
               void* q8_dst, unsigned int* rows_done, void* stream, const PeerFan* fan = nullptr);
}  // namespace
}  // namespace llmp_b200

int llmp_b200_vecq(int type, const llmp_b200_vecq_desc* desc, int variant, void* stream) {
  return llmp_b200::LaunchVecQ(type, desc, variant, false, nullptr, nullptr, nullptr, stream);
}

int llmp_b200_vecq_f32(int type, const llmp_b200_vecq_desc* desc, void* q8_out, void* stream) {
  return llmp_b200::LaunchVecQ(type, desc, -1, true, q8_out, nullptr, nullptr, stream);
}

int llmp_b200_vecq_q8(int type, const llmp_b200_vecq_desc* desc, void* q8_dst, uint32_t* rows_done,
                      void* stream) {
  if (q8_dst == nullptr || rows_done == nullptr) {
    return llmp_b200::Reject("vecq_q8: the output blocks and the row counters");
  }
  return llmp_b200::LaunchVecQ(type, desc, -1, false, nullptr, q8_dst, rows_done, stream);
}

int llmp_b200_vecq_fan(int type, const llmp_b200_vecq_desc* desc, int variant,
                       const llmp_b200_peer_fan* fan, void* stream) {
  using namespace llmp_b200;
  if (fan == nullptr || fan->world < 1 || fan->world > 32 || fan->words == nullptr ||
      fan->step == nullptr || fan->base < 0 || fan->tag < 0 || fan->tag > 255) {
    return Reject("vecq_fan: 1 to 32 ranks' word vectors, the step word, a base and a tag of 0 to 255");
  }
  PeerFan f{};
  f.words = reinterpret_cast<unsigned long long* const*>(fan->words);
  f.step = fan->step;
  f.world = fan->world;
  f.base = fan->base;
  f.tag = fan->tag;
  return LaunchVecQ(type, desc, variant, false, nullptr, nullptr, nullptr, stream, &f);
}

size_t llmp_b200_vecq_q8_scratch(int nrows, int tokens) {
  if (nrows < 1 || tokens < 1) return 0;
  return static_cast<size_t>(tokens) * static_cast<size_t>((nrows + 31) / 32) * sizeof(uint32_t);
}

}  // extern "C"

namespace llmp_b200 {
namespace {
// The rowlane geometry a default launch takes for p tokens a pass.  By default a
// CTA owns its SM, unless half an SM holds the CTA's whole row range at no worse
// a lane use: then the next kernel on the stream, a programmatic dependent,
// becomes resident and fetches early.  (A looser rule sped the down projection up
// alone, 5.6 against 6.8 us, but slowed the FFN chain it sits in, 2,377 against
// 2,742 GB/s.)
bool ChooseRowLane(const Desc& d, int p, RowLanePlan* lanes) {
  RowLanePlan half;
  bool ok = PlanRowLane(d, p, SmCount(), 0, false, lanes);
  if (PlanRowLane(d, p, SmCount(), 0, true, &half) && half.stages == half.steps &&
      (!ok || half.score >= 0.95 * lanes->score)) {
    *lanes = half;
    ok = true;
  }
  return ok;
}

int LaunchVecQ(int type, const llmp_b200_vecq_desc* desc, int variant, bool f32_input, void* q8_out,
               void* q8_dst, unsigned int* rows_done, void* stream, const PeerFan* fan) {
  if (desc == nullptr) return Reject("vecq: null descriptor");
  bool q8_fast = false;
  if (const int status = Check(type, *desc, &q8_fast); status != 0) return status;
  if (variant < -2 || variant >= kVariantCount) return Reject("vecq: no variant %d", variant);
  if (fan != nullptr && desc->tokens != 1) return Reject("vecq_fan: one token a call");
  if (const int status = DeviceStatus(); status != 0) return status;
  const Desc& d = *desc;
  const bool glu = d.glu != LLMP_B200_GLU_NONE;
  // Tokens a pass: the dense pairs are the tokens; a routed expert's pairs
  // are at most used * tokens, usually few.
  int p = 1;
  const int most = d.ids != nullptr ? std::min(d.tokens, 8) : d.tokens;
  while (p < most && p < 8) p *= 2;
  while (p > 1 && StageBytes(d.ncols_x, p) > 200 * 1024) p /= 2;
  // variant -1: the fastest measured configuration of this very product, when the table
  // has it (the bits of a token may then differ between token counts, as the reference's
  // MMVQ's do); a configuration that turns the product down falls through to the rule
  // below.  variant -2: the rule below alone, whose row-lane geometry is the one-token
  // plan's whatever the token count (what llmp_b200_mmvq_rows runs on).
  if (variant == -1 && type == LLMP_B200_TYPE_Q4_K && d.ids == nullptr && d.used == 1 &&
      d.tokens <= 8 && !f32_input && q8_dst == nullptr && d.stride_row == d.ncols_x / 256) {
    for (int i = 0; i < kMeasuredRankCount; ++i) {
      const MeasuredRank& r = kMeasuredRanks[i];
      if (r.k != d.ncols_x || r.n != d.nrows || (r.glu != 0) != glu || r.tokens != p) continue;
      for (int v = 0; v < kVariantCount; ++v) {
        if (std::strcmp(kVariants[v].name, r.variant) != 0) continue;
        if (v == kRowLaneVariant) break;  // the rule below is that kernel
        const int status = LaunchVecQ(type, desc, v, false, nullptr, nullptr, nullptr, stream, fan);
        if (status <= 0) return status;   // queued, or failed after queueing
        break;                            // refused cleanly: the rule below
      }
      break;
    }
  }
  if (variant == -2) variant = -1;
  const int slots = d.ids != nullptr ? d.used * d.tokens : d.used;
  auto* s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (MoreType(type)) {
    if (variant >= 0 || f32_input || q8_dst != nullptr || fan != nullptr) {
      return Reject("vecq: this block type has one launch configuration and no fused forms");
    }
    if (slots > 65535) return Reject("vecq: grid too large");
    e = LaunchMore(type, d, p, s);
    if (e != cudaSuccess) return Failed(e, "vecq launch");
    return 0;
  }
  // Dense products whose rows start on 16-byte boundaries stream through the
  // TMA ring; the rest (routed, grouped, more than 8 tokens, odd alignment)
  // take the register-staged kernel.
  StreamPlan plan;
  const bool dense = d.ids == nullptr && d.used == 1 && d.tokens <= (type == LLMP_B200_TYPE_Q4_K ? 8 : 4);
  const bool q4 = type == LLMP_B200_TYPE_Q4_K;
  const bool stream_ok =
      dense && (q4 || q8_fast) && Aligned(d.w, 16) && (d.g == nullptr || Aligned(d.g, 16)) &&
      PlanStream(d, q4 ? (p == 1 ? 256 : 64) : 128, q4 ? 144 : 34, q4 ? 256 : 32, p, SmCount(),
                 &plan);
  RowLanePlan lanes;
  const bool aligned16 = Aligned(d.w, 16) && (d.g == nullptr || Aligned(d.g, 16));
  if (variant >= kRowMmaVariant) {
    RowMmaPlan tiles{};
    const int ctas = kVariants[variant].u == 0 ? 1 : kVariants[variant].u;
    const bool token_columns = kVariants[variant].r == 8;
    if (token_columns && d.tokens < 2) {
      return Reject("vecq: the token-column rowmma variants take 2 to 8 tokens");
    }
    if (!(dense && q4 && aligned16 && f32_input == false && q8_dst == nullptr &&
          PlanRowMma(d, token_columns ? 8 : p, SmCount(), &tiles, ctas, token_columns))) {
      return Reject("vecq: the rowmma variant takes dense Q4_K products of up to 8 tokens");
    }
    if (fan != nullptr) tiles.fan = *fan;
    e = token_columns ? LaunchRowMmaTokens(d, tiles, s) : LaunchRowMma(d, p, tiles, s);
    if (e != cudaSuccess) return Failed(e, "vecq rowmma launch");
    return 0;
  }
  const bool wants_rowlane = variant >= kRowLaneVariant;
  bool rowlane_ok = false;
  if (dense && q4 && Aligned(d.w, 16) && (d.g == nullptr || Aligned(d.g, 16))) {
    if (wants_rowlane) {
      rowlane_ok = PlanRowLane(d, p, SmCount(), kVariants[variant].r, kVariants[variant].u == 1,
                               &lanes);
    } else {
      // A row's sum adds its super-blocks up in an order the geometry (rows and phases
      // a warp) fixes.  So that a token gives the same bits alone or in company, more
      // tokens keep the one-token geometry and only the ring depth adapts; if that
      // does not fit, the geometry is planned afresh (and the bits may differ).
      rowlane_ok = ChooseRowLane(d, 1, &lanes);
      if (rowlane_ok && p > 1) {
        RowLanePlan more;
        if (PlanRowLane(d, p, SmCount(), lanes.rows, lanes.half != 0, &more, lanes.phases) ||
            PlanRowLane(d, p, SmCount(), lanes.rows, false, &more, lanes.phases)) {
          lanes = more;
        } else {
          rowlane_ok = ChooseRowLane(d, p, &lanes);
        }
      }
    }
  }
  if (wants_rowlane && !rowlane_ok) {
    return Reject("vecq: this rowlane variant does not take the product (dense Q4_K, <= 8 tokens)");
  }
  if (f32_input) {
    // The fused quantize-and-multiply form exists in the rowlane kernel only.
    if (!rowlane_ok || d.ncols_x % 32 != 0 || !Aligned(d.y, 16) || d.y_token % 4 != 0 ||
        d.y_token < d.ncols_x) {
      return Reject("vecq_f32: dense Q4_K products of up to 8 tokens over 16-byte aligned F32 rows");
    }
    lanes.f32_input = 1;
    lanes.q8_out = static_cast<std::uint8_t*>(q8_out);
    lanes.q8_row_blocks = (d.ncols_x + 511) / 512 * 512 / 32;
  }
  if (q8_dst != nullptr) {
    // The quantized output exists in the rowlane kernel only, for rows of whole
    // 512-value groups (a token's blocks then have no padding to fill).
    if (!rowlane_ok || d.nrows % 512 != 0 || !Aligned(q8_dst, 4) || !Aligned(rows_done, 4)) {
      return Reject("vecq_q8: dense Q4_K products of up to 8 tokens with nrows a multiple of 512");
    }
    lanes.q8_dst = static_cast<std::uint8_t*>(q8_dst);
    lanes.q8_rows_done = rows_done;
  }
  if (fan != nullptr && !(rowlane_ok && (wants_rowlane || variant < 0))) {
    // The fan-out lives in the two dense Q4_K kernels' stores only.
    return Reject("vecq_fan: dense Q4_K products of one token a call");
  }
  if (rowlane_ok && (wants_rowlane || variant < 0)) {
    if (fan != nullptr) lanes.fan = *fan;
    e = LaunchRowLane(d, p, lanes, s);
    if (e != cudaSuccess) return Failed(e, "vecq rowlane launch");
    return 0;
  }
  if (variant == kStreamVariant && !stream_ok) {
    return Reject("vecq: the stream variant takes dense products of 16-byte aligned rows only");
  }
  if (stream_ok && (variant == kStreamVariant || variant < 0)) {
    e = !q4      ? LaunchStream<Q8_0Unit<4>>(d, p, plan, s)
        : p == 1 ? LaunchStream<Q4KBlockUnit>(d, p, plan, s)
                 : LaunchStream<Q4KUnit>(d, p, plan, s);
    if (e != cudaSuccess) return Failed(e, "vecq stream launch");
    return 0;
  }
  const int v = variant >= 0 ? variant
                             : DefaultVariant(UnitsOf(type, d, q8_fast), d.nrows, slots, glu, p,
                                              SmCount());
  const Variant& cfg = kVariants[v];
  const long grid_x = (d.nrows + (cfg.warps * (32 / cfg.lpr) * cfg.r) - 1) /
                      (cfg.warps * (32 / cfg.lpr) * cfg.r);
  if (grid_x > 0x7fffffffL || slots > 65535) return Reject("vecq: grid too large");
  if (type == LLMP_B200_TYPE_Q4_K) {
    e = LaunchType<Q4KUnit>(d, p, cfg, s);
  } else if (q8_fast) {
    e = LaunchType<Q8_0Unit<4>>(d, p, cfg, s);
  } else {
    e = LaunchType<Q8_0Unit<1>>(d, p, cfg, s);
  }
  if (e != cudaSuccess) return Failed(e, "vecq launch");
  return 0;
}
}  // namespace
}  // namespace llmp_b200

extern "C" {

int llmp_b200_vecq_block_sums(int type, const void* w, const void* y, int k, int nrows,
                              int stride_row, int32_t* dots, int32_t* qsums, void* stream) {
  using namespace llmp_b200;
  if (w == nullptr || y == nullptr || dots == nullptr || k < 1 || nrows < 1) {
    return Reject("block_sums: weights, one Q8_1 row and an output");
  }
  if (const int status = DeviceStatus(); status != 0) return status;
  auto* s = static_cast<cudaStream_t>(stream);
  const auto* wp = static_cast<const std::uint8_t*>(w);
  const auto* yp = static_cast<const std::uint8_t*>(y);
  if (type == LLMP_B200_TYPE_Q4_K) {
    if (k % 256 != 0 || qsums == nullptr || !Aligned(w, 16) || !Aligned(y, 4)) {
      return Reject("block_sums: Q4_K needs k % 256 == 0, aligned operands and qsums");
    }
    const long total = static_cast<long>(nrows) * (k / 256);
    BlockSumsQ4K<<<static_cast<unsigned>((total + 127) / 128), 128, 0, s>>>(wp, yp, k, nrows,
                                                                              stride_row, dots, qsums);
  } else if (type == LLMP_B200_TYPE_Q8_0) {
    if (k % 32 != 0 || !Aligned(w, 2) || !Aligned(y, 4)) {
      return Reject("block_sums: Q8_0 needs k % 32 == 0 and aligned operands");
    }
    if (Aligned(w, 8) && stride_row % 4 == 0 && k % 128 == 0) {
      const long total = static_cast<long>(nrows) * (k / 128);
      BlockSumsQ8_0<4><<<static_cast<unsigned>((total + 127) / 128), 128, 0, s>>>(
          wp, yp, k, nrows, stride_row, dots);
    } else {
      const long total = static_cast<long>(nrows) * (k / 32);
      BlockSumsQ8_0<1><<<static_cast<unsigned>((total + 127) / 128), 128, 0, s>>>(
          wp, yp, k, nrows, stride_row, dots);
    }
  } else {
    return Reject("block_sums: type %d", type);
  }
  return Launched("block_sums launch");
}

}  // extern "C"
