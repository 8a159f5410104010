// The reference's MMVQ entry points over this build's decode products.
//
// The reference reaches GGML's mul_mat_vec_q three ways
// (src/kernels/ggml/mul_mat_q.cu:407-416 MulMatVecQ, :431-451 RunMmvqPrepared,
// :502-515 MulMatVecQGlu) and keeps a fourth, row-invariant form of its own
// (src/kernels/ggml/mmvq_rows.cu:825 MulMatVecQRows): F32 activations of 1 to 8
// columns are quantized to Q8_1 rows in scratch (cols * padded k / 32 * 36
// bytes, mul_mat_q.cu:308-312) and multiplied, or the rows arrive prepared.
// Here those are thin launchers: the Q8_1 quantizer of q8_1.cu, then the
// llmp.vecq product (vecq.cu), whose kernels already stream the weights once
// for every column.
//
// Row invariance.  The reference needs mmvq_rows because GGML's launch geometry,
// and with it the order a column's sums are added in, changes with the column
// count (mmvq_rows.cu:5-18).  Here the ordinary entries take whatever launch
// configuration measured fastest for the shape and column count (vecq_ranks.h), so
// their bits may change with the column count too; the rows entry runs the products
// under the launch rule that fixes the geometry from the one-column plan (llmp.vecq's
// variant -2), in passes of at most 8 columns: a column's F32 result is then the same
// bits alone or in any company (the weights of a 15 to 30 MB matrix stay in the 126 MB
// L2 between the passes).
#include "common.cuh"

namespace llmp_b200 {
namespace {

using Desc = llmp_b200_mmvq_desc;

constexpr int kMaxColumns = 8;        // MMVQ_MAX_BATCH_SIZE (mul_mat_q.cu:530)
constexpr int kMaxRowsColumns = 4096; // the rows entry: any verify width

int Check(const Desc& d, bool prepared, int max_cols, const char* who) {
  if (d.type != LLMP_B200_TYPE_Q8_0 && d.type != LLMP_B200_TYPE_Q4_K) {
    return Reject("%s: weight type %d is not one this build computes (Q8_0, Q4_K)", who, d.type);
  }
  const int elems = d.type == LLMP_B200_TYPE_Q4_K ? 256 : 32;
  if (d.w == nullptr || d.dst == nullptr || d.k < elems || d.k % elems != 0 || d.n < 1 ||
      d.cols < 1 || d.cols > max_cols) {
    return Reject("%s: weights, an F32 output, k a positive multiple of the block, 1 to %d columns",
                  who, max_cols);
  }
  if ((d.glu != LLMP_B200_GLU_NONE) != (d.gate != nullptr) || d.glu < 0 || d.glu > 3) {
    return Reject("%s: gate weights exactly with a GLU", who);
  }
  if (d.stride_row < d.k / elems || d.dst_col_stride < d.n) {
    return Reject("%s: strides must cover a row", who);
  }
  if (prepared) {
    if (d.q8 == nullptr || !Aligned(d.q8, 4)) {
      return Reject("%s: prepared Q8_1 rows, 4-byte aligned", who);
    }
  } else {
    if (d.x == nullptr || !Aligned(d.x, 16) || d.x_col_stride < d.k || d.x_col_stride % 4 != 0) {
      return Reject("%s: F32 activation columns of k floats, 16-byte aligned", who);
    }
    if (d.scratch == nullptr || !Aligned(d.scratch, 256)) {
      return Reject("%s: 256-byte aligned scratch of llmp_b200_mmvq_scratch(k, cols) bytes", who);
    }
  }
  return 0;
}

llmp_b200_vecq_desc ProductOf(const Desc& d, const void* q8, int first, int cols) {
  const std::int64_t row_blocks = llmp_b200_q8_1_row_blocks(d.k);
  llmp_b200_vecq_desc v{};
  v.w = d.w;
  v.g = d.gate;
  v.y = static_cast<const std::uint8_t*>(q8) + (static_cast<std::int64_t>(first) * row_blocks * 36);
  v.ids = nullptr;
  v.dst = d.dst + (static_cast<std::int64_t>(first) * d.dst_col_stride);
  v.ncols_x = d.k;
  v.nrows = d.n;
  v.stride_row = d.stride_row;
  v.stride_expert = 0;
  v.y_token = static_cast<int>(row_blocks);
  v.y_slot = 0;
  v.ids_stride = 0;
  v.used = 1;
  v.tokens = cols;
  v.dst_token = static_cast<int>(d.dst_col_stride);
  v.dst_slot = 0;
  v.glu = d.glu;
  v.limit = d.limit;
  return v;
}

// Quantize (unless prepared), then the product in passes of at most `pass` columns.
int Run(const Desc& d, bool prepared, int pass, void* stream, int variant = -1) {
  if (d.dst_col_stride > 0x7fffffffLL) return Reject("mmvq: output stride beyond int");
  const void* q8 = d.q8;
  bool queued = false;
  if (!prepared) {
    const int status = llmp_b200_q8_1_quantize(d.x, d.k, d.cols, 1, d.x_col_stride, 0, d.scratch,
                                               stream);
    if (status != 0) return status;
    q8 = d.scratch;
    queued = true;
  }
  for (int first = 0; first < d.cols; first += pass) {
    const llmp_b200_vecq_desc v = ProductOf(d, q8, first, d.cols - first < pass ? d.cols - first : pass);
    const int status = llmp_b200_vecq(d.type, &v, variant, stream);
    // Work is already queued: a refusal now is reported as a failure after queueing.
    if (status != 0) return (queued && status > 0) ? -status : status;
    queued = true;
  }
  return 0;
}

}  // namespace
}  // namespace llmp_b200

extern "C" {

size_t llmp_b200_mmvq_scratch(int k, int cols) {
  if (k < 1 || cols < 1) return 0;
  const size_t bytes = static_cast<size_t>(cols) * static_cast<size_t>(llmp_b200_q8_1_row_blocks(k)) * 36;
  return (bytes + 255) / 256 * 256;
}

int llmp_b200_mmvq(const llmp_b200_mmvq_desc* desc, void* stream) {
  using namespace llmp_b200;
  if (desc == nullptr) return Reject("mmvq: null descriptor");
  if (const int status = Check(*desc, false, kMaxColumns, "mmvq"); status != 0) return status;
  if (const int status = DeviceStatus(); status != 0) return status;
  return Run(*desc, false, kMaxColumns, stream);
}

int llmp_b200_mmvq_prepared(const llmp_b200_mmvq_desc* desc, void* stream) {
  using namespace llmp_b200;
  if (desc == nullptr) return Reject("mmvq_prepared: null descriptor");
  if (const int status = Check(*desc, true, kMaxColumns, "mmvq_prepared"); status != 0) return status;
  if (const int status = DeviceStatus(); status != 0) return status;
  return Run(*desc, true, kMaxColumns, stream);
}

int llmp_b200_mmvq_rows(const llmp_b200_mmvq_desc* desc, void* stream) {
  using namespace llmp_b200;
  if (desc == nullptr) return Reject("mmvq_rows: null descriptor");
  const bool prepared = desc->q8 != nullptr;
  if (const int status = Check(*desc, prepared, kMaxRowsColumns, "mmvq_rows"); status != 0) {
    return status;
  }
  if (desc->glu != LLMP_B200_GLU_NONE) return Reject("mmvq_rows: the row-invariant form has no fused GLU");
  if (const int status = DeviceStatus(); status != 0) return status;
  // Columns a pass: what the product's fixed-geometry kernels take at once (vecq.cu: the
  // Q4_K row-lane kernel 8 tokens, the Q8_0 stream kernel 4).
  // ... under the launch rule that keeps the one-column geometry (variant -2), not the
  // measured-rank table, whose choice may change with the column count.
  return Run(*desc, prepared, desc->type == LLMP_B200_TYPE_Q4_K ? 8 : 4, stream, -2);
}

}  // extern "C"
