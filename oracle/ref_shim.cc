// C entry points over the REFERENCE's own sources, compiled where they lie
// (oracle/Makefile target `ref`): src/format/{layout,encoding,tensor_format}.cc,
// src/kernels/reference/{decode,decode_exl3}.cc and src/base/check.cc.
// Used only by tests/ to pin the oracle: element conversions, block
// geometry, the scale-atom offset, and DecodeRows for MXFP8 in scale atoms,
// Q8_1 rows and (through the stubbed GGML traits below, which call the
// oracle) the kGgmlBlocks plumbing.  TEST INFRASTRUCTURE.
#include <cstddef>
#include <cstdint>
#include <span>
#include <vector>

#include "format/encoding.h"
#include "format/layout.h"
#include "format/tensor_format.h"
#include "ggml.h"
#include "kernels/reference/decode.h"
#include "oracle.h"

namespace {
void Q8_0ToFloat(const void* x, float* y, int64_t k) {
  orc_dequant_q8_0(static_cast<const uint8_t*>(x), k / 32, y);
}
void Q4KToFloat(const void* x, float* y, int64_t k) {
  orc_dequant_q4_k(static_cast<const uint8_t*>(x), k / 256, y);
}
const ggml_type_traits kQ8_0{Q8_0ToFloat, nullptr};
const ggml_type_traits kQ4K{Q4KToFloat, nullptr};
}  // namespace

extern "C" {
const ggml_type_traits* ggml_get_type_traits(ggml_type type) {
  if (type == ORC_TYPE_Q8_0) return &kQ8_0;
  if (type == ORC_TYPE_Q4_K) return &kQ4K;
  return nullptr;
}
bool ggml_quantize_requires_imatrix(ggml_type) { return false; }
size_t ggml_quantize_chunk(ggml_type, const float*, void*, int64_t, int64_t, int64_t,
                           const float*) {
  return 0;
}

namespace ref = llmp::kernels::reference;
namespace fmt = llmp::format;

float ref_f16_to_f32(uint16_t b) { return ref::F16ToF32(b); }
uint16_t ref_f32_to_f16(float v) { return ref::F32ToF16(v); }
float ref_bf16_to_f32(uint16_t b) { return ref::Bf16ToF32(b); }
uint16_t ref_f32_to_bf16(float v) { return ref::F32ToBf16(v); }
float ref_e4m3_to_f32(uint8_t b) { return ref::E4m3ToF32(b); }
float ref_e8m0_to_f32(uint8_t b) { return ref::E8m0ToF32(b); }
uint64_t ref_scale_atom_offset(uint64_t row, uint64_t block, uint64_t blocks) {
  return fmt::ScaleAtomOffset(row, block, blocks);
}
uint64_t ref_ggml_row_padding(void) { return fmt::kGgmlRowPadding; }

// GGML type number -> (block elements, block bytes) from the encoding table.
int ref_block_geometry(int ggml_type_number, uint64_t* elements, uint64_t* bytes) {
  for (const fmt::EncodingInfo& info : fmt::Encodings()) {
    if (info.ggml && static_cast<int>(info.ggml->type) == ggml_type_number) {
      *elements = info.ggml->block_elements;
      *bytes = info.ggml->block_bytes;
      return 0;
    }
  }
  return 1;
}

// DecodeRows of an [n, k] matrix.  kind 0: MXFP8 codes + scale atoms; 1: MXFP8
// split (scales [n, k/32]); 2: Q8_1 blocks; 3: Q8_0 blocks; 4: Q4_K blocks; 5 / 6: NVFP4
// split / scale atoms; 7 / 8: MXFP4 split / scale atoms; 9: dense BF16; 10: dense F16.
int ref_decode_rows(int kind, const uint8_t* data, uint64_t data_bytes, const uint8_t* scales,
                    uint64_t scale_bytes, uint64_t n, uint64_t k, float* out) {
  fmt::TensorFormat f;
  switch (kind) {
    case 0: f.encoding = fmt::Encoding::kMxfp8; f.layout = fmt::Layout::kScaleAtoms; break;
    case 1: f.encoding = fmt::Encoding::kMxfp8; f.layout = fmt::Layout::kSplit; break;
    case 2: f.encoding = fmt::Encoding::kQ8_1; f.layout = fmt::Layout::kGgmlBlocks; break;
    case 3: f.encoding = fmt::Encoding::kQ8_0; f.layout = fmt::Layout::kGgmlBlocks; break;
    case 4: f.encoding = fmt::Encoding::kQ4_K; f.layout = fmt::Layout::kGgmlBlocks; break;
    case 5: f.encoding = fmt::Encoding::kNvfp4; f.layout = fmt::Layout::kSplit; break;
    case 6: f.encoding = fmt::Encoding::kNvfp4; f.layout = fmt::Layout::kScaleAtoms; break;
    case 7: f.encoding = fmt::Encoding::kMxfp4; f.layout = fmt::Layout::kSplit; break;
    case 8: f.encoding = fmt::Encoding::kMxfp4; f.layout = fmt::Layout::kScaleAtoms; break;
    case 9: f.encoding = fmt::Encoding::kBF16; f.layout = fmt::Layout::kDense; break;
    case 10: f.encoding = fmt::Encoding::kF16; f.layout = fmt::Layout::kDense; break;
    default: return 100;
  }
  f.shape = {.ne = {k, n, 1, 1}, .rank = 2};
  std::vector<ref::PartView> parts;
  const auto* d = reinterpret_cast<const std::byte*>(data);
  if (kind <= 1 || (kind >= 5 && kind <= 8)) {
    parts.push_back({fmt::PartRole::kCodes, std::span<const std::byte>(d, data_bytes)});
    parts.push_back({fmt::PartRole::kBlockScales,
                     std::span<const std::byte>(reinterpret_cast<const std::byte*>(scales),
                                                scale_bytes)});
  } else {
    parts.push_back({fmt::PartRole::kData, std::span<const std::byte>(d, data_bytes)});
  }
  const auto ok = ref::DecodeRows(f, parts, 0, 0, n, std::span<float>(out, n * k));
  return ok.has_value() ? 0 : 1 + static_cast<int>(ok.error());
}
}
