// Stand-in for the one GGML header the reference's CPU decode includes
// (src/kernels/reference/decode.cc:21).  GGML itself is not vendored in the
// reference tree; only the five names decode.cc uses are declared, and
// oracle/ref_shim.cc defines them over the oracle's own block decoders.
// TEST INFRASTRUCTURE (used only to build oracle/_ref).
#pragma once
#include <cstddef>
#include <cstdint>
extern "C" {
typedef int ggml_type;
typedef void (*ggml_to_float_t)(const void* x, float* y, int64_t k);
typedef void (*ggml_from_float_t)(const float* x, void* y, int64_t k);
struct ggml_type_traits {
  ggml_to_float_t to_float;
  ggml_from_float_t from_float_ref;
};
const ggml_type_traits* ggml_get_type_traits(ggml_type type);
bool ggml_quantize_requires_imatrix(ggml_type type);
size_t ggml_quantize_chunk(ggml_type type, const float* src, void* dst, int64_t start,
                           int64_t nrows, int64_t n_per_row, const float* imatrix);
}
