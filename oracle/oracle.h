/*
 * CPU oracle for the quantized-matmul hot path.  TEST INFRASTRUCTURE ONLY:
 * the parity tests, the smoke check and the benchmark's CPU-baseline leg may
 * link this; the product library never does.
 *
 * Every function restates the arithmetic of the reference (llmp) for one step
 * of the path and cites the reference file:line it follows.  The reference
 * delegates three pieces to GGML (llama.cpp tag v0.6.0, commit d8123504...),
 * which is not vendored in the reference tree: the 36-byte Q8_1 quantizer,
 * the float evaluation order of vec_dot_q8_0_q8_1 / vec_dot_q4_K_q8_1, and
 * the 144-byte Q8_1-MMQ (DS4) activation block.  Those three are restated
 * here from GGML's published algorithm and are marked PARITY UNPINNED: no
 * golden vector of the reference covers them in this tree.  Everything else
 * (block geometry, Q4_K scale unpacking, the scalar block products, FP16 /
 * BF16 / E4M3 / E8M0 conversions, the MXFP8 quantizer, the scale-atom layout,
 * the expert counting sort, GLU and the ordered combine) follows code that is
 * in the reference tree and is pinned by the tests under tests/.
 */
#ifndef LLMP_B200_ORACLE_H_
#define LLMP_B200_ORACLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML type numbers (src/format/encoding.cc:111-115). */
enum { ORC_TYPE_Q4_0 = 2, ORC_TYPE_Q5_0 = 6, ORC_TYPE_Q8_0 = 8, ORC_TYPE_Q8_1 = 9, ORC_TYPE_Q4_K = 12,
       ORC_TYPE_Q5_K = 13, ORC_TYPE_Q6_K = 14, ORC_TYPE_IQ4_NL = 20 };
enum { ORC_Q8_0_BYTES = 34, ORC_Q8_1_BYTES = 36, ORC_Q4_K_BYTES = 144, ORC_Q8_1_MMQ_BYTES = 144 };
enum { ORC_GLU_NONE = 0, ORC_GLU_SWIGLU = 1, ORC_GLU_SWIGLU_CLAMP = 2, ORC_GLU_GEGLU = 3 };

/* ---- element conversions (src/kernels/reference/decode.cc:341-427) ---- */
float orc_f16_to_f32(uint16_t bits);
uint16_t orc_f32_to_f16(float value);
float orc_bf16_to_f32(uint16_t bits);
uint16_t orc_f32_to_bf16(float value);
float orc_e4m3_to_f32(uint8_t bits);
float orc_e8m0_to_f32(uint8_t bits);
float orc_e2m1_to_f32(uint8_t code);   /* low nibble */
float orc_ue4m3_to_f32(uint8_t bits);  /* NVFP4 block scale: NaN from 0x7F up */
uint8_t orc_f32_to_e4m3_satfinite(float value);

/* ---- block geometry ---- */
int64_t orc_block_elems(int type);
int64_t orc_block_bytes(int type);
int64_t orc_q8_padded(int64_t k);             /* k rounded up to 512 */
int64_t orc_q8_row_blocks(int64_t k);         /* Q8_1 blocks in a padded row */

/* ---- weight decode ---- */
void orc_dequant_q8_0(const uint8_t* blocks, int64_t nblocks, float* out);
void orc_dequant_q4_k(const uint8_t* blocks, int64_t nblocks, float* out);
void orc_q4_k_scales(const uint8_t* block, int sc[8], int mn[8]);

/* ---- Q8_1 activation quantizer (PARITY UNPINNED) ---- */
void orc_quantize_q8_1(const float* x, int64_t k, int64_t rows, int64_t row_stride, uint8_t* out);
void orc_dequant_q8_1(const uint8_t* blocks, int64_t nblocks, float* out);
/* Q4_0, Q5_0, IQ4_NL, Q5_K, Q6_K (GGML's published block formats); 0, or 1 for another type. */
int orc_dequant_more(int type, const uint8_t* blocks, int64_t nblocks, float* out);

/* ---- per-block integer sums (bit-exact contract) ---- */
/* Q8_0: sums[b] = sum_i w.q[i]*y.q[i] for each of k/32 blocks. */
void orc_q8_0_block_sums(const uint8_t* w_row, const uint8_t* y_row, int64_t k, int32_t* sums);
/* Q4_K: for each of k/32 sub-blocks, dots[g] = sum code*q, qsums[g] = sum q. */
void orc_q4_k_block_sums(const uint8_t* w_row, const uint8_t* y_row, int64_t k, int32_t* dots,
                         int32_t* qsums);

/* ---- scalar block products in double (tests/unit/dsv4_fast_test.cc:136-194) ---- */
double orc_q8_0_block_product(const uint8_t* w, const uint8_t* q8);
double orc_q4_k_block_product(const uint8_t* w, const uint8_t* q8_8blocks);

/* ---- GLU (src/kernels/ggml/vecq.cu:184-195) ---- */
float orc_glu(int glu, float gate, float up, float limit);

/* ---- llmp.vecq (src/kernels/ggml/vecq.h:23-42, vecq.cu:457-665) ---- */
typedef struct {
  const void* w;
  const void* g;
  const void* y;
  const int32_t* ids;
  float* dst;
  int ncols_x, nrows, stride_row, stride_expert, y_token, y_slot, ids_stride, used, tokens,
      dst_token, dst_slot, glu;
  float limit;
} orc_vecq_desc;
/* F32 result, accumulated in float in block order.  If dst64/abs64 are not
 * NULL (dense, no GLU only) they receive, laid out as dst, the sum in double
 * of the scalar block products and the sum of the magnitudes of their terms
 * (per block for Q8_0; per 32-value sub-block scale and minimum term for Q4_K). */
int orc_vecq(int type, const orc_vecq_desc* d, double* dst64, double* abs64, int threads);

/* ---- Q8_1-MMQ activation blocks, DS4 layout (PARITY UNPINNED) ---- */
/* x: F32 [cols][k] with row stride; out: block_q8_1_mmq[k/128][cols]. */
void orc_quantize_mmq_q8_1_ds4(const float* x, int64_t k, int64_t cols, int64_t row_stride,
                               const int32_t* ids_src, uint8_t* out);
/* D[col][n] = W_q4k[n][k] . X_q8mmq[col][k]; dst column stride in floats.
 * ids_dst / expert_bounds NULL: dense. */
/* sums[(col * n + row) * (k / 32) + group]: the exact int32 group sums of the dense product. */
void orc_mmq_block_sums(const uint8_t* w, int64_t stride_row_blocks, const uint8_t* yq,
                        int64_t ncols, int64_t k, int64_t n, int32_t* sums);
void orc_mmq_q4_k(const uint8_t* w, int64_t stride_row_blocks, int64_t stride_expert_blocks,
                  const uint8_t* yq, int64_t ncols_y, const int32_t* ids_dst,
                  const int32_t* expert_bounds, int experts, float* dst, int64_t dst_col_stride,
                  int64_t k, int64_t n, double* dst64, int threads);

/* ---- MXFP8 (src/kernels/ggml/mxfp8_quant.cuh:22-46, llmp_ops.cu:610-663) ---- */
uint32_t orc_mxfp8_scale_code(float amax);
uint64_t orc_scale_atom_offset(uint64_t row, uint64_t block, uint64_t blocks);
uint64_t orc_mxfp8_rows_scales_offset(uint64_t rows, uint64_t k);
uint64_t orc_mxfp8_rows_bytes(uint64_t rows, uint64_t k);
/* x F32 (is_bf16=0) or BF16 bits (is_bf16=1), row stride in elements. */
void orc_mxfp8_quantize(const void* x, int is_bf16, int64_t row_stride, int64_t k, int64_t rows,
                        uint8_t* codes, uint8_t* scales);
void orc_mxfp8_swizzle(const uint8_t* in, uint8_t* out, int64_t n, int64_t blocks);
void orc_mxfp8_dequant(const uint8_t* codes, const uint8_t* scales_atoms, int64_t rows, int64_t k,
                       float* out);
/* D[m][n] = sum_k A[m][k] B[n][k]; d is F32 or BF16 bits; d64 optional. */
void orc_mxfp8_gemm(int m, int n, int k, const uint8_t* a, const uint8_t* a_scales,
                    const uint8_t* b, const uint8_t* b_scales, void* d, int bf16, double* d64,
                    int threads);

/* ---- MoE route / combine (src/kernels/ggml/moe_layout.h:47-83, llmp_moe.cu:81-160, 393-435) ---- */
/* The decode module's vector products with F32 activations
 * (src/kernels/decode/templates.cuh:83-186, decoders.cuh:106-125, 193-220,
 * products.h:96-147): a warp a weight row, lane l takes the 16-value segments l,
 * l + 32, ... with one fused multiply-add a value in order, the lanes meet in a
 * butterfly over lanes 16, 8, 4, 2, 1 apart, the sum times the row's tensor scale.
 * decoder: 0 Q8_0 blocks (v = d * q), 1 MXFP8 with row-major scales, 2 MXFP8 with
 * scale atoms (v = e4m3 * 2^(e - 127)), 3 dense BF16, 4 dense F16, 5 / 6 NVFP4 (E2M1 codes, a
 * UE4M3 scale per 16) with row-major scales / scale atoms, 7 / 8 MXFP4 (E2M1 codes, an E8M0
 * scale per 32) likewise.  y[t * y_stride + j] for t < rows, j <
 * outputs.  glu < 0: plain product of (data, scales); else the GLU of the gate
 * operand (data, scales, row first) and the up operand (data2, scales2, row
 * first2), kinds as orc_glu. */
void orc_decode_vector(int decoder, const uint8_t* data, const uint8_t* scales, int64_t row_bytes,
                       const uint8_t* data2, const uint8_t* scales2, int64_t k,
                       const float* tensor_scale, int64_t rows_per_scale, int64_t first,
                       int64_t first2, int64_t outputs, int glu, float limit, const float* x,
                       int64_t rows, int64_t x_stride, float* y, int64_t y_stride);

/* decode::RunRows: y[i][0..k) = decoded row ids[i] times its tensor scale (zeros and *bad = 1
 * for an id outside the n rows). */
void orc_decode_rows(int decoder, const uint8_t* data, const uint8_t* scales, int64_t row_bytes,
                     int64_t k, int64_t n, const float* tensor_scale, int64_t rows_per_scale,
                     const int32_t* ids, int64_t count, float* y, int32_t* bad);

int64_t orc_moe_route_ints(int64_t experts, int64_t used, int64_t tokens);
void orc_moe_route(const int32_t* ids, int ids_stride, int experts, int used, int tokens,
                   int32_t* out);
/* dst[t][width] = sum_j rows[position[t*used+j]][:] * weights[t*used+j], slot order. */
void orc_moe_combine(const float* rows, const int32_t* position, const float* weights, int used,
                     int tokens, int width, float* dst);

#ifdef __cplusplus
}
#endif
#endif
