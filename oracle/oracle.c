/*
 * CPU oracle for the quantized-matmul hot path: TEST INFRASTRUCTURE, never
 * linked into the product library.  See oracle.h for what is pinned and what
 * is restated from the un-vendored GGML dependency ("PARITY UNPINNED").
 *
 * Build: see oracle/Makefile (-O2 -ffp-contract=off so that no multiply-add is
 * fused behind the source's back; -pthread for the threaded products).
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>

/* A static split of [0, n) over `threads` POSIX threads (the timed CPU
 * baseline's parallelism: whole output rows per thread, no shared writes). */
typedef void (*orc_range_fn)(int64_t begin, int64_t end, void* ctx);
typedef struct { orc_range_fn fn; void* ctx; int64_t begin, end; } orc_task;
static void* orc_task_main(void* p) {
  orc_task* t = (orc_task*)p;
  t->fn(t->begin, t->end, t->ctx);
  return NULL;
}
static void orc_parallel_for(int64_t n, int threads, orc_range_fn fn, void* ctx) {
  if (threads > 256) threads = 256;
  if (threads <= 1 || n <= 1) { fn(0, n, ctx); return; }
  if (threads > n) threads = (int)n;
  pthread_t tid[256];
  orc_task task[256];
  for (int i = 0; i < threads; ++i) {
    task[i].fn = fn; task[i].ctx = ctx;
    task[i].begin = n * i / threads; task[i].end = n * (i + 1) / threads;
    if (i + 1 == threads) { orc_task_main(&task[i]); }
    else if (pthread_create(&tid[i], NULL, orc_task_main, &task[i]) != 0) { orc_task_main(&task[i]); tid[i] = 0; task[i].fn = NULL; }
  }
  for (int i = 0; i + 1 < threads; ++i) if (task[i].fn) pthread_join(tid[i], NULL);
}

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint16_t load_u16(const uint8_t* p) { uint16_t v; memcpy(&v, p, 2); return v; }
static inline void store_u16(uint8_t* p, uint16_t v) { memcpy(p, &v, 2); }

/* ------------------------------------------------------------------------- */
/* Element conversions: src/kernels/reference/decode.cc:341-427.             */
/* ------------------------------------------------------------------------- */

float orc_f16_to_f32(uint16_t bits) {
  const float sign = (bits & 0x8000u) ? -1.0f : 1.0f;
  const unsigned e = (bits >> 10) & 31u, m = bits & 1023u;
  if (e == 31) return m ? NAN : sign * INFINITY;
  if (e == 0) return sign * ldexpf((float)m, -24);
  return sign * ldexpf((float)(1024u + m), (int)e - 25);
}

/* Round to nearest even; decode.cc:355-383. */
uint16_t orc_f32_to_f16(float value) {
  const uint32_t x = f32_bits(value);
  const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
  const uint32_t mag = x & 0x7FFFFFFFu;
  if (mag >= 0x7F800000u) return (uint16_t)(sign | (mag > 0x7F800000u ? 0x7E00u : 0x7C00u));
  if (mag >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);
  if (mag < 0x38800000u) {
    const uint32_t e = mag >> 23, shift = 126u - e;
    if (e == 0 || shift > 24) return sign;
    const uint32_t sig = (mag & 0x7FFFFFu) | 0x800000u;
    uint32_t q = sig >> shift;
    const uint32_t rest = sig & ((1u << shift) - 1u), half = 1u << (shift - 1u);
    if (rest > half || (rest == half && (q & 1u))) ++q;
    return (uint16_t)(sign | q);
  }
  const uint32_t rounded = mag + 0xFFFu + ((mag >> 13) & 1u);
  return (uint16_t)(sign | ((rounded - 0x38000000u) >> 13));
}

float orc_bf16_to_f32(uint16_t bits) { return bits_f32((uint32_t)bits << 16); }

uint16_t orc_f32_to_bf16(float value) {
  const uint32_t x = f32_bits(value);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
  return (uint16_t)((x + 0x7FFFu + ((x >> 16) & 1u)) >> 16);
}

float orc_e4m3_to_f32(uint8_t bits) {
  const float sign = (bits & 0x80u) ? -1.0f : 1.0f;
  const unsigned e = (bits >> 3) & 15u, m = bits & 7u;
  if (e == 15 && m == 7) return NAN;
  if (e == 0) return sign * ldexpf((float)m, -9);
  return sign * ldexpf((float)(8u + m), (int)e - 10);
}

float orc_e8m0_to_f32(uint8_t bits) {
  if (bits == 0xFF) return NAN;
  return ldexpf(1.0f, (int)bits - 127);
}

/* Nearest-even E4M3 with saturation to +-448 and NaN kept: the conversion
 * mxfp8_quant.cuh:38-46 asks of the device (__NV_SATFINITE, __NV_E4M3). */
uint8_t orc_f32_to_e4m3_satfinite(float value) {
  const uint32_t x = f32_bits(value);
  const uint8_t sign = (uint8_t)((x >> 24) & 0x80u);
  const uint32_t mag = x & 0x7FFFFFFFu;
  if (mag > 0x7F800000u) return (uint8_t)(sign | 0x7Fu);
  if (mag >= 0x43E00000u) return (uint8_t)(sign | 0x7Eu); /* >= 448 */
  if (mag < 0x3C800000u) { /* below 2^-6: subnormal, units of 2^-9 */
    const float q = nearbyintf(bits_f32(mag) * 512.0f); /* exact scaling, ties to even */
    return (uint8_t)(sign | (uint8_t)q);
  }
  uint32_t r = (mag + 0x7FFFFu + ((mag >> 20) & 1u)) >> 20; /* biased exponent : 3-bit mantissa */
  r -= (127u - 7u) << 3;
  if (r > 0x7Eu) r = 0x7Eu;
  return (uint8_t)(sign | r);
}

/* ------------------------------------------------------------------------- */
/* Block geometry: src/format/encoding.cc:111-115, src/format/layout.h:97.   */
/* ------------------------------------------------------------------------- */

int64_t orc_block_elems(int type) {
  switch (type) {
    case ORC_TYPE_Q8_0: case ORC_TYPE_Q8_1: case ORC_TYPE_Q4_0: case ORC_TYPE_Q5_0:
    case ORC_TYPE_IQ4_NL: return 32;
    case ORC_TYPE_Q4_K: case ORC_TYPE_Q5_K: case ORC_TYPE_Q6_K: return 256;
  }
  return 0;
}
int64_t orc_block_bytes(int type) {
  switch (type) {
    case ORC_TYPE_Q8_0: return ORC_Q8_0_BYTES;
    case ORC_TYPE_Q8_1: return ORC_Q8_1_BYTES;
    case ORC_TYPE_Q4_K: return ORC_Q4_K_BYTES;
    case ORC_TYPE_Q4_0: case ORC_TYPE_IQ4_NL: return 18;
    case ORC_TYPE_Q5_0: return 22;
    case ORC_TYPE_Q5_K: return 176;
    case ORC_TYPE_Q6_K: return 210;
  }
  return 0;
}
int64_t orc_q8_padded(int64_t k) { return (k + 511) / 512 * 512; }
int64_t orc_q8_row_blocks(int64_t k) { return orc_q8_padded(k) / 32; }

/* ------------------------------------------------------------------------- */
/* Weight decode.                                                            */
/* ------------------------------------------------------------------------- */

/* Q8_0: FP16 d then 32 int8; value d*q (src/kernels/decode/decoders.cuh:106-125). */
void orc_dequant_q8_0(const uint8_t* blocks, int64_t nblocks, float* out) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t* p = blocks + b * ORC_Q8_0_BYTES;
    const float d = orc_f16_to_f32(load_u16(p));
    for (int i = 0; i < 32; ++i) out[b * 32 + i] = d * (float)(int8_t)p[2 + i];
  }
}

/* Q4_K's 6-bit scales and minima: tests/unit/dsv4_fast_test.cc:176-182. */
void orc_q4_k_scales(const uint8_t* block, int sc[8], int mn[8]) {
  const uint8_t* s = block + 4;
  for (int g = 0; g < 8; ++g) {
    sc[g] = g < 4 ? (s[g] & 63) : ((s[g + 4] & 15) | ((s[g - 4] >> 6) << 4));
    mn[g] = g < 4 ? (s[g + 4] & 63) : ((s[g + 4] >> 4) | ((s[g] >> 6) << 4));
  }
}

/* Q4_K: W[g,i] = d*sc_g*code - dmin*m_g; byte j of 32-byte chunk c holds
 * sub-block 2c (low nibble) and 2c+1 (high): dsv4_fast_test.cc:183-192. */
void orc_dequant_q4_k(const uint8_t* blocks, int64_t nblocks, float* out) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t* p = blocks + b * ORC_Q4_K_BYTES;
    const float d = orc_f16_to_f32(load_u16(p)), dmin = orc_f16_to_f32(load_u16(p + 2));
    int sc[8], mn[8];
    orc_q4_k_scales(p, sc, mn);
    const uint8_t* codes = p + 16;
    for (int g = 0; g < 8; ++g) {
      const float dl = d * (float)sc[g], ml = dmin * (float)mn[g];
      for (int i = 0; i < 32; ++i) {
        const int code = (codes[(g / 2) * 32 + i] >> ((g % 2) * 4)) & 15;
        out[b * 256 + g * 32 + i] = dl * (float)code - ml;
      }
    }
  }
}

/* The other block types the reference's llmp.vecq hands to GGML's vec_dot functions
 * (src/kernels/ggml/vecq.cu:54-96).  Their layouts are GGML's published block formats
 * (ggml-common.h of the pinned GGML v0.6.0, absent from the reference tree); each decoder
 * below is checked bit for bit against gguf-py's dequantizer (tests/golden/gguf_blocks.npz).
 *   Q4_0   18 B: FP16 d, 16 bytes: value i = low nibble of byte i, value i + 16 = its high
 *          nibble; w = d * (code - 8).
 *   Q5_0   22 B: FP16 d, 32 fifth bits (bit i: value i), 16 bytes as Q4_0; w = d * (code - 16).
 *   IQ4_NL 18 B: as Q4_0 with the nibble an index into a fixed table of 16 int8 levels.
 *   Q5_K   176 B: FP16 d, FP16 dmin, Q4_K's 12 scale bytes, 32 bytes of fifth bits (byte l:
 *          bit g of value l of sub-block g), 128 nibble bytes as Q4_K; w = d*sc*code - dmin*m.
 *   Q6_K   210 B: 128 bytes of low nibbles, 64 bytes of two-bit tops, 16 int8 scales (one per
 *          16 values), FP16 d last; per 128-value half: byte l of the lows' first 32 gives
 *          values l (low) and l + 64 (high), byte l + 32 values l + 32 and l + 96, byte l of the
 *          tops their bits 4-5 in that order; w = d * scale * (code - 32). */
static const int8_t kIq4NlLevels[16] = {-127, -104, -83, -65, -49, -35, -22, -10,
                                        1,    13,   25,  38,  53,  69,  89,  113};

int orc_dequant_more(int type, const uint8_t* blocks, int64_t nblocks, float* out) {
  for (int64_t b = 0; b < nblocks; ++b) {
    if (type == ORC_TYPE_Q4_0 || type == ORC_TYPE_IQ4_NL) {
      const uint8_t* p = blocks + b * 18;
      const float d = orc_f16_to_f32(load_u16(p));
      for (int i = 0; i < 16; ++i) {
        const int lo = p[2 + i] & 15, hi = p[2 + i] >> 4;
        if (type == ORC_TYPE_Q4_0) {
          out[b * 32 + i] = d * (float)(lo - 8);
          out[b * 32 + 16 + i] = d * (float)(hi - 8);
        } else {
          out[b * 32 + i] = d * (float)kIq4NlLevels[lo];
          out[b * 32 + 16 + i] = d * (float)kIq4NlLevels[hi];
        }
      }
    } else if (type == ORC_TYPE_Q5_0) {
      const uint8_t* p = blocks + b * 22;
      const float d = orc_f16_to_f32(load_u16(p));
      const uint32_t top = (uint32_t)p[2] | ((uint32_t)p[3] << 8) | ((uint32_t)p[4] << 16) |
                           ((uint32_t)p[5] << 24);
      for (int i = 0; i < 16; ++i) {
        const int lo = (p[6 + i] & 15) | (int)(((top >> i) & 1u) << 4);
        const int hi = (p[6 + i] >> 4) | (int)(((top >> (i + 16)) & 1u) << 4);
        out[b * 32 + i] = d * (float)(lo - 16);
        out[b * 32 + 16 + i] = d * (float)(hi - 16);
      }
    } else if (type == ORC_TYPE_Q5_K) {
      const uint8_t* p = blocks + b * 176;
      const float d = orc_f16_to_f32(load_u16(p)), dmin = orc_f16_to_f32(load_u16(p + 2));
      int sc[8], mn[8];
      orc_q4_k_scales(p, sc, mn);
      const uint8_t* tops = p + 16;
      const uint8_t* codes = p + 48;
      for (int g = 0; g < 8; ++g) {
        const float dl = d * (float)sc[g], ml = dmin * (float)mn[g];
        for (int i = 0; i < 32; ++i) {
          const int code = ((codes[(g / 2) * 32 + i] >> ((g % 2) * 4)) & 15) |
                           (((tops[i] >> g) & 1) << 4);
          out[b * 256 + g * 32 + i] = dl * (float)code - ml;
        }
      }
    } else if (type == ORC_TYPE_Q6_K) {
      const uint8_t* p = blocks + b * 210;
      const float d = orc_f16_to_f32(load_u16(p + 208));
      for (int half = 0; half < 2; ++half) {
        const uint8_t* lows = p + 64 * half;
        const uint8_t* tops = p + 128 + 32 * half;
        const int8_t* scales = (const int8_t*)(p + 192 + 8 * half);
        float* y = out + b * 256 + 128 * half;
        for (int l = 0; l < 32; ++l) {
          const int is = l / 16;
          const int q1 = ((lows[l] & 15) | (((tops[l] >> 0) & 3) << 4)) - 32;
          const int q2 = ((lows[l + 32] & 15) | (((tops[l] >> 2) & 3) << 4)) - 32;
          const int q3 = ((lows[l] >> 4) | (((tops[l] >> 4) & 3) << 4)) - 32;
          const int q4 = ((lows[l + 32] >> 4) | (((tops[l] >> 6) & 3) << 4)) - 32;
          y[l] = d * (float)scales[is] * (float)q1;
          y[l + 32] = d * (float)scales[is + 2] * (float)q2;
          y[l + 64] = d * (float)scales[is + 4] * (float)q3;
          y[l + 96] = d * (float)scales[is + 6] * (float)q4;
        }
      }
    } else {
      return 1;
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------- */
/* Q8_1 activation blocks.  PARITY UNPINNED (GGML quantize_q8_1, called at   */
/* src/kernels/ggml/vecq.cu:1107).  Contract as the reference words it       */
/* (src/ir/op.h:399-405; dsv4_fast_test.cc:131-135): block of 32, max-abs,   */
/* d = amax/127 and the sum of the ORIGINAL inputs both stored as FP16,      */
/* q = roundf(x/d), rows zero-padded to a multiple of 512 values.            */
/* The 32-value sum follows a warp butterfly: partners 16, 8, 4, 2, 1 apart. */
/* ------------------------------------------------------------------------- */

static void q8_1_block(const float* x, int valid, uint8_t* out) {
  float v[32], s[32];
  float amax = 0.0f;
  for (int i = 0; i < 32; ++i) {
    v[i] = i < valid ? x[i] : 0.0f;
    s[i] = v[i];
    amax = fmaxf(amax, fabsf(v[i]));
  }
  for (int off = 16; off > 0; off >>= 1)
    for (int i = 0; i < off; ++i) s[i] = s[i] + s[i + off];
  const float d = amax / 127.0f;
  store_u16(out, orc_f32_to_f16(d));
  store_u16(out + 2, orc_f32_to_f16(s[0]));
  for (int i = 0; i < 32; ++i) {
    const int8_t q = amax == 0.0f ? 0 : (int8_t)roundf(v[i] / d);
    out[4 + i] = (uint8_t)q;
  }
}

void orc_quantize_q8_1(const float* x, int64_t k, int64_t rows, int64_t row_stride, uint8_t* out) {
  const int64_t blocks = orc_q8_row_blocks(k);
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t b = 0; b < blocks; ++b) {
      const int64_t left = k - b * 32;
      static const float zeros[32] = {0};
      q8_1_block(left > 0 ? x + r * row_stride + b * 32 : zeros,
                 left >= 32 ? 32 : (left > 0 ? (int)left : 0),
                 out + (r * blocks + b) * ORC_Q8_1_BYTES);
    }
  }
}

/* d*q: src/kernels/reference/decode.cc:163-176. */
void orc_dequant_q8_1(const uint8_t* blocks, int64_t nblocks, float* out) {
  for (int64_t b = 0; b < nblocks; ++b) {
    const uint8_t* p = blocks + b * ORC_Q8_1_BYTES;
    const float d = orc_f16_to_f32(load_u16(p));
    for (int i = 0; i < 32; ++i) out[b * 32 + i] = d * (float)(int8_t)p[4 + i];
  }
}

/* ------------------------------------------------------------------------- */
/* Per-block integer sums: the bit-exact part of the contract.               */
/* ------------------------------------------------------------------------- */

static inline int32_t q8_0_isum(const uint8_t* w, const uint8_t* y) {
  int32_t s = 0;
  for (int i = 0; i < 32; ++i) s += (int32_t)(int8_t)w[2 + i] * (int32_t)(int8_t)y[4 + i];
  return s;
}

void orc_q8_0_block_sums(const uint8_t* w_row, const uint8_t* y_row, int64_t k, int32_t* sums) {
  for (int64_t b = 0; b < k / 32; ++b)
    sums[b] = q8_0_isum(w_row + b * ORC_Q8_0_BYTES, y_row + b * ORC_Q8_1_BYTES);
}

static inline void q4_k_isums(const uint8_t* w, const uint8_t* y8, int32_t dots[8],
                              int32_t qsums[8]) {
  const uint8_t* codes = w + 16;
  for (int g = 0; g < 8; ++g) {
    const uint8_t* a = y8 + g * ORC_Q8_1_BYTES;
    int32_t p = 0, s = 0;
    for (int i = 0; i < 32; ++i) {
      const int code = (codes[(g / 2) * 32 + i] >> ((g % 2) * 4)) & 15;
      const int q = (int8_t)a[4 + i];
      p += code * q;
      s += q;
    }
    dots[g] = p;
    qsums[g] = s;
  }
}

void orc_q4_k_block_sums(const uint8_t* w_row, const uint8_t* y_row, int64_t k, int32_t* dots,
                         int32_t* qsums) {
  for (int64_t b = 0; b < k / 256; ++b)
    q4_k_isums(w_row + b * ORC_Q4_K_BYTES, y_row + b * 8 * ORC_Q8_1_BYTES, dots + b * 8,
               qsums + b * 8);
}

/* ------------------------------------------------------------------------- */
/* Scalar block products in double.                                          */
/* ------------------------------------------------------------------------- */

/* Q8_0 x Q8_1: d8_0 * d8_1 * sumi (src/kernels/ggml/vecq.cu:398-418). */
double orc_q8_0_block_product(const uint8_t* w, const uint8_t* q8) {
  return (double)orc_f16_to_f32(load_u16(w)) * (double)orc_f16_to_f32(load_u16(q8)) *
         (double)q8_0_isum(w, q8);
}

/* tests/unit/dsv4_fast_test.cc:167-194 (Q4KBlockProduct). */
double orc_q4_k_block_product(const uint8_t* w, const uint8_t* q8) {
  int sc[8], mn[8];
  int32_t dots[8], qsums[8];
  orc_q4_k_scales(w, sc, mn);
  q4_k_isums(w, q8, dots, qsums);
  const double d = orc_f16_to_f32(load_u16(w)), dmin = orc_f16_to_f32(load_u16(w + 2));
  double total = 0;
  for (int g = 0; g < 8; ++g) {
    const double d8 = orc_f16_to_f32(load_u16(q8 + g * ORC_Q8_1_BYTES));
    total += d8 * (d * sc[g] * dots[g] - dmin * mn[g] * qsums[g]);
  }
  return total;
}

/* ------------------------------------------------------------------------- */
/* GLU: src/kernels/ggml/vecq.cu:184-195.  GeGLU is the tanh GELU GGML's     */
/* ggml_cuda_op_gelu_single evaluates: 0.5x(1+tanh(sqrt(2/pi)x(1+0.044715x^2))). */
/* ------------------------------------------------------------------------- */

static float silu_f(float x) { return x / (1.0f + expf(-x)); }
static float gelu_tanh_f(float x) {
  const float a = 0.044715f, c = 0.79788456080286535587989211986876f;
  return 0.5f * x * (1.0f + tanhf(c * x * (1.0f + a * x * x)));
}

float orc_glu(int glu, float gate, float up, float limit) {
  if (glu == ORC_GLU_GEGLU) return gelu_tanh_f(gate) * up;
  if (glu == ORC_GLU_SWIGLU_CLAMP) {
    gate = fminf(gate, limit);
    up = fmaxf(fminf(up, limit), -limit);
  }
  return silu_f(gate) * up;
}

/* ------------------------------------------------------------------------- */
/* llmp.vecq: src/kernels/ggml/vecq.cu:457-665 (dense, grouped, routed; GLU). */
/* Float evaluation per block (PARITY UNPINNED beyond the integer sums):     */
/*   Q8_0  acc += d8_0 * d8_1 * (float)sumi                (vecq.cu:398-418) */
/*   Q4_K  per super-block sumf_d = sum_g d8_g*(float)(dot_g*sc_g),          */
/*         sumf_m = sum_g d8_g*(float)(qsum_g*m_g), acc += d*sumf_d - dmin*sumf_m */
/*         (GGML vec_dot_q4_K_q8_1, named at vecq.cu:72-73).                 */
/* ------------------------------------------------------------------------- */

static float row_dot_f32(int type, const uint8_t* w, const uint8_t* y, int64_t k, double* sum64,
                         double* abs64) {
  float acc = 0.0f;
  double s64 = 0, a64 = 0;
  if (type == ORC_TYPE_Q8_0) {
    for (int64_t b = 0; b < k / 32; ++b) {
      const uint8_t* wb = w + b * ORC_Q8_0_BYTES;
      const uint8_t* yb = y + b * ORC_Q8_1_BYTES;
      const float d0 = orc_f16_to_f32(load_u16(wb)), d1 = orc_f16_to_f32(load_u16(yb));
      acc += d0 * d1 * (float)q8_0_isum(wb, yb);
      if (sum64) {
        const double p = orc_q8_0_block_product(wb, yb);
        s64 += p;
        a64 += fabs(p);
      }
    }
  } else {
    for (int64_t b = 0; b < k / 256; ++b) {
      const uint8_t* wb = w + b * ORC_Q4_K_BYTES;
      const uint8_t* yb = y + b * 8 * ORC_Q8_1_BYTES;
      int sc[8], mn[8];
      int32_t dots[8], qsums[8];
      orc_q4_k_scales(wb, sc, mn);
      q4_k_isums(wb, yb, dots, qsums);
      float sumf_d = 0.0f, sumf_m = 0.0f;
      for (int g = 0; g < 8; ++g) {
        const float d8 = orc_f16_to_f32(load_u16(yb + g * ORC_Q8_1_BYTES));
        sumf_d += d8 * (float)(dots[g] * sc[g]);
        sumf_m += d8 * (float)(qsums[g] * mn[g]);
      }
      const float d = orc_f16_to_f32(load_u16(wb)), dmin = orc_f16_to_f32(load_u16(wb + 2));
      acc += d * sumf_d - dmin * sumf_m;
      if (sum64) {
        s64 += orc_q4_k_block_product(wb, yb);
        /* magnitude of the terms the sum is made of: per 32-value sub-block the
         * scale product and the minimum product */
        for (int g = 0; g < 8; ++g) {
          const double d8 = orc_f16_to_f32(load_u16(yb + g * ORC_Q8_1_BYTES));
          a64 += fabs(d8 * (double)d * sc[g] * dots[g]) + fabs(d8 * (double)dmin * mn[g] * qsums[g]);
        }
      }
    }
  }
  if (sum64) *sum64 = s64;
  if (abs64) *abs64 = a64;
  return acc;
}

typedef struct { int type; const orc_vecq_desc* d; double* dst64; double* abs64; } vecq_ctx;

static void vecq_range(int64_t begin, int64_t end, void* ctxp) {
  const vecq_ctx* c = (const vecq_ctx*)ctxp;
  const orc_vecq_desc* d = c->d;
  const int type = c->type;
  double* dst64 = c->dst64;
  double* abs64 = c->abs64;
  const int64_t bb = orc_block_bytes(type);
  for (int64_t item = begin; item < end; ++item) {
    {
      const int p = (int)(item / d->nrows), row = (int)(item % d->nrows);
      const int t = p / d->used, slot = p % d->used;
      int expert = slot; /* dense: used == 1, expert 0; grouped: matrix `slot` */
      if (d->ids) {
        expert = d->ids[t * d->ids_stride + slot];
      }
      const uint8_t* y =
          (const uint8_t*)d->y + ((int64_t)t * d->y_token + (int64_t)slot * d->y_slot) * ORC_Q8_1_BYTES;
      const int64_t wat = ((int64_t)expert * d->stride_expert + (int64_t)row * d->stride_row) * bb;
      const int64_t at = (int64_t)t * d->dst_token + (int64_t)slot * d->dst_slot + row;
      double s64 = 0, a64 = 0;
      float up = row_dot_f32(type, (const uint8_t*)d->w + wat, y, d->ncols_x, dst64 ? &s64 : NULL,
                             dst64 ? &a64 : NULL);
      if (d->glu != ORC_GLU_NONE) {
        const float gate = row_dot_f32(type, (const uint8_t*)d->g + wat, y, d->ncols_x, NULL, NULL);
        up = orc_glu(d->glu, gate, up, d->limit);
      }
      d->dst[at] = up;
      if (dst64) dst64[at] = s64;
      if (abs64) abs64[at] = a64;
    }
  }
}

int orc_vecq(int type, const orc_vecq_desc* d, double* dst64, double* abs64, int threads) {
  if (type != ORC_TYPE_Q8_0 && type != ORC_TYPE_Q4_K) return 1;
  vecq_ctx c = {type, d, dst64, abs64};
  orc_parallel_for((int64_t)d->tokens * d->used * d->nrows, threads, vecq_range, &c);
  return 0;
}

/* ------------------------------------------------------------------------- */
/* Q8_1-MMQ activation blocks, DS4 layout.  PARITY UNPINNED (GGML            */
/* quantize_mmq_q8_1, called at src/kernels/ggml/mul_mat_q.cu:606-610, 806;  */
/* the in-tree restatement of its D2S6 sibling is mul_mat_q_glu.cu:170-218). */
/* Block = 4 x (FP16 d, FP16 s) then 128 int8; blocks ordered [k/128][col].  */
/* Per 32 values: d_inv = 127/amax, q = roundf(x*d_inv), d = 1/d_inv, s =    */
/* sum of the original values: four per lane left to right, then an 8-lane   */
/* butterfly (partners 4, 2, 1 lanes apart).                                 */
/* ------------------------------------------------------------------------- */

void orc_quantize_mmq_q8_1_ds4(const float* x, int64_t k, int64_t cols, int64_t row_stride,
                               const int32_t* ids_src, uint8_t* out) {
  const int64_t kb = k / 128;
  for (int64_t c = 0; c < cols; ++c) {
    const float* row = x + (ids_src ? ids_src[c] : c) * row_stride;
    for (int64_t b = 0; b < kb; ++b) {
      uint8_t* blk = out + (b * cols + c) * ORC_Q8_1_MMQ_BYTES;
      for (int g = 0; g < 4; ++g) {
        const float* v = row + b * 128 + g * 32;
        float amax = 0.0f, lane[8];
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
        for (int l = 0; l < 8; ++l) lane[l] = ((v[4 * l] + v[4 * l + 1]) + v[4 * l + 2]) + v[4 * l + 3];
        for (int off = 4; off > 0; off >>= 1)
          for (int l = 0; l < off; ++l) lane[l] = lane[l] + lane[l + off];
        float d = 0.0f;
        if (amax > 0.0f) {
          const float d_inv = 127.0f / amax;
          for (int i = 0; i < 32; ++i) blk[16 + g * 32 + i] = (uint8_t)(int8_t)roundf(v[i] * d_inv);
          d = 1.0f / d_inv;
        } else {
          memset(blk + 16 + g * 32, 0, 32);
        }
        store_u16(blk + g * 4, orc_f32_to_f16(d));
        store_u16(blk + g * 4 + 2, orc_f32_to_f16(lane[0]));
      }
    }
  }
}

/* ------------------------------------------------------------------------- */
/* MMQ, Q4_K x Q8_1-MMQ (PARITY UNPINNED for the float part; GGML mul_mat_q, */
/* called at src/kernels/ggml/mul_mat_q.cu:67-130, 453-462; tile loop shape  */
/* in-tree at mul_mat_q_glu.cu:93-135).  Per 32-group: int32 C = sum code*q; */
/* the tile loader forms (d*sc, -dmin*m) in HALF precision; then in float    */
/*   sum += dmA.x * dsB.x * (float)C;  sum += dmA.y * dsB.y                  */
/* with dsB = (d, s) of the activation group (s = stored sum of inputs).     */
/* ------------------------------------------------------------------------- */

static inline float half_mul(float a, float b) { return orc_f16_to_f32(orc_f32_to_f16(a * b)); }

typedef struct {
  const uint8_t* we; int64_t stride_row_blocks; const uint8_t* yq; int64_t ncols_y;
  const int32_t* ids_dst; float* dst; int64_t dst_col_stride; int64_t k; double* dst64;
  int64_t c0, c1;
} mmq_ctx;

static void mmq_range(int64_t begin, int64_t end, void* ctxp) {
  const mmq_ctx* x = (const mmq_ctx*)ctxp;
  const uint8_t* we = x->we; const int64_t stride_row_blocks = x->stride_row_blocks;
  const uint8_t* yq = x->yq; const int64_t ncols_y = x->ncols_y; const int32_t* ids_dst = x->ids_dst;
  float* dst = x->dst; const int64_t dst_col_stride = x->dst_col_stride; double* dst64 = x->dst64;
  const int64_t c0 = x->c0, c1 = x->c1, sbs = x->k / 256;
  {
    for (int64_t row = begin; row < end; ++row) {
      const uint8_t* wr = we + row * stride_row_blocks * ORC_Q4_K_BYTES;
      for (int64_t c = c0; c < c1; ++c) {
        float sum = 0.0f;
        double s64 = 0;
        for (int64_t sb = 0; sb < sbs; ++sb) {
          const uint8_t* wb = wr + sb * ORC_Q4_K_BYTES;
          const float d = orc_f16_to_f32(load_u16(wb)), dmin = orc_f16_to_f32(load_u16(wb + 2));
          int sc[8], mn[8];
          orc_q4_k_scales(wb, sc, mn);
          const uint8_t* codes = wb + 16;
          for (int g = 0; g < 8; ++g) {
            const int64_t kk = sb * 256 + g * 32;
            const uint8_t* yb = yq + ((kk / 128) * ncols_y + c) * ORC_Q8_1_MMQ_BYTES;
            const int gi = (int)((kk % 128) / 32);
            const float d8 = orc_f16_to_f32(load_u16(yb + gi * 4));
            const float s8 = orc_f16_to_f32(load_u16(yb + gi * 4 + 2));
            const int8_t* q = (const int8_t*)(yb + 16 + gi * 32);
            int32_t C = 0;
            for (int i = 0; i < 32; ++i)
              C += ((codes[(g / 2) * 32 + i] >> ((g % 2) * 4)) & 15) * (int32_t)q[i];
            const float ax = half_mul(d, (float)sc[g]);
            const float ay = half_mul(-dmin, (float)mn[g]);
            sum += ax * d8 * (float)C;
            sum += ay * s8;
            s64 += (double)ax * (double)d8 * (double)C + (double)ay * (double)s8;
          }
        }
        const int64_t col = ids_dst ? ids_dst[c] : c;
        dst[col * dst_col_stride + row] = sum;
        if (dst64) dst64[col * dst_col_stride + row] = s64;
      }
    }
  }
}

/* The exact int32 sums the MMQ folds: sums[(col * n + row) * (k / 32) + group] =
 * sum over the group's 32 values of code * q (the quantity the reference checks bit for bit
 * against GGML, tests/unit/dsv4_fast_test.cc:511-540). */
void orc_mmq_block_sums(const uint8_t* w, int64_t stride_row_blocks, const uint8_t* yq,
                        int64_t ncols, int64_t k, int64_t n, int32_t* sums) {
  const int64_t groups = k / 32;
  for (int64_t c = 0; c < ncols; ++c)
    for (int64_t row = 0; row < n; ++row)
      for (int64_t g = 0; g < groups; ++g) {
        const uint8_t* wb = w + (row * stride_row_blocks + g / 8) * ORC_Q4_K_BYTES;
        const uint8_t* codes = wb + 16 + ((g % 8) / 2) * 32;
        const uint8_t* yb = yq + ((g / 4) * ncols + c) * ORC_Q8_1_MMQ_BYTES;
        const int8_t* q = (const int8_t*)(yb + 16 + (g % 4) * 32);
        int32_t C = 0;
        for (int i = 0; i < 32; ++i) C += ((codes[i] >> ((g % 2) * 4)) & 15) * (int32_t)q[i];
        sums[(c * n + row) * groups + g] = C;
      }
}

void orc_mmq_q4_k(const uint8_t* w, int64_t stride_row_blocks, int64_t stride_expert_blocks,
                  const uint8_t* yq, int64_t ncols_y, const int32_t* ids_dst,
                  const int32_t* expert_bounds, int experts, float* dst, int64_t dst_col_stride,
                  int64_t k, int64_t n, double* dst64, int threads) {
  const int ne = expert_bounds ? experts : 1;
  for (int e = 0; e < ne; ++e) {
    mmq_ctx c;
    c.we = w + (int64_t)e * stride_expert_blocks * ORC_Q4_K_BYTES;
    c.stride_row_blocks = stride_row_blocks; c.yq = yq; c.ncols_y = ncols_y; c.ids_dst = ids_dst;
    c.dst = dst; c.dst_col_stride = dst_col_stride; c.k = k; c.dst64 = dst64;
    c.c0 = expert_bounds ? expert_bounds[e] : 0;
    c.c1 = expert_bounds ? expert_bounds[e + 1] : ncols_y;
    if (c.c1 > c.c0) orc_parallel_for(n, threads, mmq_range, &c);
  }
}

/* ------------------------------------------------------------------------- */
/* MXFP8: src/kernels/ggml/mxfp8_quant.cuh:22-46, llmp_ops.cu:610-663,       */
/* mxfp8_cutlass.h:30-54, moe_cutlass.h:42-46 == src/format/layout.h:107-112. */
/* ------------------------------------------------------------------------- */

uint32_t orc_mxfp8_scale_code(float amax) {
  const uint32_t bits = f32_bits(amax * (1.0f / 448.0f));
  uint32_t e = (bits >> 23) & 0xFFu;
  if (bits & 0x7FFFFFu) ++e;
  return e > 253u ? 253u : e;
}

/* ------------------------------------------------------------------------- */
/* Decode module, vector products (templates.cuh:83-186).                      */
/* ------------------------------------------------------------------------- */
uint64_t orc_scale_atom_offset(uint64_t row, uint64_t block, uint64_t blocks);
float orc_e2m1_to_f32(uint8_t code);
float orc_ue4m3_to_f32(uint8_t bits);

/* decoders.cuh:106-125 (Q8_0: half a block a segment), 193-220 (MXFP8). */
static void decode_segment(int decoder, const uint8_t* data, const uint8_t* scales,
                           int64_t row_bytes, int64_t k, int64_t row, int64_t seg, float v[16]) {
  if (decoder == 0) {
    const uint8_t* block = data + row * row_bytes + (seg / 2) * ORC_Q8_0_BYTES;
    const float d = orc_f16_to_f32(load_u16(block));
    const int8_t* q = (const int8_t*)(block + 2 + (seg & 1) * 16);
    for (int i = 0; i < 16; ++i) v[i] = d * (float)q[i];
    return;
  }
  if (decoder == 1 || decoder == 2) {
    const uint8_t e = decoder == 1
                          ? scales[row * (k / 32) + seg / 2]
                          : scales[orc_scale_atom_offset((uint64_t)row, (uint64_t)(seg / 2),
                                                         (uint64_t)(k / 32))];
    const float s = orc_e8m0_to_f32(e);
    const uint8_t* c = data + row * row_bytes + seg * 16;
    for (int i = 0; i < 16; ++i) v[i] = orc_e4m3_to_f32(c[i]) * s;
    return;
  }
  if (decoder == 3 || decoder == 4) { /* dense BF16 / F16 (decoders.cuh:73-103) */
    const uint8_t* c = data + row * row_bytes + seg * 32;
    for (int i = 0; i < 16; ++i) {
      const uint16_t bits = load_u16(c + 2 * i);
      v[i] = decoder == 3 ? orc_bf16_to_f32(bits) : orc_f16_to_f32(bits);
    }
    return;
  }
  /* E2M1 codes, value 2 i in byte i's low nibble; NVFP4 (5 split, 6 atoms): a UE4M3 scale
   * per 16; MXFP4 (7 split, 8 atoms): an E8M0 scale per 32 (decoders.cuh:57-71, 125-150,
   * 222-239). */
  const int nv = decoder == 5 || decoder == 6, atoms = decoder == 6 || decoder == 8;
  const int64_t blocks = nv ? k / 16 : k / 32, block = nv ? seg : seg / 2;
  const uint8_t code = atoms ? scales[orc_scale_atom_offset((uint64_t)row, (uint64_t)block,
                                                            (uint64_t)blocks)]
                             : scales[row * blocks + block];
  const float s = nv ? orc_ue4m3_to_f32(code) : orc_e8m0_to_f32(code);
  const uint8_t* c = data + row * row_bytes + seg * 8;
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = orc_e2m1_to_f32(c[i] & 15u) * s;
    v[2 * i + 1] = orc_e2m1_to_f32(c[i] >> 4) * s;
  }
}

/* E2M1: sign, two exponent bits (bias 1), one mantissa bit: +-{0, .5, 1, 1.5, 2, 3, 4, 6}
 * (src/kernels/device/float_formats.cuh:12-15). */
float orc_e2m1_to_f32(uint8_t code) {
  static const float magnitude[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  const float m = magnitude[code & 7u];
  return (code & 8u) ? -m : m;
}
/* NVFP4's block scale: E4M3's value for 0x00-0x7E, NaN from 0x7F up (float_formats.cuh:30-35). */
float orc_ue4m3_to_f32(uint8_t bits) {
  return bits >= 0x7Fu ? bits_f32(0x7fc00000u) : orc_e4m3_to_f32(bits);
}

/* decode::RunRows (templates.cuh:441-466): the decoded rows ids[i] times the tensor scale; an
 * id outside the matrix gives zeros and sets *bad. */
void orc_decode_rows(int decoder, const uint8_t* data, const uint8_t* scales, int64_t row_bytes,
                     int64_t k, int64_t n, const float* tensor_scale, int64_t rows_per_scale,
                     const int32_t* ids, int64_t count, float* y, int32_t* bad) {
  for (int64_t i = 0; i < count; ++i) {
    float* out = y + i * k;
    if (ids[i] < 0 || ids[i] >= n) {
      memset(out, 0, (size_t)k * sizeof(float));
      if (bad) *bad = 1;
      continue;
    }
    const float scale = tensor_scale ? tensor_scale[ids[i] / rows_per_scale] : 1.0f;
    for (int64_t seg = 0; seg < k / 16; ++seg) {
      float v[16];
      decode_segment(decoder, data, scales, row_bytes, k, ids[i], seg, v);
      for (int j = 0; j < 16; ++j) out[seg * 16 + j] = v[j] * scale;
    }
  }
}

static float decode_row_dot(int decoder, const uint8_t* data, const uint8_t* scales,
                            int64_t row_bytes, int64_t k, int64_t row, const float* x) {
  float lane[32];
  const int64_t segs = k / 16;
  for (int l = 0; l < 32; ++l) {
    float acc = 0.0f;
    for (int64_t seg = l; seg < segs; seg += 32) {
      float v[16];
      decode_segment(decoder, data, scales, row_bytes, k, row, seg, v);
      for (int i = 0; i < 16; ++i) acc = fmaf(v[i], x[seg * 16 + i], acc);
    }
    lane[l] = acc;
  }
  for (int offset = 16; offset > 0; offset >>= 1) {
    float next[32];
    for (int l = 0; l < 32; ++l) next[l] = lane[l] + lane[l ^ offset];
    memcpy(lane, next, sizeof(lane));
  }
  return lane[0];
}

void orc_decode_vector(int decoder, const uint8_t* data, const uint8_t* scales, int64_t row_bytes,
                       const uint8_t* data2, const uint8_t* scales2, int64_t k,
                       const float* tensor_scale, int64_t rows_per_scale, int64_t first,
                       int64_t first2, int64_t outputs, int glu, float limit, const float* x,
                       int64_t rows, int64_t x_stride, float* y, int64_t y_stride) {
  for (int64_t j = 0; j < outputs; ++j) {
    const float scale = tensor_scale ? tensor_scale[(first + j) / rows_per_scale] : 1.0f;
    const float scale2 = tensor_scale ? tensor_scale[(first2 + j) / rows_per_scale] : 1.0f;
    for (int64_t t = 0; t < rows; ++t) {
      const float* xt = x + t * x_stride;
      const float a = decode_row_dot(decoder, data, scales, row_bytes, k, first + j, xt) * scale;
      if (glu < 0) {
        y[t * y_stride + j] = a;
      } else {
        const float u = decode_row_dot(decoder, data2, scales2, row_bytes, k, first2 + j, xt) * scale2;
        y[t * y_stride + j] = orc_glu(glu, a, u, limit);
      }
    }
  }
}

uint64_t orc_scale_atom_offset(uint64_t row, uint64_t block, uint64_t blocks) {
  return (((row / 128) * (blocks / 4) + (block / 4)) * 512) + ((row % 32) * 16) +
         (((row % 128) / 32) * 4) + (block % 4);
}

uint64_t orc_mxfp8_rows_scales_offset(uint64_t rows, uint64_t k) {
  return (rows * k + 255) / 256 * 256;
}
uint64_t orc_mxfp8_rows_bytes(uint64_t rows, uint64_t k) {
  return orc_mxfp8_rows_scales_offset(rows, k) + ((rows + 127) / 128 * 128) * (k / 32);
}

void orc_mxfp8_quantize(const void* x, int is_bf16, int64_t row_stride, int64_t k, int64_t rows,
                        uint8_t* codes, uint8_t* scales) {
  const int64_t blocks = k / 32, padded = (rows + 127) / 128 * 128;
  for (int64_t r = 0; r < padded; ++r) {
    for (int64_t b = 0; b < blocks; ++b) {
      const uint64_t at = orc_scale_atom_offset((uint64_t)r, (uint64_t)b, (uint64_t)blocks);
      if (r >= rows) {
        scales[at] = 0;
        continue;
      }
      float v[32], amax = 0.0f;
      for (int j = 0; j < 32; ++j) {
        const int64_t i = r * row_stride + b * 32 + j;
        v[j] = is_bf16 ? orc_bf16_to_f32(((const uint16_t*)x)[i]) : ((const float*)x)[i];
        amax = fmaxf(amax, fabsf(v[j]));
      }
      const uint32_t e = orc_mxfp8_scale_code(amax);
      const float inverse = bits_f32((254u - e) << 23);
      for (int j = 0; j < 32; ++j)
        codes[r * k + b * 32 + j] = orc_f32_to_e4m3_satfinite(v[j] * inverse);
      scales[at] = (uint8_t)e;
    }
  }
}

void orc_mxfp8_swizzle(const uint8_t* in, uint8_t* out, int64_t n, int64_t blocks) {
  const int64_t padded = (n + 127) / 128 * 128;
  for (int64_t r = 0; r < padded; ++r)
    for (int64_t b = 0; b < blocks; ++b)
      out[orc_scale_atom_offset((uint64_t)r, (uint64_t)b, (uint64_t)blocks)] =
          r < n ? in[r * blocks + b] : 0;
}

/* E4M3 * 2^(s-127): tests/unit/reference_decode_test.cc:531-568. */
void orc_mxfp8_dequant(const uint8_t* codes, const uint8_t* scales_atoms, int64_t rows, int64_t k,
                       float* out) {
  const int64_t blocks = k / 32;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t b = 0; b < blocks; ++b) {
      const float s = orc_e8m0_to_f32(
          scales_atoms[orc_scale_atom_offset((uint64_t)r, (uint64_t)b, (uint64_t)blocks)]);
      for (int j = 0; j < 32; ++j)
        out[r * k + b * 32 + j] = orc_e4m3_to_f32(codes[r * k + b * 32 + j]) * s;
    }
}

/* D[m,n] = A[m,k] . B[n,k]^T over the decoded operands, accumulated in
 * double (the check tests/unit/qwen38_fast_test.cc:714-780 makes), stored as
 * F32 or nearest-even BF16 (mxfp8_cutlass.h:56-79). */
typedef struct { const float* af; const float* bf; int n, k; void* d; int bf16; double* d64; } gemm_ctx;

static void gemm_range(int64_t begin, int64_t end, void* ctxp) {
  const gemm_ctx* c = (const gemm_ctx*)ctxp;
  const float* af = c->af; const float* bf = c->bf; const int n = c->n, k = c->k;
  void* d = c->d; const int bf16 = c->bf16; double* d64 = c->d64;
  for (int64_t i = begin; i < end; ++i) {
    for (int j = 0; j < n; ++j) {
      double acc = 0;
      const float* ar = af + (size_t)i * k;
      const float* br = bf + (size_t)j * k;
      for (int x = 0; x < k; ++x) acc += (double)ar[x] * (double)br[x];
      if (bf16) ((uint16_t*)d)[(size_t)i * n + j] = orc_f32_to_bf16((float)acc);
      else ((float*)d)[(size_t)i * n + j] = (float)acc;
      if (d64) d64[(size_t)i * n + j] = acc;
    }
  }
}

void orc_mxfp8_gemm(int m, int n, int k, const uint8_t* a, const uint8_t* a_scales,
                    const uint8_t* b, const uint8_t* b_scales, void* d, int bf16, double* d64,
                    int threads) {
  float* af = (float*)malloc((size_t)m * k * sizeof(float));
  float* bf = (float*)malloc((size_t)n * k * sizeof(float));
  orc_mxfp8_dequant(a, a_scales, m, k, af);
  orc_mxfp8_dequant(b, b_scales, n, k, bf);
  gemm_ctx c = {af, bf, n, k, d, bf16, d64};
  orc_parallel_for(m, threads, gemm_range, &c);
  free(af);
  free(bf);
}

/* ------------------------------------------------------------------------- */
/* MoE route: src/kernels/ggml/moe_layout.h:47-83, llmp_moe.cu:81-160.       */
/* ------------------------------------------------------------------------- */

int64_t orc_moe_route_ints(int64_t experts, int64_t used, int64_t tokens) {
  const int64_t slots = used * tokens, chunks = (tokens + 63) / 64;
  return 2 * (experts + 1) + 3 * slots + chunks * experts;
}

void orc_moe_route(const int32_t* ids, int ids_stride, int experts, int used, int tokens,
                   int32_t* out) {
  const int64_t slots = (int64_t)used * tokens, chunks = (tokens + 63) / 64;
  int32_t* offsets = out;
  int32_t* scale_rows = out + (experts + 1);
  int32_t* position = out + 2 * (experts + 1);
  int32_t* token = position + slots;
  int32_t* expert = token + slots;
  int32_t* counts = expert + slots;
  for (int64_t i = 0; i < slots; ++i) token[i] = expert[i] = -1;
  memset(counts, 0, (size_t)(chunks * experts) * sizeof(int32_t));
  for (int t = 0; t < tokens; ++t)
    for (int j = 0; j < used; ++j) {
      const int e = ids[(int64_t)t * ids_stride + j];
      if (e >= 0 && e < experts) counts[(int64_t)(t / 64) * experts + e]++;
    }
  offsets[0] = 0;
  scale_rows[0] = 0;
  for (int e = 0; e < experts; ++e) {
    int running = 0;
    for (int64_t c = 0; c < chunks; ++c) {
      const int v = counts[c * experts + e];
      counts[c * experts + e] = running;
      running += v;
    }
    offsets[e + 1] = offsets[e] + running;
    scale_rows[e + 1] = scale_rows[e] + (running + 127) / 128 * 128;
  }
  int32_t* placed = (int32_t*)calloc((size_t)experts, sizeof(int32_t));
  for (int64_t c = 0; c < chunks; ++c) {
    memset(placed, 0, (size_t)experts * sizeof(int32_t));
    const int t1 = (int)((c + 1) * 64 < tokens ? (c + 1) * 64 : tokens);
    for (int t = (int)(c * 64); t < t1; ++t)
      for (int j = 0; j < used; ++j) {
        const int64_t slot = (int64_t)t * used + j;
        const int e = ids[(int64_t)t * ids_stride + j];
        if (e < 0 || e >= experts) {
          position[slot] = -1;
          continue;
        }
        const int row = offsets[e] + counts[c * experts + e] + placed[e]++;
        position[slot] = row;
        token[row] = t;
        expert[row] = e;
      }
  }
  free(placed);
}

/* Ordered weighted sum over a token's slots (llmp_moe.cu:393-435, without the
 * NVFP4 global scales and the shared expert): e_j = row * w_j, acc = e_0,
 * acc += e_j; a slot whose id was outside the experts contributes NaN. */
void orc_moe_combine(const float* rows, const int32_t* position, const float* weights, int used,
                     int tokens, int width, float* dst) {
  for (int t = 0; t < tokens; ++t)
    for (int c = 0; c < width; ++c) {
      float acc = 0.0f;
      for (int j = 0; j < used; ++j) {
        const int p = position[(int64_t)t * used + j];
        const float v = p >= 0 ? rows[(int64_t)p * width + c] : NAN;
        const float e = v * weights[(int64_t)t * used + j];
        acc = j == 0 ? e : acc + e;
      }
      dst[(int64_t)t * width + c] = acc;
    }
}
