/*
 * llmp_b200: B200 (sm_100a) kernels for llmp's quantized matrix products,
 * behind a C ABI shaped on the reference's own CUDA-type-free launch structs.
 *
 * Conventions (the reference's, src/kernels/ggml/mxfp8_cutlass.h:73-79 and
 * src/kernels/common/selected_operation.h:26-35, 129-160):
 *   - every pointer is a caller-owned DEVICE address unless a comment says
 *     host; scratch is caller-allocated, 256-byte aligned, sized by the
 *     matching *_scratch() call;
 *   - a call only queues work on `stream` (a cudaStream_t passed as void*):
 *     it never synchronizes, never allocates, and does nothing that depends
 *     on a device value reaching the host;
 *   - return 0: queued.  >0: refused before anything was queued (the shape or
 *     an operand is not one this build takes; llmp_b200_last_error() says
 *     why).  <0: a CUDA call failed after work may have been queued; the
 *     caller must treat its stream's context as faulted;
 *   - results are deterministic: no floating-point atomics, fixed summation
 *     orders; a token's sums do not depend on which other tokens share a call
 *     when the launch configuration is the same (see llmp_b200_vecq's variants);
 *   - thread-compatible: one stream per calling thread.
 *
 * There is no CPU fallback: on a machine without an sm_100 GPU every launch
 * entry point returns LLMP_B200_NO_DEVICE.
 */
#ifndef LLMP_B200_H_
#define LLMP_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLMP_B200_OK 0
#define LLMP_B200_REJECTED 1  /* shape / operand not taken; nothing queued */
#define LLMP_B200_NO_DEVICE 2 /* no sm_100 device is current; nothing queued */

/* GGML type numbers of the block encodings (src/format/encoding.cc:111-115). */
#define LLMP_B200_TYPE_Q8_0 8
#define LLMP_B200_TYPE_Q8_1 9
#define LLMP_B200_TYPE_Q4_K 12
/* The other block types of the reference's llmp.vecq (src/kernels/ggml/vecq.cu:54-96) that this
 * build's llmp_b200_vecq also takes, dense or grouped, 1 to 16 tokens, with or without a GLU:
 * one launch configuration each, not tuned.  Numbers are GGML's type ids. */
#define LLMP_B200_TYPE_Q4_0 2
#define LLMP_B200_TYPE_Q5_0 6
#define LLMP_B200_TYPE_Q5_K 13
#define LLMP_B200_TYPE_Q6_K 14
#define LLMP_B200_TYPE_IQ4_NL 20

/* VecQGlu (src/kernels/ggml/llmp_ops.h:1072). */
#define LLMP_B200_GLU_NONE 0
#define LLMP_B200_GLU_SWIGLU 1
#define LLMP_B200_GLU_SWIGLU_CLAMP 2
#define LLMP_B200_GLU_GEGLU 3

/* Replaces mxfp8::Available / moe::GroupedGemmAvailable
 * (src/kernels/ggml/mxfp8_cutlass.h:71, moe_cutlass.h:66): 1 when the current
 * device is compute capability 10.0 and the kernels were built for it. */
int llmp_b200_available(void);
/* SM count of the current device (the `sms` argument the reference's
 * launchers take), or 0. */
int llmp_b200_sm_count(void);
/* Thread-local text for the last non-zero status on this thread. */
const char* llmp_b200_last_error(void);

/* Diagnostics, no reference counterpart: how many bounded device-side waits
 * (an mbarrier that a bulk copy should have completed) ran out, plus how many
 * device-resident operands a kernel refused to read (a grouped product's
 * expert whose pointers or pitch its loads could not take), since the library
 * was loaded.  0 on a healthy device with well-formed operands; synchronizes the device, so it
 * is for tests and post-mortems, never for the launch path.  -1: unreadable. */
int llmp_b200_device_faults(void);
/* The same count, which is then set back to zero (synchronizes the device too). */
int llmp_b200_device_faults_clear(void);
/* Diagnostics, no reference counterpart: runs the give-up path of the library's bounded
 * waits once, harmlessly.  One warp waits at most `polls` polls (1..4096; a pending poll
 * suspends for about a microsecond) on a barrier nothing will ever arrive at, gives up,
 * raises llmp_b200_device_faults() by one and writes 1 to *status (a device int32).  The
 * context stays usable: a test follows it with an ordinary launch. */
int llmp_b200_wait_selftest(int polls, int32_t* status, void* stream);

/* ------------------------------------------------------------------ Q8_1 */
/* Replaces RunQuantizeQ8 (src/kernels/ggml/vecq.cu:1095-1111), which calls
 * GGML's quantize_row_q8_1_cuda.  x: F32 [k, rows, planes], strides in
 * floats.  out: Q8_1 blocks (36 bytes: FP16 d, FP16 sum of the inputs, 32
 * int8), each of the rows*planes rows padded with zero blocks to a multiple
 * of 512 values (llmp_b200_q8_1_row_blocks(k) blocks a row). */
int64_t llmp_b200_q8_1_row_blocks(int64_t k);
int llmp_b200_q8_1_quantize(const float* x, int64_t k, int64_t rows, int64_t planes,
                            int64_t stride_row, int64_t stride_plane, void* out, void* stream);

/* ------------------------------------------------------------------ vecq */
/* Field for field the reference's VecQDesc (src/kernels/ggml/vecq.h:23-42):
 * weight offsets count the weight type's blocks, activation offsets count
 * Q8_1 blocks, destination offsets count floats. */
typedef struct llmp_b200_vecq_desc {
  const void* w;      /* weights (the up projection with a GLU) */
  const void* g;      /* gate weights, or NULL */
  const void* y;      /* Q8_1 activations */
  const int32_t* ids; /* NULL: dense / grouped; else I32 [used, tokens] */
  float* dst;
  int ncols_x;       /* k */
  int nrows;         /* n */
  int stride_row;    /* weight blocks between rows */
  int stride_expert; /* weight blocks between experts / groups */
  int y_token;       /* Q8_1 blocks between tokens' rows */
  int y_slot;        /* between slots' rows (per-slot activations), else 0 */
  int ids_stride;    /* ids between tokens */
  int used;          /* slots a token (1 when dense) */
  int tokens;        /* 1..16 (the reference's bound); routed: up to 128, used * tokens <= 1024 */
  int dst_token;     /* floats */
  int dst_slot;
  int glu;           /* LLMP_B200_GLU_* */
  float limit;       /* clamp of LLMP_B200_GLU_SWIGLU_CLAMP */
} llmp_b200_vecq_desc;

/* Replaces VecQVariants / VecQVariantName / LaunchVecQ
 * (src/kernels/ggml/vecq.h:44-49) together with the operand checks of
 * CheckVecQ (src/kernels/ggml/llmp_ops.cc:2915-2982).  Types: Q8_0, Q4_K.
 * variant >= 0: that launch configuration (status > 0 if it does not take the product).
 * variant -1: the configuration that measured fastest on B200 for this very (k, n, GLU,
 * token count) when the rank table has it, else the rule for the shape; a token's F32 bits
 * may then differ between token counts (as the reference's MMVQ's do).
 * variant -2: the rule for the shape alone, whose geometry is the one-token plan's whatever
 * the token count: a token's bits do not depend on its company (the reference's
 * row_invariant capability; llmp_b200_mmvq_rows runs on it). */
int llmp_b200_vecq_variants(void);
const char* llmp_b200_vecq_variant_name(int variant);
int llmp_b200_vecq(int type, const llmp_b200_vecq_desc* desc, int variant, void* stream);
/* The measured rank table (the role of src/kernels/ggml/measured_ranks.h and
 * src/execution/rank_data.h): row i names the launch configuration that measured fastest on
 * B200 for the dense Q4_K product (k, n, fused GLU, tokens a pass) and its time.  Returns the
 * configuration's name ("" past the table). */
int llmp_b200_vecq_rank_count(void);
const char* llmp_b200_vecq_rank(int row, int* k, int* n, int* glu, int* tokens, float* microseconds);

/* The product with its activation quantization fused: the reference lowers a
 * shared QuantizeQ8 node in front of its products (src/kernels/ggml/shared_q8.h
 * :20-47, vecq.cu:1095-1175); here desc->y points at the F32 activations
 * themselves ([k, tokens], y_token FLOATS between tokens) and every CTA
 * quantizes them to Q8_1 in shared memory with the quantizer's arithmetic, so
 * the sums are the two-call path's bit for bit and one launch is saved.  Taken
 * for dense Q4_K products of up to 8 tokens (others: status > 0, use the two
 * calls).  q8_out (or NULL): receives the Q8_1 blocks of the first k / 32
 * blocks of each token's row, rows llmp_b200_q8_1_row_blocks(k) blocks apart. */
int llmp_b200_vecq_f32(int type, const llmp_b200_vecq_desc* desc, void* q8_out, void* stream);

/* The product with the quantization of its OUTPUT fused: in the decode graph a
 * product's F32 result usually feeds the QuantizeQ8 node of the next product
 * (src/kernels/ggml/vecq.cu:1095-1111 after :1168; shared_q8.h:20-47).  This
 * entry writes desc->dst as llmp_b200_vecq does and, besides, the Q8_1 blocks of
 * every token's output row into q8_dst ([tokens][nrows / 32] blocks of 36 bytes):
 * the warp that completes a 32-row block quantizes it with the quantizer's
 * arithmetic, so the blocks equal llmp_b200_q8_1_quantize(dst) bit for bit and
 * one launch is saved (on B200 the counting tail costs the product about what
 * the launch costs: measure before preferring it).  Taken for dense Q4_K
 * products of up to 8 tokens whose nrows is a multiple of 512 (others:
 * status > 0, use the two calls).
 * rows_done: llmp_b200_vecq_q8_scratch(nrows, tokens) bytes of device memory,
 * zero before the first call; every call leaves them zero.  Calls that share
 * rows_done must be ordered on a stream. */
size_t llmp_b200_vecq_q8_scratch(int nrows, int tokens);
int llmp_b200_vecq_q8(int type, const llmp_b200_vecq_desc* desc, void* q8_dst, uint32_t* rows_done,
                      void* stream);

/* ------------------------------------------------------------------ MMVQ */
/* The operands of the reference's MMVQ calls (GGML's mul_mat_vec_q as
 * src/kernels/ggml/mul_mat_q.cu:407-451, 502-515 reaches it): dense weights [n][k] in
 * blocks, F32 activation columns (or their prepared Q8_1 rows), F32 output columns. */
typedef struct llmp_b200_mmvq_desc {
  int type;                /* LLMP_B200_TYPE_Q8_0 / _Q4_K */
  const void* w;           /* weight blocks; with a GLU the up projection */
  const void* gate;        /* MulMatVecQGlu: the gate's blocks (same shape), else NULL */
  int glu;                 /* LLMP_B200_GLU_* */
  float limit;
  const float* x;          /* F32 [k, cols]: columns x_col_stride floats apart, 16-byte aligned */
  int64_t x_col_stride;
  const void* q8;          /* prepared Q8_1 rows (llmp_b200_q8_1_row_blocks(k) blocks a column), or NULL */
  float* dst;              /* F32 [n, cols]: columns dst_col_stride floats apart */
  int64_t dst_col_stride;
  int k, n, cols;
  int stride_row;          /* weight blocks between rows */
  void* scratch;           /* llmp_b200_mmvq_scratch(k, cols) bytes, 256-byte aligned (unused when prepared) */
} llmp_b200_mmvq_desc;
/* Replaces PlanMulMatVecQ's draw (mul_mat_q.cu:308-312): the Q8_1 rows of cols columns. */
size_t llmp_b200_mmvq_scratch(int k, int cols);
/* Replaces MulMatVecQ and, with `gate`, MulMatVecQGlu (mul_mat_q.cu:407-416, 502-515): quantize
 * the 1 to 8 columns of x into scratch, then dst[:, c] = W . x[:, c] (or the GLU of the gate and
 * up products).  Two launches: the Q8_1 quantizer and the llmp.vecq product. */
int llmp_b200_mmvq(const llmp_b200_mmvq_desc* desc, void* stream);
/* Replaces RunMmvqPrepared (mul_mat_q.cu:431-451): the same product over prepared rows
 * (desc->q8), which another product may share; nothing is quantized, scratch is unused. */
int llmp_b200_mmvq_prepared(const llmp_b200_mmvq_desc* desc, void* stream);
/* Replaces MulMatVecQRows (src/kernels/ggml/mmvq_rows.cu:825; kernel :319-452): every column's
 * F32 result is the one-column product's, bit for bit, whatever the column count (a
 * speculative verify's rows equal the decode steps they stand for).  Takes any column
 * count up to 4096 (the reference: 8) in passes that keep the one-column launch geometry;
 * x or prepared q8.  No fused GLU. */
int llmp_b200_mmvq_rows(const llmp_b200_mmvq_desc* desc, void* stream);

/* ------------------------------------------------------------------ peer exchange */
/* The all-gather after an N-column sharded projection (the reference's kAllGather node,
 * src/ir/op.h:246-250, src/planner/partition.h:39-56, src/components/ffn.cc:67-81) without a
 * collective library: llmp_b200_peer_publish stores this rank's slice into every rank's copy of
 * the gathered vector (plain stores into memory of the other GPUs, mapped through CUDA IPC)
 * and raises a flag word on each; the consumer begins by waiting, with a bound, for every
 * rank's flag (llmp_b200_q8_1_quantize_gathered, or llmp_b200_peer_wait alone).  One process a
 * GPU.  Memory that other processes map comes from llmp_b200_peer_alloc (zeroed; the one place
 * this library allocates, because an exportable allocation must be a whole one). */
#define LLMP_B200_PEER_HANDLE_BYTES 64
int llmp_b200_peer_alloc(size_t bytes, void** ptr);
int llmp_b200_peer_free(void* ptr);
int llmp_b200_peer_export(const void* ptr, void* handle /* 64 bytes out */);
int llmp_b200_peer_import(const void* handle, void** ptr);  /* another process's allocation */
int llmp_b200_peer_close(void* ptr);
typedef struct llmp_b200_peer_site {
  int world, rank;
  void* const* buffers;    /* device array [world]: every rank's copy of the gathered vector ([rank]: local) */
  int32_t* const* flags;   /* device array [world]: every rank's flag words, I32 [sites][world], zeroed */
  const int32_t* step;     /* device word, this rank's: the step number flags are compared with */
  int site;                /* which exchange of the step: its own row of flags */
} llmp_b200_peer_site;
/* Raises the step word by one: once at the start of a step (a captured graph replays it). */
int llmp_b200_peer_begin_step(int32_t* step, void* stream);
/* slice (bytes, 16-byte aligned, the kernel before's output) -> offset in every rank's buffer,
 * then flags[to][site][rank] = step on every rank `to`. */
int llmp_b200_peer_publish(const llmp_b200_peer_site* site, const void* slice, size_t offset,
                           size_t bytes, void* stream);
/* Waits until local_flags[site][r] has reached the step number for every r, polling each at
 * most `polls` times about 0.1 us apart.  A wait that runs out writes 1 to *status (a device
 * int32, may be NULL), raises llmp_b200_device_faults() by one and RETURNS: the stream always
 * finishes. */
int llmp_b200_peer_wait(const llmp_b200_peer_site* site, const int32_t* local_flags, int polls,
                        int32_t* status, void* stream);
/* llmp_b200_q8_1_quantize of one plane whose input is a gathered vector: every CTA first waits
 * as llmp_b200_peer_wait does. */
int llmp_b200_q8_1_quantize_gathered(const float* x, int64_t k, int64_t rows, int64_t stride_row,
                                     void* out, const llmp_b200_peer_site* site,
                                     const int32_t* local_flags, int polls, int32_t* status,
                                     void* stream);
/* Publish, wait and quantize in ONE launch: stores `slice` (the kernel before's output) into
 * every rank's buffer of the site and flags it, waits for every rank's flag, then quantizes the
 * F32 vector x of k values (the gathered vector itself, or another input when the exchange is
 * waited for as back-pressure only). */
int llmp_b200_q8_1_quantize_exchange(const float* x, int64_t k, void* out,
                                     const llmp_b200_peer_site* site, const int32_t* local_flags,
                                     const void* slice, size_t offset, size_t bytes, int polls,
                                     int32_t* status, void* stream);

/* The in-band form of the exchange: no flag words, no fence, no publishing kernel.  A value
 * travels as one 8-byte word {F32 bits, tag}, tag = (step << 8) | an exchange number of 0 to
 * 255, and it is the PRODUCT KERNEL that stores token 0's results, tagged, into every rank's
 * vector of words at words[r] + base + row (as well as into desc->dst); a reader polls each word
 * it needs until it carries the expected tag.  Dense Q4_K products of one token (the two
 * kernels of the decode step). */
typedef struct llmp_b200_peer_fan {
  int world;
  uint64_t* const* words;  /* device array [world]: every rank's vector (llmp_b200_peer_alloc, zeroed) */
  const int32_t* step;     /* this rank's step word */
  int base;                /* word index of this rank's first row */
  int tag;
} llmp_b200_peer_fan;
int llmp_b200_vecq_fan(int type, const llmp_b200_vecq_desc* desc, int variant,
                       const llmp_b200_peer_fan* fan, void* stream);
/* The Q8_1 quantizer of one row of k values that arrive as such words (x NULL), each polled
 * at most `polls` times about 0.1 us apart; or of x (words NULL).  `hold` (or NULL): another
 * run of hold_count words whose arrival under hold_tag is waited for first, values unused.  A
 * word that does not arrive writes 1 to *status, raises llmp_b200_device_faults() and the
 * kernel carries on. */
int llmp_b200_q8_1_quantize_words(const float* x, const uint64_t* words, int tag, int64_t k,
                                  const uint64_t* hold, int64_t hold_count, int hold_tag,
                                  const int32_t* step, void* out, int polls, int32_t* status,
                                  void* stream);

/* Verification entry with no reference counterpart as a separate call: the
 * int32 per-block sums the product kernels form (the quantity the reference
 * checks bit for bit, tests/unit/dsv4_fast_test.cc:511-540), for nrows weight
 * rows against ONE Q8_1 row.  Q8_0: dots[row][k/32].  Q4_K: dots[row][k/32]
 * (sum code*q per 32-value sub-block) and qsums[row][k/32] (sum q). */
int llmp_b200_vecq_block_sums(int type, const void* w, const void* y, int k, int nrows,
                              int stride_row, int32_t* dots, int32_t* qsums, void* stream);

/* ------------------------------------------------------------------ MMQ */
/* Replaces GGML's quantize_mmq_q8_1_cuda as the reference calls it
 * (src/kernels/ggml/mul_mat_q.cu:606-610, 806; the D2S6 sibling is restated
 * in-tree at mul_mat_q_glu.cu:170-218).  x: F32 or BF16 [k, rows], row stride
 * in elements.  out: block_q8_1_mmq in the DS4 layout (144 bytes: four (FP16
 * d, FP16 sum of the inputs) pairs, then 128 int8), ordered [k / 128][cols].
 * ids_src (device, or NULL): column c quantizes input row ids_src[c] (the
 * scatter to an expert-sorted order). */
int64_t llmp_b200_mmq_q8_1_bytes(int64_t k, int64_t cols);
int llmp_b200_mmq_quantize(const void* x, int is_bf16, int64_t row_stride, int64_t k, int64_t cols,
                           const int32_t* ids_src, void* out, void* stream);

/* The operands GGML's mmq_args carry as the reference fills them
 * (src/kernels/ggml/mul_mat_q.cu:632-658). */
typedef struct llmp_b200_mmq_desc {
  int type;                     /* LLMP_B200_TYPE_Q4_K */
  const void* w;                /* weight blocks [experts][nrows][k / 256] */
  const void* y;                /* Q8_1-MMQ blocks [k / 128][ncols] */
  const int32_t* ids_dst;       /* device: sorted column -> output column, or NULL */
  const int32_t* expert_bounds; /* device: experts + 1 column bounds, or NULL (dense) */
  float* dst;                   /* F32 [out column][nrows], dst_col_stride floats apart */
  int k, nrows, ncols;          /* ncols: columns of y */
  int stride_row;               /* weight blocks between rows */
  int stride_expert;            /* weight blocks between experts */
  int dst_col_stride;
  int experts;                  /* with expert_bounds */
  int max_cols_per_expert;      /* host-known bound on an expert's columns (<= ncols) */
  const void* w_slab;           /* the weights as llmp_b200_q4k_relayout left them, or NULL
                                   (then `w` is read; with a slab `w` may be NULL) */
  void* scratch;                /* llmp_b200_mmq_scratch() bytes, 256-byte aligned, or NULL */
} llmp_b200_mmq_desc;

/* The reference's import-time expert relayout (src/import/expert_relayout.h,
 * src/kernels/ggml/moe_layout.h:8-24, src/engine/expert_slab.h:22-36: GGML blocks to the
 * tensor core's layout, once at load time), for Q4_K and tcgen05: per expert the 4-bit codes
 * as int8 rows K-major (what kind::i8 reads through a swizzled tensor map), the groups'
 * (d * sc)_half as F32 in [128 rows][k-step] tiles, the groups' (-dmin * m)_half as FP16
 * K-major.  Lossless: every value of the blocks is kept, only rearranged and widened
 * (1.19 bytes a weight against 0.56).  w: Q4_K blocks [experts][nrows][k / 256], stride_row
 * blocks between rows, stride_expert blocks between experts.  slab: llmp_b200_q4k_slab_bytes
 * bytes, 256-byte aligned.  One launch; nothing else is allocated or synchronized. */
size_t llmp_b200_q4k_slab_bytes(int nrows, int k, int experts);
int llmp_b200_q4k_relayout(const void* w, int nrows, int k, int stride_row, int64_t stride_expert,
                           int experts, void* slab, void* stream);

/* Replace PlanMulMatQ's scratch sizing and MulMatQ / RunExpertProducts
 * (src/kernels/ggml/mul_mat_q.cu:317-397, 453-462, 551-737): D[col][row] =
 * W[row] . Y[col] with exact int32 group sums on tcgen05 (kind::i8) and the
 * F32 scale fold of GGML's MMQ.  The weights are read from desc->w_slab when given;
 * else they are relaid into desc->scratch first (llmp_b200_mmq_scratch bytes: the slab's
 * size; one more launch); with neither, the kernel unpacks the raw blocks itself, k-step
 * by k-step, which is the slowest of the three and needs no memory.  There is no stream-k
 * fixup pass. */
size_t llmp_b200_mmq_scratch(const llmp_b200_mmq_desc* desc, int sms);
int llmp_b200_mmq(const llmp_b200_mmq_desc* desc, int sms, void* stream);
/* The gate | up product with the GLU and the requantization in its write-back (the reference's
 * MulMatQGlu, src/kernels/ggml/mul_mat_q_glu.cu:143-218): instead of F32 [2 * inter] a column,
 * the Q8_1-MMQ blocks of glu(gate . y, up . y), [inter / 128][ncols] x 144 bytes, which the
 * down product reads.  The weights come as a slab whose rows interleave gate and up rows
 * (llmp_b200_q4k_relayout_glu at load time: the source holds inter gate rows, then inter up
 * rows, per expert); desc->nrows = 2 * inter (a multiple of 64), desc->dst is unused,
 * desc->ids_dst NULL.  The blocks equal, bit for bit, what llmp_b200_moe_glu_quantize makes of
 * the F32 product. */
int llmp_b200_q4k_relayout_glu(const void* w, int inter, int k, int stride_row, int64_t stride_expert,
                               int experts, void* slab, void* stream);
int llmp_b200_mmq_glu(const llmp_b200_mmq_desc* desc, int glu, float limit, void* blocks,
                      void* stream);

/* Verification entry with no reference counterpart as a separate call: the dense product as
 * llmp_b200_mmq queues it and, besides, the exact int32 sums C = sum code * q of every
 * (column, weight row, 32-value group), read out of tensor memory before the fold:
 * sums[(col * nrows + row) * (k / 32) + group] (the quantity the reference checks bit for
 * bit against GGML, tests/unit/dsv4_fast_test.cc:511-540). */
int llmp_b200_mmq_block_sums(const llmp_b200_mmq_desc* desc, int32_t* sums, void* stream);

/* ------------------------------------------------------------------ MoE */
/* Replaces RunMoeRoute (src/kernels/ggml/llmp_moe.cu:760; kernels :81-160).
 * ids: I32 [used, tokens], ids_stride ints between tokens.  out: the I32 blob
 * of moe::RouteLayout (moe_layout.h:47-83), llmp_b200_moe_route_ints() ints:
 *   offsets[experts+1]     expert e's rows are offsets[e]..offsets[e+1] of the
 *                          sorted order (slots in token order within an expert)
 *   scale_rows[experts+1]  prefix of each expert's rows rounded up to 128
 *   position[slots]        each slot's sorted row (slot = t * used + j; -1 for
 *                          an id outside the experts)
 *   token[slots], expert[slots]   each sorted row's token and expert (rows no
 *                          slot reaches hold 0)
 *   counts[chunks*experts] the counting blocks' work space (64 tokens a chunk) */
int64_t llmp_b200_moe_route_ints(int experts, int used, int tokens);
int llmp_b200_moe_route(const int32_t* ids, int ids_stride, int experts, int used, int tokens,
                        int32_t* out, void* stream);

/* Shaped on moe::GroupedGemm (src/kernels/ggml/moe_cutlass.h:48-63).  The
 * reference multiplies NVFP4 operands; this build's experts are Q4_K blocks
 * and its activations Q8_1-MMQ blocks, so `a` holds the blocks' scales and no
 * separate scale arrays are passed. */
typedef struct llmp_b200_grouped_gemm_desc {
  int groups;               /* experts */
  int n;                    /* output features (weight rows an expert) */
  int k;                    /* a multiple of 256 */
  int rows;                 /* sorted activation rows (columns of `a`) */
  const int32_t* offsets;   /* device, groups + 1: a route's offsets */
  const void* a;            /* Q8_1-MMQ blocks [k / 128][rows], expert-sorted rows */
  const void* weights;      /* Q4_K blocks: expert e at weights + e * expert_stride */
  uint64_t expert_stride;   /* bytes, a multiple of 144 */
  void* d;                  /* F32 [rows][n] */
  void* scratch;            /* llmp_b200_grouped_gemm_scratch() bytes, 256-byte aligned */
  const void* weights_slab; /* the experts as llmp_b200_q4k_relayout(weights, n, k, k / 256,
                               expert_stride / 144, groups) left them, or NULL: then the
                               kernel unpacks `weights` itself (slower) */
} llmp_b200_grouped_gemm_desc;

/* Replace moe::GroupedGemmAvailable / GroupedGemmScratch / RunGroupedGemm
 * (moe_cutlass.h:64-76): per expert e, D_e[M_e, n] = A_e[M_e, k] . W_e^T with the
 * arithmetic of llmp_b200_mmq.  The tile list is built on the device from
 * `offsets` into `scratch` (the reference's SetupGroups), then the tensor-core
 * kernel runs one CTA a listed tile. */
int llmp_b200_grouped_gemm_available(void);
size_t llmp_b200_grouped_gemm_scratch(int groups, int rows, int sms);
int llmp_b200_grouped_gemm(const llmp_b200_grouped_gemm_desc* gemm, int sms, void* stream);
/* The grouped gate | up product with the GLU write-back (see llmp_b200_mmq_glu): gemm->n = 2 * inter,
 * gemm->weights_slab from llmp_b200_q4k_relayout_glu, gemm->d unused; blocks: Q8_1-MMQ
 * [inter / 128][rows]. */
int llmp_b200_grouped_gemm_glu(const llmp_b200_grouped_gemm_desc* gemm, int glu, float limit,
                               void* blocks, int sms, void* stream);

/* No counterpart in the reference.  The grouped GEMM for callers that have no
 * way to hand over scratch: code running where device allocation is off the
 * table (a latency-critical serving loop that must never take the allocator's
 * device-wide synchronization, a host that pre-sized all of its memory and has
 * none left to carve a work area from, a plug-in boundary whose contract
 * forbids the callee's caller from allocating on its behalf).  It is
 * llmp_b200_grouped_gemm with the tile list kept in a 6,400-byte array built
 * into the library's device image instead of `scratch` (which is ignored and
 * may be NULL).  It calls no allocator of any kind.
 *   - Limits: at most 256 groups and 65,536 sorted rows; larger problems are
 *     refused (status > 0) with a message naming the limits.
 *   - The first call on each device looks the array's device address up
 *     (cudaGetSymbolAddress); make that first call before starting any stream
 *     capture.
 *   - All calls on a device share the one array: two calls whose kernels may
 *     overlap on the GPU (different streams, no ordering) race on it.  Calls
 *     ordered on one stream are safe; each rebuilds the list it uses. */
int llmp_b200_grouped_gemm_static(const llmp_b200_grouped_gemm_desc* gemm, int sms, void* stream);

/* Replaces llmp.moe.glu_quantize (llmp_moe.cu:348-392) for this build's
 * activation format: gate_up F32 [2 f, rows] (gate then up in a row); out:
 * Q8_1-MMQ blocks [f / 128][rows] of glu(gate, up). */
int llmp_b200_moe_glu_quantize(const float* gate_up, int64_t row_stride, int f, int64_t rows,
                               int glu, float limit, void* out, void* stream);

/* Expert-parallel dispatch (the reference models expert parallelism as a partition of whole
 * experts, src/planner/partition.h:57-67, src/components/moe.cc:521-531, with kAllToAll as its
 * exchange, src/ir/op.h:246-250): packs this rank's (token, slot) rows for an all-to-all of
 * FIXED size, so no split size ever reaches the host.  Rank r owns experts [r, r + 1) * experts /
 * world.  `route` is llmp_b200_moe_route's blob over the slots' owner ranks (ids / (experts /
 * world), world "experts").  Lane i of destination r, send_rows[(r * capacity + i) * hidden ..],
 * takes the i-th row bound for r in (token, slot) order and send_ids[r * capacity + i] its
 * expert's index on r (unused lanes: -1).  home[slot] is the lane the slot's result comes back
 * in after the return all-to-all (the `position` of llmp_b200_moe_combine over the returned
 * rows), -1 for an id outside the experts.  A row beyond a destination's capacity is dropped,
 * counted in *dropped (a device int the caller zeroes) and its home is -1. */
int llmp_b200_moe_ep_pack(const float* x, int64_t x_stride, int hidden, const int32_t* ids,
                          int ids_stride, int used, int tokens, int experts, int world, int capacity,
                          const int32_t* route, float* send_rows, int32_t* send_ids, int32_t* home,
                          int32_t* dropped, void* stream);

/* The routed block for 1 to 16 tokens as ONE launch: what the reference runs as llmp.q8_1,
 * llmp.vecq with ids and a GLU, llmp.q8_1, llmp.vecq per slot and llmp.moe.combine
 * (src/kernels/ggml/vecq.cu:457-665, llmp_moe.cu:393-435; src/components/moe.cc's decode
 * branch).  dst[t] = sum over the token's slots j, in slot order, of weights[t][j] *
 * (down_e . Q8_1(glu(gate_e . Q8_1(x_t), up_e . Q8_1(x_t)))), e = ids[t][j]; a slot outside
 * the experts contributes NaN.  A cooperative launch of one CTA an SM with one grid barrier,
 * waited for with a bound (it raises llmp_b200_device_faults() and stores nothing if it
 * runs out).  scratch: llmp_b200_moe_decode_scratch() bytes, 256-byte aligned, its first 256
 * bytes zeroed ONCE (not between calls). */
typedef struct llmp_b200_moe_decode_desc {
  const float* x;          /* F32 [tokens, hidden], rows x_stride floats apart, 16-byte aligned */
  int64_t x_stride;
  const int32_t* ids;      /* I32 [tokens, used], rows ids_stride apart */
  int ids_stride;
  const float* weights;    /* F32 [tokens, used], packed */
  const void* gate_up;     /* Q4_K [experts][2 * inter][hidden / 256]: gate rows, then up rows */
  const void* down;        /* Q4_K [experts][hidden][inter / 256] */
  int experts, used, tokens, hidden, inter;
  int glu;                 /* LLMP_B200_GLU_SWIGLU / _SWIGLU_CLAMP / _GEGLU */
  float limit;
  float* dst;              /* F32 [tokens, hidden], rows dst_stride floats apart */
  int64_t dst_stride;
  void* scratch;
} llmp_b200_moe_decode_desc;
size_t llmp_b200_moe_decode_scratch(int used, int tokens, int inter);
int llmp_b200_moe_decode(const llmp_b200_moe_decode_desc* desc, void* stream);

/* Replaces llmp.moe.combine_sorted (llmp_moe.cu:393-435) without NVFP4's global
 * scales and the shared expert: dst[t] = sum over the token's slots, in slot
 * order, of rows[position[t * used + j]] * weights[t * used + j].  position NULL: the rows
 * are already in slot order (row t * used + j), as the routed decode products leave them. */
int llmp_b200_moe_combine(const float* rows, int64_t row_stride, const int32_t* position,
                          const float* weights, int used, int tokens, int width, float* dst,
                          void* stream);

/* ------------------------------------------------------------------ MXFP8 */
/* MXFP8: E4M3 codes with one E8M0 scale per 32 values along K.  Scales live in
 * "scale atoms" (src/format/layout.h:97-112, == moe_cutlass.h:42-46 SfOffset):
 * 128 rows x 4 scales per 512-byte atom, atoms along K first, rows padded to a
 * multiple of 128 with zero scales.  The atom is also the layout tcgen05.cp
 * reads, so the GEMM copies atoms unchanged. */
uint64_t llmp_b200_mxfp8_padded_rows(uint64_t rows);
uint64_t llmp_b200_mxfp8_scale_offset(uint64_t row, uint64_t block, uint64_t blocks);

/* Replaces RunMxfp8Quantize (src/kernels/ggml/llmp_ops.cu:868; kernel :610-650,
 * arithmetic mxfp8_quant.cuh:22-46).  x: F32 or BF16 [k, rows], row stride in
 * elements.  codes: rows * k bytes.  scales: padded_rows(rows) * k / 32 bytes
 * in scale atoms (the caller places them; RowsLayout of mxfp8_cutlass.h:42-49
 * puts them 256-byte aligned after the codes). */
int llmp_b200_mxfp8_quantize(const void* x, int is_bf16, int64_t row_stride, int k, int rows,
                             void* codes, void* scales, void* stream);
/* Replaces RunMxfp8Swizzle (llmp_ops.cu:895; kernel :652-663): weight scales
 * [n, k/32] row-major -> scale atoms of padded_rows(n) rows. */
int llmp_b200_mxfp8_swizzle(const void* in, void* out, int n, int blocks, void* stream);

/* Replaces RunMxfp8MulMatVec (src/kernels/ggml/llmp_ops.cu:744; kernels :145-423):
 * the decode product for up to 16 activation columns.  codes: E4M3 [k, n];
 * scales: E8M0 [k / 32, n] ROW-MAJOR (not atoms); x: F32 columns x_stride floats
 * apart; y: F32 [n] per column, y_stride floats apart. */
int llmp_b200_mxfp8_mul_mat_vec(const void* codes, const void* scales, const float* x,
                                int64_t x_stride, float* y, int64_t y_stride, int n, int k,
                                int columns, void* stream);

/* ---- The decode module's vector products (F32 activations, no Q8_1) ----
 * Replace decode::RunVector and decode::RunVectorGlu (src/kernels/decode/products.h:96-147;
 * kernels templates.cuh:116-186) for the decoders this build has: Q8_0 blocks
 * (decoders.cuh:106-125) and MXFP8 with row-major scales or scale atoms (:193-220).
 * The operand has the fields of decode::Operand (operand.h:71-93) those decoders read.
 * y[t * y_stride + j] = tensor_scale(row) * sum_k W[first + j, k] * x[t * x_stride + k] for
 * t < rows (1..16) and j < outputs, summed in the reference's order (a warp a row, lane l the
 * 16-value segments l, l + 32, ..., a butterfly over the lanes), so the F32 results are the
 * reference's bit for bit. */
#define LLMP_B200_DECODER_Q8_0_BLOCKS 0
#define LLMP_B200_DECODER_MXFP8_SPLIT 1  /* scales [rows, k / 32] row-major */
#define LLMP_B200_DECODER_MXFP8_ATOMS 2  /* scales in 128 x 4 scale atoms */
/* The vector and row products also take (decoders.cuh:73-103, 125-150, 222-239): */
#define LLMP_B200_DECODER_BF16_DENSE 3
#define LLMP_B200_DECODER_F16_DENSE 4
#define LLMP_B200_DECODER_NVFP4_SPLIT 5  /* E2M1 codes k / 2 bytes a row, UE4M3 scales k / 16 a row */
#define LLMP_B200_DECODER_NVFP4_ATOMS 6  /* the same scales in scale atoms (k % 64 == 0) */
#define LLMP_B200_DECODER_MXFP4_SPLIT 7  /* E2M1 codes, E8M0 scales k / 32 a row */
#define LLMP_B200_DECODER_MXFP4_ATOMS 8  /* the same scales in scale atoms (k % 128 == 0) */
typedef struct llmp_b200_decode_operand {
  const void* data;           /* Q8_0 blocks, or E4M3 codes */
  const void* scales;         /* MXFP8: E8M0 scales; Q8_0: unused */
  const float* tensor_scale;  /* or NULL: row r takes tensor_scale[r / rows_per_scale] */
  uint32_t k;                 /* values a row */
  uint32_t rows;              /* rows of the matrix */
  uint32_t rows_per_scale;
  uint32_t decoder;           /* LLMP_B200_DECODER_* */
  uint64_t row_bytes;         /* bytes of a row of data */
} llmp_b200_decode_operand;
typedef struct llmp_b200_decode_product {
  llmp_b200_decode_operand w;
  uint64_t first, outputs;
  const float* x;
  uint64_t rows, x_stride;    /* strides in floats */
  float* y;
  uint64_t y_stride;
} llmp_b200_decode_product;
int llmp_b200_decode_vector(const llmp_b200_decode_product* product, void* stream);
/* decode::RunRows (products.h:170-186; kernel templates.cuh:441-466): y[i, 0..k) = the decoded
 * row ids[i] of the weight times its tensor scale, for i < count (an embedding lookup).  An id
 * outside the matrix gives a zero row and sets *bad (a device int, or NULL) to 1.  y rows are
 * y_stride floats apart, 16-byte aligned. */
int llmp_b200_decode_rows(const llmp_b200_decode_operand* weight, const int32_t* ids, uint64_t count,
                          float* y, uint64_t y_stride, int32_t* bad, void* stream);
/* decode::RunMatrix with MatrixPath::kMma (products.h:116-120; tile kernel templates.cuh:
 * 236-440): any number of activation rows; weights and activations are rounded to the
 * decoder's MMA element (FP16 for Q8_0 blocks, BF16 for MXFP8: DecoderMmaElement) and
 * multiplied on the tensor cores with F32 accumulation, here tcgen05 kind::f16 over the whole
 * K in tensor memory.  Results agree with the reference's mma.sync tiles to F32 summation
 * order.  The FMA path (MatrixPath::kFma, for devices without tensor cores) is not provided. */
int llmp_b200_decode_matrix(const llmp_b200_decode_product* product, void* stream);
/* decode::RunGrouped (products.h:149-168): for each expert e, its pairs p in [offsets[e],
 * offsets[e + 1]) compute y[pair_out[p] (or p), j] = sum_k W_e[first + j, k] * x[pair_rows[p], k]
 * with the matrix product's numerics.  `format` gives the experts' decoder, k and rows (its
 * pointers are unused); `experts` is a DEVICE array of experts_count operands; offsets,
 * pair_rows and pair_out (or NULL) are device I32 arrays.  As in the reference the device
 * skips an expert whose operand is not of the format, a pair past `pairs`, and one naming a
 * row past x_rows or y_rows.  The reference's rows_hint (its tile choice) has no use here. */
typedef struct llmp_b200_decode_grouped_product {
  llmp_b200_decode_operand format;
  const llmp_b200_decode_operand* experts;
  uint64_t experts_count;
  uint64_t first, outputs;
  const int32_t* offsets;
  const int32_t* pair_rows;
  const int32_t* pair_out;
  uint64_t pairs;
  const float* x;
  uint64_t x_rows, x_stride;
  float* y;
  uint64_t y_rows, y_stride;
} llmp_b200_decode_grouped_product;
int llmp_b200_decode_grouped(const llmp_b200_decode_grouped_product* product, void* stream);
/* out[t, j] = glu(gate[t, j], up[t, j]) of rows gate_first + j and up_first + j; glu is
 * LLMP_B200_GLU_SWIGLU, _SWIGLU_CLAMP (limit) or _GEGLU (tanh): ir::GluKind 0, 3 and 2 of
 * templates.cuh:75-95; the erf GeGLU (1) is refused. */
typedef struct llmp_b200_decode_glu_product {
  llmp_b200_decode_operand gate;
  uint64_t gate_first;
  llmp_b200_decode_operand up;
  uint64_t up_first;
  uint64_t outputs;
  int glu;
  float limit;
  const float* x;
  uint64_t rows, x_stride;
  float* y;
  uint64_t y_stride;
} llmp_b200_decode_glu_product;
int llmp_b200_decode_vector_glu(const llmp_b200_decode_glu_product* product, void* stream);

/* Field for field mxfp8::Gemm (src/kernels/ggml/mxfp8_cutlass.h:56-68). */
typedef struct llmp_b200_mxfp8_gemm_desc {
  int m, n, k;
  const void* a;        /* codes, m rows of k */
  const void* a_scales; /* scale atoms */
  const void* b;        /* codes, n rows of k */
  const void* b_scales; /* scale atoms */
  void* d;              /* m rows of n */
  int bf16;             /* D in BF16, else F32 */
  void* scratch;        /* llmp_b200_mxfp8_gemm_scratch() bytes (0: may be NULL) */
} llmp_b200_mxfp8_gemm_desc;

/* Replace mxfp8::Available / Scratch / Run (mxfp8_cutlass.h:70-79): D[m,n] =
 * A[m,k] . B[n,k]^T with F32 accumulation on tcgen05 (kind::mxf8f6f4
 * block_scale).  k % 128 == 0.  sms <= 0: every SM of the device. */
int llmp_b200_mxfp8_gemm_available(void);
size_t llmp_b200_mxfp8_gemm_scratch(const llmp_b200_mxfp8_gemm_desc* gemm, int sms);
int llmp_b200_mxfp8_gemm(const llmp_b200_mxfp8_gemm_desc* gemm, int sms, void* stream);
/* The same product by a named kernel: 0 the rule llmp_b200_mxfp8_gemm follows (CTA pairs once
 * m exceeds one 128-row tile), 1 one CTA a 128 x 192 tile, 2 a pair of CTAs (cta_group::2) a
 * 256 x 192 tile.  The kernels accumulate a tile's k-steps in the same order, so their
 * results are the same bits; the entry exists for measurement and tests. */
int llmp_b200_mxfp8_gemm_variant(const llmp_b200_mxfp8_gemm_desc* gemm, int sms, int variant,
                                 void* stream);
/* How many CTA pairs of the pair kernel the current device holds at once (0: none). */
int llmp_b200_mxfp8_gemm_resident_pairs(void);

#ifdef __cplusplus
}
#endif
#endif /* LLMP_B200_H_ */
