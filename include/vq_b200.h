/*
 * C ABI of the B200 (sm_100a) quantized-ops library, libvq_b200.so.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*), launches on that stream and returns 0 on success or a
 * negative VQ_E* code; vq_last_error() then describes the failure.  Nothing
 * here synchronises the device or allocates device memory unless stated.
 * Inputs are never written.  Tensors are dense row-major unless stated.
 *
 * Each declaration names the operator of the reference project
 * (voyager_compiler, paths relative to its checkout) whose arithmetic the
 * entry point reproduces bit for bit.
 */
#ifndef VQ_B200_H
#define VQ_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* storage dtypes of tensors crossing the ABI */
enum { VQ_BF16 = 0, VQ_F16 = 1, VQ_F32 = 2 };

/* error codes */
enum {
  VQ_OK = 0,
  VQ_EINVAL = -1,     /* bad argument (shape, dtype, alignment, mode) */
  VQ_ECUDA = -2,      /* a CUDA runtime/driver call failed */
  VQ_EUNSUPPORTED = -3,
  VQ_ETIMEOUT = -4    /* a bounded device-side wait ran out */
};

/*
 * How a value is rounded onto a format's grid.  VQ_ROUND_TABLE gathers from
 * the caller's 65 536-entry bfloat16 table (always exact for any table); the
 * other modes are arithmetic forms that the host selects only after checking
 * that they reproduce the supplied table on all 65 536 bfloat16 inputs.
 */
enum {
  VQ_ROUND_NONE = 0,      /* keep the scaled value */
  VQ_ROUND_TABLE = 1,     /* table[bits(bf16(v))] */
  VQ_ROUND_INT = 2,       /* clamp(rint(v), lo, hi), zero keeps its sign */
  VQ_ROUND_MINIFLOAT = 3, /* saturating RNE onto an (emin, mbits, max) grid */
  VQ_ROUND_STEPS = 4,     /* <= 32 levels: threshold search on the bf16 bits */
  VQ_ROUND_SEARCH = 5,    /* searchsorted over float edges (codebook encode) */
  VQ_ROUND_STOCHASTIC = 6 /* Philox stochastic rounding between sorted levels */
};

#define VQ_MAX_STEPS 32

typedef struct VqRound {
  int32_t mode;
  const void* table;      /* TABLE: device uint16[65536] (bf16 bits) */
  float lo, hi;           /* INT: bounds */
  int32_t emin, mbits;    /* MINIFLOAT: min normal exponent, mantissa bits */
  float max_norm;         /* MINIFLOAT: saturation magnitude */
  int32_t is_signed;      /* MINIFLOAT: 0 takes |v| first */
  /* STEPS: device uint16[2 * n_steps]: first n_steps exclusive upper keys (in
     the value-ordered key space of bf16 bit patterns: negatives below
     positives), then n_steps level values as bf16 bits.  Level k is chosen for
     keys in [key[k-1], key[k]); nan_value is the result for a NaN input. */
  int32_t n_steps;
  const void* steps;
  uint16_t nan_value;
  /* SEARCH / STOCHASTIC: device float arrays */
  const float* edges;     /* SEARCH: ascending edges, result = #edges < v */
  const float* levels;    /* SEARCH (optional: value per index) / STOCHASTIC */
  int32_t n_edges;
  int32_t n_levels;
  const int64_t* seed;    /* STOCHASTIC: device int64 scalar */
} VqRound;

/* Broadcast geometry of a per-block parameter tensor against a dense input
 * viewed as up to VQ_MAX_DIMS collapsed dimensions (outermost first):
 * parameter index = sum_d (coord_d / div[d]) * stride[d]. */
#define VQ_MAX_DIMS 5
typedef struct VqBroadcast {
  int32_t ndim;
  int64_t size[VQ_MAX_DIMS];
  int64_t div[VQ_MAX_DIMS];
  int64_t stride[VQ_MAX_DIMS];
} VqBroadcast;

const char* vq_last_error(void);
int vq_version(void);

/* quantized_ops::vmap -- src/voyager_compiler/ops/quantized.py:151-184.
 * out[i] = T(table[bits(bf16(in[i]))]); in/out are n elements of `dtype`. */
int vq_vmap(const void* in, void* out, int dtype, const VqRound* round, int64_t n, void* stream);

/* quantized_ops::quantize -- ops/quantized.py:458-515 (with repeat_per_block
 * :124-144).  out = round(in / scale [+ zero_point]) with every step rounded to
 * `dtype`.  `zero_point` may be NULL.  `geom` maps an element to its scale.
 * `param_dtype` is the dtype of scale and zero_point: equal to `dtype`, or
 * VQ_F32 for a single-element scale used at full precision. */
int vq_quantize(const void* in, const void* scale, const void* zero_point, void* out, int dtype,
                int param_dtype, const VqBroadcast* geom, const VqRound* round, void* stream);

/* quantized_ops::dequantize -- ops/quantized.py:527-571.
 * out = round_out((round_in(in) - zero_point) * scale). */
int vq_dequantize(const void* in, const void* scale, const void* zero_point, void* out, int dtype,
                  int param_dtype, const VqBroadcast* geom, const VqRound* round_in,
                  const VqRound* round_out, void* stream);

/* Packed integer codes for a 2-bit (or 4-bit) KV cache: the storage form of the
 * codes quantized_ops::quantize_affine yields for a KIVI cache
 * (examples/language_modeling/quantization_configs.py:171-207; the reference keeps
 * them as bfloat16-valued tensors and its quant_folding pass,
 * codegen/transform/quant_folding.py:2391-2547, reads them back through one fused
 * dequantize).  Element i of the row-major tensor sits in byte i / (8 / bits) at
 * bit bits * (i % (8 / bits)).
 *
 * vq_pack_codes: `codes` holds n integers in [0, 2^bits) as values of `dtype`.
 * vq_unpack_dequantize: out = round_out((code - zero_point) * scale), bit for bit
 * what vq_dequantize gives on the unpacked codes (the fused decode + re-encode of
 * quant_folding.py:2524-2527 when round_out is the re-encoding table); geom,
 * param_dtype and the roundings are as for vq_dequantize; `dtype` is out's. */
int vq_pack_codes(const void* codes, int dtype, void* packed, int bits, int64_t n, void* stream);
int vq_unpack_dequantize(const void* packed, int bits, const void* scale, const void* zero_point, void* out,
                         int dtype, int param_dtype, const VqBroadcast* geom, const VqRound* round_out,
                         void* stream);

/* Outlier side stream -- quantized_ops::filter_outlier (ops/quantized.py:1323-1373)
 * and quantized_ops::spmm_csr (:1574-1644), built on the device with no host read
 * (the reference calls .item() and is not graph-capturable).
 *
 * An element is an outlier when |x| >= threshold (threshold already rounded to the
 * tensor's dtype).  Per [rows, cols] matrix the stored outliers (zero values are not
 * stored) form a CSR matrix of fixed capacity: data / indices hold `capacity` entries
 * (caller pre-fills 0 and -1), entries beyond the capacity are dropped in row-major order.
 *
 * vq_outlier_count: counts[row] for the [rows_total, cols] view of the input.
 * vq_outlier_fill: row_start is [batches, rows + 1], the exclusive prefix sums of the
 *   counts per matrix (not clamped); writes data, indices and inlier = x with outliers zeroed.
 * vq_spmm_csr: out[b][r][n] = sum_e data[b][e] * B[b][indices[b][e]][n] over row r's
 *   entries, float32 accumulation in entry order, rounded to out_dtype.  Row pointers are
 *   rebased on indptr[b][0] and clamped to the stored span; B element (k, n) of batch b is
 *   at B[b * strideB + k * ld_k + n * ld_n] (strideB = 0 shares one B). */
int vq_outlier_count(const void* in, int dtype, int32_t* counts, int64_t rows_total, int64_t cols, float threshold,
                     void* stream);
int vq_outlier_fill(const void* in, int dtype, void* inlier, void* data, int32_t* indices, const int32_t* row_start,
                    int64_t batches, int64_t rows, int64_t cols, float threshold, int64_t capacity, void* stream);
int vq_spmm_csr(const void* data, int data_dtype, const int32_t* indices, const int32_t* indptr, const void* B,
                int b_dtype, void* out, int out_dtype, int64_t batches, int64_t rows, int64_t N, int64_t K,
                int64_t capacity, int64_t strideB, int64_t ld_k, int64_t ld_n, void* stream);

/* Microscaling block geometry: the input is a dense [O, A, M, B, I] tensor
 * whose blocks span block_a consecutive indices of A and block_b of B (1 =
 * axis not blocked); scales are dense [O, ceil(A/block_a), M, ceil(B/block_b), I]. */
typedef struct VqBlocks {
  int64_t O, A, M, B, I;
  int32_t block_a, block_b;
} VqBlocks;

/* Scale rule of calculate_mx_qparam -- ops/quantized.py:966-1031 with
 * quantization/mx_utils.py:16-125. */
typedef struct VqScaleRule {
  float quant_max;
  int32_t power_of_two;       /* 2**(floor(log2 amax) - floor(log2 quant_max)) */
  const void* global_scale;   /* device scalar, or NULL */
  int32_t global_scale_dtype; /* its dtype */
  VqRound scale_round;        /* rounding of the scale (NONE or a table form) */
} VqScaleRule;

/* quantized_ops::calculate_mx_qparam -- ops/quantized.py:966-1031. */
int vq_mx_qparam(const void* in, void* scale_out, int dtype, const VqBlocks* blocks,
                 const VqScaleRule* rule, void* stream);

/* quantized_ops::quantize_mx -- ops/quantized.py:1080-1115: per-block scale,
 * then codes = round(in / (scale [* global_scale])). */
int vq_quantize_mx(const void* in, void* scale_out, void* codes_out, int dtype, const VqBlocks* blocks,
                   const VqScaleRule* rule, const VqRound* round, void* stream);

/* quantized_ops::quantize_affine -- ops/quantized.py:1227-1283: per-block
 * min/max -> scale and zero point (optionally table-rounded) -> codes.
 * Blocks lie along B only (block_a must be 1). */
int vq_quantize_affine(const void* in, void* scale_out, void* zero_out, void* codes_out, int dtype,
                       const VqBlocks* blocks, float quant_min, float quant_max,
                       const VqRound* scale_round, const VqRound* round, void* stream);

/* quantized_ops::dequantize_mx / _decode_and_scale -- ops/quantized.py:574-591,
 * 1125-1149.  out = code[in] * scale [* global_scale]; `code` (n_code entries of
 * `dtype`), `scale` and `global_scale` may each be NULL. */
int vq_dequantize_mx(const void* in, const void* scale, const void* code, int32_t n_code,
                     const void* global_scale, int global_scale_dtype, void* out, int dtype,
                     const VqBroadcast* geom, void* stream);

/* max |x| over n elements, written as a float to *out (device).  The amax
 * that calculate_global_scale (quantization/fake_quantize.py:142-160) and the
 * per-tensor scale rule (fake_quantize.py:406-437) start from.  `out` must
 * be zeroed by the caller; NaN inputs give NaN. */
int vq_amax(const void* in, int dtype, int64_t n, float* out, void* stream);

/* One step of the delayed-scaling observer, FusedAmaxObsFakeQuantize._update_amax_scale
 * (quantization/fake_quantize.py:406-437), on device state.  ring: [length, channels] of
 * `dtype`, the last `length` absolute maxima per channel in ring order; position: [channels]
 * int32, where each channel writes next (start both zeroed); scale: [channels] of `dtype`
 * (start at 1).  The call sets scale from the ring as it stood before this tensor
 * (max / quant_max in `dtype`; unchanged while that max is 0, infinite or NaN; rounded up to a
 * power of two when power_of_two != 0), then stores this tensor's amax (one value of
 * amax_dtype shared by all channels when amax_count == 1, else one per channel) and advances
 * the ring.  No host state: the call can be captured in a CUDA graph. */
int vq_amax_history_update(void* ring, int dtype, int64_t length, int64_t channels, int32_t* position,
                           const void* amax, int amax_dtype, int64_t amax_count, float quant_max,
                           int power_of_two, void* scale, void* stream);

/* hadamard_rotate -- ops/quantized.py:1038-1067: each run of 16 elements along the
 * middle axis of a dense [O, A, I] tensor is multiplied by the float32 16x16
 * `matrix` (device, row-major; out_j = sum_k in_k * matrix[k][j]) in fp32; A is
 * zero padded to a multiple of 16 and `out` is dense [O, ceil16(A), I]. */
int vq_hadamard_rotate(const void* in, void* out, int dtype, const float* matrix, int64_t O, int64_t A,
                       int64_t I, void* stream);

/* One block of the GPTQ column sweep -- quantization/gptq.py: block_scale (85-143)
 * and quantize_block (189-220), as compensate_weight (223-308) calls them.
 * work/out are fp32 [rows, K]; columns [start, start+n) (n <= 128) are rounded one
 * by one against each row's scale, errors over the pivots of U (fp32 [K, K], the
 * upper Cholesky factor of the inverse Hessian) are propagated inside the block and
 * written to deltas (fp32 [rows, n]).  affine = 0: microscaling scale amax/quant_max
 * through scale_round (shrink = 1 adds the reference's five-candidate search, weighted
 * by salience[K]); affine = 1: group-wise affine scale and zero point
 * (ops/quantized.py:1268-1281 applied to the block), which the reference's GPTQ lacks. */
int vq_gptq_block(float* work, float* out, float* deltas, const float* U, const float* salience,
                  int64_t rows, int64_t K, int64_t start, int64_t n, int affine, float quant_min,
                  float quant_max, int shrink, const VqRound* scale_round, const VqRound* round,
                  void* stream);

/* The trailing update of compensate_weight (quantization/gptq.py:302-303):
 * work[:, start+n:] -= deltas @ U[start:start+n, start+n:], fp32, products summed in
 * ascending column order. */
int vq_gptq_update(float* work, const float* deltas, const float* U, int64_t rows, int64_t K,
                   int64_t start, int64_t n, void* stream);

/* One whole GPTQ block step (vq_gptq_block followed by vq_gptq_update) that needs
 * no buffer for the per-column errors and performs no allocation of any kind.
 * It has no counterpart in the reference.  It is meant for hosts that cannot
 * allocate device memory while they run: a runtime working inside a fixed,
 * fully planned arena, or a plugin in a process that forbids cudaMalloc after
 * start-up.  The errors are kept in an 8 MiB array built into the library
 * (resident on every GPU that loads it, until the process exits), so
 * rows * n must not exceed 2 097 152 values (for example 16 384 rows of a
 * 128-column block); larger calls fail with VQ_EINVAL and a message saying so.
 * The first call on a device looks up the array's address (cudaGetSymbolAddress)
 * with that device current; make that first call before any stream capture.
 * All calls on a device share the array: calls that may overlap on the GPU
 * (different streams without ordering between them) race on it and must be
 * serialised by the caller.  Inputs, outputs and stream are as for
 * vq_gptq_block. */
int vq_gptq_block_step_static(float* work, float* out, const float* U, const float* salience,
                              int64_t rows, int64_t K, int64_t start, int64_t n, int affine,
                              float quant_min, float quant_max, int shrink, const VqRound* scale_round,
                              const VqRound* round, void* stream);

/* operand element kinds of the tensor-core GEMM */
enum { VQ_IN_BF16 = 0, VQ_IN_F16 = 1, VQ_IN_E4M3 = 2, VQ_IN_E5M2 = 3 };

/* The contraction of quantized_ops::linear_mx / matmul_mx (ops/quantized.py:662-805,
 * through quantized_ops::linear / matmul, ops/layout.py:231-284) and of the
 * real-FP8 linear (backend/gpu/fp8.py:372-429):
 *   C[b][m][n] = round(alpha * sum_k A[b][m][k] * B[b][n][k] + bias[n])
 * A is [batch, M, K] and B is [batch, N, K], both K-contiguous with leading
 * dimensions lda / ldb and batch strides strideA / strideB (in elements; a
 * batch stride of 0 shares the operand).  Products are accumulated in fp32 on
 * the tensor cores; alpha (device scalar, may be NULL) and bias (device [N],
 * may be NULL) are applied in fp32 as two separately rounded operations; the
 * result is rounded once to out_dtype.  Operand pointers, leading dimensions
 * and batch strides must be multiples of 16 bytes. */
int vq_gemm_tn(const void* A, const void* B, void* C, int in_kind, int out_dtype, int64_t M, int64_t N,
               int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t batch, int64_t strideA,
               int64_t strideB, int64_t strideC, const void* alpha, int alpha_dtype, const void* bias,
               int bias_dtype, void* stream);

/* vq_gemm_tn with a richer epilogue.  alpha_cols (device [N] of alpha_cols_dtype,
 * may be NULL) multiplies column n after alpha and before the bias: the
 * per-output-channel scale of fp8_linear (backend/gpu/fp8.py:372-400, scale
 * [1, N]), and what lets linears that share an input and differ in their
 * per-tensor scales run as one GEMM.  residual (device [batch, M, N] of the
 * output dtype with leading dimension ldr and batch stride strideR, may be NULL,
 * must not alias C) is added after the rounding to out_dtype and the sum is
 * rounded again, which is `x + linear(...)` of a decoder layer in one pass.
 * causal_mode / causal_period describe the two matmuls of causal attention, where
 * row r of A and C belongs to position t = r % causal_period of a sequence:
 *   1  elements C[r][n] with n > t are never read by the caller (the masked scores
 *      of Q K^T): tiles made only of such elements may be left unwritten;
 *   2  A[r][k] is zero for k > t (the probabilities of P V): the contraction of a
 *      tile may stop after the largest t among its rows.
 * Both are permissions, not requests: results the caller may read are unchanged.
 * gate_scale (device scalar of gate_scale_dtype, may be NULL) selects the gated
 * (SwiGLU) epilogue for a B whose rows interleave 32 rows of the gate projection
 * with the matching 32 rows of the up projection: C is then [batch, M, N / 2]
 * e4m3 bytes (ldc and strideC in bytes, rows 16-byte aligned) holding
 *   e4m3(bf16(bf16(bf16(silu(g)) * u) / gate_scale)),  g, u = bf16(alpha * alpha_cols * acc)
 * -- gate/up linears, SiLU, product and the FP8 cast of the next linear's input
 * (backend/gpu/fp8.py:253-261) in one kernel, with every bfloat16 rounding of the
 * unfused sequence.  out_dtype must be VQ_BF16, N a multiple of 64, no bias or residual.
 * round_acc != 0 rounds the float32 accumulator to out_dtype before alpha, alpha_cols and
 * the bias are applied: the two roundings of a converted per-tensor graph, which runs
 * `aten.linear` / `aten.matmul` on the codes (one rounding to the tensor dtype) and then
 * `dequantize` by s_a * s_w (a second one; quantization/quantize_pt2e.py:563-626).  With
 * round_acc == 0 the product is rounded once, as fp8_linear's scaled GEMM does
 * (backend/gpu/fp8.py:372-400).
 * epi == NULL is vq_gemm_tn. */
typedef struct VqGemmEpilogue {
  const void* alpha_cols;
  int32_t alpha_cols_dtype;
  const void* residual;
  int64_t ldr, strideR;
  int32_t causal_mode;
  int64_t causal_period;
  const void* gate_scale;
  int32_t gate_scale_dtype;
  int32_t round_acc;
} VqGemmEpilogue;
int vq_gemm_tn_ex(const void* A, const void* B, void* C, int in_kind, int out_dtype, int64_t M, int64_t N,
                  int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t batch, int64_t strideA,
                  int64_t strideB, int64_t strideC, const void* alpha, int alpha_dtype, const void* bias,
                  int bias_dtype, const VqGemmEpilogue* epi, void* stream);

/* The contraction of linear_mx / matmul_mx (ops/quantized.py:662-805) taken straight from
 * the block-scaled operands: C = alpha * (bf16(A * a_scale) . bf16(B * b_scale)^T) + bias with
 * A [batch, M, K] and B [batch or 1, N, K] bfloat16 codes, K contiguous, and one bfloat16 scale
 * per `block_size` consecutive elements of K ([batch, M, ceil(K / block_size)] and
 * [batch or 1, N, ceil(K / block_size)], contiguous; a null scale pointer takes that operand
 * as it is).  The product code * scale is rounded to bfloat16 once, as _decode_and_scale
 * (ops/quantized.py:574-591) does, but inside the GEMM's main loop: the dequantized
 * operands are never written to device memory.  block_size is a power of two >= 8.
 * Alignment rules, alpha and bias as vq_gemm_tn.  VQ_EUNSUPPORTED on a device that cannot
 * co-schedule CTA pairs (the caller then dequantizes and calls vq_gemm_tn). */
int vq_gemm_mx(const void* A, const void* a_scale, const void* B, const void* b_scale, int64_t block_size, void* C,
               int out_dtype, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t batch,
               int64_t strideA, int64_t strideB, int64_t strideC, const void* alpha, int alpha_dtype,
               const void* bias, int bias_dtype, void* stream);

/* Real FP8 codes for the tensor-core GEMM, the cast the reference's GPU backend
 * makes before torch._scaled_mm (backend/gpu/fp8.py:253-309): out[i] is the
 * e4m3 / e5m2 byte of round_bf16(in[i] / scale), i.e. the byte encoding of the
 * value quantized_ops::quantize (ops/quantized.py:458-515) yields with that
 * format's table.  `in` is bfloat16, `format` VQ_IN_E4M3 or VQ_IN_E5M2, `scale`
 * holds one element (elems_per_scale = 0) or one per elems_per_scale consecutive
 * elements (a multiple of 16; per-row scales of a weight).  n must be a multiple
 * of 16 and both buffers 16-byte aligned. */
int vq_quantize_fp8(const void* in, const void* scale, int scale_dtype, void* out, int format, int64_t n,
                    int64_t elems_per_scale, void* stream);

/* Attention probabilities as FP8 codes in one pass over the scores: per row,
 *   s = bf16(score * score_scale); s = bf16(s + mask[row % mask_rows]);
 *   p = bf16(softmax_fp32(s)); out = fp8(bf16(p / out_scale))
 * -- the scale / mask / softmax / quantize sequence between the two attention
 * matmuls of an eager-attention graph (ops/quantized.py:900-925 has the same
 * sequence inside sdpa_mx), whose last step is the FP8 cast of
 * backend/gpu/fp8.py:253-309.  scores: bfloat16 [rows, cols]; out: bytes
 * [rows, cols]; mask: bfloat16 [mask_rows, cols] or NULL; causal_period T > 0
 * additionally masks columns > (row % T) without reading them.  cols must be a
 * multiple of 8 and at most 4096. */
int vq_softmax_quantize_fp8(const void* scores, void* out, int64_t rows, int64_t cols, float score_scale,
                            const void* mask, int64_t mask_rows, int64_t causal_period,
                            const void* out_scale, int out_scale_dtype, int format, void* stream);

/* Causal self-attention of a per-tensor FP8 decoder layer in one kernel: the two
 * attention matmuls (backend/gpu/fp8.py:253-309, fp8_bmm) with the scale / causal
 * mask / softmax / FP8 cast of the probabilities between them and the FP8 cast
 * of the context after them, every bfloat16 rounding of the separate operators
 * kept:
 *   scores = bf16(q8 k8^T * alpha_qk); s = bf16(scores * score_scale), keys > query masked
 *   p8 = e4m3(bf16(bf16(softmax_fp32(s)) / p_scale))
 *   ctx = bf16(p8 v8 * alpha_pv); out8 = e4m3(bf16(ctx / ctx_scale))
 * With round_acc != 0 both products are first rounded to bfloat16 and then scaled,
 * scores = bf16(bf16(q8 k8^T) * alpha_qk) and ctx = bf16(bf16(p8 v8) * alpha_pv): the
 * matmul-then-dequantize pair of a converted graph (see VqGemmEpilogue.round_acc).
 * q8: e4m3 [kv_heads, groups * T, 128], the query heads of a KV group stacked
 * along the rows; k8: e4m3 [kv_heads, T, 128]; vt8: e4m3 [kv_heads, 128, T].
 * out8 (or NULL): e4m3 [T, ld8], head h = kv * groups + g at columns [128 h, +128);
 * out16 (or NULL): bfloat16 ctx [kv_heads, groups * T, 128].  The scalars are
 * device pointers of the given dtypes.  head_dim must be 128 and T a multiple of
 * 128, else VQ_EUNSUPPORTED.  vq_attention_status reports (and optionally
 * clears) VQ_ETIMEOUT if a wait inside the kernel ran out; it synchronises. */
int vq_attention_fp8(const void* q8, const void* k8, const void* vt8, void* out8, int64_t ld8, void* out16,
                     int64_t T, int64_t kv_heads, int64_t groups, int64_t head_dim, const void* alpha_qk,
                     int alpha_qk_dtype, float score_scale, const void* p_scale, int p_scale_dtype,
                     const void* alpha_pv, int alpha_pv_dtype, const void* ctx_scale, int ctx_scale_dtype,
                     int round_acc, void* stream);
int vq_attention_status(int reset);

/* Causal self-attention on bfloat16 operands in one kernel: the matmul / scale + mask / softmax /
 * matmul nodes of an eager attention in a converted graph whose attention matmuls stay in
 * bfloat16 (the recipes that quantize only the linears: aten.matmul or quantized_ops::matmul,
 * ops/layout.py:281-290, around aten.softmax), every bfloat16 rounding of the separate nodes kept:
 *   scores = bf16(q k^T); s = bf16(scores * score_scale), keys > query masked
 *   p = bf16(softmax_fp32(s)); out = bf16(p v)
 * (round_acc == 0 skips the first rounding: the scores stay in float32 until they are scaled).
 * q: [kv_heads, groups * T, 128], the query heads of a KV group stacked along the rows;
 * k: [kv_heads, T, 128]; vt: [kv_heads, 128, T] (V transposed); out: [T, ldo] with head
 * h = kv * groups + g at columns [128 h, +128).  head_dim must be 128 and T a multiple of 128,
 * else VQ_EUNSUPPORTED.  The score and probability matrices never leave the SM.
 * vq_attention_status covers this kernel too. */
int vq_attention_bf16(const void* q, const void* k, const void* vt, void* out, int64_t ldo, int64_t T,
                      int64_t kv_heads, int64_t groups, int64_t head_dim, float score_scale, int round_acc,
                      void* stream);

/* RMSNorm's backward of a training step: the input gradient (plus the residual stream's) and
 * the weight gradient from one read of the rows -- the operator
 * voyager_gpu::rmsnorm_backward(Tensor[] gradients, Tensor x, Tensor rsqrt, Tensor weight,
 * Tensor? residual) -> (Tensor, Tensor) of backend/gpu/rmsnorm.py:133-182, whose Triton kernels
 * (:56-135) this replaces with the same rounding steps: dy = the gradients summed (bfloat16 after
 * each addition), dw = sum over rows of bf16(dy * bf16(x * r)), g = bf16(dy * w),
 * dx = bf16(g * r + (sum_k g x * -0.5 * r^3 / cols) * 2 x) (+ residual).  All row tensors are
 * contiguous bfloat16 [rows, cols]; rsqrt_rows float32 [rows]; weight and dw bfloat16 [cols];
 * dy1, dy2 and residual may be NULL (gradients = 1..3).  partial_dw is scratch of
 * vq_rmsnorm_backward_programs(rows, cols) * cols floats.  cols: a multiple of 8, at most 8192. */
int64_t vq_rmsnorm_backward_programs(int64_t rows, int64_t cols);
int vq_rmsnorm_backward(const void* dy0, const void* dy1, const void* dy2, int gradients, const void* x,
                        const float* rsqrt_rows, const void* weight, const void* residual, void* dx,
                        float* partial_dw, void* dw, int64_t rows, int64_t cols, void* stream);

/* SwiGLU in bfloat16 with the tensor-wide amax the next cast needs: out = bf16(bf16(silu(gate)) * up) for
 * gate / up [rows, cols] with row strides ld_gate / ld_up (the halves of a merged projection's output need no
 * copy), out [rows, cols] dense, and *amax (float32, zero on entry) raised to max |out| by atomicMax -- aten.silu,
 * aten.mul and the amax of calculate_global_scale (quantization/fake_quantize.py:142-160) in one pass. */
int vq_silu_mul_amax(const void* gate, const void* up, void* out, void* amax, int64_t rows, int64_t cols,
                     int64_t ld_gate, int64_t ld_up, void* stream);

/* Rotate-half RoPE of x [T, heads, d] (bfloat16; element (t, h, j) at x + t * in_stride_t + h * in_stride_h + j,
 * so a slice of a merged projection's output needs no copy) written to out + h * out_stride_h + t * out_stride_t
 * + j: head-major for the attention kernel.  cos / sin: bfloat16 [T, d].  y = bf16(bf16(x * cos) + bf16(rot(x) *
 * sin)), rot(x) = (-x[d/2:], x[:d/2]): the graph's mul / cat / neg / add nodes with their roundings. */
int vq_rope_heads_bf16(const void* x, const void* cosv, const void* sinv, void* out, int64_t T, int64_t heads, int64_t d,
                       int64_t in_stride_t, int64_t in_stride_h, int64_t out_stride_t, int64_t out_stride_h,
                       void* stream);

/* One decode step's RoPE and cache append on the merged q/k/v projection qkv [B, (q_heads + 2 kv_heads) * d]
 * (bfloat16): query head h, rotated, to q_out [B, q_heads, d]; key head h, rotated, to
 * k_dst + (b * kv_heads + h) * kv_stride; value head h, unchanged, to v_dst + (b * kv_heads + h) * kv_stride
 * -- k_dst / v_dst point at this step's slot of a [B, kv_heads, R, d] window, kv_stride = R * d elements.
 * cos / sin: bfloat16 [d] shared by all sequences (cs_stride = 0) or one row per sequence (cs_stride elements
 * apart).  y = bf16(bf16(x * cos) + bf16(rot(x) * sin)), rot(x) = (-x[d/2:], x[:d/2]): HF rotate_half
 * RoPE as the graph's mul / cat / neg / add nodes compute it, then the index-copy of the cache update. */
int vq_rope_decode_append(const void* qkv, const void* cosv, const void* sinv, void* q_out, void* k_dst, void* v_dst,
                          int64_t B, int64_t q_heads, int64_t kv_heads, int64_t d, int64_t kv_stride,
                          int64_t cs_stride, void* stream);

/* A per-tensor e4m3 cast applied and undone, plus an optional addend, in one pass:
 *   out = bf16(dequantize(quantize(x, scale, qmap = fp8_e4m3), scale) + y)
 * -- the quantize -> dequantize pair a converted graph puts on a residual stream
 * (quantized_ops::quantize / ::dequantize, ops/quantized.py:458-571) followed by aten.add, with each
 * node's bfloat16 rounding: q = e4m3(bf16(x / s)) saturating at 448, d = bf16(q * s), out = bf16(d + y).
 * x, y (or NULL), out: bfloat16, n elements (a multiple of 8), 16-byte aligned. */
int vq_fp8_roundtrip_add(const void* x, const void* y, void* out, int64_t n, const void* scale, int scale_dtype,
                         void* stream);

/* FP8 casts fused with the bfloat16 operation that feeds them in a per-tensor FP8
 * decoder layer.  The reference's converted graph runs the producer (RMSNorm,
 * rotary embedding, SiLU * up, a transpose) as separate aten nodes and then
 * quantized_ops::quantize (ops/quantized.py:458-515), whose FP8 byte form is
 * backend/gpu/fp8.py:253-261; its one fused cast is the cast + transpose of
 * backend/gpu/fp8.py:272-369.  Each entry keeps the
 * bfloat16 roundings of the unfused sequence and writes e4m3 bytes of
 * round_bf16(y / scale); scale holds one element of scale_dtype.  All inputs are
 * bfloat16, contiguous and 16-byte aligned.
 *
 * vq_rmsnorm_quantize_fp8: y = bf16(x * rsqrt(mean(x^2) + eps) * weight), x [rows, cols],
 *   cols a multiple of 8 and at most 8192.
 * vq_silu_mul_quantize_fp8: y = bf16(bf16(silu(gate)) * up); gate / up are [rows, cols]
 *   with row strides ld_gate / ld_up (two halves of one merged projection's output),
 *   out is dense; cols and the strides are multiples of 8.
 * vq_rope_quantize_fp8: element (t, h, j) of a [T, heads, d] activation is read at
 *   x[t * in_stride_t + h * in_stride_h + j] and its byte written at
 *   out[t * out_stride_t + h * out_stride_h + j] (strides in elements, multiples of 8),
 *   so one call also moves between token-major [T, heads, d] and head-major
 *   [heads, T, d] layouts.  cos / sin are [T, d] or both NULL (no rotation);
 *   y = bf16(bf16(x * cos) + bf16(rotate_half(x) * sin)).  d must be a multiple of 16.
 * vq_transpose_quantize_fp8: x [T, heads, d] with ldx elements between consecutive t
 *   (heads * d when dense) -> out bytes [heads, d, T] (the value
 *   operand of P @ V as a K-major B matrix; heads = 1 is the matrix transpose of
 *   quantize_fp8_transpose, backend/gpu/fp8.py:342-369).  codes, if not NULL, also
 *   receives the bytes in x's own layout; amax_bits, if not NULL, is an int32 the
 *   caller has zeroed that is raised to the bfloat16 bit pattern of max |x| (NaN
 *   orders above every number).  format is VQ_IN_E4M3 or VQ_IN_E5M2; no alignment
 *   or divisibility requirement. */
int vq_rmsnorm_quantize_fp8(const void* x, const void* weight, void* out, int64_t rows, int64_t cols, float eps,
                            const void* scale, int scale_dtype, void* stream);
int vq_silu_mul_quantize_fp8(const void* gate, const void* up, void* out, int64_t rows, int64_t cols,
                             int64_t ld_gate, int64_t ld_up, const void* scale, int scale_dtype, void* stream);
int vq_rope_quantize_fp8(const void* x, const void* cosv, const void* sinv, void* out, int64_t T, int64_t heads,
                         int64_t d, int64_t in_stride_t, int64_t in_stride_h, int64_t out_stride_t,
                         int64_t out_stride_h, const void* scale, int scale_dtype, void* stream);
/* The three casts between a merged q/k/v projection and vq_attention_fp8 as one launch: vq_rope_quantize_fp8 of the
 * query heads q [T, q_heads, d] and of the key heads k [T, kv_heads, d] (head-major e4m3 outputs [heads, T, d]) and
 * vq_transpose_quantize_fp8 of the value heads v [T, kv_heads, d] (vt_out [kv_heads, d, T]); q, k and v are bfloat16
 * column slices of one matrix with `ld` elements between tokens, cos / sin are [T, d] bfloat16, each scale holds one
 * element.  Results equal the three separate calls bit for bit.  d % 16 == 0, ld % 8 == 0, 16-byte aligned inputs. */
int vq_qkv_post_fp8(const void* q, const void* k, const void* v, int64_t ld, const void* cosv, const void* sinv,
                    void* q_out, void* k_out, void* vt_out, int64_t T, int64_t q_heads, int64_t kv_heads, int64_t d,
                    const void* q_scale, int q_scale_dtype, const void* k_scale, int k_scale_dtype,
                    const void* v_scale, int v_scale_dtype, void* stream);
int vq_transpose_quantize_fp8(const void* x, void* out, void* codes, void* amax_bits, int format, int64_t T,
                              int64_t heads, int64_t d, int64_t ldx, const void* scale, int scale_dtype,
                              void* stream);

/* NVFP4 operands for the block-scaled GEMM, the cast of the reference's
 * backend/gpu/nvfp4.py (cast_nvfp4:683-739, _cast_tile:262-372): codes are e2m1,
 * two per byte (even element in the low nibble), rows of K/2 bytes; scales are
 * e4m3 bytes, one per 16 elements, in 512-byte tiles of 128 rows x 4 scales
 * (byte (r%32)*16 + (r/32)*4 + s of tile row_block * K/64 + k64_block).
 * vq_nvfp4_scale_bytes gives the size of that buffer, which the caller zeroes
 * when rows is not a multiple of 128.  K must be a multiple of 64.
 *
 * vq_quantize_nvfp4 casts bfloat16 [rows, K] with the arithmetic of
 * quantized_ops::quantize_mx (ops/quantized.py:1080-1115) for an e2m1 table,
 * an e4m3 scale table, quant_max 6 and the given global scale (device scalar).
 * vq_pack_nvfp4 packs that operator's own outputs (bfloat16-valued codes
 * [rows, K], bfloat16 scales [rows, K/16]) and sets *bad_flag (device int) to 1
 * if a value is not representable (pack_nvfp4, backend/gpu/nvfp4.py:1045-1091). */
int64_t vq_nvfp4_scale_bytes(int64_t rows, int64_t K);
int vq_quantize_nvfp4(const void* in, const void* global_scale, int global_scale_dtype, void* codes,
                      void* scales, int64_t rows, int64_t K, void* stream);
int vq_pack_nvfp4(const void* codes_in, const void* scales_in, void* codes, void* scales, int64_t rows,
                  int64_t K, int* bad_flag, void* stream);

/* NVFP4 linear on the tensor cores' native block-scaled MMA (nvfp4_linear,
 * backend/gpu/nvfp4.py:1101-1151; numerically linear_mx, ops/quantized.py:662-723,
 * on the same codes and scales):
 *   C[b][m][n] = round(alpha * sum_k (A[b][m][k] sa[b][m][k/16]) (B[b][n][k] sb[b][n][k/16]) + bias[n])
 * A [batch, M, K/2] and B [batch, N, K/2] are packed codes, sfa / sfb their scale
 * tiles (per batch element, as above), alpha the product of the two global scales
 * (device scalar or NULL), fp32 accumulation, one rounding to out_dtype. */
int vq_gemm_nvfp4(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int out_dtype,
                  int64_t M, int64_t N, int64_t K, int64_t ldc, int64_t batch, int64_t strideC,
                  const void* alpha, int alpha_dtype, const void* bias, int bias_dtype, void* stream);

/* vq_gemm_nvfp4 with one more factor per output column (device [N] of alpha_cols_dtype, may be
 * NULL), applied after alpha: linears that read one packed activation but carry different
 * weight global scales (q/k/v, gate/up of a decoder layer) run as one GEMM, column n scaled by
 * its own linear's alpha (backend/gpu/nvfp4.py:1101-1152 applies one alpha per linear). */
int vq_gemm_nvfp4_ex(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int out_dtype, int64_t M,
                     int64_t N, int64_t K, int64_t ldc, int64_t batch, int64_t strideC, const void* alpha,
                     int alpha_dtype, const void* bias, int bias_dtype, const void* alpha_cols, int alpha_cols_dtype,
                     void* stream);

/* Token-row exchanges of a tensor-parallel layer by plain loads from peer memory (NVLink), for ranks whose
 * buffers are mapped into one another's address space (symmetric memory).  peer_ptrs: a HOST array of `world`
 * device pointers, one buffer per rank (this rank's own at its index), 16-byte aligned.  Neither kernel waits on
 * another GPU: the caller orders them after the buffers' producers with a cross-rank barrier.
 *   vq_peer_gather      out[p * chunk_bytes + i] = peer[p][i]: all-gather of every rank's chunk (chunk_bytes a
 *                       multiple of 16) into this GPU's `out` (world * chunk_bytes)
 *   vq_peer_reduce_rows out[i] = sum_p peer[p][rank * chunk_floats + i], p = 0 .. world-1 in that order:
 *                       reduce-scatter of float32 partial sums (chunk_floats a multiple of 4) into `out`
 * They stand where ncclAllGather / ncclReduceScatter stand in the row-parallel linears of a layer short enough
 * for the collectives' latency to dominate it. */
int vq_peer_gather(const void* const* peer_ptrs, int64_t world, int64_t chunk_bytes, void* out, void* stream);
int vq_peer_reduce_rows(const void* const* peer_ptrs, int64_t world, int64_t rank, int64_t chunk_floats, void* out,
                        void* stream);
/* out[0] = max over ranks of the float32 at the start of each rank's buffer: all-reduce(max) of a tensor's amax. */
int vq_peer_max(const void* const* peer_ptrs, int64_t world, void* out, void* stream);

/* Synchronising health check for the GEMM kernels: returns VQ_ETIMEOUT if any
 * launch since the last reset gave up on a bounded barrier wait (its output is
 * then invalid).  No counterpart in the reference. */
int vq_gemm_status(int reset);

/* The KIVI cache read for 2-bit codes of a bfloat16 [outer, T, D] tensor: quantized_ops::dequantize(
 * codes, scale, zero_point, axes, block) (ops/quantized.py:527-571; codegen/transform/
 * quant_folding.py:2391-2547) straight from packed bytes (element i of the row-major tensor in
 * byte i / 4 at bit 2 (i % 4)), out = bf16(bf16(code - zero_point) * scale).  along_channels == 0:
 * groups of `block` positions per channel (keys; parameters [outer, T / block, D]); != 0: groups of
 * `block` channels per position (values; parameters [outer, T, D / block]).  The general layouts,
 * other widths and the fused re-encode stay with vq_unpack_dequantize. */
int vq_kivi_read_2bit(const void* packed, const void* scale, const void* zero_point, void* out, int64_t outer,
                      int64_t T, int64_t D, int along_channels, int64_t block, void* stream);

/* One decode step's attention straight from the packed KIVI cache, for every (sequence, KV head) pair
 * `outer`: the nodes
 *   k = dequantize(k_codes, k_scale, k_zero); v = dequantize(v_codes, v_scale, v_zero)   (as vq_kivi_read_2bit)
 *   scores = cat(matmul(q, k^T), matmul(q, k_res^T)); p = bf16(softmax_fp32(bf16(scores * score_scale)))
 *   out = bf16(matmul(p[:, :Tm], v)) + bf16(matmul(p[:, Tm:], v_res))
 * of the graph (quantized_ops::dequantize, ops/quantized.py:527-571, emitted for the cache by
 * codegen/transform/quant_folding.py:2391-2547, and the eager attention around it) with every node's
 * bfloat16 rounding, without writing the dequantized cache.  q, out: bfloat16 [outer, G, 128] (the G query
 * heads of the KV head); k_packed / v_packed: 2-bit codes [outer, Tm, 128] (four per byte); k_scale,
 * k_zero: bfloat16 [outer, Tm / k_block, 128]; v_scale, v_zero: bfloat16 [outer, Tm, 128 / v_block];
 * k_res, v_res: the newest R positions in bfloat16, [outer, R, 128].  VQ_EUNSUPPORTED unless D == 128,
 * G <= 8, k_block a multiple of 64 dividing Tm, v_block 32, 64 or 128, R a multiple of 16 and the
 * G * (Tm + R) * 6 bytes of scores fit in shared memory beside two staged chunks (G = 4: about 4600
 * positions) (the caller then reads the cache with
 * vq_kivi_read_2bit and runs the nodes one by one). */
int vq_kivi_decode_attention(const void* q, const void* k_packed, const void* k_scale, const void* k_zero,
                             const void* v_packed, const void* v_scale, const void* v_zero, const void* k_res,
                             const void* v_res, void* out, int64_t outer, int64_t G, int64_t Tm, int64_t R, int64_t D,
                             int64_t k_block, int64_t v_block, float score_scale, void* stream);

/* Weight-streaming microscaling linear for a decode step (M <= 32 activation rows), on a weight
 * stored packed: w_packed [N, K / 2] holds two 4-bit codebook indices per byte (even element in
 * the low nibble), w_scale [N, K / block_size] its bfloat16 block scales, w_levels the 16
 * bfloat16 codebook entries.  It computes quantized_ops::linear_mx (ops/quantized.py:662-723)
 * for such a weight -- both operands read back as bf16(level * scale) (:574-591), float32
 * products and sum, alpha, bias, one rounding -- without ever materialising the weight's
 * bfloat16-valued index tensor (0.53 bytes per parameter from memory instead of 2).  The
 * activation a [M, K] (row pitch lda, bfloat16) holds values, or codebook indices when a_levels
 * (n_a_levels bfloat16 entries) is given; a_scale [M, K / block_size] may be NULL.
 * K is a multiple of 128; block_size a multiple of 32 dividing K.  workspace is
 * vq_gemm_lut4_workspace_floats(M, N, K) floats of device scratch (contents irrelevant);
 * counters is vq_gemm_lut4_counters(N) ints that must be zero before the first call and are
 * left zero by every call (calls sharing them must not overlap on the device). */
int64_t vq_gemm_lut4_workspace_floats(int64_t M, int64_t N, int64_t K);
int64_t vq_gemm_lut4_counters(int64_t N);
int vq_gemm_lut4(const void* a, int64_t lda, const void* a_scale, const void* a_levels, int n_a_levels, int64_t M,
                 const void* w_packed, const void* w_scale, const void* w_levels, int block_size, void* out,
                 int out_dtype, int64_t N, int64_t K, const void* alpha, int alpha_dtype, const void* bias,
                 int bias_dtype, float* workspace, int* counters, void* stream);

/* Packs bfloat16-valued codebook indices codes [rows, K] (each 0..15, what quantize_mx returns
 * for a lookup format with an index table, quantize_pt2e.py:754-791) into vq_gemm_lut4's
 * w_packed layout.  *bad (device int, zeroed by the caller) is set if a value is not such an index. */
int vq_pack_lut4(const void* codes, void* packed, int64_t rows, int64_t K, int* bad, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VQ_B200_H */
