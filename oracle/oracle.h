/*
 * CPU oracle for the quantized-matmul path: a plain-C restatement of the CATLASS CPU goldens.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or calls this code; it exists so
 * that the CUDA kernels can be checked against an independent, obviously-correct implementation, and so
 * that a CPU baseline can be timed next to the GPU numbers.
 *
 * Parity status of each function is stated beside it:
 *   - "pinned: reference golden"  the restatement is checked against the reference's own C++ golden
 *                                 (compiled from the reference tree into oracle/_ref) and against
 *                                 committed vectors produced by it;
 *   - "pinned: reference python"  checked against committed vectors produced by the reference's Python
 *                                 data generators;
 *   - "parity unpinned"           the reference holds no golden for this exact formula; the restatement
 *                                 follows the published formula only.
 */
#ifndef CB200_ORACLE_H
#define CB200_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Layout tags (same numbering as the shipped C ABI). */
#define ORC_ROW_MAJOR 0
#define ORC_COL_MAJOR 1

/*
 * Dense W8A8 with per-token / per-channel dequant.            [pinned: reference golden]
 * Follows golden::QuantMatmul, examples/common/golden/matmul.hpp:303-324:
 *   acc[i,j]  = sum_k int32(A[i,k]) * int32(B[k,j])
 *   out[i,j]  = (float(acc) * scale[j]) * perToken[i]      (two separate fp32 multiplies, left to right)
 * A is m x k, B is k x n, each row- or column-major; out is row-major fp32.
 * acc (may be NULL) receives the raw int32 accumulators, row-major.
 */
void orc_quant_matmul(uint32_t m, uint32_t n, uint32_t k,
                      const int8_t *a, int layout_a, const int8_t *b, int layout_b,
                      const float *scale, const float *per_token, float *out, int32_t *acc);

/*
 * Grouped slice-M W8A8 with per-token dequant.                [pinned: reference golden]
 * Follows golden::ComputeGroupedMatmulPerTokenDequant, examples/common/golden/matmul.hpp:271-301:
 * group_list holds ascending prefix sums of rows; group g owns rows [group_list[g-1], group_list[g]),
 * uses weight matrix B + g*k*n and channel scales scale + g*n.  Rows at or beyond group_list[G-1]
 * are left untouched.
 */
void orc_grouped_quant_matmul_slice_m(uint32_t m, uint32_t n, uint32_t k, uint32_t group_count,
                                      const int64_t *group_list, const int8_t *a,
                                      const int8_t *b, int layout_b, const float *scale,
                                      const float *per_token, float *out, int32_t *acc);

/*
 * Grouped slice-M W8A8 with per-tensor / per-channel dequant. [pinned: reference golden]
 * Follows golden::ComputeGroupedMatmulFixpipeDequant, examples/common/golden/matmul.hpp:234-269:
 *   quant_mode 0: out = float(acc) * scale_per_tensor;  quant_mode 1: out = float(acc) * per_channel_scale[j]
 * (one [n] vector shared by every group; no per-token factor).
 */
void orc_grouped_matmul_fixpipe_dequant(uint32_t m, uint32_t n, uint32_t k, uint32_t group_count,
                                        const int64_t *group_list, const int8_t *a, const int8_t *b,
                                        int layout_b, int quant_mode, float scale_per_tensor,
                                        const float *per_channel_scale, float *out, int32_t *acc);

/*
 * Grouped slice-K W8A8 with per-token dequant.                [pinned: reference golden]
 * Follows golden::ComputeGroupedMatmulSliceKPerTokenDequant, examples/common/golden/matmul.hpp:326-359:
 * group_list holds ascending prefix sums over K; group g multiplies A[:, k_{g-1}:k_g] (A column-major m x k)
 * with B[k_{g-1}:k_g, :] (row-major k x n) into its own m x n output block out + g*m*n, scaled by
 * scale[g*n + j] and per_token[g*m + i].
 */
void orc_grouped_quant_matmul_slice_k(uint32_t m, uint32_t n, uint32_t k, uint32_t group_count,
                                      const int64_t *group_list, const int8_t *a, const int8_t *b,
                                      const float *scale, const float *per_token, float *out, int32_t *acc);

/*
 * W4A8 with per-group weight scales.                          [parity unpinned]
 * The reference holds a per-TENSOR W4A8 golden only (examples/32_w4a8_matmul/gen_data.py:111-131,
 * out = 1.5 * (A @ B)); the per-group formula restated here is:
 *   acc_g[i,j] = sum_{kk in group g} int32(A[i,kk]) * int32(W[kk,j])          (int32, exact)
 *   y[i,j]     = fma(float(acc_g), sw[g,j], y)    (fp32, one rounding per group; g ascending from y = 0)
 *   out[i,j]   = y * sa[i]
 * Weights are signed 4-bit, packed two per byte along K: byte t of column j holds W[2t,j] in bits 0-3
 * and W[2t+1,j] in bits 4-7 (nibble order of examples/32_w4a8_matmul/gen_data.py:102-105), columns
 * stored one after another (column-major B, ceil(k/2) bytes per column).  The last group is shorter when
 * group_size does not divide k.
 *
 * Which fp32 reading this is.  "Rescale each group's int32 sum and add in fp32" can be read fused (one rounding
 * per group, as here) or unfused (round the product, then the sum).  Nothing in the reference decides between
 * them; the fused form is the definition here because it is the more accurate one and what a GPU does at full
 * rate.  So that parity does not rest on this choice alone, orc_w4a8_matmul_per_group_readings returns the
 * UNFUSED fp32 result, the exact result in double, and sum_g |acc_g * sw| * |sa|: every fp32 evaluation in any
 * order lies within (number of groups) * 2^-24 * that magnitude of the exact value.
 */
void orc_w4a8_matmul_per_group(uint32_t m, uint32_t n, uint32_t k, uint32_t group_size,
                               const int8_t *a, const uint8_t *w_packed, const float *sw,
                               const float *sa, float *out);

void orc_w4a8_matmul_per_group_readings(uint32_t m, uint32_t n, uint32_t k, uint32_t group_size,
                                        const int8_t *a, const uint8_t *w_packed, const float *sw,
                                        const float *sa, float *out_unfused, double *out_exact,
                                        double *abs_terms);

/*
 * W4A8 per-tensor (the reference's example 32).               [pinned: reference python]
 * out[i,j] = scalar * float(sum_k A[i,k]*W[k,j])   (examples/32_w4a8_matmul/gen_data.py:111-131).
 */
void orc_w4a8_matmul_per_tensor(uint32_t m, uint32_t n, uint32_t k, const int8_t *a,
                                const uint8_t *w_packed, float scalar, float *out);

/* Unpack one signed 4-bit value (sign-extend bits 0-3). */
static inline int orc_int4(uint8_t nibble) { return (int)((nibble & 0xF) ^ 8) - 8; }

/*
 * MX (OCP microscaling) helpers.                              [pinned: reference python]
 * Follow examples/53_ascend950_fp8_mx_matmul/gen_data.py:186-207 (shared exponent),
 * :216-265 (snap to grid, ties toward zero), and examples/54_ascend950_fp4_mx_matmul/gen_data.py:46-95.
 *
 * orc_mx_quantize: rows x cols fp32 matrix, blocks of 32 along the contiguous (cols) axis.
 *   fmt = 0: E4M3 (emax 8, max 448);  fmt = 1: E2M1 (emax 2, max 6).
 *   q      : one byte per element (E4M3 bit pattern, or E2M1 code 0..15 in the low nibble)
 *   sf     : rows x ceil(cols/32) E8M0 bytes (exponent + 127)
 *   deq    : (may be NULL) dequantised fp32 values, rows x cols
 */
#define ORC_MX_E4M3 0
#define ORC_MX_E2M1 1
void orc_mx_quantize(uint32_t rows, uint32_t cols, int fmt, const float *x, uint8_t *q, uint8_t *sf,
                     float *deq);
float orc_e4m3_to_float(uint8_t v);

/*
 * Per-token int8 quantisation of activations (the step in front of the W8A8 matmuls; the reference has no
 * implementation of it: parity unpinned, this file is the definition the library's header states):
 *   amax = max |x| over the row; scale = amax / 127; inv = 127 / amax (0 for an all-zero row);
 *   q = clamp(rint(x * inv), -127, 127), one fp32 multiply, round half to even.
 */
void orc_quantize_per_token_int8(uint32_t rows, uint32_t cols, const float *x, int8_t *q, float *scale);
float orc_e2m1_to_float(uint8_t v);
float orc_e8m0_to_float(uint8_t v);

/*
 * MX block-scaled matmul golden: out = A_deq @ B_deq in fp32 (gen_data.py:417 of example 53).
 * aq: m x k element bytes, row-major (K contiguous); bq: n x k element bytes (column-major B, K contiguous);
 * sfa: m x ceil(k/32), sfb: n x ceil(k/32).  Products are accumulated in double and rounded once to fp32,
 * which lies inside the reference's own tolerance band (rtol 1/128) around its fp32 matmul.
 */
void orc_mx_matmul(uint32_t m, uint32_t n, uint32_t k, int fmt, const uint8_t *aq, const uint8_t *sfa,
                   const uint8_t *bq, const uint8_t *sfb, float *out);

/* fp32 -> bf16 bits, round to nearest even (NaN kept quiet). */
uint16_t orc_bf16_rne(float x);
void orc_bf16_rne_array(const float *x, uint16_t *y, size_t count);
float orc_bf16_to_float(uint16_t v);

/* fp32 -> fp16 bits, round to nearest even (overflow to infinity, gradual underflow). */
uint16_t orc_f16_rne(float x);
void orc_f16_rne_array(const float *x, uint16_t *y, size_t count);

#ifdef __cplusplus
}
#endif
/*
 * SwiGLU + MX quantisation epilogue of the grouped MXFP8 matmul      [pinned: reference python]
 * (experimental/gmm/ascend950_fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant/compare.py:31-121).
 *   orc_swiglu_bf16         c [m][n] fp32 -> s_bits [m][n/2] bf16 bit patterns
 *   orc_mx_quant_bf16_e4m3  s_bits [rows][cols], cols % 32 == 0 -> q [rows][cols] E4M3, scale [rows][cols/32] E8M0
 *   orc_e4m3_rne_sat        nearest E4M3 code, ties to even, saturating at 448
 */
uint8_t orc_e4m3_rne_sat(float x);
void orc_swiglu_bf16(const float *c, uint64_t m, uint64_t n, uint16_t *s_bits);
void orc_mx_quant_bf16_e4m3(const uint16_t *s_bits, uint64_t rows, uint64_t cols, uint8_t *q, uint8_t *scale);

#endif
