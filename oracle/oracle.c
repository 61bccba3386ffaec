/*
 * CPU oracle: plain-C restatement of the CATLASS CPU goldens for the quantized-matmul path.
 * TEST INFRASTRUCTURE ONLY - see oracle.h for what each function follows and how it is pinned.
 *
 * Build with -ffp-contract=off: the goldens multiply and add in separate fp32 operations and the
 * comparisons against the GPU are bit-exact, so the compiler must not fuse them.
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ bf16 */

uint16_t orc_bf16_rne(float x)
{
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) { /* NaN: keep sign, force quiet */
        return (uint16_t)((u >> 16) | 0x0040u);
    }
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

void orc_bf16_rne_array(const float *x, uint16_t *y, size_t count)
{
    for (size_t i = 0; i < count; ++i) {
        y[i] = orc_bf16_rne(x[i]);
    }
}

float orc_bf16_to_float(uint16_t v)
{
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* ------------------------------------------------------------------ W8A8 */

/* acc_row[j] = sum_k a_row[k] * B[k,j] for one row of A. Loop order is chosen per layout so that the
 * inner loop walks memory contiguously; integer sums do not depend on the order. */
static void int8_row_times_matrix(uint32_t n, uint32_t k, const int8_t *a_row, size_t a_stride,
                                  const int8_t *b, int layout_b, int32_t *acc_row)
{
    if (layout_b == ORC_COL_MAJOR) { /* column j is k contiguous bytes */
        for (uint32_t j = 0; j < n; ++j) {
            const int8_t *col = b + (size_t)j * k;
            int32_t s = 0;
            for (uint32_t kk = 0; kk < k; ++kk) {
                s += (int32_t)a_row[(size_t)kk * a_stride] * (int32_t)col[kk];
            }
            acc_row[j] = s;
        }
    } else { /* row kk of B is n contiguous bytes */
        for (uint32_t j = 0; j < n; ++j) {
            acc_row[j] = 0;
        }
        for (uint32_t kk = 0; kk < k; ++kk) {
            int32_t av = (int32_t)a_row[(size_t)kk * a_stride];
            const int8_t *row = b + (size_t)kk * n;
            for (uint32_t j = 0; j < n; ++j) {
                acc_row[j] += av * (int32_t)row[j];
            }
        }
    }
}

void orc_quant_matmul(uint32_t m, uint32_t n, uint32_t k, const int8_t *a, int layout_a,
                      const int8_t *b, int layout_b, const float *scale, const float *per_token,
                      float *out, int32_t *acc)
{
    int32_t *row_acc = (int32_t *)malloc(sizeof(int32_t) * (n ? n : 1));
    for (uint32_t i = 0; i < m; ++i) {
        const int8_t *a_row = (layout_a == ORC_ROW_MAJOR) ? a + (size_t)i * k : a + i;
        size_t a_stride = (layout_a == ORC_ROW_MAJOR) ? 1 : m;
        int8_row_times_matrix(n, k, a_row, a_stride, b, layout_b, row_acc);
        for (uint32_t j = 0; j < n; ++j) {
            float t = (float)row_acc[j] * scale[j];
            out[(size_t)i * n + j] = t * per_token[i];
        }
        if (acc) {
            memcpy(acc + (size_t)i * n, row_acc, sizeof(int32_t) * n);
        }
    }
    free(row_acc);
}

void orc_grouped_quant_matmul_slice_m(uint32_t m, uint32_t n, uint32_t k, uint32_t group_count,
                                      const int64_t *group_list, const int8_t *a, const int8_t *b,
                                      int layout_b, const float *scale, const float *per_token,
                                      float *out, int32_t *acc)
{
    (void)m;
    int32_t *row_acc = (int32_t *)malloc(sizeof(int32_t) * (n ? n : 1));
    int64_t start_row = 0;
    for (uint32_t g = 0; g < group_count; ++g) {
        const int8_t *bg = b + (size_t)g * k * n;
        const float *sg = scale + (size_t)g * n;
        for (int64_t i = start_row; i < group_list[g]; ++i) {
            int8_row_times_matrix(n, k, a + (size_t)i * k, 1, bg, layout_b, row_acc);
            for (uint32_t j = 0; j < n; ++j) {
                float t = (float)row_acc[j] * sg[j];
                out[(size_t)i * n + j] = t * per_token[i];
            }
            if (acc) {
                memcpy(acc + (size_t)i * n, row_acc, sizeof(int32_t) * n);
            }
        }
        start_row = group_list[g]; /* as the golden does, also for a list that is not ascending */
    }
    free(row_acc);
}

void orc_grouped_matmul_fixpipe_dequant(uint32_t m, uint32_t n, uint32_t k, uint32_t group_count,
                                        const int64_t *group_list, const int8_t *a, const int8_t *b,
                                        int layout_b, int quant_mode, float scale_per_tensor,
                                        const float *per_channel_scale, float *out, int32_t *acc)
{
    (void)m;
    int32_t *row_acc = (int32_t *)malloc(sizeof(int32_t) * (n ? n : 1));
    int64_t start_row = 0;
    for (uint32_t g = 0; g < group_count; ++g) {
        const int8_t *bg = b + (size_t)g * k * n;
        for (int64_t i = start_row; i < group_list[g]; ++i) {
            int8_row_times_matrix(n, k, a + (size_t)i * k, 1, bg, layout_b, row_acc);
            for (uint32_t j = 0; j < n; ++j) {
                float s = quant_mode == 0 ? scale_per_tensor : per_channel_scale[j];
                out[(size_t)i * n + j] = (float)row_acc[j] * s;
            }
            if (acc) {
                memcpy(acc + (size_t)i * n, row_acc, sizeof(int32_t) * n);
            }
        }
        start_row = group_list[g];
    }
    free(row_acc);
}

void orc_grouped_quant_matmul_slice_k(uint32_t m, uint32_t n, uint32_t k, uint32_t group_count,
                                      const int64_t *group_list, const int8_t *a, const int8_t *b,
                                      const float *scale, const float *per_token, float *out, int32_t *acc)
{
    (void)k;
    int32_t *row_acc = (int32_t *)malloc(sizeof(int32_t) * (n ? n : 1));
    int64_t start = 0;
    for (uint32_t g = 0; g < group_count; ++g) {
        int64_t end = group_list[g];
        uint32_t kg = end > start ? (uint32_t)(end - start) : 0;
        float *og = out + (size_t)g * m * n;
        for (uint32_t i = 0; i < m; ++i) {
            /* A is column-major: element (i, kk) at a[kk * m + i]; B row-major: row kk at b + kk * n */
            int8_row_times_matrix(n, kg, a + (size_t)start * m + i, m, b + (size_t)start * n, ORC_ROW_MAJOR, row_acc);
            for (uint32_t j = 0; j < n; ++j) {
                float t = (float)row_acc[j] * scale[(size_t)g * n + j];
                og[(size_t)i * n + j] = t * per_token[(size_t)g * m + i];
            }
            if (acc) {
                memcpy(acc + ((size_t)g * m + i) * n, row_acc, sizeof(int32_t) * n);
            }
        }
        start = end;
    }
    free(row_acc);
}

/* ------------------------------------------------------------------ fp16 */

uint16_t orc_f16_rne(float x)
{
    uint32_t u;
    memcpy(&u, &x, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t abs = u & 0x7fffffffu;
    if (abs > 0x7f800000u) {
        return (uint16_t)(sign | 0x7e00u); /* NaN */
    }
    if (abs >= 0x477ff000u) { /* >= 65520: rounds to infinity */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (abs < 0x33000001u) { /* <= 2^-25: rounds to zero (the tie 2^-25 goes to even = 0) */
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(abs >> 23) - 127;
    uint32_t mant = (abs & 0x7fffffu) | 0x800000u; /* 24 bits */
    uint32_t shift = e < -14 ? (uint32_t)(13 + (-14 - e)) : 13u; /* bits dropped */
    uint32_t kept = mant >> shift;
    uint32_t rem = mant & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (kept & 1u))) {
        ++kept;
    }
    uint32_t r;
    if (e < -14) {
        r = kept; /* subnormal (a carry into 0x400 is the smallest normal, correctly encoded) */
    } else {
        r = ((uint32_t)(e + 15) << 10) + (kept - 0x400u); /* a mantissa carry bumps the exponent */
    }
    return (uint16_t)(sign | r);
}

void orc_f16_rne_array(const float *x, uint16_t *y, size_t count)
{
    for (size_t i = 0; i < count; ++i) {
        y[i] = orc_f16_rne(x[i]);
    }
}

/* ------------------------------------------------------------------ W4A8 */

void orc_w4a8_matmul_per_group_readings(uint32_t m, uint32_t n, uint32_t k, uint32_t group_size,
                                        const int8_t *a, const uint8_t *w_packed, const float *sw,
                                        const float *sa, float *out_unfused, double *out_exact,
                                        double *abs_terms)
{
    uint32_t groups = (k + group_size - 1) / group_size;
    size_t col_bytes = (k + 1) / 2;
    for (uint32_t i = 0; i < m; ++i) {
        const int8_t *a_row = a + (size_t)i * k;
        for (uint32_t j = 0; j < n; ++j) {
            const uint8_t *col = w_packed + (size_t)j * col_bytes;
            float y = 0.0f;
            double y64 = 0.0, mag = 0.0;
            for (uint32_t g = 0; g < groups; ++g) {
                int32_t s = 0;
                uint32_t k0 = g * group_size;
                uint32_t k1 = k0 + group_size < k ? k0 + group_size : k;
                for (uint32_t kk = k0; kk < k1; ++kk) {
                    uint8_t byte = col[kk >> 1];
                    int w = (kk & 1) ? orc_int4(byte >> 4) : orc_int4(byte & 0xF);
                    s += (int32_t)a_row[kk] * w;
                }
                float scale = sw[(size_t)g * n + j];
                float prod = (float)s * scale; /* rounded product: the unfused reading */
                y = y + prod;
                y64 += (double)s * (double)scale;
                mag += fabs((double)s * (double)scale);
            }
            if (out_unfused) {
                out_unfused[(size_t)i * n + j] = y * sa[i];
            }
            if (out_exact) {
                out_exact[(size_t)i * n + j] = y64 * (double)sa[i];
            }
            if (abs_terms) {
                abs_terms[(size_t)i * n + j] = mag * fabs((double)sa[i]);
            }
        }
    }
}

void orc_w4a8_matmul_per_group(uint32_t m, uint32_t n, uint32_t k, uint32_t group_size,
                               const int8_t *a, const uint8_t *w_packed, const float *sw,
                               const float *sa, float *out)
{
    uint32_t groups = (k + group_size - 1) / group_size; /* the last group may be shorter */
    size_t col_bytes = (k + 1) / 2;
    for (uint32_t i = 0; i < m; ++i) {
        const int8_t *a_row = a + (size_t)i * k;
        for (uint32_t j = 0; j < n; ++j) {
            const uint8_t *col = w_packed + (size_t)j * col_bytes;
            float y = 0.0f;
            for (uint32_t g = 0; g < groups; ++g) {
                int32_t s = 0;
                uint32_t k0 = g * group_size;
                uint32_t k1 = k0 + group_size < k ? k0 + group_size : k;
                for (uint32_t kk = k0; kk < k1; ++kk) {
                    uint8_t byte = col[kk >> 1];
                    int w = (kk & 1) ? orc_int4(byte >> 4) : orc_int4(byte & 0xF);
                    s += (int32_t)a_row[kk] * w;
                }
                y = fmaf((float)s, sw[(size_t)g * n + j], y);
            }
            out[(size_t)i * n + j] = y * sa[i];
        }
    }
}

void orc_w4a8_matmul_per_tensor(uint32_t m, uint32_t n, uint32_t k, const int8_t *a,
                                const uint8_t *w_packed, float scalar, float *out)
{
    size_t col_bytes = (k + 1) / 2;
    for (uint32_t i = 0; i < m; ++i) {
        const int8_t *a_row = a + (size_t)i * k;
        for (uint32_t j = 0; j < n; ++j) {
            const uint8_t *col = w_packed + (size_t)j * col_bytes;
            int32_t s = 0;
            for (uint32_t kk = 0; kk < k; ++kk) {
                uint8_t byte = col[kk >> 1];
                int w = (kk & 1) ? orc_int4(byte >> 4) : orc_int4(byte & 0xF);
                s += (int32_t)a_row[kk] * w;
            }
            out[(size_t)i * n + j] = scalar * (float)s;
        }
    }
}

/* ------------------------------------------------------------------ MX */

float orc_e4m3_to_float(uint8_t v)
{
    int sign = v >> 7;
    int e = (v >> 3) & 0xF;
    int mant = v & 7;
    float r;
    if (e == 0xF && mant == 7) {
        r = NAN;
    } else if (e == 0) {
        r = ldexpf((float)mant, -9); /* subnormal: mant/8 * 2^-6 */
    } else {
        r = ldexpf((float)(8 + mant), e - 10); /* (1+mant/8) * 2^(e-7) */
    }
    return sign ? -r : r;
}

float orc_e2m1_to_float(uint8_t v)
{
    static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float r = mag[v & 7];
    return (v & 8) ? -r : r;
}

float orc_e8m0_to_float(uint8_t v)
{
    if (v == 0xFF) {
        return NAN;
    }
    return ldexpf(1.0f, (int)v - 127);
}

/* Snap |x| to the nearest representable magnitude of the format; on a tie take the smaller magnitude
 * (the reference's lowest-index argmin rule).  Returns the element code without sign. */
static uint8_t snap_magnitude(float mag, int fmt)
{
    int count = (fmt == ORC_MX_E4M3) ? 127 : 8; /* E4M3 code 0x7F is NaN: 0..0x7E are magnitudes */
    int lo = 0;
    int hi = count - 1;
    /* largest code whose value <= mag */
    while (lo < hi) {
        int mid = (lo + hi + 1) / 2;
        float v = (fmt == ORC_MX_E4M3) ? orc_e4m3_to_float((uint8_t)mid) : orc_e2m1_to_float((uint8_t)mid);
        if (v <= mag) {
            lo = mid;
        } else {
            hi = mid - 1;
        }
    }
    if (lo == count - 1) {
        return (uint8_t)lo;
    }
    float lower = (fmt == ORC_MX_E4M3) ? orc_e4m3_to_float((uint8_t)lo) : orc_e2m1_to_float((uint8_t)lo);
    float upper =
        (fmt == ORC_MX_E4M3) ? orc_e4m3_to_float((uint8_t)(lo + 1)) : orc_e2m1_to_float((uint8_t)(lo + 1));
    return ((mag - lower) <= (upper - mag)) ? (uint8_t)lo : (uint8_t)(lo + 1);
}

void orc_quantize_per_token_int8(uint32_t rows, uint32_t cols, const float *x, int8_t *q, float *scale)
{
    for (uint32_t r = 0; r < rows; ++r) {
        const float *xr = x + (size_t)r * cols;
        float amax = 0.0f;
        for (uint32_t c = 0; c < cols; ++c) {
            const float a = fabsf(xr[c]);
            amax = a > amax ? a : amax;
        }
        const float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
        scale[r] = amax / 127.0f;
        for (uint32_t c = 0; c < cols; ++c) {
            const float t = nearbyintf(xr[c] * inv);  /* round half to even (default rounding mode) */
            q[(size_t)r * cols + c] = (int8_t)(t > 127.0f ? 127.0f : (t < -127.0f ? -127.0f : t));
        }
    }
}

void orc_mx_quantize(uint32_t rows, uint32_t cols, int fmt, const float *x, uint8_t *q, uint8_t *sf,
                     float *deq)
{
    const int emax = (fmt == ORC_MX_E4M3) ? 8 : 2;
    const float max_value = (fmt == ORC_MX_E4M3) ? 448.0f : 6.0f;
    const uint8_t sign_bit = (fmt == ORC_MX_E4M3) ? 0x80 : 0x08;
    uint32_t blocks = (cols + 31) / 32;
    for (uint32_t r = 0; r < rows; ++r) {
        for (uint32_t b = 0; b < blocks; ++b) {
            uint32_t c0 = b * 32;
            uint32_t c1 = c0 + 32 < cols ? c0 + 32 : cols;
            float max_abs = 0.0f;
            for (uint32_t c = c0; c < c1; ++c) {
                float v = fabsf(x[(size_t)r * cols + c]);
                if (v > max_abs) {
                    max_abs = v;
                }
            }
            int exp = 0;
            if (!(max_abs < 1e-12f)) {
                uint32_t bits;
                memcpy(&bits, &max_abs, 4);
                exp = (int)((bits >> 23) & 0xFF) - 127 - emax;
                if (exp < -128) {
                    exp = -128;
                }
                if (exp > 127) {
                    exp = 127;
                }
            }
            /* torch.float8_e8m0fnu stores 2^exp as exp+127; 2^-128 is not representable and rounds
             * to the smallest code. */
            int code = exp + 127;
            if (code < 0) {
                code = 0;
            }
            sf[(size_t)r * blocks + b] = (uint8_t)code;
            float scale = ldexpf(1.0f, exp);
            for (uint32_t c = c0; c < c1; ++c) {
                float v = x[(size_t)r * cols + c] / scale;
                if (v > max_value) {
                    v = max_value;
                }
                if (v < -max_value) {
                    v = -max_value;
                }
                uint8_t code_mag = snap_magnitude(fabsf(v), fmt);
                uint8_t out = code_mag;
                if (v < 0.0f && code_mag != 0) {
                    out |= sign_bit;
                }
                q[(size_t)r * cols + c] = out;
                if (deq) {
                    float e = (fmt == ORC_MX_E4M3) ? orc_e4m3_to_float(out) : orc_e2m1_to_float(out);
                    deq[(size_t)r * cols + c] = e * scale;
                }
            }
        }
    }
}

void orc_mx_matmul(uint32_t m, uint32_t n, uint32_t k, int fmt, const uint8_t *aq, const uint8_t *sfa,
                   const uint8_t *bq, const uint8_t *sfb, float *out)
{
    uint32_t blocks = (k + 31) / 32;
    float *a_deq = (float *)malloc(sizeof(float) * (size_t)(k ? k : 1));
    float *b_deq = (float *)malloc(sizeof(float) * (size_t)n * (k ? k : 1));
    for (uint32_t j = 0; j < n; ++j) {
        for (uint32_t kk = 0; kk < k; ++kk) {
            uint8_t e = bq[(size_t)j * k + kk];
            float v = (fmt == ORC_MX_E4M3) ? orc_e4m3_to_float(e) : orc_e2m1_to_float(e);
            b_deq[(size_t)j * k + kk] = v * orc_e8m0_to_float(sfb[(size_t)j * blocks + kk / 32]);
        }
    }
    for (uint32_t i = 0; i < m; ++i) {
        for (uint32_t kk = 0; kk < k; ++kk) {
            uint8_t e = aq[(size_t)i * k + kk];
            float v = (fmt == ORC_MX_E4M3) ? orc_e4m3_to_float(e) : orc_e2m1_to_float(e);
            a_deq[kk] = v * orc_e8m0_to_float(sfa[(size_t)i * blocks + kk / 32]);
        }
        for (uint32_t j = 0; j < n; ++j) {
            const float *bc = b_deq + (size_t)j * k;
            double s = 0.0;
            for (uint32_t kk = 0; kk < k; ++kk) {
                s += (double)a_deq[kk] * (double)bc[kk];
            }
            out[(size_t)i * n + j] = (float)s;
        }
    }
    free(a_deq);
    free(b_deq);
}

/* ------------------------------------------------------------------ SwiGLU + MX quantisation epilogue */

/* Nearest E4M3 (fn: no infinities, max 448) code, ties to even, saturating; NaN -> 0x7F.
 * What torch's float32 -> float8_e4m3fn conversion does after the golden's clamp to +-448
 * (experimental/gmm/ascend950_fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant/compare.py:106-108). */
uint8_t orc_e4m3_rne_sat(float x)
{
    uint32_t bits;
    memcpy(&bits, &x, 4);
    const uint8_t sign = (uint8_t)((bits >> 24) & 0x80u);
    if (x != x) {
        return 0x7F;
    }
    float mag = fabsf(x);
    if (mag >= 448.0f) {
        return (uint8_t)(sign | 0x7E);
    }
    /* grid spacing: 2^-9 below 2^-6 (subnormals), else 2^(e-3) for 2^e <= mag < 2^(e+1) */
    int e;
    (void)frexpf(mag, &e);   /* mag = f * 2^e, f in [0.5, 1) -> exponent of the leading bit is e - 1 */
    int lead = e - 1;
    if (mag == 0.0f || lead < -6) {
        lead = -6;
    }
    const float step = ldexpf(1.0f, lead - 3);
    const float scaled = mag / step;            /* exact: a power-of-two division */
    float r = nearbyintf(scaled);               /* default rounding mode: ties to even */
    /* r is in [0, 16]; 16 means the next binade's first value */
    int ri = (int)r;
    int exp_field = lead + 7;                   /* bias 7 */
    if (lead == -6 && ri < 8) {
        return (uint8_t)(sign | (uint8_t)ri);   /* subnormal (exp field 0) */
    }
    if (ri == 16) {
        ri = 8;
        exp_field += 1;
    }
    return (uint8_t)(sign | (uint8_t)(exp_field << 3) | (uint8_t)(ri - 8));
}

/* S = bf16_rne(act / (1 + exp(-act)) * gate) with act = c[:, :n/2], gate = c[:, n/2:], every step in fp32:
 * compare.py:31-39 (swiglu) and :174-175 (the rounding to bfloat16) of the example named above. */
void orc_swiglu_bf16(const float *c, uint64_t m, uint64_t n, uint16_t *s_bits)
{
    const uint64_t h = n / 2;
    for (uint64_t i = 0; i < m; ++i) {
        for (uint64_t j = 0; j < h; ++j) {
            const float act = c[i * n + j];
            const float gate = c[i * n + h + j];
            const float t1 = -act;
            const float t2 = expf(t1);
            const float t3 = t2 + 1.0f;
            const float t4 = act / t3;
            const float t5 = t4 * gate;
            s_bits[i * h + j] = orc_bf16_rne(t5);
        }
    }
}

/* MX quantisation of bf16 values along the contiguous axis, 32 per block, to E4M3 + E8M0:
 * compare.py:41-121 (mx_quant_dtype 36) of the example named above, itself a restatement of the device
 * epilogue's integer arithmetic on bf16 exponent fields (include/catlass/epilogue/tile/tile_swiglu_mx_quant.hpp:167-215).
 * s_bits [rows][cols] (cols a multiple of 32), q [rows][cols], scale [rows][cols/32]. */
void orc_mx_quant_bf16_e4m3(const uint16_t *s_bits, uint64_t rows, uint64_t cols, uint8_t *q, uint8_t *scale)
{
    const uint64_t blocks = cols / 32;
    for (uint64_t i = 0; i < rows; ++i) {
        for (uint64_t b = 0; b < blocks; ++b) {
            const uint16_t *x = s_bits + i * cols + b * 32;
            uint32_t max_exp = 0;
            for (int e = 0; e < 32; ++e) {
                const uint32_t ex = x[e] & 0x7f80u;
                max_exp = ex > max_exp ? ex : max_exp;
            }
            const int finite = max_exp != 0x7f80u;
            const int nonzero = max_exp != 0;
            const uint32_t clamped = max_exp <= 0x0400u ? 0x0400u : max_exp;
            const uint32_t shared = clamped - 0x0400u;
            uint32_t sv = shared >> 7;
            sv = finite ? sv : 0xffu;
            sv = nonzero ? sv : 0u;
            uint32_t hs = 0x7f00u - shared;
            hs = finite ? hs : 0x7f81u;
            hs = nonzero ? hs : 0u;
            hs = shared == 0x7f00u ? 0x0040u : hs;
            const float inv = orc_bf16_to_float((uint16_t)hs);
            scale[i * blocks + b] = (uint8_t)sv;
            for (int e = 0; e < 32; ++e) {
                /* bf16 * bf16 -> bf16: the exact product, rounded once */
                const float prod = orc_bf16_to_float(x[e]) * inv;
                float f = orc_bf16_to_float(orc_bf16_rne(prod));
                if (f > 448.0f) {
                    f = 448.0f;
                } else if (f < -448.0f) {
                    f = -448.0f;
                }
                q[i * cols + b * 32 + e] = orc_e4m3_rne_sat(f);
            }
        }
    }
}
