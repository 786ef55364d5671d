/*
 * kaio_oracle.c -- CPU restatement of the KAIO quantized-inference ops.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the parity checker and the timed CPU
 * baseline.  Nothing in the shipped library links, loads or calls it; the
 * product path is the CUDA library and it fails loudly when that is missing.
 *
 * Every function follows one of the CPU reference functions that the KAIO
 * repository keeps inside its own GPU tests (paths are relative to the KAIO
 * source tree):
 *
 *   matmul_int8      kaio-ops/tests/matmul_int8_e2e.rs:20-34      (cpu_reference)
 *   pack_s4          kaio-ops/tests/matmul_int4_e2e.rs:37-54      (pack_s4_weights)
 *   matmul_int4      kaio-ops/tests/matmul_int4_e2e.rs:60-95      (cpu_reference_matmul_int4)
 *   qkv_int8         kaio-ops/tests/qkv_project_int8_e2e.rs:48-72 (cpu_reference_qkv_int8)
 *   qkv_int4         kaio-ops/tests/qkv_project_int4_e2e.rs:70-100 (cpu_reference_qkv_int4)
 *   attention        kaio-ops/tests/common/mod.rs:163-235         (cpu_attention_f16xf16_f32)
 *   quantisers       examples/int8_matmul/src/main.rs:41-61, examples/int4_matmul/src/main.rs:48-85
 *
 * Parity pin: the restatement is checked against the known-answer vectors those
 * tests hold (0x11111111 / 0xFFFFFFFF pack words and the [8,-8,0,0] product,
 * the -1024 / -64 / 384 / {K,2K,3K} canaries, causal row 0 == V row 0) in
 * tests/test_oracle_golden.py.  The "extended" functions at the end (per-row x
 * per-column INT8 scales, f16 output, per-column QKV scales, strided multi-head
 * attention) have no counterpart in KAIO: for those, parity is unpinned.
 *
 * Arithmetic rules kept from the reference:
 *   - s32 accumulation is exact; the scale is one cast then one f32 multiply;
 *   - f16 <-> f32 conversions are IEEE round-to-nearest-even (half::f16);
 *   - every f32 sum runs over k (or j) in ascending order, one add per term,
 *     with no fused multiply-add (compile with -ffp-contract=off).
 *
 * Rows are independent, so the outer row loop is an OpenMP parallel-for; that
 * changes no per-element operation order.  `row0`/`row1` select a row range
 * [row0,row1) so a caller can time or check a bounded sample of a big shape;
 * rows outside the range are left untouched.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define KAIO_EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------ f16 */

/* f16 bits -> f32, exact. */
KAIO_EXPORT float kaio_oracle_f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* f32 -> f16 bits, round-to-nearest-even, overflow to inf (half::f16::from_f32). */
KAIO_EXPORT uint16_t kaio_oracle_f32_to_f16(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) { /* inf / nan */
        if (ax > 0x7F800000u)
            return (uint16_t)(sign | 0x7E00u | ((ax >> 13) & 0x3FFu));
        return (uint16_t)(sign | 0x7C00u);
    }
    if (ax >= 0x477FF000u) /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7C00u);
    if (ax < 0x33000001u) /* <= 2^-25 rounds to zero (tie goes to even = 0) */
        return (uint16_t)sign;
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
    uint32_t shift;
    uint32_t half_exp;
    if (e < -14) { /* subnormal result */
        shift = (uint32_t)(13 + (-14 - e));
        half_exp = 0;
    } else {
        shift = 13;
        half_exp = (uint32_t)(e + 15);
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u)))
        q++;
    uint32_t out;
    if (half_exp == 0)
        out = q; /* may carry into exponent 1: correct */
    else
        out = ((half_exp - 1) << 10) + q; /* q holds the implicit bit */
    return (uint16_t)(sign | out);
}

/* ------------------------------------------------------------ f16 GEMM (matmul_tc) */

/* kaio-ops/tests/common/mod.rs:37-54 (cpu_matmul_f16xf16_f32): both operands widened to f32,
 * sum += av * bv in f32, k ascending. */
KAIO_EXPORT void kaio_oracle_matmul_f16(const uint16_t *a, const uint16_t *b, uint32_t m,
                                        uint32_t n, uint32_t k, uint32_t row0, uint32_t row1,
                                        float *out)
{
    (void)m;
#pragma omp parallel for schedule(static)
    for (int64_t i = row0; i < (int64_t)row1; i++) {
        for (uint32_t j = 0; j < n; j++) {
            float sum = 0.0f;
            for (uint32_t p = 0; p < k; p++) {
                float av = kaio_oracle_f16_to_f32(a[(size_t)i * k + p]);
                float bv = kaio_oracle_f16_to_f32(b[(size_t)p * n + j]);
                sum += av * bv;
            }
            out[(size_t)i * n + j] = sum;
        }
    }
}

/* ------------------------------------------------------------ W8A8 GEMM */

/* kaio-ops/tests/matmul_int8_e2e.rs:20-34.  acc_out (may be NULL) receives the
 * exact s32 accumulators so the GPU accumulators can be compared bit for bit. */
KAIO_EXPORT void kaio_oracle_matmul_int8(const int8_t *a, const int8_t *b, float scale,
                                         uint32_t m, uint32_t n, uint32_t k, uint32_t row0,
                                         uint32_t row1, float *out, int32_t *acc_out)
{
    (void)m;
#pragma omp parallel for schedule(static)
    for (int64_t i = row0; i < (int64_t)row1; i++) {
        int32_t *acc = (int32_t *)calloc(n, sizeof(int32_t));
        for (uint32_t kk = 0; kk < k; kk++) {
            int32_t av = a[(size_t)i * k + kk];
            const int8_t *brow = b + (size_t)kk * n;
            for (uint32_t j = 0; j < n; j++)
                acc[j] += av * (int32_t)brow[j];
        }
        for (uint32_t j = 0; j < n; j++) {
            out[(size_t)i * n + j] = (float)acc[j] * scale;
            if (acc_out)
                acc_out[(size_t)i * n + j] = acc[j];
        }
        free(acc);
    }
}

/* Extended (no KAIO counterpart): C = ((acc as f32) * a_scale[i]) * w_scale[j]. */
KAIO_EXPORT void kaio_oracle_matmul_int8_scaled(const int8_t *a, const int8_t *b,
                                                const float *a_scale, const float *w_scale,
                                                uint32_t m, uint32_t n, uint32_t k, uint32_t row0,
                                                uint32_t row1, float *out)
{
    (void)m;
#pragma omp parallel for schedule(static)
    for (int64_t i = row0; i < (int64_t)row1; i++) {
        int32_t *acc = (int32_t *)calloc(n, sizeof(int32_t));
        for (uint32_t kk = 0; kk < k; kk++) {
            int32_t av = a[(size_t)i * k + kk];
            const int8_t *brow = b + (size_t)kk * n;
            for (uint32_t j = 0; j < n; j++)
                acc[j] += av * (int32_t)brow[j];
        }
        for (uint32_t j = 0; j < n; j++) {
            float t = (float)acc[j] * a_scale[i];
            out[(size_t)i * n + j] = t * w_scale[j];
        }
        free(acc);
    }
}

/* ------------------------------------------------------------ W4A16 GEMM */

/* kaio-ops/tests/matmul_int4_e2e.rs:37-54.  w is the logical [K,N] row-major
 * matrix of values in [-8,7]; out is u32[(K/8)*N], word (k/8) of column j at
 * index (k/8) + j*(K/8), nibble k%8 at bits [4*(k%8), 4*(k%8)+4). */
KAIO_EXPORT void kaio_oracle_pack_s4(const int8_t *w, uint32_t k, uint32_t n, uint32_t *out)
{
    uint32_t k_words = k / 8;
    for (uint32_t col = 0; col < n; col++) {
        for (uint32_t wi = 0; wi < k_words; wi++) {
            uint32_t word = 0;
            for (uint32_t nib = 0; nib < 8; nib++) {
                int8_t val = w[(size_t)(wi * 8 + nib) * n + col];
                word |= ((uint32_t)val & 0xFu) << (4 * nib);
            }
            out[wi + (size_t)col * k_words] = word;
        }
    }
}

/* The dequantised weight exactly as the reference computes it:
 * nibble -> sign-extend -> f32 -> f16 -> (f16 * f16 scale, evaluated in f32,
 * rounded to f16) -> f32.  kaio-ops/tests/matmul_int4_e2e.rs:73-87. */
static inline float dequant_s4(const uint32_t *w_packed, const uint16_t *scales, uint32_t kk,
                               uint32_t j, uint32_t n, uint32_t k_words, uint32_t group_size)
{
    uint32_t word = w_packed[(kk / 8) + (size_t)j * k_words];
    uint32_t nibble = (word >> (4 * (kk % 8))) & 0xFu;
    int32_t s = ((int32_t)(nibble << 28)) >> 28;
    uint16_t raw = kaio_oracle_f32_to_f16((float)s);
    float scale = kaio_oracle_f16_to_f32(scales[(size_t)(kk / group_size) * n + j]);
    uint16_t scaled = kaio_oracle_f32_to_f16(kaio_oracle_f16_to_f32(raw) * scale);
    return kaio_oracle_f16_to_f32(scaled);
}

/* Dequantise the whole [K,N] matrix once (row-major f32); shared by all rows. */
static float *dequant_matrix_s4(const uint32_t *w_packed, const uint16_t *scales, uint32_t n,
                                uint32_t k, uint32_t group_size)
{
    float *w = (float *)malloc((size_t)k * n * sizeof(float));
    uint32_t k_words = k / 8;
#pragma omp parallel for schedule(static)
    for (int64_t kk = 0; kk < (int64_t)k; kk++)
        for (uint32_t j = 0; j < n; j++)
            w[(size_t)kk * n + j] =
                dequant_s4(w_packed, scales, (uint32_t)kk, j, n, k_words, group_size);
    return w;
}

/* kaio-ops/tests/matmul_int4_e2e.rs:60-95.  out_f32 and out_f16 may each be
 * NULL; out_f16 = f16_rn(acc) is the extended f16-output form (the same narrow
 * as kaio-ops/tests/qkv_project_int4_e2e.rs:96). */
KAIO_EXPORT void kaio_oracle_matmul_int4(const uint16_t *a, const uint32_t *w_packed,
                                         const uint16_t *scales, uint32_t m, uint32_t n,
                                         uint32_t k, uint32_t group_size, uint32_t row0,
                                         uint32_t row1, float *out_f32, uint16_t *out_f16)
{
    (void)m;
    float *w = dequant_matrix_s4(w_packed, scales, n, k, group_size);
#pragma omp parallel for schedule(static)
    for (int64_t i = row0; i < (int64_t)row1; i++) {
        float *acc = (float *)calloc(n, sizeof(float));
        for (uint32_t kk = 0; kk < k; kk++) {
            float av = kaio_oracle_f16_to_f32(a[(size_t)i * k + kk]);
            const float *wrow = w + (size_t)kk * n;
            for (uint32_t j = 0; j < n; j++)
                acc[j] += av * wrow[j];
        }
        for (uint32_t j = 0; j < n; j++) {
            if (out_f32)
                out_f32[(size_t)i * n + j] = acc[j];
            if (out_f16)
                out_f16[(size_t)i * n + j] = kaio_oracle_f32_to_f16(acc[j]);
        }
        free(acc);
    }
    free(w);
}

/* ------------------------------------------------------------ fused QKV */

/* One projection of kaio-ops/tests/qkv_project_int8_e2e.rs:48-72 (W8A16):
 * out = f16_rn((sum_k f32(x) * f32(f16(w))) * scale).  col_scale (may be NULL)
 * is the extended per-column form: scale is replaced by col_scale[j]. */
KAIO_EXPORT void kaio_oracle_qkv_int8(const uint16_t *x, const int8_t *w, float scale,
                                      const float *col_scale, uint32_t m, uint32_t n, uint32_t k,
                                      uint32_t row0, uint32_t row1, uint16_t *out)
{
    (void)m;
#pragma omp parallel for schedule(static)
    for (int64_t i = row0; i < (int64_t)row1; i++) {
        float *acc = (float *)calloc(n, sizeof(float));
        for (uint32_t kk = 0; kk < k; kk++) {
            float xv = kaio_oracle_f16_to_f32(x[(size_t)i * k + kk]);
            const int8_t *wrow = w + (size_t)kk * n;
            for (uint32_t j = 0; j < n; j++)
                acc[j] += xv * (float)wrow[j]; /* s8 -> f16 -> f32 is exact */
        }
        for (uint32_t j = 0; j < n; j++) {
            float s = col_scale ? col_scale[j] : scale;
            out[(size_t)i * n + j] = kaio_oracle_f32_to_f16(acc[j] * s);
        }
        free(acc);
    }
}

/* One projection of the W8A8 fused QKV op (extended: the reference's INT8 QKV op is W8A16, so
 * parity is unpinned by reference tests).  Built from two reference pieces: the symmetric
 * per-tensor quantiser of examples/int8_matmul/src/main.rs:41-61 applied to each row of x
 * (s_x = max|x| / 127, 1 for an all-zero row; xq = clamp(round(x / s_x), -127, 127), round half
 * away from zero, x widened from f16 to f32 exactly) and cpu_reference of
 * kaio-ops/tests/matmul_int8_e2e.rs:20-34 (exact s32 accumulation, one cast, then f32
 * multiplies): out = f16_rn(((acc as f32) * s_x[i]) * col_scale[j]).  acc_out (may be NULL)
 * receives the s32 accumulators, xq_out / sx_out (may be NULL) the quantised row. */
KAIO_EXPORT void kaio_oracle_qkv_w8a8(const uint16_t *x, const int8_t *w, const float *col_scale,
                                      uint32_t m, uint32_t n, uint32_t k, uint32_t row0,
                                      uint32_t row1, uint16_t *out, int32_t *acc_out,
                                      int8_t *xq_out, float *sx_out)
{
    (void)m;
#pragma omp parallel for schedule(static)
    for (int64_t i = row0; i < (int64_t)row1; i++) {
        int32_t *acc = (int32_t *)calloc(n, sizeof(int32_t));
        int8_t *xq = (int8_t *)malloc(k);
        float mx = 0.0f;
        for (uint32_t kk = 0; kk < k; kk++) {
            float a = fabsf(kaio_oracle_f16_to_f32(x[(size_t)i * k + kk]));
            mx = a > mx ? a : mx;
        }
        float s = (mx == 0.0f) ? 1.0f : mx / 127.0f;
        for (uint32_t kk = 0; kk < k; kk++) {
            float v = roundf(kaio_oracle_f16_to_f32(x[(size_t)i * k + kk]) / s);
            v = v < -127.0f ? -127.0f : (v > 127.0f ? 127.0f : v);
            xq[kk] = (int8_t)v;
        }
        for (uint32_t kk = 0; kk < k; kk++) {
            const int32_t xv = xq[kk];
            const int8_t *wrow = w + (size_t)kk * n;
            for (uint32_t j = 0; j < n; j++)
                acc[j] += xv * (int32_t)wrow[j];
        }
        for (uint32_t j = 0; j < n; j++) {
            out[(size_t)i * n + j] = kaio_oracle_f32_to_f16(((float)acc[j] * s) * col_scale[j]);
            if (acc_out)
                acc_out[(size_t)i * n + j] = acc[j];
        }
        if (xq_out)
            memcpy(xq_out + (size_t)i * k, xq, k);
        if (sx_out)
            sx_out[i] = s;
        free(xq);
        free(acc);
    }
}

/* One projection of kaio-ops/tests/qkv_project_int4_e2e.rs:70-100. */
KAIO_EXPORT void kaio_oracle_qkv_int4(const uint16_t *x, const uint32_t *w_packed,
                                      const uint16_t *scales, uint32_t m, uint32_t n, uint32_t k,
                                      uint32_t group_size, uint32_t row0, uint32_t row1,
                                      uint16_t *out)
{
    kaio_oracle_matmul_int4(x, w_packed, scales, m, n, k, group_size, row0, row1, NULL, out);
}

/* ------------------------------------------------------------ attention */

/* kaio-ops/tests/common/mod.rs:163-235, generalised only in addressing: each
 * of q/k/v/out has a row stride (in elements) so one head of a [rows, H*D]
 * projection output can be addressed in place.  With strides d_k, d_k, d_v,
 * d_v this is the reference function.  f32 throughout, true -inf mask, expf,
 * divide by the row sum; out_f16 (may be NULL) = f16_rn(out) is the extended
 * f16-output form. */
KAIO_EXPORT void kaio_oracle_attention(const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                       uint32_t seq_q, uint32_t seq_k, uint32_t d_k, uint32_t d_v,
                                       uint32_t q_stride, uint32_t k_stride, uint32_t v_stride,
                                       uint32_t out_stride, int causal, uint32_t row0,
                                       uint32_t row1, float *out_f32, uint16_t *out_f16)
{
    (void)seq_q;
    float inv_sqrt_dk = 1.0f / sqrtf((float)d_k);
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t i = row0; i < (int64_t)row1; i++) {
        float *row = (float *)malloc((size_t)seq_k * sizeof(float));
        float *qf = (float *)malloc((size_t)d_k * sizeof(float));
        float *o = (float *)calloc(d_v, sizeof(float));
        for (uint32_t d = 0; d < d_k; d++)
            qf[d] = kaio_oracle_f16_to_f32(q[(size_t)i * q_stride + d]);
        for (uint32_t j = 0; j < seq_k; j++) {
            float dot = 0.0f;
            for (uint32_t d = 0; d < d_k; d++)
                dot += qf[d] * kaio_oracle_f16_to_f32(k[(size_t)j * k_stride + d]);
            row[j] = dot * inv_sqrt_dk;
            if (causal && j > (uint32_t)i)
                row[j] = -INFINITY;
        }
        float mx = -INFINITY;
        for (uint32_t j = 0; j < seq_k; j++)
            mx = row[j] > mx ? row[j] : mx;
        float sum = 0.0f;
        for (uint32_t j = 0; j < seq_k; j++) {
            float e = (row[j] == -INFINITY) ? 0.0f : expf(row[j] - mx);
            row[j] = e;
            sum += e;
        }
        if (sum > 0.0f)
            for (uint32_t j = 0; j < seq_k; j++)
                row[j] /= sum;
        for (uint32_t j = 0; j < seq_k; j++) {
            float p = row[j];
            const uint16_t *vrow = v + (size_t)j * v_stride;
            for (uint32_t d = 0; d < d_v; d++)
                o[d] += p * kaio_oracle_f16_to_f32(vrow[d]);
        }
        for (uint32_t d = 0; d < d_v; d++) {
            if (out_f32)
                out_f32[(size_t)i * out_stride + d] = o[d];
            if (out_f16)
                out_f16[(size_t)i * out_stride + d] = kaio_oracle_f32_to_f16(o[d]);
        }
        free(row);
        free(qf);
        free(o);
    }
}

/* ----------------------------------------------------- gated activation */

/* cpu_reference of examples/fused_silu_gate/src/main.rs:23-33: widen to f64,
 * sig = 1 / (1 + exp(-x)), out = (x * sig * gate) as f32. */
KAIO_EXPORT void kaio_oracle_silu_gate_f32(const float *x, const float *gate, float *out, size_t n)
{
    for (size_t i = 0; i < n; i++) {
        double xi = (double)x[i], gi = (double)gate[i];
        double sig = 1.0 / (1.0 + exp(-xi));
        out[i] = (float)(xi * sig * gi);
    }
}

/* The same on f16 matrices with row strides (elements): the f64 result is narrowed to f32 as
 * above and then rounded once to f16. */
KAIO_EXPORT void kaio_oracle_silu_gate_f16(const uint16_t *x, const uint16_t *gate, uint16_t *out,
                                           uint32_t rows, uint32_t cols, uint32_t x_ld,
                                           uint32_t gate_ld, uint32_t out_ld)
{
    for (uint32_t r = 0; r < rows; r++)
        for (uint32_t c = 0; c < cols; c++) {
            double xi = (double)kaio_oracle_f16_to_f32(x[(size_t)r * x_ld + c]);
            double gi = (double)kaio_oracle_f16_to_f32(gate[(size_t)r * gate_ld + c]);
            double sig = 1.0 / (1.0 + exp(-xi));
            out[(size_t)r * out_ld + c] = kaio_oracle_f32_to_f16((float)(xi * sig * gi));
        }
}

/* ----------------------------------------------------------- quantisers */

/* derive_scale + quantize of examples/int8_matmul/src/main.rs:41-61, applied per row:
 * scale = max|x| / 127 (1 if zero); q = clamp(round(x / scale), -127, 127); `round` is
 * round-half-away-from-zero like Rust's f32::round. */
KAIO_EXPORT void kaio_oracle_quantize_rows_int8(const float *x, uint32_t m, uint32_t k, int8_t *q,
                                                float *scale)
{
    for (uint32_t i = 0; i < m; i++) {
        float mx = 0.0f;
        for (uint32_t j = 0; j < k; j++) {
            float a = fabsf(x[(size_t)i * k + j]);
            mx = a > mx ? a : mx;
        }
        float s = (mx == 0.0f) ? 1.0f : mx / 127.0f;
        scale[i] = s;
        for (uint32_t j = 0; j < k; j++) {
            float v = roundf(x[(size_t)i * k + j] / s);
            v = v < -127.0f ? -127.0f : (v > 127.0f ? 127.0f : v);
            q[(size_t)i * k + j] = (int8_t)v;
        }
    }
}

/* quantize_gptq_lite of examples/int4_matmul/src/main.rs:48-85: per (column, group):
 * scale = max|w| / 7 (1 if zero), stored as f16; q = clamp(round(w / scale_f32), -8, 7). */
KAIO_EXPORT void kaio_oracle_quantize_gptq_lite(const float *w, uint32_t k, uint32_t n,
                                                uint32_t group_size, int8_t *q, uint16_t *scales)
{
    uint32_t groups = k / group_size;
    for (uint32_t col = 0; col < n; col++) {
        for (uint32_t g = 0; g < groups; g++) {
            float mx = 0.0f;
            for (uint32_t kk = g * group_size; kk < (g + 1) * group_size; kk++) {
                float a = fabsf(w[(size_t)kk * n + col]);
                mx = a > mx ? a : mx;
            }
            float s = (mx == 0.0f) ? 1.0f : mx / 7.0f;
            scales[(size_t)g * n + col] = kaio_oracle_f32_to_f16(s);
            for (uint32_t kk = g * group_size; kk < (g + 1) * group_size; kk++) {
                float v = roundf(w[(size_t)kk * n + col] / s);
                v = v < -8.0f ? -8.0f : (v > 7.0f ? 7.0f : v);
                q[(size_t)kk * n + col] = (int8_t)v;
            }
        }
    }
}

/* ---------------------------------------------------------------- misc */

/* Sets the number of OpenMP threads of the following calls (a launcher such as torchrun exports
 * OMP_NUM_THREADS=1 to its workers; a timed CPU baseline wants all the host's cores). */
KAIO_EXPORT void kaio_oracle_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0)
        omp_set_num_threads(n);
#else
    (void)n;
#endif
}

KAIO_EXPORT int kaio_oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
