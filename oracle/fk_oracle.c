/*
 * fk_oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT.
 *
 * A plain-C restatement of the CPU references the ferro-kittens examples check
 * their two kernels against, used only as the checker in tests, in the smoke
 * run and as the timed CPU baseline of the benchmark. Nothing in the library
 * links, loads or calls this file.
 *
 * Parity is pinned: the reference's algorithm for this path lives in its own
 * repository (no third-party dependency carries it), and the restatement is
 * held to the known answers its tests state -- the exact integer GEMM gate
 * (examples/src/gemm.rs:422-451, 544-578), the attention lattice and f64 row
 * reference with its 2^-8 bound (examples/src/flash_forward.rs:313-440, 475),
 * the bf16 rounding rule, and the fixtures under tests/golden/.
 *
 * Each function cites the reference lines it follows.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int fko_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the timed baseline sets its own count. */
void fko_set_threads(int count) {
#ifdef _OPENMP
    if (count > 0) omp_set_num_threads(count);
#else
    (void)count;
#endif
}

/* ---------------------------------------------------------------- bf16 */

/* examples/src/gemm.rs:444-447 -- round-to-nearest-even fp32 -> bf16. */
uint16_t fko_to_bf16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    return (uint16_t)((bits + (0x7fffu + ((bits >> 16) & 1u))) >> 16);
}

/* examples/src/gemm.rs:449-451 */
float fko_from_bf16(uint16_t bits) {
    uint32_t wide = (uint32_t)bits << 16;
    float value;
    memcpy(&value, &wide, 4);
    return value;
}

/* Round-to-nearest-even fp32 -> fp16 (IEEE binary16), what `half::f16::from_f32` does for the
 * operands of examples/src/gemm_sol.rs:1241-1249. Handles normals, subnormals, overflow to
 * infinity and NaN. */
uint16_t fko_to_f16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    const uint32_t sign = (bits >> 16) & 0x8000u;
    const uint32_t magnitude = bits & 0x7fffffffu;
    if (magnitude >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (magnitude > 0x7f800000u ? 0x200u : 0u));
    if (magnitude >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* rounds to >= 65520: infinity */
    if (magnitude < 0x38800000u) {                                   /* below 2^-14: subnormal */
        if (magnitude < 0x33000000u) return (uint16_t)sign;          /* below 2^-25: zero */
        const uint32_t shift = 126u - (magnitude >> 23);             /* 14..24 */
        const uint32_t mantissa = (magnitude & 0x7fffffu) | 0x800000u;
        const uint32_t kept = mantissa >> shift;
        const uint32_t rest = mantissa & ((1u << shift) - 1u), halfway = 1u << (shift - 1u);
        return (uint16_t)(sign | (kept + ((rest > halfway || (rest == halfway && (kept & 1u))) ? 1u : 0u)));
    }
    const uint32_t rebased = magnitude - 0x38000000u; /* exponent bias 127 -> 15 */
    const uint32_t kept = rebased >> 13, rest = rebased & 0x1fffu;
    return (uint16_t)(sign | (kept + ((rest > 0x1000u || (rest == 0x1000u && (kept & 1u))) ? 1u : 0u)));
}

/* What the copy engine's reduce-add leaves in a bf16 destination: the sum of the two bf16
 * values rounded once to bf16 (`tma_store_add_2d`, src/shared.rs:974-1009: "the add happens at
 * the destination in the element's own type ... with round-to-nearest"). The sum is formed in
 * double, where it is exact for operands within 2^40 of each other. */
uint16_t fko_bf16_add(uint16_t held, uint16_t added) {
    const double sum = (double)fko_from_bf16(held) + (double)fko_from_bf16(added);
    /* double -> bf16 in one rounding: go through the bit pattern of the double. */
    uint64_t bits;
    memcpy(&bits, &sum, 8);
    const uint64_t sign = bits >> 63;
    const int64_t exponent = (int64_t)((bits >> 52) & 0x7ff) - 1023;
    if (sum == 0.0) return (uint16_t)(sign << 15);
    if (exponent > 127) return (uint16_t)((sign << 15) | 0x7f80u);
    if (exponent < -126) return fko_to_bf16((float)sum); /* subnormal range: not reached by the tests */
    const uint64_t mantissa = bits & 0xfffffffffffffull; /* 52 bits; keep 7 */
    uint64_t kept = mantissa >> 45;
    const uint64_t rest = mantissa & ((1ull << 45) - 1), halfway = 1ull << 44;
    uint64_t biased = (uint64_t)(exponent + 127);
    if (rest > halfway || (rest == halfway && (kept & 1))) {
        if (++kept == 128) {
            kept = 0;
            ++biased;
        }
    }
    if (biased >= 255) return (uint16_t)((sign << 15) | 0x7f80u);
    return (uint16_t)((sign << 15) | (biased << 7) | kept);
}

/* ---------------------------------------------------------------- GEMM operands */

/* `exp2_approx` (src/reg.rs:81-93): clamp to +-125, split x = n + f with f in [-0.5, 0.5] by the
 * 1.5 * 2^23 shift, a degree-3 polynomial for 2^f (C0..C3 as the reference spells them), n added into
 * the exponent field. Plain fp32 multiplies and adds in the reference's order, no fused operations:
 * compile with -ffp-contract=off semantics in mind (the expression below is written so that a
 * contraction cannot change it: every product is stored to a float first). The reference's own
 * test holds it to a relative error under 1e-4 over [-125, 125] (src/reg.rs:2047-2062). */
float fko_exp2_approx(float x) {
    const float shift = 12582912.0f; /* 1.5 * 2^23 */
    const float c0 = 0.99992807f, c1 = 0.69326099f, c2 = 0.24261112f, c3 = 0.05517167f;
    x = fminf(fmaxf(x, -125.0f), 125.0f);
    volatile float shifted = x + shift;
    uint32_t shifted_bits;
    float shifted_value = shifted;
    memcpy(&shifted_bits, &shifted_value, sizeof shifted_bits);
    const int32_t integer = (int32_t)shifted_bits - 0x4b400000;
    volatile float whole = shifted_value - shift;
    volatile float fraction = x - whole;
    volatile float t3 = fraction * c3;
    volatile float s2 = c2 + t3;
    volatile float t2 = fraction * s2;
    volatile float s1 = c1 + t2;
    volatile float t1 = fraction * s1;
    volatile float poly = c0 + t1;
    float poly_value = poly;
    uint32_t poly_bits;
    memcpy(&poly_bits, &poly_value, sizeof poly_bits);
    poly_bits = (uint32_t)((int32_t)poly_bits + (int32_t)((uint32_t)integer << 23));
    float out;
    memcpy(&out, &poly_bits, sizeof out);
    return out;
}

/* examples/src/gemm.rs:434-436 */
float fko_gemm_a_value(size_t row, size_t depth) { return (float)((row * 5 + depth * 3) % 7) - 3.0f; }

/* examples/src/gemm.rs:438-440 */
float fko_gemm_b_value(size_t column, size_t depth) {
    return (float)((column * 4 + depth * 5) % 21) - 10.0f;
}

/* examples/src/gemm.rs:455-464 -- a [rows, k] operand as bf16 words, K contiguous
 * (the reference packs two per u32, low half first: the same bytes). */
void fko_gemm_stage(int which, size_t rows, size_t k, uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (size_t row = 0; row < rows; ++row)
        for (size_t depth = 0; depth < k; ++depth)
            out[row * k + depth] =
                fko_to_bf16(which == 0 ? fko_gemm_a_value(row, depth) : fko_gemm_b_value(row, depth));
}

/* examples/src/gemm_sol.rs:1241-1249 -- the same operands staged as fp16 words. */
void fko_gemm_stage_f16(int which, size_t rows, size_t k, uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (size_t row = 0; row < rows; ++row)
        for (size_t depth = 0; depth < k; ++depth)
            out[row * k + depth] =
                fko_to_f16(which == 0 ? fko_gemm_a_value(row, depth) : fko_gemm_b_value(row, depth));
}

/* examples/src/gemm.rs:544-578 -- compare an observed bf16 C element by element
 * with == against the 7 x 21 distinct dot products the operands' periods leave.
 * Returns the number of wrong elements; *worst receives the worst relative
 * error against the exact fp32 value; first_wrong (may be null) the flat index
 * of the first mismatch. */
size_t fko_gemm_check_c(const uint16_t* observed, size_t m, size_t n, size_t k, double* worst,
                        size_t* first_wrong) {
    float exact[7 * 21];
    uint16_t reference[7 * 21];
    for (size_t cell = 0; cell < 7 * 21; ++cell) {
        float sum = 0.0f;
        for (size_t depth = 0; depth < k; ++depth)
            sum += fko_gemm_a_value(cell / 21, depth) * fko_gemm_b_value(cell % 21, depth);
        exact[cell] = sum;
        reference[cell] = fko_to_bf16(sum);
    }
    size_t wrong = 0, first = (size_t)-1;
    double worst_seen = 0.0;
    for (size_t row = 0; row < m; ++row) {
        for (size_t column = 0; column < n; ++column) {
            const size_t cell = (row % 7) * 21 + column % 21;
            const uint16_t value = observed[row * n + column];
            if (value != reference[cell]) {
                if (wrong == 0) first = row * n + column;
                ++wrong;
            }
            if (exact[cell] != 0.0f) {
                const double error = fabs((double)(fko_from_bf16(value) - exact[cell]) / (double)exact[cell]);
                if (error > worst_seen) worst_seen = error;
            }
        }
    }
    if (worst) *worst = worst_seen;
    if (first_wrong) *first_wrong = first;
    return wrong;
}

/* The reference value of one cell, for a caller that wants the expected C. */
uint16_t fko_gemm_expected(size_t row, size_t column, size_t k) {
    float sum = 0.0f;
    for (size_t depth = 0; depth < k; ++depth)
        sum += fko_gemm_a_value(row % 7, depth) * fko_gemm_b_value(column % 21, depth);
    return fko_to_bf16(sum);
}

/* The same cell before its rounding: the running fp32 sum check_c's `exact` holds (:545-551), for the
 * fused epilogue's oracle (bias and unary map apply to this value, then one rounding). */
float fko_gemm_exact(size_t row, size_t column, size_t k) {
    float sum = 0.0f;
    for (size_t depth = 0; depth < k; ++depth)
        sum += fko_gemm_a_value(row % 7, depth) * fko_gemm_b_value(column % 21, depth);
    return sum;
}

/* ---------------------------------------------------------------- GEMM over arbitrary bf16 inputs
 *
 * The same contraction check_c's `exact` performs (:545-551: a running fp32
 * sum over depth of a*b, then one rounding to bf16), over caller-supplied
 * bf16 operands: rows [row0, row0+rows) of C = A . B^T, A [m, k], B [n, k].
 * c_bf16 and/or c_f64 may be null; c_f64 receives the f64-accumulated value
 * for error bounds. Output buffers hold `rows * n` elements.
 */
void fko_gemm_rows(const uint16_t* a, const uint16_t* b, size_t n, size_t k, size_t row0, size_t rows,
                   uint16_t* c_bf16, double* c_f64) {
    /* Widen the slab of A once; B rows are widened per column block. */
    float* a_wide = (float*)malloc(rows * k * sizeof(float));
    for (size_t i = 0; i < rows * k; ++i) a_wide[i] = fko_from_bf16(a[row0 * k + i]);
#pragma omp parallel
    {
        float* b_wide = (float*)malloc(k * sizeof(float));
#pragma omp for schedule(dynamic, 16)
        for (size_t column = 0; column < n; ++column) {
            for (size_t depth = 0; depth < k; ++depth) b_wide[depth] = fko_from_bf16(b[column * k + depth]);
            for (size_t row = 0; row < rows; ++row) {
                const float* a_row = a_wide + row * k;
                if (c_bf16) {
                    float sum = 0.0f;
                    for (size_t depth = 0; depth < k; ++depth) sum += a_row[depth] * b_wide[depth];
                    c_bf16[row * n + column] = fko_to_bf16(sum);
                }
                if (c_f64) {
                    double sum = 0.0;
                    for (size_t depth = 0; depth < k; ++depth) sum += (double)a_row[depth] * (double)b_wide[depth];
                    c_f64[row * n + column] = sum;
                }
            }
        }
        free(b_wide);
    }
    free(a_wide);
}

/* ---------------------------------------------------------------- attention operands */

/* examples/src/flash_forward.rs:326-334 */
static size_t permutation(size_t tensor, size_t head, size_t row, size_t column) {
    const size_t stride = 11 + 2 * ((row + 17 * tensor) % 63);
    return (53 * head + 37 * row + stride * column + 71 * tensor) % 128;
}
size_t fko_flash_permutation(size_t tensor, size_t head, size_t row, size_t column) {
    return permutation(tensor, head, row, column);
}

/* examples/src/flash_forward.rs:341-347 */
float fko_flash_q_value(size_t head, size_t row, size_t dim) {
    return dim == 0 ? 2.0f : ((float)permutation(0, head, row, dim) - 64.0f) / 64.0f;
}
/* examples/src/flash_forward.rs:349-355 */
float fko_flash_k_value(size_t head, size_t row, size_t dim) {
    return dim == 0 ? (float)row / 8.0f : ((float)permutation(1, head, row, dim) - 64.0f) / 64.0f;
}
/* examples/src/flash_forward.rs:360-362 */
float fko_flash_v_value(size_t head, size_t row, size_t dim) {
    return 1.0f + (float)permutation(2, head, row, dim) / 64.0f;
}

/* examples/src/flash_forward.rs:382-393 -- [heads, sequence, 128] bf16, head-major. */
void fko_flash_stage(int which, size_t sequence, size_t heads, uint16_t* out) {
    for (size_t head = 0; head < heads; ++head)
        for (size_t row = 0; row < sequence; ++row)
            for (size_t dim = 0; dim < 128; ++dim) {
                const float value = which == 0   ? fko_flash_q_value(head, row, dim)
                                    : which == 1 ? fko_flash_k_value(head, row, dim)
                                                 : fko_flash_v_value(head, row, dim);
                out[(head * sequence + row) * 128 + dim] = fko_to_bf16(value);
            }
}

/* examples/src/flash_forward.rs:419-440 -- the straightforward stable softmax
 * times V for query rows [row0, row0+rows) of one [sequence, 128] plane, in
 * f64 over the bf16 inputs: scores, subtract the row max, exponentiate, weight
 * V, divide by the sum. The reference is causal only (keys 0..=row); `causal`
 * == 0 attends all `sequence` keys, which is the same function over a longer
 * key range. lse (may be null) receives max + ln(sum), the natural-log
 * normaliser the row's softmax divides by.
 */
void fko_flash_rows(const uint16_t* q, const uint16_t* k, const uint16_t* v, size_t sequence,
                    size_t row0, size_t rows, double scale, int causal, double* out, double* lse) {
#pragma omp parallel
    {
        double* weights = (double*)malloc(sequence * sizeof(double));
#pragma omp for schedule(dynamic, 4)
        for (size_t r = 0; r < rows; ++r) {
            const size_t row = row0 + r;
            const size_t keys = causal ? row + 1 : sequence;
            double qw[128];
            for (size_t d = 0; d < 128; ++d) qw[d] = (double)fko_from_bf16(q[row * 128 + d]);
            double max = -INFINITY;
            for (size_t key = 0; key < keys; ++key) {
                double dot = 0.0;
                for (size_t d = 0; d < 128; ++d) dot += qw[d] * (double)fko_from_bf16(k[key * 128 + d]);
                weights[key] = scale * dot;
                if (weights[key] > max) max = weights[key];
            }
            double total = 0.0;
            for (size_t key = 0; key < keys; ++key) {
                weights[key] = exp(weights[key] - max);
                total += weights[key];
            }
            double acc[128];
            for (size_t d = 0; d < 128; ++d) acc[d] = 0.0;
            for (size_t key = 0; key < keys; ++key) {
                const double w = weights[key];
                for (size_t d = 0; d < 128; ++d) acc[d] += w * (double)fko_from_bf16(v[key * 128 + d]);
            }
            for (size_t d = 0; d < 128; ++d) out[r * 128 + d] = acc[d] / total;
            if (lse) lse[r] = max + log(total);
        }
        free(weights);
    }
}

/* ---------------------------------------------------------------- row kernels */

/* examples/src/softmax.rs:195-202 -- every row a permutation of the multiples of 1/8 below 16. */
static size_t softmax_permutation(size_t plane, size_t row, size_t column) {
    const size_t stride = 11 + 2 * (row / 128 % 63);
    return (53 * plane + 37 * row + stride * column) % 128;
}
float fko_softmax_input(size_t plane, size_t row, size_t column) {
    return (float)softmax_permutation(plane, row, column) / 8.0f;
}
/* examples/src/softmax.rs:204-215 -- [planes, rows, 128] bf16. */
void fko_softmax_stage(size_t rows, size_t planes, uint16_t* out) {
    for (size_t plane = 0; plane < planes; ++plane)
        for (size_t row = 0; row < rows; ++row)
            for (size_t column = 0; column < 128; ++column)
                out[(plane * rows + row) * 128 + column] = fko_to_bf16(fko_softmax_input(plane, row, column));
}
/* The closed form the reference checks its seed against (:276-279): weight 2^(p/8 - 127/8) over
 * the sum of all 128 weights. */
double fko_softmax_expected(size_t plane, size_t row, size_t column) {
    double total = 0.0;
    for (size_t value = 0; value < 128; ++value) total += exp2((double)value / 8.0 - 127.0 / 8.0);
    return exp2((double)softmax_permutation(plane, row, column) / 8.0 - 127.0 / 8.0) / total;
}
/* The kernel's function over arbitrary bf16 rows (softmax.rs:137-160), in f64:
 * 2^(x - max) / sum over the 128 columns of each row. */
void fko_softmax_rows(const uint16_t* x, size_t rows, double* out) {
#pragma omp parallel for schedule(static)
    for (size_t row = 0; row < rows; ++row) {
        double peak = -INFINITY, total = 0.0;
        for (size_t c = 0; c < 128; ++c) {
            const double v = (double)fko_from_bf16(x[row * 128 + c]);
            if (v > peak) peak = v;
        }
        for (size_t c = 0; c < 128; ++c) {
            out[row * 128 + c] = exp2((double)fko_from_bf16(x[row * 128 + c]) - peak);
            total += out[row * 128 + c];
        }
        for (size_t c = 0; c < 128; ++c) out[row * 128 + c] /= total;
    }
}

/* examples/src/layernorm.rs:330-352 -- the seed and the parameter vectors. */
static size_t layernorm_permutation(size_t row, size_t column) {
    const size_t stride = 11 + 2 * (row / 128 % 63);
    return (37 * row + stride * column) % 128;
}
float fko_layernorm_value(size_t p, size_t row) {
    const float magnitude = 16.0f + (float)(p % 32) / 2.0f;
    const float boost = (float)(1 << (1 + row % 3));
    const float sign[4] = {1.0f, -0.5f, boost, -boost / 2.0f};
    return magnitude * sign[p / 32];
}
float fko_layernorm_input(size_t row, size_t column) {
    return fko_layernorm_value(layernorm_permutation(row, column), row);
}
float fko_layernorm_gamma(size_t column) { return 1.0f + (float)column / 128.0f; }
float fko_layernorm_beta(size_t column) { return 2.0f + (float)column / 64.0f; }
void fko_layernorm_stage(size_t rows, uint16_t* x, uint16_t* gamma, uint16_t* beta) {
    for (size_t row = 0; row < rows; ++row)
        for (size_t column = 0; column < 128; ++column)
            x[row * 128 + column] = fko_to_bf16(fko_layernorm_input(row, column));
    for (size_t column = 0; column < 128; ++column) {
        gamma[column] = fko_to_bf16(fko_layernorm_gamma(column));
        beta[column] = fko_to_bf16(fko_layernorm_beta(column));
    }
}
/* examples/src/layernorm.rs:354-360, 425-433 -- per-row statistics in f64, population variance,
 * gamma * (x - mean) / sqrt(var + eps) + beta; over arbitrary bf16 inputs. */
void fko_layernorm_rows(const uint16_t* x, const uint16_t* gamma, const uint16_t* beta, size_t rows,
                        double epsilon, double* out) {
#pragma omp parallel for schedule(static)
    for (size_t row = 0; row < rows; ++row) {
        double mean = 0.0, variance = 0.0;
        for (size_t c = 0; c < 128; ++c) mean += (double)fko_from_bf16(x[row * 128 + c]);
        mean /= 128.0;
        for (size_t c = 0; c < 128; ++c) {
            const double d = (double)fko_from_bf16(x[row * 128 + c]) - mean;
            variance += d * d;
        }
        const double deviation = 1.0 / sqrt(variance / 128.0 + epsilon);
        for (size_t c = 0; c < 128; ++c)
            out[row * 128 + c] = (double)fko_from_bf16(gamma[c]) *
                                     (((double)fko_from_bf16(x[row * 128 + c]) - mean) * deviation) +
                                 (double)fko_from_bf16(beta[c]);
    }
}
/* examples/src/layernorm.rs:480-489, 560-566 -- the same statistic over each [128, 128] tile. */
void fko_groupnorm_tiles(const uint16_t* x, size_t rows, double epsilon, double* out) {
#pragma omp parallel for schedule(static)
    for (size_t tile = 0; tile < rows / 128; ++tile) {
        const uint16_t* in = x + tile * 128 * 128;
        double mean = 0.0, variance = 0.0;
        for (size_t i = 0; i < 128 * 128; ++i) mean += (double)fko_from_bf16(in[i]);
        mean /= 128.0 * 128.0;
        for (size_t i = 0; i < 128 * 128; ++i) {
            const double d = (double)fko_from_bf16(in[i]) - mean;
            variance += d * d;
        }
        const double deviation = 1.0 / sqrt(variance / (128.0 * 128.0) + epsilon);
        for (size_t i = 0; i < 128 * 128; ++i)
            out[tile * 128 * 128 + i] = ((double)fko_from_bf16(in[i]) - mean) * deviation;
    }
}

/* ---------------------------------------------------------------- attention backward
 *
 * The gradients of the function fko_flash_rows computes, for one [sequence, 128] plane, in f64
 * over bf16 inputs: P from the stable softmax of the scaled scores, dV = P^T dO, dP = dO V^T,
 * dS = P * (dP - rowsum(P * dP)), dQ = scale dS K, dK = scale dS^T Q. The reference has no
 * backward; this restates the textbook derivative of its forward (examples/src/flash_forward.rs:419-440).
 */
void fko_flash_backward(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* d_out,
                        size_t sequence, double scale, int causal, double* dq, double* dk, double* dv) {
    for (size_t i = 0; i < sequence * 128; ++i) dq[i] = dk[i] = dv[i] = 0.0;
    double* weights = (double*)malloc(sequence * sizeof(double));
    double* slopes = (double*)malloc(sequence * sizeof(double));
    for (size_t row = 0; row < sequence; ++row) {
        const size_t keys = causal ? row + 1 : sequence;
        double qw[128], gw[128];
        for (size_t d = 0; d < 128; ++d) {
            qw[d] = (double)fko_from_bf16(q[row * 128 + d]);
            gw[d] = (double)fko_from_bf16(d_out[row * 128 + d]);
        }
        double max = -INFINITY, total = 0.0, inner = 0.0;
        for (size_t key = 0; key < keys; ++key) {
            double dot = 0.0, slope = 0.0;
            for (size_t d = 0; d < 128; ++d) {
                dot += qw[d] * (double)fko_from_bf16(k[key * 128 + d]);
                slope += gw[d] * (double)fko_from_bf16(v[key * 128 + d]);
            }
            weights[key] = scale * dot;
            slopes[key] = slope;
            if (weights[key] > max) max = weights[key];
        }
        for (size_t key = 0; key < keys; ++key) {
            weights[key] = exp(weights[key] - max);
            total += weights[key];
        }
        for (size_t key = 0; key < keys; ++key) {
            weights[key] /= total;
            inner += weights[key] * slopes[key];
        }
        for (size_t key = 0; key < keys; ++key) {
            const double p = weights[key], ds = scale * p * (slopes[key] - inner);
            for (size_t d = 0; d < 128; ++d) {
                dv[key * 128 + d] += p * gw[d];
                dq[row * 128 + d] += ds * (double)fko_from_bf16(k[key * 128 + d]);
                dk[key * 128 + d] += ds * qw[d];
            }
        }
    }
    free(weights);
    free(slopes);
}
