/*
 * CPU oracle for the FP8 skinny GEMM. TEST INFRASTRUCTURE ONLY: it is the checker for the CUDA
 * path (tests/, the smoke check, and the CPU-baseline leg of the benchmark) and is never called,
 * linked or loaded by the shipped library or the Python package.
 *
 * It restates, in plain C, the arithmetic the reference (huggingface/hf-rocm-kernels) defines
 * for this path:
 *   - quantisation to fp8:   hf_rocm_kernels/utils/fp8.py:17-29
 *         q = clamp(x * (1/scale), -448, 448) -> e4m3fn (round to nearest even); the byte 0x80
 *         (-0) becomes 0x00; the same byte reinterpreted as e4m3fnuz is worth half as much.
 *   - the expected result:   hf_rocm_kernels/operators/skinny_gemm/reference.py:18-25
 *         out = cast(scale_a * scale_b * (A . B))   (torch._scaled_mm there)
 *   - the in-place contract: hf_rocm_kernels/operators/skinny_gemm/wrapped.py:115 and
 *     csrc/op_src/skinny_gemm/consumers/mfma_16x16x32_consumer.cu:113-168
 *         D <- D_in + scale * (A . W^T), D_in being zeros or the broadcast bias.
 *
 * Parity pin: the reference holds no golden vectors for this path (its own test is a
 * differential test against torch._scaled_mm on an AMD GPU, tests/test_skinny_gemm.py:21-36).
 * The quantiser here is pinned bit-for-bit against outputs of the reference's own fp8.py run on
 * CPU, and the GEMM against torch._scaled_mm (the function the reference calls) run on CPU on
 * the same bytes; both sets of vectors live in tests/golden/.
 *
 * Two accumulations are offered. "exact" sums in double: every e4m3 x e4m3 product is a
 * multiple of 2^-18 below 2^18 and K <= 2^15 of them sum without rounding in 53 bits, so the
 * double sum IS the mathematical dot product. "f32" sums in float in index order, a plain
 * "dequantised fp32 matmul on host".
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>

/* kind: 0 = e4m3fn (OCP: bias 7, 0x7f/0xff NaN, max 448), 1 = e4m3fnuz (bias 8, 0x80 NaN). */
float hfrk_oracle_fp8_to_f32(uint8_t bits, int kind) {
    const int sign = bits >> 7;
    const int exp = (bits >> 3) & 0xf;
    const int man = bits & 0x7;
    const int bias = kind == 1 ? 8 : 7;
    float v;
    if (kind == 1 && bits == 0x80) return NAN;
    if (kind == 0 && exp == 15 && man == 7) return NAN;
    if (exp == 0) {
        v = ldexpf((float)man, 1 - bias - 3);
    } else {
        v = ldexpf((float)(8 + man), exp - bias - 3);
    }
    return sign ? -v : v;
}

void hfrk_oracle_fp8_table(float* table256, int kind) {
    for (int i = 0; i < 256; ++i) table256[i] = hfrk_oracle_fp8_to_f32((uint8_t)i, kind);
}

/* Round-to-nearest-even conversion of a finite float in [-448, 448] to e4m3fn bits. */
static uint8_t f32_to_e4m3fn_rne(float x) {
    const uint8_t sign = signbit(x) ? 0x80 : 0x00;
    float a = fabsf(x);
    if (isnan(a)) return (uint8_t)(sign | 0x7f);
    if (a > 448.0f) a = 448.0f;
    int e;
    (void)frexpf(a, &e);          /* a = f * 2^e, f in [0.5, 1) -> unbiased exponent e - 1 */
    int ue = e - 1;
    if (a == 0.0f || ue < -6) ue = -6; /* subnormal range shares the exponent of the smallest normal */
    const float quantum = ldexpf(1.0f, ue - 3);
    /* a / quantum is exact (power-of-two scaling); nearbyintf rounds half to even by default. */
    float steps = nearbyintf(a / quantum);
    if (steps >= 16.0f) { /* rounded up into the next binade */
        steps = 8.0f;
        ue += 1;
    }
    uint8_t bits;
    if (steps < 8.0f) {
        bits = (uint8_t)steps; /* subnormal (ue == -6): exponent field 0 */
    } else {
        bits = (uint8_t)(((ue + 7) << 3) | ((int)steps - 8));
    }
    return (uint8_t)(sign | bits);
}

/* fp8_quantize of the reference (utils/fp8.py:17-29). Writes the bytes; the value of a byte is
 * hfrk_oracle_fp8_to_f32(byte, 0) when read as e4m3fn, half of that when read as e4m3fnuz
 * (zero_negative_zero = 1 reproduces the reference's 0x80 -> 0x00 step). */
void hfrk_oracle_quantize(const float* x, int64_t count, float scale, int zero_negative_zero, uint8_t* out) {
    const float inv = 1.0f / scale;
    for (int64_t i = 0; i < count; ++i) {
        float v = x[i] * inv;
        if (v < -448.0f) v = -448.0f;
        if (v > 448.0f) v = 448.0f;
        uint8_t b = f32_to_e4m3fn_rne(v);
        if (zero_negative_zero && b == 0x80) b = 0x00;
        out[i] = b;
    }
}

/* ref[m][n] = d_in[m][n] + scale * sum_k A[m][k] * W[n][k]
 *   A : m x k bytes, contiguous          W : n rows of k bytes, pitch w_row_stride
 *   d_in : m x n floats or NULL (zeros)  ref : m x n floats
 *   exact = 1: the sum is taken in double and rounded once to float, then the scale and d_in are
 *              applied in float with one fused multiply-add (what the CUDA epilogue does);
 *   exact = 0: float accumulation in index order.
 * scale is the caller's scale times 0.5 per e4m3fnuz operand, applied by the caller.
 * Columns are shared out over hfrk_oracle_set_num_threads() POSIX threads. */
typedef struct {
    const uint8_t* W;
    const float* a32;
    const float* d_in;
    const float* table;
    float* ref;
    float scale;
    int m, n, k, exact, col_begin, col_end;
    int64_t w_row_stride;
} oracle_job;

static void* oracle_worker(void* arg) {
    const oracle_job* job = (const oracle_job*)arg;
    const int m = job->m, n = job->n, k = job->k;
    float* w32 = (float*)malloc((size_t)k * sizeof(float));
    for (int col = job->col_begin; col < job->col_end; ++col) {
        const uint8_t* w_row = job->W + (size_t)col * job->w_row_stride;
        for (int kk = 0; kk < k; ++kk) w32[kk] = job->table[w_row[kk]];
        for (int row = 0; row < m; ++row) {
            const float* a_row = job->a32 + (size_t)row * k;
            float dot;
            if (job->exact) {
                /* Exact sums do not depend on the order, so eight independent lanes (which the
                 * compiler may keep in vector registers) give the same double as one. */
                double lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                int kk = 0;
                for (; kk + 8 <= k; kk += 8) {
                    for (int l = 0; l < 8; ++l) lanes[l] += (double)a_row[kk + l] * (double)w32[kk + l];
                }
                double acc = 0.0;
                for (; kk < k; ++kk) acc += (double)a_row[kk] * (double)w32[kk];
                for (int l = 0; l < 8; ++l) acc += lanes[l];
                dot = (float)acc;
            } else {
                float acc = 0.0f;
                for (int kk = 0; kk < k; ++kk) acc += a_row[kk] * w32[kk];
                dot = acc;
            }
            const float base = job->d_in ? job->d_in[(size_t)row * n + col] : 0.0f;
            job->ref[(size_t)row * n + col] = fmaf(dot, job->scale, base);
        }
    }
    free(w32);
    return NULL;
}

static int g_threads = 1;

int hfrk_oracle_num_threads(void) { return g_threads; }

void hfrk_oracle_set_num_threads(int threads) {
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    g_threads = threads;
}

void hfrk_oracle_skinny_gemm(const uint8_t* A, const uint8_t* W, const float* d_in, float scale, int m, int n,
                             int k, int64_t w_row_stride, int exact, float* ref) {
    float table[256];
    hfrk_oracle_fp8_table(table, 0);
    float* a32 = (float*)malloc((size_t)m * k * sizeof(float));
    for (int64_t i = 0; i < (int64_t)m * k; ++i) a32[i] = table[A[i]];

    int threads = g_threads < n ? g_threads : n;
    if (threads < 1) threads = 1;
    oracle_job jobs[256];
    pthread_t handles[256];
    const int per = (n + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        oracle_job* j = &jobs[t];
        j->W = W; j->a32 = a32; j->d_in = d_in; j->table = table; j->ref = ref; j->scale = scale;
        j->m = m; j->n = n; j->k = k; j->exact = exact; j->w_row_stride = w_row_stride;
        j->col_begin = t * per < n ? t * per : n;
        j->col_end = (t + 1) * per < n ? (t + 1) * per : n;
    }
    for (int t = 1; t < threads; ++t) pthread_create(&handles[t], NULL, oracle_worker, &jobs[t]);
    oracle_worker(&jobs[0]);
    for (int t = 1; t < threads; ++t) pthread_join(handles[t], NULL);
    free(a32);
}
