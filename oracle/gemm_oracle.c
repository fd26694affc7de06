/*
 * CPU oracle for D = alpha * A * B^T + beta * C  (TEST INFRASTRUCTURE, never a product path).
 *
 * A is m x k row-major, Bt is B stored transposed as n x k row-major, C and D are m x n row-major
 * fp32. Inputs are IEEE fp16 or bfloat16 bit patterns (uint16_t); accumulation is fp32.
 *
 * The arithmetic restates the reference's host check, matmul_test.h:294-298 and :316-320
 * (MatmulTestGemmSquare::IsCorrect / GetNumIncorrect):
 *
 *     temp = 0;  for k in 0..K-1 (ascending):  temp += float(A[i*K+k]) * float(Bt[j*K+k]);
 *     D[i*N+j] = alpha * temp + beta * C[i*N+j];
 *
 * with every operation rounded to fp32 separately (no fused multiply-add; build with
 * -ffp-contract=off). The reference indexes Bt with pitch dim.n (matmul_test.h:296,318), which
 * equals K only for its square problems; this file uses pitch K so m != n != k works.
 *
 * Only tests, the smoke check and the bench's CPU-baseline legs may call this file. The
 * shipped library has no CPU path.
 *
 * Parity is pinned: tests/golden holds outputs of this file that were checked element-for-element
 * (tolerance 0) against the reference's own GetNumIncorrect compiled from matmul_test.h
 * (oracle/ref_driver.cpp -> oracle/_ref/libref_matmul.so).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---------- input-type decoding -------------------------------------------------------- */

static inline float half_bits_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: value = man * 2^-24, exact in fp32 */
            float f = (float)man * 5.9604644775390625e-8f;
            memcpy(&bits, &f, 4);
            bits |= sign;
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

static inline float bf16_bits_to_float(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

/* dtype: 0 = fp16, 1 = bf16 */
static inline float decode(uint16_t v, int dtype) {
    return dtype ? bf16_bits_to_float(v) : half_bits_to_float(v);
}

void oracle_to_float(const uint16_t *src, float *dst, int64_t count, int dtype) {
    for (int64_t i = 0; i < count; ++i) dst[i] = decode(src[i], dtype);
}

/* ---------- the matmul ------------------------------------------------------------------ */

/* Scalar form, literally the reference's triple loop (matmul_test.h:312-320). Used for small
 * cases and to validate the blocked form below. */
void oracle_gemm_scalar(const uint16_t *A, const uint16_t *Bt, const float *C, float *D,
                        float alpha, float beta, int64_t M, int64_t N, int64_t K, int dtype) {
    for (int64_t i = 0; i < M; ++i) {
        for (int64_t j = 0; j < N; ++j) {
            float temp = 0.0f;
            for (int64_t k = 0; k < K; ++k) {
                temp += decode(A[i * K + k], dtype) * decode(Bt[j * K + k], dtype);
            }
            D[i * N + j] = alpha * temp + beta * (C ? C[i * N + j] : 0.0f);
        }
    }
}

/* Row-range form. Each output element still sees the same ascending-k chain of separately
 * rounded multiply and add, so results are bit-identical to oracle_gemm_scalar; only the loop
 * nest differs: B is pre-transposed to k x n fp32 so that the compiler can carry JB independent
 * accumulation chains (different j) through the k loop. Rows [row_begin, row_end) of D are
 * produced; threads (OpenMP) split rows. Returns 0, or -1 if memory could not be had. */
#define JB 64
int oracle_gemm_rows(const uint16_t *A, const uint16_t *Bt, const float *C, float *D,
                     float alpha, float beta, int64_t M, int64_t N, int64_t K, int dtype,
                     int64_t row_begin, int64_t row_end, int num_threads) {
    (void)M;
    float *Bf = (float *)malloc((size_t)K * (size_t)N * sizeof(float)); /* k x n */
    if (!Bf) return -1;
#ifdef _OPENMP
    if (num_threads > 0) omp_set_num_threads(num_threads);
#else
    (void)num_threads;
#endif
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < N; ++j)
        for (int64_t k = 0; k < K; ++k) Bf[k * N + j] = decode(Bt[j * K + k], dtype);

#pragma omp parallel
    {
        float *arow = (float *)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(dynamic, 1)
        for (int64_t i = row_begin; i < row_end; ++i) {
            for (int64_t k = 0; k < K; ++k) arow[k] = decode(A[i * K + k], dtype);
            for (int64_t j0 = 0; j0 < N; j0 += JB) {
                int64_t jn = (N - j0 < JB) ? (N - j0) : JB;
                float acc[JB];
                for (int64_t jj = 0; jj < JB; ++jj) acc[jj] = 0.0f;
                if (jn == JB) {
                    for (int64_t k = 0; k < K; ++k) {
                        const float a = arow[k];
                        const float *b = Bf + k * N + j0;
                        for (int jj = 0; jj < JB; ++jj) acc[jj] += a * b[jj];
                    }
                } else {
                    for (int64_t k = 0; k < K; ++k) {
                        const float a = arow[k];
                        const float *b = Bf + k * N + j0;
                        for (int64_t jj = 0; jj < jn; ++jj) acc[jj] += a * b[jj];
                    }
                }
                for (int64_t jj = 0; jj < jn; ++jj) {
                    int64_t o = i * N + j0 + jj;
                    D[o] = alpha * acc[jj] + beta * (C ? C[o] : 0.0f);
                }
            }
        }
        free(arow);
    }
    free(Bf);
    return 0;
}

int oracle_gemm(const uint16_t *A, const uint16_t *Bt, const float *C, float *D, float alpha,
                float beta, int64_t M, int64_t N, int64_t K, int dtype, int num_threads) {
    return oracle_gemm_rows(A, Bt, C, D, alpha, beta, M, N, K, dtype, 0, M, num_threads);
}

/* Scattered elements in fp32 (reference order) and in fp64 (to show how much of a deviation is
 * the reference's own rounding). idx holds `count` linear indices i*N+j. */
void oracle_gemm_elements(const uint16_t *A, const uint16_t *Bt, const float *C, float alpha,
                          float beta, int64_t N, int64_t K, int dtype, const int64_t *idx,
                          int64_t count, float *out32, double *out64) {
#pragma omp parallel for schedule(dynamic, 16)
    for (int64_t t = 0; t < count; ++t) {
        int64_t i = idx[t] / N, j = idx[t] % N;
        float temp = 0.0f;
        double temp64 = 0.0;
        for (int64_t k = 0; k < K; ++k) {
            float a = decode(A[i * K + k], dtype), b = decode(Bt[j * K + k], dtype);
            temp += a * b;
            temp64 += (double)a * (double)b;
        }
        float c = C ? C[idx[t]] : 0.0f;
        if (out32) out32[t] = alpha * temp + beta * c;
        if (out64) out64[t] = (double)alpha * temp64 + (double)beta * (double)c;
    }
}

/* ---------- comparison, in the reference's terms --------------------------------------- */

/* Count of elements with |expected - got| > atol: GetNumIncorrect's criterion
 * (matmul_test.h:320). NaN in either operand counts as incorrect here. */
int64_t oracle_count_incorrect(const float *expected, const float *got, int64_t count, float atol) {
    int64_t bad = 0;
    for (int64_t i = 0; i < count; ++i) {
        float d = fabsf(expected[i] - got[i]);
        if (!(d <= atol)) ++bad;
    }
    return bad;
}

/* Closed form for the constant-matrix correctness family (matmul_test.h:279-281):
 * alpha * (a*b) * K + beta * c, evaluated in fp32 in that order. */
float oracle_constant_expected(float a, float b, float c, float alpha, float beta, int64_t K) {
    return alpha * (a * b) * (float)K + beta * c;
}

/* ---------- seeded synthetic inputs ---------------------------------------------------- */
/* Independent restatement of the generator the library ships (synth.h in the package): a
 * counter-based hash, so element `index` of tensor `tensor_id` under `seed` can be produced
 * anywhere without materialising the rest. Tests check the two agree bit for bit. */

static inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

static inline uint64_t synth_key(uint64_t seed, uint64_t tensor_id) {
    return splitmix64(seed ^ (tensor_id * 0xD1B54A32D192ED03ull));
}

static inline uint64_t synth_hash(uint64_t key, uint64_t index, uint64_t lane) {
    return splitmix64(key + index * 0x9E3779B97F4A7C15ull + lane * 0xC2B2AE3D27D4EB4Full);
}

/* uniform in [-1, 1): 24 random bits b -> b * 2^-23 - 1 (exact in fp32) */
static inline float synth_uniform(uint64_t key, uint64_t index) {
    uint32_t b = (uint32_t)(synth_hash(key, index, 0) >> 40);
    return (float)b * 1.1920928955078125e-7f - 1.0f;
}

/* approximately N(0, sigma^2): sum of twelve 16-bit uniforms (Irwin-Hall), integer arithmetic
 * up to one final fp32 multiply, so host and device agree exactly. Support is +-6 sigma. */
static inline float synth_normal(uint64_t key, uint64_t index, float sigma) {
    int32_t s = 0;
    for (uint64_t lane = 1; lane <= 3; ++lane) {
        uint64_t h = synth_hash(key, index, lane);
        s += (int32_t)(h & 0xFFFF) + (int32_t)((h >> 16) & 0xFFFF) + (int32_t)((h >> 32) & 0xFFFF) +
             (int32_t)(h >> 48);
    }
    float z = (float)(s - 393210) * 1.52587890625e-5f; /* (sum - 12*65535/2) / 65536, exact */
    return z * sigma;
}

static inline uint16_t float_to_half_bits(float f) { /* round to nearest even */
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | ((ax > 0x7F800000u) ? 0x200u : 0u));
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to inf */
    if (ax < 0x33000001u) return (uint16_t)sign;               /* <= 2^-25 rounds to zero */
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7FFFFFu) | 0x800000u;
    uint32_t shift, hexp;
    if (e < -14) { shift = (uint32_t)(13 + (-14 - e)); hexp = 0; } else { shift = 13; hexp = (uint32_t)(e + 15); }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
    uint32_t out = (hexp == 0) ? q : (((hexp - 1u) << 10) + q); /* q carries the implicit bit */
    return (uint16_t)(sign | out);
}

static inline uint16_t float_to_bf16_bits(float f) { /* round to nearest even */
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7FFFu + lsb;
    return (uint16_t)(x >> 16);
}

/* dist: 0 = uniform[-1,1), 1 = normal(0, sigma). dtype: 0 = fp16, 1 = bf16. */
void oracle_fill_u16(uint16_t *dst, int64_t begin, int64_t count, uint64_t seed, uint64_t tensor_id,
                     int dist, float sigma, int dtype) {
    uint64_t key = synth_key(seed, tensor_id);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        uint64_t index = (uint64_t)(begin + i);
        float v = dist ? synth_normal(key, index, sigma) : synth_uniform(key, index);
        dst[i] = dtype ? float_to_bf16_bits(v) : float_to_half_bits(v);
    }
}

void oracle_fill_f32(float *dst, int64_t begin, int64_t count, uint64_t seed, uint64_t tensor_id,
                     int dist, float sigma) {
    uint64_t key = synth_key(seed, tensor_id);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        uint64_t index = (uint64_t)(begin + i);
        dst[i] = dist ? synth_normal(key, index, sigma) : synth_uniform(key, index);
    }
}

int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
