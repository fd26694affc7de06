// C entry points around the REFERENCE's own host check, compiled from the reference tree where it
// lies (the header is included, never copied): matmul_test.h, class MatmulTestGemmSquare, methods
// GetNumIncorrect (matmul_test.h:307-326) and IsCorrect (matmul_test.h:275-305).
//
// TEST INFRASTRUCTURE. Built only by oracle/Makefile into oracle/_ref/libref_matmul.so, and only
// where the reference tree is present. It is used (1) to pin oracle/gemm_oracle.c: the oracle's
// output is handed to GetNumIncorrect with atol = 0, and a count of 0 means every element equals
// what the reference's loop computes; (2) as the timed CPU baseline ("kind": "reference").
//
// The class owns its operands in private vectors sized dim_max^2 and only exposes const pointers
// (matmul_test.h:244-261); this driver writes seeded data through those pointers, which is what a
// harness that wanted reproducible inputs would have to do, the class itself seeding from the clock
// (matmul_test.h:239). The constant-value constructor is used because it does not call rand().
//
// The reference reads B^T with row pitch dim.n (matmul_test.h:318), so a problem handed to it
// must have n == k; m may be smaller (a slab of rows). dim_max must be >= n.

#include <cstdint>
#include <cstring>
#include <new>
#include "cuda_fp16.h"
#include "cuda_bf16.h"
#include "matmul_test.h"

namespace {

template <typename DT>
struct Session {
    matmul_test::MatmulTestGemmSquare<DT, float> mt;
    int n;
    explicit Session(int n_) : mt(n_, 64), n(n_) {}
};

template <typename DT>
void *create(int n) {
    return new (std::nothrow) Session<DT>(n);
}

template <typename DT>
int load(void *h, const uint16_t *A, const uint16_t *Bt, const float *C, int m) {
    Session<DT> *s = static_cast<Session<DT> *>(h);
    const size_t n = s->n;
    if (m < 0 || static_cast<size_t>(m) > n) return -1;
    std::memcpy(const_cast<DT *>(s->mt.GetA()), A, size_t(m) * n * sizeof(uint16_t));
    std::memcpy(const_cast<DT *>(s->mt.GetB()), Bt, n * n * sizeof(uint16_t));
    if (C) std::memcpy(const_cast<float *>(s->mt.GetC()), C, size_t(m) * n * sizeof(float));
    else std::memset(const_cast<float *>(s->mt.GetC()), 0, size_t(m) * n * sizeof(float));
    return 0;
}

template <typename DT>
int count_incorrect(void *h, const float *res, int m, float alpha, float beta, float atol) {
    Session<DT> *s = static_cast<Session<DT> *>(h);
    const size_t n = s->n;
    std::memcpy(s->mt.GetRes(), res, size_t(m) * n * sizeof(float));
    matmul_test::MatDim dim = {m, s->n, s->n};
    return s->mt.GetNumIncorrect(s->mt.GetRes(), dim, alpha, beta, atol);
}

}  // namespace

extern "C" {

// dtype: 0 = fp16 (the reference's DT = half), 1 = bf16 (instantiated with __nv_bfloat16; the
// reference never does, but its template accepts it and only float values are compared).
void *ref_create(int n, int dtype) { return dtype ? create<__nv_bfloat16>(n) : create<half>(n); }

void ref_destroy(void *h, int dtype) {
    if (dtype) delete static_cast<Session<__nv_bfloat16> *>(h);
    else delete static_cast<Session<half> *>(h);
}

// A: m x n, Bt: n x n, C: m x n or null (taken as zeros).
int ref_load(void *h, int dtype, const uint16_t *A, const uint16_t *Bt, const float *C, int m) {
    return dtype ? load<__nv_bfloat16>(h, A, Bt, C, m) : load<half>(h, A, Bt, C, m);
}

// Runs the reference's full recompute of the m x n result and returns how many elements of `res`
// differ from it by more than atol. This call IS the reference's CPU matmul; timing it times it.
int ref_count_incorrect(void *h, int dtype, const float *res, int m, float alpha, float beta, float atol) {
    return dtype ? count_incorrect<__nv_bfloat16>(h, res, m, alpha, beta, atol)
                 : count_incorrect<half>(h, res, m, alpha, beta, atol);
}

// The reference's own <half, half> check (every launcher is also instantiated with DT_ACC = half,
// matmul_shmem_tc_async.cu:411-478): the product accumulated IN HALF (each += rounds to fp16) and
// compared in half with Abs(half) (matmul_test.h:33, :316-320). A: m x n, Bt: n x n, C and res:
// m x n, all fp16 bit patterns; C may be null (zeros). Returns the count of elements off by more
// than atol.
int ref_half_count_incorrect(int n, const uint16_t *A, const uint16_t *Bt, const uint16_t *C, const uint16_t *res, int m,
                             float alpha, float beta, float atol) {
    matmul_test::MatmulTestGemmSquare<half, half> mt(n, 64);
    std::memcpy(const_cast<half *>(mt.GetA()), A, size_t(m) * n * 2);
    std::memcpy(const_cast<half *>(mt.GetB()), Bt, size_t(n) * n * 2);
    if (C) std::memcpy(const_cast<half *>(mt.GetC()), C, size_t(m) * n * 2);
    else std::memset(const_cast<half *>(mt.GetC()), 0, size_t(m) * n * 2);
    std::memcpy(mt.GetRes(), res, size_t(m) * n * 2);
    matmul_test::MatDim dim = {m, n, n};
    return mt.GetNumIncorrect(mt.GetRes(), dim, __float2half(alpha), __float2half(beta), __float2half(atol));
}

// The constant-matrix family (A = 1, B = 10, C = 1; matmul_test.h:227-232) judged by the
// reference's closed form (matmul_test.h:279-288). res is n x n. Returns 1 if correct.
int ref_constant_is_correct(const float *res, int n, float alpha, float beta, float atol) {
    matmul_test::MatmulTestGemmSquare<half, float> mt(n, 64);
    std::memcpy(mt.GetRes(), res, size_t(n) * n * sizeof(float));
    matmul_test::MatDim dim = {n, n, n};
    return mt.IsCorrect(mt.GetRes(), dim, alpha, beta, atol) ? 1 : 0;
}

}  // extern "C"
