// Stand-in for Apple's <Accelerate/Accelerate.h>, used only to compile the
// reference's CPU ops on Linux as a test oracle.  Plain loops with the
// documented vDSP / vForce / CBLAS semantics; nothing here is product code.
#pragma once
#include <cmath>
#include <cstddef>

typedef unsigned long vDSP_Length;
typedef long vDSP_Stride;

enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112 };

static inline void vDSP_vadd(const float *a, vDSP_Stride ia, const float *b, vDSP_Stride ib,
                             float *c, vDSP_Stride ic, vDSP_Length n) {
  for (vDSP_Length i = 0; i < n; ++i) c[i * ic] = a[i * ia] + b[i * ib];
}
static inline void vDSP_vmul(const float *a, vDSP_Stride ia, const float *b, vDSP_Stride ib,
                             float *c, vDSP_Stride ic, vDSP_Length n) {
  for (vDSP_Length i = 0; i < n; ++i) c[i * ic] = a[i * ia] * b[i * ib];
}
static inline void vDSP_vsmul(const float *a, vDSP_Stride ia, const float *s, float *c,
                              vDSP_Stride ic, vDSP_Length n) {
  for (vDSP_Length i = 0; i < n; ++i) c[i * ic] = a[i * ia] * (*s);
}
static inline void vDSP_vsadd(const float *a, vDSP_Stride ia, const float *s, float *c,
                              vDSP_Stride ic, vDSP_Length n) {
  for (vDSP_Length i = 0; i < n; ++i) c[i * ic] = a[i * ia] + (*s);
}
static inline void vDSP_vneg(const float *a, vDSP_Stride ia, float *c, vDSP_Stride ic,
                             vDSP_Length n) {
  for (vDSP_Length i = 0; i < n; ++i) c[i * ic] = -a[i * ia];
}
// C (M rows x N cols) = transpose of A (N rows x M cols).
static inline void vDSP_mtrans(const float *a, vDSP_Stride ia, float *c, vDSP_Stride ic,
                               vDSP_Length M, vDSP_Length N) {
  for (vDSP_Length r = 0; r < M; ++r)
    for (vDSP_Length q = 0; q < N; ++q) c[(r * N + q) * ic] = a[(q * M + r) * ia];
}
static inline void vvexpf(float *y, const float *x, const int *n) {
  for (int i = 0; i < *n; ++i) y[i] = std::exp(x[i]);
}
static inline void vvrecf(float *y, const float *x, const int *n) {
  for (int i = 0; i < *n; ++i) y[i] = 1.0f / x[i];
}
static inline void cblas_sgemm(CBLAS_ORDER, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int M, int N,
                               int K, float alpha, const float *A, int lda, const float *B,
                               int ldb, float beta, float *C, int ldc) {
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      float acc = 0.f;
      for (int k = 0; k < K; ++k) {
        float a = (ta == CblasNoTrans) ? A[i * lda + k] : A[k * lda + i];
        float b = (tb == CblasNoTrans) ? B[k * ldb + j] : B[j * ldb + k];
        acc += a * b;
      }
      C[i * ldc + j] = alpha * acc + beta * C[i * ldc + j];
    }
}
