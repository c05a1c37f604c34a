/* accelerate_shim.h -- portable-C stand-ins for the Apple Accelerate (vDSP / vForce /
 * cblas) calls that the reference's CPU operator headers make.
 *
 * TEST INFRASTRUCTURE ONLY.  This header exists so that the reference headers
 * (training/stories_cpu_ops.h, training/training_dynamic/cpu_ops.h) compile with gcc on
 * Linux straight from where they lie, without the Objective-C config headers they
 * normally include.  Nothing in the shipped library includes it.
 *
 * Every routine follows Apple's documented element-wise definition in fp32 with libm.
 * Bit-exactness with Apple's vvexpf / vvrsqrtf is not claimed; the parity tolerance
 * (1e-5 relative) covers the difference.
 */
#ifndef ACCELERATE_SHIM_H
#define ACCELERATE_SHIM_H

#include <math.h>
#include <stdint.h>
#include <stddef.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef unsigned long vDSP_Length;
typedef long vDSP_Stride;

/* C[i] = A[i] * B[i] */
static inline void vDSP_vmul(const float *A, vDSP_Stride IA, const float *B, vDSP_Stride IB,
                             float *C, vDSP_Stride IC, vDSP_Length N) {
    for (vDSP_Length i = 0; i < N; i++) C[i * IC] = A[i * IA] * B[i * IB];
}
/* C[i] = A[i] + B[i] */
static inline void vDSP_vadd(const float *A, vDSP_Stride IA, const float *B, vDSP_Stride IB,
                             float *C, vDSP_Stride IC, vDSP_Length N) {
    for (vDSP_Length i = 0; i < N; i++) C[i * IC] = A[i * IA] + B[i * IB];
}
/* C[i] = A[i] - B[i]  -- note the operand order: the FIRST argument is subtracted. */
static inline void vDSP_vsub(const float *B, vDSP_Stride IB, const float *A, vDSP_Stride IA,
                             float *C, vDSP_Stride IC, vDSP_Length N) {
    for (vDSP_Length i = 0; i < N; i++) C[i * IC] = A[i * IA] - B[i * IB];
}
/* C[i] = A[i] * b */
static inline void vDSP_vsmul(const float *A, vDSP_Stride IA, const float *b,
                              float *C, vDSP_Stride IC, vDSP_Length N) {
    const float s = *b;
    for (vDSP_Length i = 0; i < N; i++) C[i * IC] = A[i * IA] * s;
}
/* C[i] = A[i] + b */
static inline void vDSP_vsadd(const float *A, vDSP_Stride IA, const float *b,
                              float *C, vDSP_Stride IC, vDSP_Length N) {
    const float s = *b;
    for (vDSP_Length i = 0; i < N; i++) C[i * IC] = A[i * IA] + s;
}
/* D[i] = A[i] * b + C[i] */
static inline void vDSP_vsma(const float *A, vDSP_Stride IA, const float *b,
                             const float *C, vDSP_Stride IC, float *D, vDSP_Stride ID,
                             vDSP_Length N) {
    const float s = *b;
    for (vDSP_Length i = 0; i < N; i++) D[i * ID] = A[i * IA] * s + C[i * IC];
}
/* D[i] = A[i] * b + c */
static inline void vDSP_vsmsa(const float *A, vDSP_Stride IA, const float *b, const float *c,
                              float *D, vDSP_Stride ID, vDSP_Length N) {
    const float s = *b, t = *c;
    for (vDSP_Length i = 0; i < N; i++) D[i * ID] = A[i * IA] * s + t;
}
/* C[i] = -A[i] */
static inline void vDSP_vneg(const float *A, vDSP_Stride IA, float *C, vDSP_Stride IC,
                             vDSP_Length N) {
    for (vDSP_Length i = 0; i < N; i++) C[i * IC] = -A[i * IA];
}
/* *c = sum A[i] */
static inline void vDSP_sve(const float *A, vDSP_Stride IA, float *c, vDSP_Length N) {
    float s = 0.0f;
    for (vDSP_Length i = 0; i < N; i++) s += A[i * IA];
    *c = s;
}
/* *c = max A[i] */
static inline void vDSP_maxv(const float *A, vDSP_Stride IA, float *c, vDSP_Length N) {
    float m = -INFINITY;
    for (vDSP_Length i = 0; i < N; i++) if (A[i * IA] > m) m = A[i * IA];
    *c = m;
}
/* *c = min A[i] */
static inline void vDSP_minv(const float *A, vDSP_Stride IA, float *c, vDSP_Length N) {
    float m = INFINITY;
    for (vDSP_Length i = 0; i < N; i++) if (A[i * IA] < m) m = A[i * IA];
    *c = m;
}
/* *c = max |A[i]| */
static inline void vDSP_maxmgv(const float *A, vDSP_Stride IA, float *c, vDSP_Length N) {
    float m = 0.0f;
    for (vDSP_Length i = 0; i < N; i++) { float a = fabsf(A[i * IA]); if (a > m) m = a; }
    *c = m;
}
/* *c = sum A[i] * B[i] */
static inline void vDSP_dotpr(const float *A, vDSP_Stride IA, const float *B, vDSP_Stride IB,
                              float *c, vDSP_Length N) {
    float s = 0.0f;
    for (vDSP_Length i = 0; i < N; i++) s += A[i * IA] * B[i * IB];
    *c = s;
}
/* C is the M x N transpose of the N x M matrix A: C[m*N + n] = A[n*M + m] */
static inline void vDSP_mtrans(const float *A, vDSP_Stride IA, float *C, vDSP_Stride IC,
                               vDSP_Length M, vDSP_Length N) {
    for (vDSP_Length m = 0; m < M; m++)
        for (vDSP_Length n = 0; n < N; n++)
            C[(m * N + n) * IC] = A[(n * M + m) * IA];
}
/* vForce: y[i] = 1/sqrt(x[i]) ; exp(x[i]) ; 1/x[i] */
static inline void vvrsqrtf(float *y, const float *x, const int *n) {
    for (int i = 0; i < *n; i++) y[i] = 1.0f / sqrtf(x[i]);
}
static inline void vvexpf(float *y, const float *x, const int *n) {
    for (int i = 0; i < *n; i++) y[i] = expf(x[i]);
}
static inline void vvrecf(float *y, const float *x, const int *n) {
    for (int i = 0; i < *n; i++) y[i] = 1.0f / x[i];
}
/* Y[i*incY] = X[i*incX] */
static inline void cblas_scopy(int N, const float *X, int incX, float *Y, int incY) {
    for (int i = 0; i < N; i++) Y[(size_t)i * incY] = X[(size_t)i * incX];
}

#endif /* ACCELERATE_SHIM_H */
