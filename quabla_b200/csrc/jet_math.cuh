// Jet arithmetic shared by every kernel: derivatives of tanh as polynomials in
// t = tanh(z) and the Faa di Bruno composition of a univariate Taylor jet with
// tanh, forwards and transposed.
//
// The reference reaches the same quantities by re-differentiating the IR nodes
// of the tanh chain rule s * (1 - t*t) once per autodiff level
// (crates/quabla-core/src/tensor_ir/elementwise.rs:416-468); here the closed
// forms are evaluated in registers.
#pragma once
#include <cuda_runtime.h>
#include <math.h>

namespace qb {

constexpr int MAX_DIRS = 8;      // derivative directions per point set
constexpr int MAX_ORDER = 4;     // highest derivative order along a direction
constexpr int MAX_STREAMS = 17;  // 1 + sum of orders, bounded for kernel arguments

// Streams of one point set: stream 0 is the primal; direction j of order k_j owns
// streams base[j] .. base[j] + k_j - 1 (first .. k_j-th derivative along it).
//
// Merged second-order stream (merged != 0): when the residual needs second derivatives only as one
// weighted sum M = sum_j c_j d^2u/ds_j^2 (a Laplacian), the directions j carry first order only and
// one extra stream, the last, carries M: through an affine layer it maps like every other stream,
// and through the activation f as  h_M = f'(z_0) z_M + f''(z_0) sum_j c_j z1_j^2.
struct JetSpec {
    int S;
    int ndirs;
    int order[MAX_DIRS];
    int base[MAX_DIRS];
    int merged;
    double merge_w[MAX_DIRS];  // c_j (0 for directions outside the sum)
};

// Signature codes at or above SIG_MERGED denote (code - SIG_MERGED) plus the merged stream.
constexpr int SIG_MERGED = 1000000;

// The weights c_j in the arithmetic type of a kernel, passed by value.
template <typename T>
struct MergeW {
    T w[MAX_DIRS];
};

template <typename T>
__device__ __forceinline__ T qb_tanh(T x);
template <>
__device__ __forceinline__ float qb_tanh<float>(float x) {
    return tanhf(x);
}
template <>
__device__ __forceinline__ double qb_tanh<double>(double x) {
    return tanh(x);
}

__device__ __forceinline__ void qb_sincos(float x, float* s, float* c) { sincosf(x, s, c); }
__device__ __forceinline__ void qb_sincos(double x, double* s, double* c) { sincos(x, s, c); }

// Hidden-layer activations (qb200_activation in the C ABI).
constexpr int ACT_TANH = 0;
constexpr int ACT_SIN = 1;
constexpr int ACT_SIGMOID = 2;
constexpr int ACT_SOFTPLUS = 3;
constexpr int ACT_SILU = 4;
constexpr int ACT_GELU = 5;

__device__ __forceinline__ float qb_exp(float x) { return expf(x); }
__device__ __forceinline__ double qb_exp(double x) { return exp(x); }
__device__ __forceinline__ float qb_log1p(float x) { return log1pf(x); }
__device__ __forceinline__ double qb_log1p(double x) { return log1p(x); }

// The logistic function s(z) and its first five derivatives, ds[k] = k-th derivative at z.  s is evaluated as
// the reference composes it, where(z > 0, 1 / (1 + e), e / (1 + e)) with e = exp(-|z|), which never overflows
// (crates/quabla-python/src/composite.rs:178-199); the derivatives are polynomials in s: with p = s (1 - s) and
// q = 1 - 2 s they are p, p q, p (q^2 - 2 p), p q (q^2 - 8 p), p (q^4 - 22 p q^2 + 16 p^2).
template <typename T>
__device__ __forceinline__ void logistic_derivs(T z, T* ds) {
    const T e = qb_exp(-fabs(z));
    const T s = z > T(0) ? T(1) / (T(1) + e) : e / (T(1) + e);
    const T p = s * (T(1) - s), q = T(1) - T(2) * s, q2 = q * q;
    ds[0] = s;
    ds[1] = p;
    ds[2] = p * q;
    ds[3] = p * (q2 - T(2) * p);
    ds[4] = p * q * (q2 - T(8) * p);
    ds[5] = p * (q2 * q2 - T(22) * p * q2 + T(16) * p * p);
}

// t1..t5 = the first five derivatives of the activation at z.  For tanh they are polynomials in
// t = tanh(z); for sin they cycle through cos, -sin, -cos, sin, cos.
template <typename T>
struct TanhD {
    T t1, t2, t3, t4, t5;
    __device__ __forceinline__ TanhD() {}
    // Activation `act` at z; *value receives the activation itself.
    __device__ __forceinline__ TanhD(T z, int act, T* value) {
        if (act >= ACT_SIGMOID) {
            T ds[6];
            if (act == ACT_GELU) {
                // x * s(v(x)), v = c (x + a x^3), c = 2 sqrt(2 / pi) (python/quabla/_ops.py:481-505); beyond
                // |x| = 40 the reference returns x or -0 with a constant derivative.
                if (fabs(z) > T(40)) {
                    *value = z > T(0) ? z : T(-0.0);
                    t1 = z > T(0) ? T(1) : T(0);
                    t2 = t3 = t4 = t5 = T(0);
                    return;
                }
                const T c = T(1.5957691216057308), a = T(0.044715);
                const T v1 = c * (T(1) + T(3) * a * z * z), v2 = T(6) * a * c * z, v3 = T(6) * a * c;
                logistic_derivs(c * (z + a * z * z * z), ds);
                // Derivatives of S(x) = s(v(x)) (Faa di Bruno; the fourth derivative of v is zero), then of x S(x).
                const T S0 = ds[0];
                const T S1 = ds[1] * v1;
                const T S2 = ds[2] * v1 * v1 + ds[1] * v2;
                const T S3 = ds[3] * v1 * v1 * v1 + T(3) * ds[2] * v1 * v2 + ds[1] * v3;
                const T S4 = ds[4] * v1 * v1 * v1 * v1 + T(6) * ds[3] * v1 * v1 * v2 +
                             ds[2] * (T(3) * v2 * v2 + T(4) * v1 * v3);
                const T S5 = ds[5] * v1 * v1 * v1 * v1 * v1 + T(10) * ds[4] * v1 * v1 * v1 * v2 +
                             ds[3] * (T(15) * v1 * v2 * v2 + T(10) * v1 * v1 * v3) + ds[2] * T(10) * v2 * v3;
                *value = z * S0;
                t1 = z * S1 + S0;
                t2 = z * S2 + T(2) * S1;
                t3 = z * S3 + T(3) * S2;
                t4 = z * S4 + T(4) * S3;
                t5 = z * S5 + T(5) * S4;
                return;
            }
            logistic_derivs(z, ds);
            if (act == ACT_SIGMOID) {
                *value = ds[0];
                t1 = ds[1]; t2 = ds[2]; t3 = ds[3]; t4 = ds[4]; t5 = ds[5];
            } else if (act == ACT_SOFTPLUS) {
                // relu(z) + log1p(exp(-|z|)) (composite.rs:201-209); its derivative is the logistic function.
                *value = fmax(z, T(0)) + qb_log1p(qb_exp(-fabs(z)));
                t1 = ds[0]; t2 = ds[1]; t3 = ds[2]; t4 = ds[3]; t5 = ds[4];
            } else {  // ACT_SILU: z * s(z) (python/quabla/_ops.py:475-478)
                *value = z * ds[0];
                t1 = z * ds[1] + ds[0];
                t2 = z * ds[2] + T(2) * ds[1];
                t3 = z * ds[3] + T(3) * ds[2];
                t4 = z * ds[4] + T(4) * ds[3];
                t5 = z * ds[5] + T(5) * ds[4];
            }
            return;
        }
        if (act == ACT_SIN) {
            T sn, cs;
            qb_sincos(z, &sn, &cs);
            *value = sn;
            t1 = cs;
            t2 = -sn;
            t3 = -cs;
            t4 = sn;
            t5 = cs;
        } else {
            const T t = qb_tanh<T>(z);
            *value = t;
            *this = TanhD(t);
        }
    }
    __device__ __forceinline__ explicit TanhD(T t) {
        t1 = T(1) - t * t;
        t2 = T(-2) * t * t1;
        t3 = T(-2) * (t1 * t1 + t * t2);
        t4 = T(-2) * (T(3) * t1 * t2 + t * t3);
        t5 = T(-2) * (T(3) * t2 * t2 + T(4) * t1 * t3 + t * t4);
    }
};

// h_m = d^m tanh(z(s)) / ds^m from z_m = d^m z / ds^m, m = 1..K.
template <typename T, int K>
__device__ __forceinline__ void jet_compose(const TanhD<T>& d, const T* z, T* h) {
    const T z1 = z[0];
    h[0] = d.t1 * z1;
    if (K >= 2) {
        h[1] = d.t2 * z1 * z1 + d.t1 * z[1];
    }
    if (K >= 3) {
        h[2] = d.t3 * z1 * z1 * z1 + T(3) * d.t2 * z1 * z[1] + d.t1 * z[2];
    }
    if (K >= 4) {
        const T z1s = z1 * z1;
        h[3] = d.t4 * z1s * z1s + T(6) * d.t3 * z1s * z[1] +
               d.t2 * (T(3) * z[1] * z[1] + T(4) * z1 * z[2]) + d.t1 * z[3];
    }
}

// Transpose of jet_compose: from cotangents g_m of h_m produce cotangents of
// z_m (written to gz) and return the contribution to the cotangent of z_0
// (through the dependence of t1..t4 on z_0).
template <typename T, int K>
__device__ __forceinline__ T jet_compose_transposed(const TanhD<T>& d, const T* z, const T* g, T* gz) {
    const T z1 = z[0];
    T z0bar = d.t2 * z1 * g[0];
    T a1 = d.t1 * g[0];
    T a2 = T(0), a3 = T(0);
    if (K >= 2) {
        z0bar += (d.t3 * z1 * z1 + d.t2 * z[1]) * g[1];
        a1 += T(2) * d.t2 * z1 * g[1];
        a2 = d.t1 * g[1];
    }
    if (K >= 3) {
        z0bar += (d.t4 * z1 * z1 * z1 + T(3) * d.t3 * z1 * z[1] + d.t2 * z[2]) * g[2];
        a1 += (T(3) * d.t3 * z1 * z1 + T(3) * d.t2 * z[1]) * g[2];
        a2 += T(3) * d.t2 * z1 * g[2];
        a3 = d.t1 * g[2];
    }
    if (K >= 4) {
        const T z1s = z1 * z1;
        z0bar += (d.t5 * z1s * z1s + T(6) * d.t4 * z1s * z[1] +
                  d.t3 * (T(3) * z[1] * z[1] + T(4) * z1 * z[2]) + d.t2 * z[3]) * g[3];
        a1 += (T(4) * d.t4 * z1s * z1 + T(12) * d.t3 * z1 * z[1] + T(4) * d.t2 * z[2]) * g[3];
        a2 += (T(6) * d.t3 * z1s + T(6) * d.t2 * z[1]) * g[3];
        a3 += T(4) * d.t2 * z1 * g[3];
        gz[3] = d.t1 * g[3];
    }
    gz[0] = a1;
    if (K >= 2) gz[1] = a2;
    if (K >= 3) gz[2] = a3;
    return z0bar;
}

// Merged stream through the activation.  q = sum_j c_j z1_j^2 over the PRE-activation first-order
// streams; zM the pre-activation merged stream.
template <typename T>
__device__ __forceinline__ T merged_compose(const TanhD<T>& d, T q, T zM) {
    return d.t1 * zM + d.t2 * q;
}
// Transpose: gM is the cotangent of h_M.  Returns the contribution to the cotangent of z_0, writes
// the cotangent of z_M to *gzM; the caller adds  2 f''(z_0) c_j z1_j gM  to the cotangent of z1_j
// (merged_first_order_factor gives 2 f'' gM).
template <typename T>
__device__ __forceinline__ T merged_compose_transposed(const TanhD<T>& d, T q, T zM, T gM, T* gzM) {
    *gzM = d.t1 * gM;
    return (d.t2 * zM + d.t3 * q) * gM;
}
template <typename T>
__device__ __forceinline__ T merged_first_order_factor(const TanhD<T>& d, T gM) {
    return T(2) * d.t2 * gM;
}

}  // namespace qb
