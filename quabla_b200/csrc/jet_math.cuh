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

// t1..t5 = the first five derivatives of the activation at z.  For tanh they are polynomials in
// t = tanh(z); for sin they cycle through cos, -sin, -cos, sin, cos.
template <typename T>
struct TanhD {
    T t1, t2, t3, t4, t5;
    __device__ __forceinline__ TanhD() {}
    // Activation `act` at z; *value receives the activation itself.
    __device__ __forceinline__ TanhD(T z, int act, T* value) {
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
