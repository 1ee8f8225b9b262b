// Vectorised tanh-jet kernels of the layer-wise engine for the common derivative signatures.
//
// Activations are [S][C][d] (stream-major planes of `plane` = C*d elements).  A thread owns 16 bytes
// of every plane (4 floats or 2 doubles of consecutive units): it issues the S (forward) or 2S+1
// (backward) 16-byte loads up front, runs the Faa di Bruno composition with the signature known at
// compile time (all stream loops unroll, no local memory), and stores 16 bytes per plane.  The
// generic jet_forward_kernel / jet_backward_kernel (layer_kernels.cuh) remain for other signatures
// and for planes that are not a multiple of 16 bytes.
//
// These kernels are HBM-bound: 2*S*plane elements of traffic forward, (3S+1)*plane backward.
// Blocks have JET_BLOCK = 128 threads: with at most 112 registers per thread such a block fits on an SM beside
// a CTA of the tensor-core GEMM (320 threads x 160 registers, ~210 KB of shared memory), so the jet kernels of
// one chunk can run under the GEMMs of another chunk issued on a second stream.
#pragma once
#include "fused_kernel.cuh"  // Sig<CODE>, jet_apply
#include "jet_math.cuh"

namespace qb {

constexpr int JET_BLOCK = 128;

template <typename T>
struct JetVec;
template <>
struct JetVec<float> {
    static constexpr int V = 4;
    typedef float4 type;
    static __device__ __forceinline__ void unpack(const float4& q, float (&v)[4]) {
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
    static __device__ __forceinline__ float4 pack(const float (&v)[4]) { return make_float4(v[0], v[1], v[2], v[3]); }
};
template <>
struct JetVec<double> {
    static constexpr int V = 2;
    typedef double2 type;
    static __device__ __forceinline__ void unpack(const double2& q, double (&v)[2]) {
        v[0] = q.x; v[1] = q.y;
    }
    static __device__ __forceinline__ double2 pack(const double (&v)[2]) { return make_double2(v[0], v[1]); }
};

// Forward jet composition on the S streams of one (point, unit) for activation `act`.
template <typename T, typename SG, typename MW>
__device__ __forceinline__ void jet_apply_act(T (&v)[SG::S], int act, const MW& mw) {
    T value;
    const TanhD<T> d(v[0], act, &value);
    T hM = T(0);
    if (SG::merged) hM = merged_compose(d, merged_square_sum<T, SG, MW>(v, mw), v[SG::MS]);
    v[0] = value;
#pragma unroll
    for (int j = 0; j < SG::ndirs; ++j) {
        T z[MAX_ORDER], h[MAX_ORDER];
        const int K = SG::order(j);
        const int b = SG::base(j);
#pragma unroll
        for (int m = 0; m < MAX_ORDER; ++m) z[m] = m < K ? v[b + m] : T(0);
        switch (K) {
            case 1: jet_compose<T, 1>(d, z, h); break;
            case 2: jet_compose<T, 2>(d, z, h); break;
            case 3: jet_compose<T, 3>(d, z, h); break;
            default: jet_compose<T, 4>(d, z, h); break;
        }
#pragma unroll
        for (int m = 0; m < MAX_ORDER; ++m)
            if (m < K) v[b + m] = h[m];
    }
    if (SG::merged) v[SG::MS] = hM;
}

// H = tanh-jet(Z), all streams.
template <typename T, int CODE>
__global__ void __launch_bounds__(JET_BLOCK) jet_forward_sig_kernel(const T* __restrict__ Z, T* __restrict__ H, long long plane,
                                                              int act, MergeW<T> mw) {
    typedef Sig<CODE> SG;
    typedef JetVec<T> JV;
    typedef typename JV::type VT;
    constexpr int S = SG::S, V = JV::V;
    const long long nvec = plane / V;
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < nvec; e += (long long)gridDim.x * blockDim.x) {
        VT q[S];
#pragma unroll
        for (int s = 0; s < S; ++s) q[s] = reinterpret_cast<const VT*>(Z + (long long)s * plane)[e];
        T lanes[S][V];
#pragma unroll
        for (int s = 0; s < S; ++s) JV::unpack(q[s], lanes[s]);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            T v[S];
#pragma unroll
            for (int s = 0; s < S; ++s) v[s] = lanes[s][i];
            jet_apply_act<T, SG>(v, act, mw.w);
#pragma unroll
            for (int s = 0; s < S; ++s) lanes[s][i] = v[s];
        }
#pragma unroll
        for (int s = 0; s < S; ++s) reinterpret_cast<VT*>(H + (long long)s * plane)[e] = JV::pack(lanes[s]);
    }
}

// In place: G (cotangents of H) becomes the cotangents of Z.  With HEAD the incoming cotangents are
// not read but formed on the fly as Uhat[s][point] * w_head[unit] (the head layer's data gradient),
// which saves writing and re-reading that [S][C][d] array.
template <typename T, int CODE, bool HEAD>
__global__ void __launch_bounds__(JET_BLOCK) jet_backward_sig_kernel(const T* __restrict__ Z, const T* __restrict__ Hprimal,
                                                               T* __restrict__ G, long long plane,
                                                               const T* __restrict__ Uhat, const T* __restrict__ w_head,
                                                               int d, long long C, int act, T* __restrict__ bias_partial,
                                                               MergeW<T> mw) {
    typedef Sig<CODE> SG;
    typedef JetVec<T> JV;
    typedef typename JV::type VT;
    constexpr int S = SG::S, V = JV::V;
    const long long nvec = plane / V;
    // Bias gradient (column sums of the primal pre-activation cotangents), when asked for: the
    // grid stride is a multiple of the layer width, so a thread always owns the same V units.
    T bsum[V];
#pragma unroll
    for (int i = 0; i < V; ++i) bsum[i] = T(0);
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < nvec; e += (long long)gridDim.x * blockDim.x) {
        VT qz[S], qg[S];
        // tanh rebuilds its derivatives from the saved activation, other activations from z_0.
        const VT qt = reinterpret_cast<const VT*>(act == ACT_TANH ? Hprimal : Z)[e];
#pragma unroll
        for (int s = 0; s < S; ++s) {
            // The transposed composition never reads z_0 itself (t replaces it).
            if (s > 0) qz[s] = reinterpret_cast<const VT*>(Z + (long long)s * plane)[e];
            if (!HEAD) qg[s] = reinterpret_cast<const VT*>(G + (long long)s * plane)[e];
        }
        T t[V], zl[S][V], gl[S][V];
        JV::unpack(qt, t);
        if (HEAD) {
            const long long elem = e * V, point = elem / d;
            T wv[V];
            JV::unpack(reinterpret_cast<const VT*>(w_head)[(elem - point * d) / V], wv);
#pragma unroll
            for (int s = 0; s < S; ++s) {
                const T u = Uhat[(long long)s * C + point];
#pragma unroll
                for (int i = 0; i < V; ++i) gl[s][i] = u * wv[i];
            }
        }
#pragma unroll
        for (int s = 0; s < S; ++s) {
            if (s > 0) JV::unpack(qz[s], zl[s]);
            if (!HEAD) JV::unpack(qg[s], gl[s]);
        }
#pragma unroll
        for (int i = 0; i < V; ++i) {
            T z[S], g[S];
            z[0] = T(0);
#pragma unroll
            for (int s = 0; s < S; ++s) {
                if (s > 0) z[s] = zl[s][i];
                g[s] = gl[s][i];
            }
            T unused;
            const TanhD<T> dv = act == ACT_TANH ? TanhD<T>(t[i]) : TanhD<T>(t[i], act, &unused);
            jet_apply_transposed_with<T, SG>(dv, z, g, mw.w);
#pragma unroll
            for (int s = 0; s < S; ++s) gl[s][i] = g[s];
        }
#pragma unroll
        for (int s = 0; s < S; ++s) reinterpret_cast<VT*>(G + (long long)s * plane)[e] = JV::pack(gl[s]);
#pragma unroll
        for (int i = 0; i < V; ++i) bsum[i] += gl[0][i];
    }
    if (bias_partial != nullptr) {
        // The block covers JET_BLOCK V / d rows of the plane: add them in row order, one partial per block.
        __shared__ T red[JET_BLOCK][V];
#pragma unroll
        for (int i = 0; i < V; ++i) red[threadIdx.x][i] = bsum[i];
        __syncthreads();
        const int groups = d / V;  // threads per row
        if ((int)threadIdx.x < groups) {
#pragma unroll
            for (int i = 0; i < V; ++i) {
                T total = red[threadIdx.x][i];
                for (int r = groups; r < JET_BLOCK; r += groups) total += red[threadIdx.x + r][i];
                bias_partial[(long long)blockIdx.x * d + threadIdx.x * V + i] = total;
            }
        }
    }
}

// Launchers: true when a compile-time signature exists for `code` and the planes can be read
// 16 bytes at a time.
template <typename T>
inline bool jet_sig_eligible(int code, long long plane, const void* a, const void* b, const void* c) {
    const bool known = code == 0 || code == 1 || code == 2 || code == 4 || code == 7 || code == 12 || code == 187 ||
                       code == SIG_MERGED + 6 || code == SIG_MERGED + 31 || code == SIG_MERGED + 156;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c);
    return known && plane % JetVec<T>::V == 0 && (bits & 15) == 0;
}

// Whether the backward kernel can also form the bias-gradient partials of a layer of width d:
// its grid stride (JET_BLOCK V elements per block) must cover whole rows.
template <typename T>
inline bool jet_bias_fusable(int d) {
    return d >= JetVec<T>::V && d % JetVec<T>::V == 0 && (JET_BLOCK * JetVec<T>::V) % d == 0;
}

inline int jet_sig_grid(long long vectors) {
    const long long blocks = (vectors + JET_BLOCK - 1) / JET_BLOCK;
    return (int)(blocks < 148 * 32 ? (blocks < 1 ? 1 : blocks) : 148 * 32);
}

// Merged codes: SIG_MERGED + 6 / 31 / 156 = two / three / four first-order directions plus the merged
// second-order stream (Laplacians in 2 and 3 dimensions; 3-D heat equation with its time direction).
template <typename T>
inline void jet_forward_sig_launch(int code, const T* Z, T* H, long long plane, int act, const MergeW<T>& mw,
                                   cudaStream_t stream) {
    const int grid = jet_sig_grid(plane / JetVec<T>::V);
#define QB_JET_FWD(CODE) jet_forward_sig_kernel<T, CODE><<<grid, JET_BLOCK, 0, stream>>>(Z, H, plane, act, mw)
    switch (code) {
        case 0: QB_JET_FWD(0); break;
        case 1: QB_JET_FWD(1); break;
        case 2: QB_JET_FWD(2); break;
        case 4: QB_JET_FWD(4); break;
        case 7: QB_JET_FWD(7); break;
        case 12: QB_JET_FWD(12); break;
        case SIG_MERGED + 6: QB_JET_FWD(SIG_MERGED + 6); break;
        case SIG_MERGED + 31: QB_JET_FWD(SIG_MERGED + 31); break;
        case SIG_MERGED + 156: QB_JET_FWD(SIG_MERGED + 156); break;
        default: QB_JET_FWD(187); break;
    }
#undef QB_JET_FWD
}

template <typename T, bool HEAD>
inline void jet_backward_sig_launch_impl(int code, const T* Z, const T* Hprimal, T* G, long long plane, const T* Uhat,
                                         const T* w_head, int d, long long C, int act, T* bias_partial,
                                         const MergeW<T>& mw, cudaStream_t stream) {
    const int grid = jet_sig_grid(plane / JetVec<T>::V);
#define QB_JET_BWD(CODE)                                                                                             \
    jet_backward_sig_kernel<T, CODE, HEAD><<<grid, JET_BLOCK, 0, stream>>>(Z, Hprimal, G, plane, Uhat, w_head, d, C, act, \
                                                                     bias_partial, mw)
    switch (code) {
        case 0: QB_JET_BWD(0); break;
        case 1: QB_JET_BWD(1); break;
        case 2: QB_JET_BWD(2); break;
        case 4: QB_JET_BWD(4); break;
        case 7: QB_JET_BWD(7); break;
        case 12: QB_JET_BWD(12); break;
        case SIG_MERGED + 6: QB_JET_BWD(SIG_MERGED + 6); break;
        case SIG_MERGED + 31: QB_JET_BWD(SIG_MERGED + 31); break;
        case SIG_MERGED + 156: QB_JET_BWD(SIG_MERGED + 156); break;
        default: QB_JET_BWD(187); break;
    }
#undef QB_JET_BWD
}

template <typename T>
inline void jet_backward_sig_launch(int code, const T* Z, const T* Hprimal, T* G, long long plane, int d, int act,
                                    T* bias_partial, const MergeW<T>& mw, cudaStream_t stream) {
    jet_backward_sig_launch_impl<T, false>(code, Z, Hprimal, G, plane, nullptr, nullptr, d, 1, act, bias_partial, mw,
                                           stream);
}

// Last hidden layer: the cotangents of H are Uhat (x) w_head, formed inside the kernel; d % V == 0
// and w_head 16-byte aligned are the caller's to check.
template <typename T>
inline void jet_backward_head_launch(int code, const T* Z, const T* Hprimal, T* G, long long plane, const T* Uhat,
                                     const T* w_head, int d, long long C, int act, T* bias_partial,
                                     const MergeW<T>& mw, cudaStream_t stream) {
    jet_backward_sig_launch_impl<T, true>(code, Z, Hprimal, G, plane, Uhat, w_head, d, C, act, bias_partial, mw, stream);
}

}  // namespace qb
