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

// The forward composition again, from the activation's derivatives d and value at z_0 and the input jets
// v[1..] (v[0] is not read): v becomes the output jets.  Same steps as jet_apply_act.
template <typename T, typename SG, typename MW>
__device__ __forceinline__ void jet_values_with(const TanhD<T>& d, T value, T (&v)[SG::S], const MW& mw) {
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

// The first hidden layer without its pre-activations in memory (KIN = number of network inputs, 1 to 4):
// z_s[point][unit] = sum_j x_s[point][j] W[j][unit] (+ b[unit] on the primal stream) costs KIN multiply-adds, so the
// jet kernels form it from the point's S input jets instead of reading an [S][C][d] array that a separate kernel
// would have written: forward that saves writing and reading Z_1, backward reading it, writing the cotangents
// of Z_1 and reading them again for the first layer's weight gradient, which the backward kernel accumulates itself
// (per-thread sums over its points, then one partial [KIN][d] per block, summed later in block order in double).
// The arithmetic of z is that of skinny_forward_kernel, term by term.
template <typename T>
struct FirstLayer {
    const T* X;     // [S][C][KIN]: input jets of the chunk
    const T* W;     // [KIN][d]
    const T* b;     // [d] or null
    T* wpartial;    // backward: [blocks][KIN][d]
    long long C;
    int d;
};

// The linear output layer on the way out of the last hidden layer's forward kernel: every warp adds its 32 V units
// of u_s[point] = sum_unit h_s[point][unit] w[unit] (a fixed shuffle tree) and writes one partial per stream, so the
// [S][C][d] activations are not read again for it; head_combine_kernel adds the d / (32 V) partials of a row in
// order, plus the bias on the primal rows.  Needs whole warps per point: d % (32 V) == 0.
template <typename T>
struct HeadDot {
    const T* w;   // [d] weights of the output layer, or null: no head product here
    T* partial;   // [S][C][d / (32 V)]
    long long C;
    int d;
};

template <typename T>
inline bool head_dot_fusable(int d) {
    return d % (32 * JetVec<T>::V) == 0;
}

template <typename T>
__global__ void head_combine_kernel(const T* __restrict__ partial, const T* __restrict__ b, T* __restrict__ U, long long rows,
                                    int per_row, long long primal_rows) {
    for (long long r = blockIdx.x * (long long)blockDim.x + threadIdx.x; r < rows; r += (long long)gridDim.x * blockDim.x) {
        T s = partial[r * per_row];
        for (int k = 1; k < per_row; ++k) s += partial[r * per_row + k];
        U[r] = s + ((b != nullptr && r < primal_rows) ? b[0] : T(0));
    }
}

template <typename T, int S, int V, int KIN>
__device__ __forceinline__ void first_layer_z(const FirstLayer<T>& f, long long point, const T (&w)[KIN][V], const T (&bv)[V],
                                              T (&x)[S][KIN], T (&z)[S][V]) {
#pragma unroll
    for (int s = 0; s < S; ++s) {
        const T* row = f.X + ((long long)s * f.C + point) * KIN;
        if constexpr (KIN * sizeof(T) == 16) {
            // One 16-byte load per stream (four float or two double inputs); the row is 16-byte aligned.
            union {
                uint4 q;
                T v[KIN];
            } u;
            u.q = __ldg(reinterpret_cast<const uint4*>(row));
#pragma unroll
            for (int j = 0; j < KIN; ++j) x[s][j] = u.v[j];
        } else {
#pragma unroll
            for (int j = 0; j < KIN; ++j) x[s][j] = __ldg(row + j);
        }
#pragma unroll
        for (int i = 0; i < V; ++i) {
            T sum = T(0);
#pragma unroll
            for (int j = 0; j < KIN; ++j) sum += x[s][j] * w[j][i];
            z[s][i] = s == 0 ? sum + bv[i] : sum;
        }
    }
}

// H = tanh-jet(Z), all streams.  With KIN > 0, Z is the first layer's product formed here (FirstLayer).
template <typename T, int CODE, int KIN = 0>
__global__ void __launch_bounds__(JET_BLOCK) jet_forward_sig_kernel(const T* __restrict__ Z, T* __restrict__ H, long long plane,
                                                              int act, MergeW<T> mw, FirstLayer<T> first, HeadDot<T> head) {
    typedef Sig<CODE> SG;
    typedef JetVec<T> JV;
    typedef typename JV::type VT;
    constexpr int S = SG::S, V = JV::V;
    const long long nvec = plane / V;
    // The grid stride is a multiple of the layer width, so a thread always owns the same V units.
    T w[KIN > 0 ? KIN : 1][V], bv[V], wh[V];
    if (head.w != nullptr) {
        const int unit0 = (int)(((blockIdx.x * (long long)blockDim.x + threadIdx.x) * V) % head.d);
#pragma unroll
        for (int i = 0; i < V; ++i) wh[i] = head.w[unit0 + i];
    }
    if (KIN > 0) {
        const int unit0 = (int)(((blockIdx.x * (long long)blockDim.x + threadIdx.x) * V) % first.d);
#pragma unroll
        for (int i = 0; i < V; ++i) {
#pragma unroll
            for (int j = 0; j < KIN; ++j) w[j][i] = first.W[(long long)j * first.d + unit0 + i];
            bv[i] = first.b != nullptr ? first.b[unit0 + i] : T(0);
        }
    }
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < nvec; e += (long long)gridDim.x * blockDim.x) {
        T lanes[S][V];
        if (KIN > 0) {
            T x[S][KIN > 0 ? KIN : 1];
            first_layer_z<T, S, V, (KIN > 0 ? KIN : 1)>(first, (e * V) / first.d, w, bv, x, lanes);
        } else {
            VT q[S];
#pragma unroll
            for (int s = 0; s < S; ++s) q[s] = reinterpret_cast<const VT*>(Z + (long long)s * plane)[e];
#pragma unroll
            for (int s = 0; s < S; ++s) JV::unpack(q[s], lanes[s]);
        }
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
        if (head.w != nullptr) {
            // A warp's 32 V elements lie in one row (d % (32 V) == 0, and the plane is whole rows, so the warp is
            // either all inside the loop or all outside).
            const long long elem = e * V, point = elem / head.d;
            const int per_row = head.d / (32 * V), slot = (int)(elem - point * head.d) / (32 * V);
#pragma unroll
            for (int s = 0; s < S; ++s) {
                T dot = T(0);
#pragma unroll
                for (int i = 0; i < V; ++i) dot += lanes[s][i] * wh[i];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                if ((threadIdx.x & 31) == 0) head.partial[((long long)s * head.C + point) * per_row + slot] = dot;
            }
        }
    }
}

// In place: G (cotangents of H) becomes the cotangents of Z.  With HEAD the incoming cotangents are
// not read but formed on the fly as Uhat[s][point] * w_head[unit] (the head layer's data gradient),
// which saves writing and re-reading that [S][C][d] array.  With KIN > 0 (FirstLayer) Z is formed here, the
// cotangents of Z are not written, and the first layer's weight gradient leaves as per-block partials.
// With HEAD and head_wpartial the kernel also rebuilds the layer's output jets from what it has loaded (the
// forward composition is a few dozen flops next to 12 planes of traffic) and accumulates the output layer's weight
// gradient sum_{s, point} h_s[point][unit] Uhat_s[point], one partial [d] per block, so that those activations are
// not read from memory a third time.
template <typename T, int CODE, bool HEAD, int KIN = 0>
__global__ void __launch_bounds__(JET_BLOCK) jet_backward_sig_kernel(const T* __restrict__ Z, const T* __restrict__ Hprimal,
                                                               T* __restrict__ G, long long plane,
                                                               const T* __restrict__ Uhat, const T* __restrict__ w_head,
                                                               int d, long long C, int act, T* __restrict__ bias_partial,
                                                               MergeW<T> mw, FirstLayer<T> first,
                                                               T* __restrict__ head_wpartial) {
    typedef Sig<CODE> SG;
    typedef JetVec<T> JV;
    typedef typename JV::type VT;
    constexpr int S = SG::S, V = JV::V;
    constexpr int KW = KIN > 0 ? KIN : 1;
    T hsum[V], us[S];
#pragma unroll
    for (int i = 0; i < V; ++i) hsum[i] = T(0);
    static_assert(!(HEAD && KIN > 0), "the first layer is not the last hidden layer here");
    const long long nvec = plane / V;
    // Bias gradient (column sums of the primal pre-activation cotangents), when asked for: the
    // grid stride is a multiple of the layer width, so a thread always owns the same V units.
    T bsum[V], w[KW][V], bv[V], wsum[KW][V];
#pragma unroll
    for (int i = 0; i < V; ++i) bsum[i] = T(0);
    if (KIN > 0) {
        const int unit0 = (int)(((blockIdx.x * (long long)blockDim.x + threadIdx.x) * V) % first.d);
#pragma unroll
        for (int i = 0; i < V; ++i) {
#pragma unroll
            for (int j = 0; j < KW; ++j) {
                w[j][i] = first.W[(long long)j * first.d + unit0 + i];
                wsum[j][i] = T(0);
            }
            bv[i] = first.b != nullptr ? first.b[unit0 + i] : T(0);
        }
    }
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < nvec; e += (long long)gridDim.x * blockDim.x) {
        VT qz[S], qg[S];
        T t[V], zl[S][V], gl[S][V], x[S][KW];
        // tanh rebuilds its derivatives from the saved activation, other activations from z_0.
        if (KIN == 0 || act == ACT_TANH) JV::unpack(reinterpret_cast<const VT*>(act == ACT_TANH ? Hprimal : Z)[e], t);
#pragma unroll
        for (int s = 0; s < S; ++s) {
            // The transposed composition never reads z_0 itself (t replaces it).
            if (KIN == 0 && s > 0) qz[s] = reinterpret_cast<const VT*>(Z + (long long)s * plane)[e];
            if (!HEAD) qg[s] = reinterpret_cast<const VT*>(G + (long long)s * plane)[e];
        }
        if (KIN > 0) {
            first_layer_z<T, S, V, KW>(first, (e * V) / first.d, w, bv, x, zl);
            if (act != ACT_TANH) {
#pragma unroll
                for (int i = 0; i < V; ++i) t[i] = zl[0][i];
            }
        }
        if (HEAD) {
            const long long elem = e * V, point = elem / d;
            T wv[V];
            JV::unpack(reinterpret_cast<const VT*>(w_head)[(elem - point * d) / V], wv);
#pragma unroll
            for (int s = 0; s < S; ++s) {
                const T u = Uhat[(long long)s * C + point];
                us[s] = u;
#pragma unroll
                for (int i = 0; i < V; ++i) gl[s][i] = u * wv[i];
            }
        }
#pragma unroll
        for (int s = 0; s < S; ++s) {
            if (KIN == 0 && s > 0) JV::unpack(qz[s], zl[s]);
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
            T value = t[i];
            const TanhD<T> dv = act == ACT_TANH ? TanhD<T>(t[i]) : TanhD<T>(t[i], act, &value);
            if (HEAD && head_wpartial != nullptr) {
                T h[S];
#pragma unroll
                for (int s = 0; s < S; ++s) h[s] = z[s];
                jet_values_with<T, SG>(dv, value, h, mw.w);
#pragma unroll
                for (int s = 0; s < S; ++s) hsum[i] += h[s] * us[s];
            }
            jet_apply_transposed_with<T, SG>(dv, z, g, mw.w);
#pragma unroll
            for (int s = 0; s < S; ++s) gl[s][i] = g[s];
        }
        if (KIN == 0) {
#pragma unroll
            for (int s = 0; s < S; ++s) reinterpret_cast<VT*>(G + (long long)s * plane)[e] = JV::pack(gl[s]);
        } else {
#pragma unroll
            for (int s = 0; s < S; ++s)
#pragma unroll
                for (int j = 0; j < KW; ++j)
#pragma unroll
                    for (int i = 0; i < V; ++i) wsum[j][i] += x[s][j] * gl[s][i];
        }
#pragma unroll
        for (int i = 0; i < V; ++i) bsum[i] += gl[0][i];
    }
    const bool head_w = HEAD && head_wpartial != nullptr;
    if (bias_partial != nullptr || KIN > 0 || head_w) {
        // The block covers JET_BLOCK V / d rows of the plane: add them in row order, one partial per block.
        // Passes: 0 the bias gradient, 1..KIN the first layer's weight gradient, KIN + 1 the output layer's.
        __shared__ T red[JET_BLOCK][V];
        const int groups = d / V;  // threads per row
        for (int pass = 0; pass <= KIN + 1; ++pass) {
            if ((pass == 0 && bias_partial == nullptr) || (pass == KIN + 1 && !head_w)) continue;
            __syncthreads();
#pragma unroll
            for (int i = 0; i < V; ++i) {
                T value = pass == 0 ? bsum[i] : hsum[i];
#pragma unroll
                for (int j = 0; j < KW; ++j)
                    if (KIN > 0 && pass == j + 1) value = wsum[j][i];
                red[threadIdx.x][i] = value;
            }
            __syncthreads();
            if ((int)threadIdx.x < groups) {
                T* out = pass == 0 ? bias_partial + (long long)blockIdx.x * d
                         : pass == KIN + 1 ? head_wpartial + (long long)blockIdx.x * d
                                           : first.wpartial + ((long long)blockIdx.x * KW + (pass - 1)) * d;
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    T total = red[threadIdx.x][i];
                    for (int r = groups; r < JET_BLOCK; r += groups) total += red[threadIdx.x + r][i];
                    out[threadIdx.x * V + i] = total;
                }
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
template <typename T, int KIN>
inline void jet_forward_sig_launch_k(int code, const T* Z, T* H, long long plane, int act, const MergeW<T>& mw,
                                     const FirstLayer<T>& first, cudaStream_t stream, const HeadDot<T>& head = HeadDot<T>()) {
    const int grid = jet_sig_grid(plane / JetVec<T>::V);
#define QB_JET_FWD(CODE) jet_forward_sig_kernel<T, CODE, KIN><<<grid, JET_BLOCK, 0, stream>>>(Z, H, plane, act, mw, first, head)
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

// `head` (optional): the output layer's product leaves as per-warp partials (HeadDot); the caller checked
// head_dot_fusable and jet_bias_fusable for this width.
template <typename T>
inline void jet_forward_sig_launch(int code, const T* Z, T* H, long long plane, int act, const MergeW<T>& mw,
                                   cudaStream_t stream, const HeadDot<T>& head = HeadDot<T>()) {
    jet_forward_sig_launch_k<T, 0>(code, Z, H, plane, act, mw, FirstLayer<T>(), stream, head);
}

// Inputs of the network (1 to 4) for which the first-layer variants exist.
inline bool jet_first_inputs_ok(int kin) { return kin >= 1 && kin <= 4; }

// H_1 straight from the input jets (FirstLayer); the caller checked jet_first_inputs_ok and jet_bias_fusable.
template <typename T>
inline void jet_forward_first_launch(int code, T* H, long long plane, int act, const MergeW<T>& mw, int kin,
                                     const FirstLayer<T>& first, cudaStream_t stream) {
    switch (kin) {
        case 1: jet_forward_sig_launch_k<T, 1>(code, nullptr, H, plane, act, mw, first, stream); break;
        case 2: jet_forward_sig_launch_k<T, 2>(code, nullptr, H, plane, act, mw, first, stream); break;
        case 3: jet_forward_sig_launch_k<T, 3>(code, nullptr, H, plane, act, mw, first, stream); break;
        default: jet_forward_sig_launch_k<T, 4>(code, nullptr, H, plane, act, mw, first, stream); break;
    }
}

template <typename T, bool HEAD, int KIN = 0>
inline void jet_backward_sig_launch_impl(int code, const T* Z, const T* Hprimal, T* G, long long plane, const T* Uhat,
                                         const T* w_head, int d, long long C, int act, T* bias_partial,
                                         const MergeW<T>& mw, cudaStream_t stream,
                                         const FirstLayer<T>& first = FirstLayer<T>(), T* head_wpartial = nullptr) {
    const int grid = jet_sig_grid(plane / JetVec<T>::V);
#define QB_JET_BWD(CODE)                                                                                                   \
    jet_backward_sig_kernel<T, CODE, HEAD, KIN><<<grid, JET_BLOCK, 0, stream>>>(Z, Hprimal, G, plane, Uhat, w_head, d, C, act, \
                                                                          bias_partial, mw, first, head_wpartial)
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

// First hidden layer (FirstLayer): G holds the cotangents of H_1 and is only read; the weight-gradient partials go to
// first.wpartial, one [kin][d] block per CTA of jet_sig_grid(plane / V).
template <typename T>
inline void jet_backward_first_launch(int code, const T* Hprimal, T* G, long long plane, int d, int act, T* bias_partial,
                                      const MergeW<T>& mw, int kin, const FirstLayer<T>& first, cudaStream_t stream) {
    switch (kin) {
        case 1: jet_backward_sig_launch_impl<T, false, 1>(code, nullptr, Hprimal, G, plane, nullptr, nullptr, d, 1, act, bias_partial, mw, stream, first); break;
        case 2: jet_backward_sig_launch_impl<T, false, 2>(code, nullptr, Hprimal, G, plane, nullptr, nullptr, d, 1, act, bias_partial, mw, stream, first); break;
        case 3: jet_backward_sig_launch_impl<T, false, 3>(code, nullptr, Hprimal, G, plane, nullptr, nullptr, d, 1, act, bias_partial, mw, stream, first); break;
        default: jet_backward_sig_launch_impl<T, false, 4>(code, nullptr, Hprimal, G, plane, nullptr, nullptr, d, 1, act, bias_partial, mw, stream, first); break;
    }
}

// Last hidden layer: the cotangents of H are Uhat (x) w_head, formed inside the kernel; d % V == 0
// and w_head 16-byte aligned are the caller's to check.
template <typename T>
inline void jet_backward_head_launch(int code, const T* Z, const T* Hprimal, T* G, long long plane, const T* Uhat,
                                     const T* w_head, int d, long long C, int act, T* bias_partial,
                                     const MergeW<T>& mw, cudaStream_t stream, T* head_wpartial = nullptr) {
    jet_backward_sig_launch_impl<T, true>(code, Z, Hprimal, G, plane, Uhat, w_head, d, C, act, bias_partial, mw, stream,
                                          FirstLayer<T>(), head_wpartial);
}

}  // namespace qb
