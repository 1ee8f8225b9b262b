// Fused engine for narrow networks: ONE persistent kernel runs, per tile of
// collocation points, the whole forward pass with all derivative streams, the
// residual program, and the whole reverse sweep, and accumulates the weight
// gradients per CTA.  Nothing but the point coordinates is read from HBM; the
// saved jets of a tile live in a per-CTA scratch that is rewritten every tile
// and therefore stays in L2.
//
// It replaces, for one point set, the reference's per-node launches of the
// vmapped value-and-gradient plan (crates/quabla-core/src/tensor_ir/cuda.rs:
// 1792-2972: one kernel per IR node; op/vjp.rs:176-209: a materialised
// [B, in, out] product per weight gradient).
//
// Shapes: every hidden layer has the same width W (16, 32 or 64), the input
// width d0 <= 4, the output width 1.  A CTA of 256 threads owns a tile of TP
// points; thread (tp, tn) holds, for 2 points x 4 units, ALL S streams in
// registers, so the tanh-jet composition and its transpose are register-only.
#pragma once
#include "jet_math.cuh"
#include "point_kernels.cuh"

namespace qb {

constexpr int FUSED_MAX_LAYERS = 12;  // hidden layers
constexpr int FUSED_THREADS = 256;

// Derivative signature as a compile-time code: sum over directions j of
// order_j * 5^j.  All loops over streams unroll completely.
template <int CODE>
struct Sig {
    static constexpr bool merged = CODE >= SIG_MERGED;  // one extra stream: the merged second order
    static constexpr int PLAIN = CODE % SIG_MERGED;
    static __host__ __device__ constexpr int order(int j) {
        int c = PLAIN;
        for (int i = 0; i < j; ++i) c /= 5;
        return c % 5;
    }
    static __host__ __device__ constexpr int count_dirs() {
        int c = PLAIN, n = 0;
        while (c > 0) {
            ++n;
            c /= 5;
        }
        return n;
    }
    static __host__ __device__ constexpr int base(int j) {
        // One pass over the digits (a nested loop here was not folded to a constant for the fourth
        // direction, which put the streams of a thread into local memory).
        int c = PLAIN, b = 1;
        for (int i = 0; i < j; ++i) {
            b += c % 5;
            c /= 5;
        }
        return b;
    }
    static constexpr int ndirs = count_dirs();
    static constexpr int S = base(ndirs) + (merged ? 1 : 0);
    static constexpr int MS = S - 1;  // the merged stream, when there is one
};

// q = sum_j c_j z1_j^2 over the first-order streams of a merged signature.
// MW is anything indexable by direction (a pointer, or the array inside a by-value kernel parameter,
// which is then read straight from parameter space).
template <typename T, typename SG, typename MW>
__device__ __forceinline__ T merged_square_sum(const T (&v)[SG::S], const MW& mw) {
    T q = T(0);
#pragma unroll
    for (int j = 0; j < SG::ndirs; ++j) q += mw[j] * v[SG::base(j)] * v[SG::base(j)];
    return q;
}

template <typename T>
struct FusedArgs {
    int L;       // hidden layers, all of width W
    int d0;      // network input width (<= 4)
    int P;       // total parameter scalars (stride of the per-CTA gradient rows)
    const T* params;
    int w_off[FUSED_MAX_LAYERS + 1];  // layer l = 0..L (L is the head)
    int b_off[FUSED_MAX_LAYERS + 1];  // -1: no bias
    const T* table;
    int ncols;
    long long n_points;
    T dirs[MAX_DIRS * 4];  // [ndirs][d0]
    T merge_w[MAX_DIRS];   // weights of the merged second-order stream (merged signatures only)
    ProgramRef prog;
    const T* cotangent;
    T weight;
    T extra;
    T* scratch_z;       // per CTA [L][S][TP][W]
    T* scratch_h;       // per CTA [L][S][TP][W]
    T* grad_cta;        // [gridDim.x][P]
    double* loss_cta;   // [gridDim.x]
    int forward_only;
    const void* weight_images;  // tensor-core variant: pre-split weight images (prep_weights_kernel)
    int* error;                 // set to 1 when a bounded wait inside the kernel gave up
};

template <typename T> struct Pack2;
template <> struct Pack2<float> { typedef float2 type; };
template <> struct Pack2<double> { typedef double2 type; };

template <typename T>
__device__ __forceinline__ void ld2(const T* p, T& a, T& b) {
    const typename Pack2<T>::type v = *reinterpret_cast<const typename Pack2<T>::type*>(p);
    a = v.x;
    b = v.y;
}
template <typename T>
__device__ __forceinline__ void st2(T* p, T a, T b) {
    typename Pack2<T>::type v;
    v.x = a;
    v.y = b;
    *reinterpret_cast<typename Pack2<T>::type*>(p) = v;
}
__device__ __forceinline__ void ld4(const float* p, float (&v)[4]) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
}
__device__ __forceinline__ void ld4(const double* p, double (&v)[4]) {
    const double2 a = *reinterpret_cast<const double2*>(p);
    const double2 b = *reinterpret_cast<const double2*>(p + 2);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void st4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void st4(double* p, const double (&v)[4]) {
    *reinterpret_cast<double2*>(p) = make_double2(v[0], v[1]);
    *reinterpret_cast<double2*>(p + 2) = make_double2(v[2], v[3]);
}

// Geometry shared by host (shared-memory size, scratch size) and device.
template <typename T, int W, int CODE>
struct FusedGeom {
    typedef Sig<CODE> sig;
    static constexpr int S = sig::S;
    static constexpr int CG = W / 4;                  // column groups (4 units each)
    static constexpr int PG = FUSED_THREADS / CG;     // point groups (2 points each)
    static constexpr int TP = 2 * PG;                 // points per tile
    static constexpr int ROWS = S * TP;
    static constexpr int ROWP = ROWS + 4;             // stride of the k-major activation buffer
    static constexpr int WP = W + 4;                  // stride of the row-major buffers
    static constexpr int MT = W / 16;                 // weight-gradient micro-tile per thread
    // shared-memory regions, in elements of T
    static constexpr int OFF_ACT = 0;                          // [W][ROWP]  k-major A operand
    static constexpr int OFF_HR = OFF_ACT + W * ROWP;          // [ROWS][WP] previous-layer jets, row-major
    static constexpr int OFF_ZR = OFF_HR + ROWS * WP;          // [ROWS][WP] pre-activation cotangents
    static constexpr int OFF_WB = OFF_ZR + ROWS * WP;          // [W][WP]    weights of the current GEMM
    static constexpr int OFF_RED = OFF_WB + W * WP;            // [PG][5][W] cross-thread reductions
    static constexpr int OFF_U = OFF_RED + PG * 5 * W;         // [S][TP]    network output streams
    static constexpr int OFF_UH = OFF_U + ROWS;                // [S][TP]    their cotangents
    static constexpr int TOTAL = OFF_UH + ROWS;
    // plus 16 bytes per instruction of the residual program, staged after these regions
    static constexpr size_t SMEM_BASE_BYTES = ((size_t)TOTAL * sizeof(T) + 15) / 16 * 16;
    static constexpr size_t SCRATCH_PER_CTA = (size_t)S * TP * W;  // elements per layer per buffer
};

// acc[s][i][j] = sum_k A[k][s*TP + 2*tp + i] * B[k][4*tn + j], k < K.
template <typename T, int S, int TP, int ROWP, int WP>
__device__ __forceinline__ void tile_gemm(const T* __restrict__ A, const T* __restrict__ B, int K, int tp, int tn,
                                          T (&acc)[S][2][4]) {
#pragma unroll
    for (int s = 0; s < S; ++s)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[s][i][j] = T(0);
#pragma unroll 4
    for (int k = 0; k < K; ++k) {
        T b[4];
        ld4(B + k * WP + 4 * tn, b);
        const T* arow = A + k * ROWP + 2 * tp;
#pragma unroll
        for (int s = 0; s < S; ++s) {
            T a0, a1;
            ld2(arow + s * TP, a0, a1);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc[s][0][j] += a0 * b[j];
                acc[s][1][j] += a1 * b[j];
            }
        }
    }
}

// Derivatives of the fused engines' activations (ACT_TANH or ACT_SIN, a compile-time choice: a run-time switch
// cost the tensor-core kernel 8 % on the tanh path) at z; *value receives the activation itself.
template <typename T, int ACT>
__device__ __forceinline__ TanhD<T> fused_activation(T z, T* value) {
    if (ACT == ACT_SIN) return TanhD<T>(z, ACT_SIN, value);
    *value = qb_tanh<T>(z);
    return TanhD<T>(*value);
}

// Forward jet composition on the S streams of one (point, unit); mw: weights of the merged stream.
template <typename T, typename SG, int ACT, typename MW>
__device__ __forceinline__ void jet_apply(T (&v)[SG::S], const MW& mw) {
    T t;
    const TanhD<T> d = fused_activation<T, ACT>(v[0], &t);
    T hM = T(0);
    if (SG::merged) hM = merged_compose(d, merged_square_sum<T, SG, MW>(v, mw), v[SG::MS]);
    v[0] = t;
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

// Transposed composition with the activation's derivatives d at z_0 given: g (cotangents of the
// post-activation streams) becomes the cotangents of the pre-activation streams z.  z[0] is not read.
template <typename T, typename SG, typename MW>
__device__ __forceinline__ void jet_apply_transposed_with(const TanhD<T>& d, const T (&z)[SG::S], T (&g)[SG::S],
                                                          const MW& mw) {
    T z0bar = d.t1 * g[0];
    T first_factor = T(0);
    if (SG::merged) {
        const T gM = g[SG::MS];
        T gzM;
        z0bar += merged_compose_transposed(d, merged_square_sum<T, SG, MW>(z, mw), z[SG::MS], gM, &gzM);
        first_factor = merged_first_order_factor(d, gM);
        g[SG::MS] = gzM;
    }
#pragma unroll
    for (int j = 0; j < SG::ndirs; ++j) {
        T zz[MAX_ORDER], gg[MAX_ORDER], gz[MAX_ORDER];
        const int K = SG::order(j);
        const int b = SG::base(j);
#pragma unroll
        for (int m = 0; m < MAX_ORDER; ++m) {
            zz[m] = m < K ? z[b + m] : T(0);
            gg[m] = m < K ? g[b + m] : T(0);
        }
        switch (K) {
            case 1: z0bar += jet_compose_transposed<T, 1>(d, zz, gg, gz); break;
            case 2: z0bar += jet_compose_transposed<T, 2>(d, zz, gg, gz); break;
            case 3: z0bar += jet_compose_transposed<T, 3>(d, zz, gg, gz); break;
            default: z0bar += jet_compose_transposed<T, 4>(d, zz, gg, gz); break;
        }
#pragma unroll
        for (int m = 0; m < MAX_ORDER; ++m)
            if (m < K) g[b + m] = gz[m];
        if (SG::merged) g[b] += first_factor * mw[j] * z[b];
    }
    g[0] = z0bar;
}

// The same, rebuilding the activation's derivatives from z_0.
template <typename T, typename SG, int ACT, typename MW>
__device__ __forceinline__ void jet_apply_transposed(const T (&z)[SG::S], T (&g)[SG::S], const MW& mw) {
    T unused;
    const TanhD<T> d = fused_activation<T, ACT>(z[0], &unused);
    jet_apply_transposed_with<T, SG, MW>(d, z, g, mw);
}

template <typename T, int W, int CODE, int ACT>
__global__ void __launch_bounds__(FUSED_THREADS, 1) fused_step_kernel(FusedArgs<T> a) {
    typedef FusedGeom<T, W, CODE> G;
    typedef Sig<CODE> SG;
    constexpr int S = G::S, TP = G::TP, CG = G::CG, PG = G::PG, ROWP = G::ROWP, WP = G::WP, ROWS = G::ROWS,
                  MT = G::MT;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* smem = reinterpret_cast<T*>(smem_raw);
    T* act = smem + G::OFF_ACT;
    T* hr = smem + G::OFF_HR;
    T* zr = smem + G::OFF_ZR;
    T* wb = smem + G::OFF_WB;
    T* red = smem + G::OFF_RED;
    T* us = smem + G::OFF_U;
    T* uh = smem + G::OFF_UH;
    int4* code = reinterpret_cast<int4*>(smem_raw + (((size_t)G::TOTAL * sizeof(T) + 15) / 16) * 16);

    const int tid = threadIdx.x;
    const int tn = tid % CG, tp = tid / CG;
    const int L = a.L, d0 = a.d0;
    const bool backward = a.forward_only == 0;
    T* my_grad = a.grad_cta + (size_t)blockIdx.x * a.P;
    T* sz = a.scratch_z + (size_t)blockIdx.x * L * G::SCRATCH_PER_CTA;
    T* sh = a.scratch_h + (size_t)blockIdx.x * L * G::SCRATCH_PER_CTA;

    for (int i = tid; i < a.prog.n_instr; i += FUSED_THREADS) code[i] = a.prog.code[i];
    if (backward)
        for (int i = tid; i < a.P; i += FUSED_THREADS) my_grad[i] = T(0);
    double loss_sum = 0.0;  // threads < TP: one point each
    const T seed = a.cotangent[0] * a.weight * a.extra;
    __syncthreads();

    const long long n_tiles = (a.n_points + TP - 1) / TP;
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const long long p0 = tile * TP;
        T acc[S][2][4];
        T x[2][4];  // the coordinates of this thread's two points
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const long long p = min(p0 + 2 * tp + i, a.n_points - 1);
#pragma unroll
            for (int k = 0; k < 4; ++k) x[i][k] = k < d0 ? a.table[p * a.ncols + k] : T(0);
        }

        // ------------------------------ forward ------------------------------
        for (int l = 0; l < L; ++l) {
            if (l == 0) {
                // First layer: K = d0 <= 4; the derivative streams see the direction vectors.
                const T* w0 = a.params + a.w_off[0];
#pragma unroll
                for (int s = 0; s < S; ++s)
#pragma unroll
                    for (int i = 0; i < 2; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) acc[s][i][j] = T(0);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (k < d0) {
                        T wrow[4];
                        ld4(w0 + k * W + 4 * tn, wrow);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            acc[0][0][j] += x[0][k] * wrow[j];
                            acc[0][1][j] += x[1][k] * wrow[j];
                        }
#pragma unroll
                        for (int dj = 0; dj < SG::ndirs; ++dj) {
                            const T v = a.dirs[dj * d0 + k];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                acc[SG::base(dj)][0][j] += v * wrow[j];
                                acc[SG::base(dj)][1][j] += v * wrow[j];
                            }
                        }
                    }
                }
            } else {
                const T* wl = a.params + a.w_off[l];
                for (int e = tid; e < W * W; e += FUSED_THREADS) wb[(e / W) * WP + (e % W)] = wl[e];
                __syncthreads();  // weights and the previous epilogue's activations are in place
                tile_gemm<T, S, TP, ROWP, WP>(act, wb, W, tp, tn, acc);
                __syncthreads();  // every thread is done reading act and wb
            }
            if (a.b_off[l] >= 0) {
                T bias[4];
                ld4(a.params + a.b_off[l] + 4 * tn, bias);
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[0][i][j] += bias[j];
            }
            // Save the pre-activations, compose with tanh, save and stage the jets.
            T* zl = sz + (size_t)l * G::SCRATCH_PER_CTA;
            T* hl = sh + (size_t)l * G::SCRATCH_PER_CTA;
            if (backward) {
#pragma unroll
                for (int s = 0; s < S; ++s)
#pragma unroll
                    for (int i = 0; i < 2; ++i) st4(zl + ((size_t)s * TP + 2 * tp + i) * W + 4 * tn, acc[s][i]);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    T v[S];
#pragma unroll
                    for (int s = 0; s < S; ++s) v[s] = acc[s][i][j];
                    jet_apply<T, SG, ACT>(v, a.merge_w);
#pragma unroll
                    for (int s = 0; s < S; ++s) acc[s][i][j] = v[s];
                }
            if (backward) {
#pragma unroll
                for (int s = 0; s < S; ++s)
#pragma unroll
                    for (int i = 0; i < 2; ++i) st4(hl + ((size_t)s * TP + 2 * tp + i) * W + 4 * tn, acc[s][i]);
            }
            if (l + 1 < L) {
#pragma unroll
                for (int s = 0; s < S; ++s)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        st2(act + (4 * tn + j) * ROWP + s * TP + 2 * tp, acc[s][0][j], acc[s][1][j]);
            }
        }

        // ------------------------- head and residual -------------------------
        T wh[4];
        ld4(a.params + a.w_off[L] + 4 * tn, wh);
#pragma unroll
        for (int s = 0; s < S; ++s)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                T dot = T(0);
#pragma unroll
                for (int j = 0; j < 4; ++j) dot += acc[s][i][j] * wh[j];
#pragma unroll
                for (int o = CG / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                if (tn == 0) us[s * TP + 2 * tp + i] = dot;
            }
        __syncthreads();
        if (tid < TP) {
            const long long p = p0 + tid;
            const bool valid = p < a.n_points;
            const long long pc = valid ? p : a.n_points - 1;
            if (a.b_off[L] >= 0) us[tid] += a.params[a.b_off[L]];
            T r[MAX_REGS];
            run_program<T>(code, a.prog.n_instr, static_cast<const T*>(a.prog.consts), a.table + pc * a.ncols, us + tid,
                           TP, r);
            if (valid) loss_sum += (double)r[a.prog.value_reg];
#pragma unroll
            for (int s = 0; s < S; ++s) {
                const int reg = a.prog.grad_regs[s];
                uh[s * TP + tid] = (valid && reg >= 0) ? seed * r[reg] : T(0);
            }
        }
        if (!backward) {
            __syncthreads();
            continue;
        }
        __syncthreads();

        // ------------------------------ backward ------------------------------
        // Head: dW = sum h * uhat, db = sum uhat(primal), G = uhat (x) w.
        {
            T ug[S][2];
#pragma unroll
            for (int s = 0; s < S; ++s) ld2(uh + s * TP + 2 * tp, ug[s][0], ug[s][1]);
            T pw[4] = {T(0), T(0), T(0), T(0)};
#pragma unroll
            for (int s = 0; s < S; ++s)
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        pw[j] += acc[s][i][j] * ug[s][i];
                        acc[s][i][j] = ug[s][i] * wh[j];
                    }
            st4(red + tp * W + 4 * tn, pw);
            __syncthreads();
            if (tid < W) {
                T total = T(0);
                for (int g = 0; g < PG; ++g) total += red[g * W + tid];
                my_grad[a.w_off[L] + tid] += total;
            }
            if (tid == 0 && a.b_off[L] >= 0) {
                T total = T(0);
                for (int p = 0; p < TP; ++p) total += uh[p];
                my_grad[a.b_off[L]] += total;
            }
            __syncthreads();
        }
        for (int l = L - 1; l >= 0; --l) {
            // acc holds the cotangents of layer l's jets; turn them into cotangents of its pre-activations.
            const T* zl = sz + (size_t)l * G::SCRATCH_PER_CTA;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                T zs[S][4];
#pragma unroll
                for (int s = 0; s < S; ++s) ld4(zl + ((size_t)s * TP + 2 * tp + i) * W + 4 * tn, zs[s]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    T z[S], g[S];
#pragma unroll
                    for (int s = 0; s < S; ++s) {
                        z[s] = zs[s][j];
                        g[s] = acc[s][i][j];
                    }
                    jet_apply_transposed<T, SG, ACT>(z, g, a.merge_w);
#pragma unroll
                    for (int s = 0; s < S; ++s) acc[s][i][j] = g[s];
                }
            }
            // Bias gradient partials (primal stream) and, for the first layer, the weight gradient partials.
            {
                T pb[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) pb[j] = acc[0][0][j] + acc[0][1][j];
                st4(red + tp * 5 * W + 4 * tn, pb);
            }
            if (l == 0) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (k < d0) {
                        T pw[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) pw[j] = x[0][k] * acc[0][0][j] + x[1][k] * acc[0][1][j];
#pragma unroll
                        for (int dj = 0; dj < SG::ndirs; ++dj) {
                            const T v = a.dirs[dj * d0 + k];
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                pw[j] += v * (acc[SG::base(dj)][0][j] + acc[SG::base(dj)][1][j]);
                        }
                        st4(red + (tp * 5 + 1 + k) * W + 4 * tn, pw);
                    }
                }
                __syncthreads();
                for (int e = tid; e < (1 + d0) * W; e += FUSED_THREADS) {
                    const int which = e / W, n = e % W;
                    T total = T(0);
                    for (int g = 0; g < PG; ++g) total += red[(g * 5 + which) * W + n];
                    if (which == 0) {
                        if (a.b_off[0] >= 0) my_grad[a.b_off[0] + n] += total;
                    } else {
                        my_grad[a.w_off[0] + (which - 1) * W + n] += total;
                    }
                }
                __syncthreads();
                break;
            }
            // Stage the operands: cotangents k-major (dgrad A) and row-major (wgrad B), the previous
            // layer's jets row-major (wgrad A), the transposed weights (dgrad B).
#pragma unroll
            for (int s = 0; s < S; ++s) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    st2(act + (4 * tn + j) * ROWP + s * TP + 2 * tp, acc[s][0][j], acc[s][1][j]);
#pragma unroll
                for (int i = 0; i < 2; ++i) st4(zr + (s * TP + 2 * tp + i) * WP + 4 * tn, acc[s][i]);
            }
            {
                const T* hp = sh + (size_t)(l - 1) * G::SCRATCH_PER_CTA;
                for (int e = tid; e < ROWS * CG; e += FUSED_THREADS) {
                    const int row = e / CG, c4 = e % CG;
                    T v[4];
                    ld4(hp + (size_t)row * W + 4 * c4, v);
                    st4(hr + row * WP + 4 * c4, v);
                }
                const T* wl = a.params + a.w_off[l];
                for (int e = tid; e < W * W; e += FUSED_THREADS) wb[(e % W) * WP + (e / W)] = wl[e];
            }
            __syncthreads();
            if (tid < W && a.b_off[l] >= 0) {
                T total = T(0);
                for (int g = 0; g < PG; ++g) total += red[g * 5 * W + tid];
                my_grad[a.b_off[l] + tid] += total;
            }
            // Weight gradient of layer l: dW[k][n] += sum_rows hr[row][k] * zr[row][n].
            {
                const int ty = tid / 16, tx = tid % 16;
                T dw[MT][MT];
#pragma unroll
                for (int i = 0; i < MT; ++i)
#pragma unroll
                    for (int j = 0; j < MT; ++j) dw[i][j] = T(0);
#pragma unroll 4
                for (int row = 0; row < ROWS; ++row) {
                    T hv[MT], zv[MT];
#pragma unroll
                    for (int i = 0; i < MT; ++i) hv[i] = hr[row * WP + ty * MT + i];
#pragma unroll
                    for (int j = 0; j < MT; ++j) zv[j] = zr[row * WP + tx * MT + j];
#pragma unroll
                    for (int i = 0; i < MT; ++i)
#pragma unroll
                        for (int j = 0; j < MT; ++j) dw[i][j] += hv[i] * zv[j];
                }
                T* gw = my_grad + a.w_off[l];
#pragma unroll
                for (int i = 0; i < MT; ++i)
#pragma unroll
                    for (int j = 0; j < MT; ++j) gw[(ty * MT + i) * W + tx * MT + j] += dw[i][j];
            }
            // Cotangents of layer l-1's jets: G = Zhat W^T.
            tile_gemm<T, S, TP, ROWP, WP>(act, wb, W, tp, tn, acc);
            __syncthreads();
        }
    }

    // Per-CTA loss partial, fixed order.
    double* lred = reinterpret_cast<double*>(hr);
    __syncthreads();
    if (tid < TP) lred[tid] = loss_sum;
    __syncthreads();
    if (tid == 0) {
        double total = 0.0;
        for (int p = 0; p < TP; ++p) total += lred[p];
        a.loss_cta[blockIdx.x] = total;
    }
}

}  // namespace qb
