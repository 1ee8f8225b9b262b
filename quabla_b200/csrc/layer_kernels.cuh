// Layer-wise engine: the kernels that run a tanh MLP of any width over a chunk
// of collocation points while carrying the primal and the derivative streams.
//
// Activation layout for a chunk of C points and a layer of width d:
//   [S][C][d], stream-major, d contiguous,
// so the S streams of a layer form ONE row-major matrix of S*C rows and every
// weight contraction is a single GEMM over all streams (the reference issues a
// batch=B, M=1 strided-batched GEMM per stream instead,
// crates/quabla-core/src/tensor_ir/cuda.rs:4936-5035).
#pragma once
#include "jet_math.cuh"

namespace qb {

// ---------------------------------------------------------------------------
// Tiled SIMT GEMM, C[m][n] = sum_k A(m,k) * B(k,n), with arbitrary element
// strides so that the same kernel serves
//   forward   Z  = H W            (A k-fast, B n-fast)
//   dgrad     G' = G W^T          (A k-fast, B k-fast)
//   wgrad     dW = H^T G          (A m-fast, B n-fast, split over k = rows)
// gridDim.z splits k; slice z writes its partial to C + z * M * N.
// ---------------------------------------------------------------------------
template <typename T>
struct GemmArgs {
    const T* A;
    const T* B;
    T* C;
    const T* bias;       // added to rows < bias_rows (the primal stream), may be null
    long long sam, sak;  // strides of A(m,k)
    long long sbk, sbn;  // strides of B(k,n)
    int M, N, K;
    int ldc;
    int bias_rows;
    int k_chunk;         // k range per grid.z slice
};

constexpr int WGRAD_ROWS_PER_SLICE = 4096;  // rows summed in the plan dtype before the double reduction
constexpr int GEMM_BM = 64;
constexpr int GEMM_BN = 64;
constexpr int GEMM_BK = 16;

template <typename T, bool A_KFAST, bool B_NFAST>
__global__ void __launch_bounds__(256) gemm_kernel(GemmArgs<T> g) {
    __shared__ T As[GEMM_BK][GEMM_BM + 4];
    __shared__ T Bs[GEMM_BK][GEMM_BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * GEMM_BM, n0 = blockIdx.x * GEMM_BN;
    const int k_begin = blockIdx.z * g.k_chunk;
    const int k_end = min(g.K, k_begin + g.k_chunk);
    T acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = T(0);

    for (int kt = k_begin; kt < k_end; kt += GEMM_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            int m, k;
            if (A_KFAST) {
                k = idx % GEMM_BK;
                m = idx / GEMM_BK;
            } else {
                m = idx % GEMM_BM;
                k = idx / GEMM_BM;
            }
            const int gm = m0 + m, gk = kt + k;
            As[k][m] = (gm < g.M && gk < k_end) ? g.A[gm * g.sam + gk * g.sak] : T(0);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            int n, k;
            if (B_NFAST) {
                n = idx % GEMM_BN;
                k = idx / GEMM_BN;
            } else {
                k = idx % GEMM_BK;
                n = idx / GEMM_BK;
            }
            const int gn = n0 + n, gk = kt + k;
            Bs[k][n] = (gn < g.N && gk < k_end) ? g.B[gk * g.sbk + gn * g.sbn] : T(0);
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GEMM_BK; ++k) {
            T a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
        }
        __syncthreads();
    }
    T* C = g.C + (long long)blockIdx.z * g.M * g.ldc;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= g.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= g.N) continue;
            T v = acc[i][j];
            if (g.bias != nullptr && gm < g.bias_rows) v += g.bias[gn];
            C[(long long)gm * g.ldc + gn] = v;
        }
    }
}

// Forward product with a narrow contraction (the first layer: K = network inputs <= 4):
// C[row][n] = sum_{j<K} A[row][j] * W[j][n] (+ bias[n] on rows < bias_rows).  A thread owns four
// consecutive columns and keeps its 4 K weights in registers; a row's A values are a broadcast load.
// HBM-bound on the write of C.
template <typename T, int K>
__global__ void __launch_bounds__(256) skinny_forward_kernel(const T* __restrict__ A, const T* __restrict__ W,
                                                             const T* __restrict__ bias, T* __restrict__ C,
                                                             long long rows, int N, int bias_rows) {
    const int groups = N / 4;                       // column groups of four per row
    const int group = threadIdx.x % groups;         // blockDim.x is a multiple of groups
    const int rows_per_block = blockDim.x / groups;
    T w[K][4], b[4];
#pragma unroll
    for (int j = 0; j < K; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) w[j][i] = W[(long long)j * N + 4 * group + i];
#pragma unroll
    for (int i = 0; i < 4; ++i) b[i] = bias != nullptr ? bias[4 * group + i] : T(0);
    for (long long row = (long long)blockIdx.x * rows_per_block + threadIdx.x / groups; row < rows;
         row += (long long)gridDim.x * rows_per_block) {
        T a[K], v[4];
#pragma unroll
        for (int j = 0; j < K; ++j) a[j] = A[row * K + j];
        const bool biased = row < bias_rows;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            T sum = T(0);
#pragma unroll
            for (int j = 0; j < K; ++j) sum += a[j] * w[j][i];
            v[i] = biased ? sum + b[i] : sum;
        }
        T* out = C + row * N + 4 * group;  // 16-byte aligned: N % 4 == 0 and C comes from cudaMalloc
        if (sizeof(T) == 4) {
            *reinterpret_cast<float4*>(out) = make_float4((float)v[0], (float)v[1], (float)v[2], (float)v[3]);
        } else {
            reinterpret_cast<double2*>(out)[0] = make_double2((double)v[0], (double)v[1]);
            reinterpret_cast<double2*>(out)[1] = make_double2((double)v[2], (double)v[3]);
        }
    }
}

// Weight gradient with one narrow side (the first layer's d_in <= 8 coordinates, the head's single
// output): P[z][m][n] = sum over the rows r of slice z of A[r][m] * B[r][n].  One thread per element
// of the wide side streams its column (coalesced across the CTA) and keeps NARROW accumulators; the
// narrow operand is a broadcast load.  HBM-bound: the wide matrix is read once.
template <typename T, int NARROW, bool NARROW_A>
__global__ void __launch_bounds__(256) skinny_wgrad_kernel(const T* __restrict__ A, const T* __restrict__ B,
                                                           T* __restrict__ P, long long rows, int M, int N, int k_chunk) {
    const int wide = NARROW_A ? N : M;
    const int col = blockIdx.x * 256 + threadIdx.x;
    if (col >= wide) return;
    const T* __restrict__ wide_ptr = NARROW_A ? B : A;
    const T* __restrict__ narrow_ptr = NARROW_A ? A : B;
    const long long r0 = (long long)blockIdx.y * k_chunk;
    const long long r1 = min(rows, r0 + (long long)k_chunk);
    T acc[NARROW];
#pragma unroll
    for (int i = 0; i < NARROW; ++i) acc[i] = T(0);
#pragma unroll 8
    for (long long r = r0; r < r1; ++r) {
        const T w = wide_ptr[r * wide + col];
#pragma unroll
        for (int i = 0; i < NARROW; ++i) acc[i] += narrow_ptr[r * NARROW + i] * w;
    }
    T* out = P + (long long)blockIdx.y * M * N;
#pragma unroll
    for (int i = 0; i < NARROW; ++i) {
        if (NARROW_A)
            out[(long long)i * N + col] = acc[i];
        else
            out[(long long)col * N + i] = acc[i];
    }
}

// Column sums of the first `rows` rows of G[rows][N] (bias gradients), split
// over rows: slice z writes partial[z][n].
template <typename T>
__global__ void __launch_bounds__(256) colsum_kernel(const T* __restrict__ G, T* __restrict__ partial, int rows,
                                                     int N, int row_chunk) {
    __shared__ T red[8][33];
    const int lane = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int n = blockIdx.x * 32 + lane;
    const int r0 = blockIdx.y * row_chunk;
    const int r1 = min(rows, r0 + row_chunk);
    T s = T(0);
    if (n < N)
        for (int r = r0 + ty; r < r1; r += 8) s += G[(long long)r * N + n];
    red[ty][lane] = s;
    __syncthreads();
    if (ty == 0 && n < N) {
        T total = red[0][lane];
#pragma unroll
        for (int i = 1; i < 8; ++i) total += red[i][lane];
        partial[(long long)blockIdx.y * N + n] = total;
    }
}

// acc[i] += sum_z partial[z][i] in double, in a fixed order: the second pass that keeps gradients
// bit-reproducible (the reference sums long axes in double as well, cuda.rs:8202-8247).  A block
// owns EX consecutive elements; thread (x, y) sums the slices z = y, y + G, ... of element x
// (G = 256 / EX groups, coalesced along x), then the G partial sums are added in y order.
// EX = 32 suits many elements and few slices, EX = 8 or 2 few elements and hundreds or thousands of slices.
template <typename T, int EX>
__global__ void __launch_bounds__(256) accumulate_partials_kernel(const T* __restrict__ partial, double* __restrict__ acc,
                                                                  int count, int slices) {
    constexpr int GROUPS = 256 / EX;
    __shared__ double part[GROUPS][EX + 1];
    const int x = threadIdx.x % EX, y = threadIdx.x / EX;
    const int i = blockIdx.x * EX + x;
    double s = 0.0;
    if (i < count) {
#pragma unroll 4
        for (int z = y; z < slices; z += GROUPS) s += (double)partial[(long long)z * count + i];
    }
    part[y][x] = s;
    __syncthreads();
    if (y == 0 && i < count) {
        double total = part[0][x];
#pragma unroll
        for (int k = 1; k < GROUPS; ++k) total += part[k][x];
        acc[i] += total;
    }
}

template <typename T>
inline void accumulate_partials_launch(const T* partial, double* acc, int count, int slices, cudaStream_t stream) {
    if (slices > 1024 && count <= 4096)  // per-block partials of the jet kernels: thousands of slices of a few hundred elements
        accumulate_partials_kernel<T, 2><<<(count + 1) / 2, 256, 0, stream>>>(partial, acc, count, slices);
    else if (slices > 256 && count <= 4096)
        accumulate_partials_kernel<T, 8><<<(count + 7) / 8, 256, 0, stream>>>(partial, acc, count, slices);
    else
        accumulate_partials_kernel<T, 32><<<(count + 31) / 32, 256, 0, stream>>>(partial, acc, count, slices);
}

// out[i] = sum_z partial[z][i], z ascending, summed in double and rounded once.
template <typename T>
__global__ void reduce_partials_kernel(const T* __restrict__ partial, T* __restrict__ out, int count, int slices) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    double s = 0.0;
#pragma unroll 8
    for (int z = 0; z < slices; ++z) s += (double)partial[(long long)z * count + i];
    out[i] = (T)s;
}

// ---------------------------------------------------------------------------
// Input streams of the first layer from the point table:
//   stream 0 = the coordinates, first-order stream of direction j = v_j,
//   every higher-order stream = 0.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void seed_input_kernel(const T* __restrict__ table, int table_cols, long long point0, int C, int d0,
                                  JetSpec spec, const T* __restrict__ dirs, T* __restrict__ H0) {
    const long long total = (long long)spec.S * C * d0;
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total;
         e += (long long)gridDim.x * blockDim.x) {
        const int k = (int)(e % d0);
        const long long r = e / d0;
        const int c = (int)(r % C);
        const int s = (int)(r / C);
        T v = T(0);
        if (s == 0) {
            v = table[(point0 + c) * table_cols + k];
        } else {
            for (int j = 0; j < spec.ndirs; ++j)
                if (s == spec.base[j]) v = dirs[j * d0 + k];
        }
        H0[e] = v;
    }
}

// H = tanh-jet(Z), all streams, one thread per (point, unit).
template <typename T>
__global__ void jet_forward_kernel(const T* __restrict__ Z, T* __restrict__ H, long long plane, JetSpec spec, int act) {
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < plane;
         e += (long long)gridDim.x * blockDim.x) {
        T t;
        const TanhD<T> d(Z[e], act, &t);
        H[e] = t;
        if (spec.merged) {
            // Reads the pre-activation first-order streams, so it goes before the loop that may run in place.
            T q = T(0);
            for (int j = 0; j < spec.ndirs; ++j) {
                const T z1 = Z[(long long)spec.base[j] * plane + e];
                q += (T)spec.merge_w[j] * z1 * z1;
            }
            const long long m = (long long)(spec.S - 1) * plane + e;
            H[m] = merged_compose(d, q, Z[m]);
        }
        for (int j = 0; j < spec.ndirs; ++j) {
            const long long off = (long long)spec.base[j] * plane + e;
            T z[MAX_ORDER], h[MAX_ORDER];
            const int K = spec.order[j];
#pragma unroll
            for (int m = 0; m < MAX_ORDER; ++m) z[m] = (m < K) ? Z[off + m * plane] : T(0);
            switch (K) {
                case 1: jet_compose<T, 1>(d, z, h); break;
                case 2: jet_compose<T, 2>(d, z, h); break;
                case 3: jet_compose<T, 3>(d, z, h); break;
                default: jet_compose<T, 4>(d, z, h); break;
            }
#pragma unroll
            for (int m = 0; m < MAX_ORDER; ++m)
                if (m < K) H[off + m * plane] = h[m];
        }
    }
}

// In place: G (cotangents of H) becomes the cotangents of Z.
template <typename T>
__global__ void jet_backward_kernel(const T* __restrict__ Z, const T* __restrict__ Hprimal, T* __restrict__ G,
                                    long long plane, JetSpec spec, int act) {
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < plane;
         e += (long long)gridDim.x * blockDim.x) {
        // tanh: derivatives from the saved activation; otherwise from the saved pre-activation.
        T unused;
        const TanhD<T> d = act == ACT_TANH ? TanhD<T>(Hprimal[e]) : TanhD<T>(Z[e], act, &unused);
        T z0bar = d.t1 * G[e];
        T first_factor = T(0);
        if (spec.merged) {
            T q = T(0);
            for (int j = 0; j < spec.ndirs; ++j) {
                const T z1 = Z[(long long)spec.base[j] * plane + e];
                q += (T)spec.merge_w[j] * z1 * z1;
            }
            const long long m = (long long)(spec.S - 1) * plane + e;
            const T gM = G[m];
            T gzM;
            z0bar += merged_compose_transposed(d, q, Z[m], gM, &gzM);
            first_factor = merged_first_order_factor(d, gM);
            G[m] = gzM;
        }
        for (int j = 0; j < spec.ndirs; ++j) {
            const long long off = (long long)spec.base[j] * plane + e;
            T z[MAX_ORDER], g[MAX_ORDER], gz[MAX_ORDER];
            const int K = spec.order[j];
#pragma unroll
            for (int m = 0; m < MAX_ORDER; ++m) {
                z[m] = (m < K) ? Z[off + m * plane] : T(0);
                g[m] = (m < K) ? G[off + m * plane] : T(0);
            }
            switch (K) {
                case 1: z0bar += jet_compose_transposed<T, 1>(d, z, g, gz); break;
                case 2: z0bar += jet_compose_transposed<T, 2>(d, z, g, gz); break;
                case 3: z0bar += jet_compose_transposed<T, 3>(d, z, g, gz); break;
                default: z0bar += jet_compose_transposed<T, 4>(d, z, g, gz); break;
            }
            if (spec.merged) gz[0] += first_factor * (T)spec.merge_w[j] * z[0];
#pragma unroll
            for (int m = 0; m < MAX_ORDER; ++m)
                if (m < K) G[off + m * plane] = gz[m];
        }
        G[e] = z0bar;
    }
}

// Last (linear, width -> 1) layer: U[row] = H[row][:] . w (+ b on the primal
// rows); one warp per row, fixed shuffle tree.
template <typename T>
__global__ void head_forward_kernel(const T* __restrict__ H, const T* __restrict__ w, const T* __restrict__ b,
                                    T* __restrict__ U, long long rows, int d, int primal_rows) {
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long r = warp; r < rows; r += nwarps) {
        T s = T(0);
        for (int k = lane; k < d; k += 32) s += H[r * d + k] * w[k];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) U[r] = s + ((b != nullptr && r < primal_rows) ? b[0] : T(0));
    }
}

// Cotangent of the last hidden layer: G[row][k] = Uhat[row] * w[k].
template <typename T>
__global__ void head_backward_kernel(const T* __restrict__ Uhat, const T* __restrict__ w, T* __restrict__ G,
                                     long long rows, int d) {
    const long long total = rows * d;
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total;
         e += (long long)gridDim.x * blockDim.x) {
        G[e] = Uhat[e / d] * w[e % d];
    }
}

}  // namespace qb
