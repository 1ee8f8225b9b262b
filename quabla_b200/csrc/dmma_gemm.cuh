// Float64 GEMM on the FP64 tensor-core path (mma.sync m8n8k4, "DMMA") for the
// layer-wise engine, with the same operand description as the SIMT gemm_kernel:
//   forward   Z  = H W            (A k-fast, B n-fast)
//   dgrad     G' = G W^T          (A k-fast, B k-fast)
//   wgrad     dW = H^T G          (A m-fast, B n-fast, split over k = rows)
//
// A CTA of 256 threads owns a 128 x 64 tile of C; warp (wm, wn) of the 4 x 2 warp grid owns
// 32 x 32 of it as 4 x 4 m8n8 accumulator tiles (64 doubles per thread).  Operand tiles of 16 k
// are staged by cp.async (16 bytes per copy, zero-filled outside the matrix) into a three-stage
// ring; every smem row stride is 4 (mod 16) doubles, which makes the 64-bit fragment loads of a
// half warp (4 k x 4 rows) fall into 16 distinct bank pairs.
//
// FP64 MMA accumulates with IEEE fused multiply-adds, so the result differs from the SIMT kernel
// only in summation order.  Measured on B200: m8n8k4 issues at 64 FMA/clk/SM, the same rate as
// DFMA; the gain over the SIMT kernel is fewer shared-memory loads and instructions per FMA
// (16 FMA per 64-bit load against 2).
#pragma once
#include <cstdint>
#include <cstdlib>

#include "layer_kernels.cuh"

namespace qb {

constexpr int DM_BM = 128;
constexpr int DM_BN = 64;
constexpr int DM_BK = 16;
constexpr int DM_STAGES = 3;
constexpr int DM_THREADS = 256;
constexpr int DM_LDK = DM_BK + 4;   // [row][k] tiles
constexpr int DM_LDAM = DM_BM + 4;  // A as [k][m]
constexpr int DM_LDBN = DM_BN + 4;  // B as [k][n]

template <bool A_KFAST>
struct DmmaATile {
    static constexpr int ELEMS = A_KFAST ? DM_BM * DM_LDK : DM_BK * DM_LDAM;
};
template <bool B_NFAST>
struct DmmaBTile {
    static constexpr int ELEMS = B_NFAST ? DM_BK * DM_LDBN : DM_BN * DM_LDK;
};
template <bool A_KFAST, bool B_NFAST>
constexpr size_t dmma_smem_bytes() {
    return (size_t)DM_STAGES * (DmmaATile<A_KFAST>::ELEMS + DmmaBTile<B_NFAST>::ELEMS) * sizeof(double);
}

__device__ __forceinline__ void dmma_m8n8k4(double (&c)[2], double a, double b) {
    asm("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
        : "+d"(c[0]), "+d"(c[1])
        : "d"(a), "d"(b));
}

// 16-byte asynchronous copy; `valid` false zero-fills the destination.
__device__ __forceinline__ void dm_copy16(double* dst, const double* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

template <bool A_KFAST, bool B_NFAST>
__global__ void __launch_bounds__(DM_THREADS, 2) dmma_gemm_kernel(GemmArgs<double> g) {
    extern __shared__ __align__(16) unsigned char dm_smem[];
    constexpr int A_ELEMS = DmmaATile<A_KFAST>::ELEMS, B_ELEMS = DmmaBTile<B_NFAST>::ELEMS;
    double* const As = reinterpret_cast<double*>(dm_smem);
    double* const Bs = As + DM_STAGES * A_ELEMS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp & 3, wn = warp >> 2;
    const int m0 = blockIdx.y * DM_BM, n0 = blockIdx.x * DM_BN;
    const int k_begin = blockIdx.z * g.k_chunk;
    const int k_end = min(g.K, k_begin + g.k_chunk);
    const int tiles = (k_end - k_begin + DM_BK - 1) / DM_BK;

    auto stage_tile = [&](int stage, int kt) {
        double* a = As + stage * A_ELEMS;
        double* b = Bs + stage * B_ELEMS;
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // A: 128 x 16 doubles = 1024 copies
            const int v = tid + i * DM_THREADS;
            if (A_KFAST) {
                const int m = v >> 3, k = (v & 7) * 2;
                const bool ok = (m0 + m < g.M) && (kt + k < k_end);
                dm_copy16(a + m * DM_LDK + k, ok ? g.A + (long long)(m0 + m) * g.sam + (kt + k) : g.A, ok);
            } else {
                const int k = v >> 6, m = (v & 63) * 2;
                const bool ok = (m0 + m < g.M) && (kt + k < k_end);
                dm_copy16(a + k * DM_LDAM + m, ok ? g.A + (long long)(kt + k) * g.sak + (m0 + m) : g.A, ok);
            }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {  // B: 16 x 64 doubles = 512 copies
            const int v = tid + i * DM_THREADS;
            if (B_NFAST) {
                const int k = v >> 5, n = (v & 31) * 2;
                const bool ok = (n0 + n < g.N) && (kt + k < k_end);
                dm_copy16(b + k * DM_LDBN + n, ok ? g.B + (long long)(kt + k) * g.sbk + (n0 + n) : g.B, ok);
            } else {
                const int n = v >> 3, k = (v & 7) * 2;
                const bool ok = (n0 + n < g.N) && (kt + k < k_end);
                dm_copy16(b + n * DM_LDK + k, ok ? g.B + (long long)(n0 + n) * g.sbn + (kt + k) : g.B, ok);
            }
        }
    };

    double acc[4][4][2];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

#pragma unroll
    for (int s = 0; s < DM_STAGES - 1; ++s) {
        if (s < tiles) stage_tile(s, k_begin + s * DM_BK);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const int fr = lane >> 2, fk = lane & 3;  // fragment row (or column) and k of this lane
    for (int t = 0; t < tiles; ++t) {
        asm volatile("cp.async.wait_group %0;" ::"n"(DM_STAGES - 2) : "memory");
        __syncthreads();  // tile t has landed for everyone; the stage of tile t-1 is free
        const int next = t + DM_STAGES - 1;
        if (next < tiles) stage_tile(next % DM_STAGES, k_begin + next * DM_BK);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const double* a = As + (t % DM_STAGES) * A_ELEMS;
        const double* b = Bs + (t % DM_STAGES) * B_ELEMS;
#pragma unroll
        for (int ks = 0; ks < DM_BK / 4; ++ks) {
            const int k = ks * 4 + fk;
            double af[4], bf[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int m = wm * 32 + i * 8 + fr;
                af[i] = A_KFAST ? a[m * DM_LDK + k] : a[k * DM_LDAM + m];
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = wn * 32 + j * 8 + fr;
                bf[j] = B_NFAST ? b[k * DM_LDBN + n] : b[n * DM_LDK + k];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) dmma_m8n8k4(acc[i][j], af[i], bf[j]);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    double* C = g.C + (long long)blockIdx.z * g.M * g.ldc;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + wm * 32 + i * 8 + fr;
        if (gm >= g.M) continue;
        const bool add_bias = g.bias != nullptr && gm < g.bias_rows;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + wn * 32 + j * 8 + 2 * fk;
            if (gn >= g.N) continue;
            double2 v = make_double2(acc[i][j][0], acc[i][j][1]);
            if (add_bias) {
                v.x += g.bias[gn];
                v.y += g.bias[gn + 1];
            }
            *reinterpret_cast<double2*>(C + (long long)gm * g.ldc + gn) = v;
        }
    }
}

inline bool dm_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Whether the operands meet the kernel's 16-byte copy rules: unit stride along the fast axis,
// even strides and extents along it, 16-byte aligned bases, C rows 16-byte aligned.
template <bool A_KFAST, bool B_NFAST>
inline bool dmma_eligible(const GemmArgs<double>& g) {
    if (!dm_aligned16(g.A) || !dm_aligned16(g.B) || !dm_aligned16(g.C) || (g.ldc & 1) || (g.N & 1)) return false;
    if (g.bias != nullptr && (reinterpret_cast<uintptr_t>(g.bias) & 7)) return false;
    if (A_KFAST) {
        if (g.sak != 1 || (g.sam & 1) || (g.K & 1) || (g.k_chunk & 1)) return false;
    } else {
        if (g.sam != 1 || (g.sak & 1) || (g.M & 1)) return false;
    }
    if (B_NFAST) {
        if (g.sbn != 1 || (g.sbk & 1)) return false;
    } else {
        if (g.sbk != 1 || (g.sbn & 1) || (g.K & 1) || (g.k_chunk & 1)) return false;
    }
    // Small outputs stay on the SIMT kernel, whose 64 x 64 tile wastes less of them.
    return g.N >= 32 && g.M >= 32;
}

inline bool dmma_enabled() {
    static const bool on = [] {
        const char* e = getenv("QB200_DMMA");
        return e == nullptr || e[0] != '0';
    }();
    return on;
}

// Launch C = A B over `slices` split-K slices with the kernel that fits: the FP64 tensor-core
// kernel for float64 operands that meet its rules, else the SIMT kernel.
template <typename T, bool A_KFAST, bool B_NFAST>
inline cudaError_t gemm_launch(const GemmArgs<T>& g, int slices, cudaStream_t stream) {
    dim3 grid((g.N + GEMM_BN - 1) / GEMM_BN, (g.M + GEMM_BM - 1) / GEMM_BM, slices);
    gemm_kernel<T, A_KFAST, B_NFAST><<<grid, 256, 0, stream>>>(g);
    return cudaGetLastError();
}

template <bool A_KFAST, bool B_NFAST>
inline cudaError_t gemm_launch_f64(const GemmArgs<double>& g, int slices, cudaStream_t stream) {
    if (dmma_enabled() && dmma_eligible<A_KFAST, B_NFAST>(g)) {
        constexpr size_t smem = dmma_smem_bytes<A_KFAST, B_NFAST>();
        cudaError_t e = cudaFuncSetAttribute(dmma_gemm_kernel<A_KFAST, B_NFAST>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        dim3 grid((g.N + DM_BN - 1) / DM_BN, (g.M + DM_BM - 1) / DM_BM, slices);
        dmma_gemm_kernel<A_KFAST, B_NFAST><<<grid, DM_THREADS, smem, stream>>>(g);
        return cudaGetLastError();
    }
    dim3 grid((g.N + GEMM_BN - 1) / GEMM_BN, (g.M + GEMM_BM - 1) / GEMM_BM, slices);
    gemm_kernel<double, A_KFAST, B_NFAST><<<grid, 256, 0, stream>>>(g);
    return cudaGetLastError();
}

template <>
inline cudaError_t gemm_launch<double, true, true>(const GemmArgs<double>& g, int slices, cudaStream_t stream) {
    return gemm_launch_f64<true, true>(g, slices, stream);
}
template <>
inline cudaError_t gemm_launch<double, true, false>(const GemmArgs<double>& g, int slices, cudaStream_t stream) {
    return gemm_launch_f64<true, false>(g, slices, stream);
}
template <>
inline cudaError_t gemm_launch<double, false, true>(const GemmArgs<double>& g, int slices, cudaStream_t stream) {
    return gemm_launch_f64<false, true>(g, slices, stream);
}

// CTA tiles of the output under the kernel gemm_launch picks (for sizing split-K slices).
inline int gemm_output_tiles(int M, int N, bool tensor_core) {
    if (tensor_core) return ((N + DM_BN - 1) / DM_BN) * ((M + DM_BM - 1) / DM_BM);
    return ((N + GEMM_BN - 1) / GEMM_BN) * ((M + GEMM_BM - 1) / GEMM_BM);
}

}  // namespace qb
