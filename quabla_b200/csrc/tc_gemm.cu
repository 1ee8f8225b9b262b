// Host side of the tcgen05 float32 GEMMs.
#include "tc_gemm.h"

#include <cstdlib>
#include <cstring>

#include "tc_gemm.cuh"

namespace qb {

bool tc_enabled() {
    const char* env = getenv("QB200_TC");
    return !(env != nullptr && strcmp(env, "0") == 0);
}

bool tc_rows_ok(int N, int K) { return N % 64 == 0 && N >= 64 && N <= 256 && K % TC_BK == 0 && K >= TC_BK; }

bool tc_wgrad_ok(int Mw, int N) { return Mw % TC_BM == 0 && N % 64 == 0 && N >= 64 && N <= 256; }

size_t tc_image_words(int K, int N) { return (size_t)4 * K * N; }

cudaError_t tc_prep_launch(const float* w, int K, int N, uint32_t* image, cudaStream_t stream) {
    const int blocks = (K * N + 255) / 256;
    tc_prep_weight_kernel<<<blocks < 296 ? blocks : 296, 256, 0, stream>>>(w, K, N, image);
    return cudaGetLastError();
}

static size_t smem_bytes(int N) { return (size_t)2 * (2 * TC_BM * TC_BK * 4 + 2 * N * TC_BK * 4) + 64; }

template <bool WGRAD>
static cudaError_t configure(int N) {
    return cudaFuncSetAttribute(reinterpret_cast<const void*>(tc_gemm_kernel<WGRAD>),
                                cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes(N));
}

cudaError_t tc_rows_launch(const float* A, int lda, const uint32_t* image, bool backward, int wK, int wN, float* C,
                           int ldc, const float* bias, int bias_rows, int M, int* error, cudaStream_t stream) {
    TcGemmArgs a;
    memset(&a, 0, sizeof(a));
    const size_t plane = (size_t)wK * wN;
    a.A = A;
    a.Bhi = image + (backward ? 2 : 0) * plane;
    a.Blo = image + (backward ? 3 : 1) * plane;
    a.C = C;
    a.bias = bias;
    a.M = M;
    a.N = backward ? wK : wN;   // output width
    a.K = backward ? wN : wK;   // contraction
    a.lda = lda;
    a.ldc = ldc;
    a.bias_rows = bias_rows;
    a.error = error;
    cudaError_t e = configure<false>(a.N);
    if (e != cudaSuccess) return e;
    tc_gemm_kernel<false><<<(M + TC_BM - 1) / TC_BM, TC_THREADS, smem_bytes(a.N), stream>>>(a);
    return cudaGetLastError();
}

cudaError_t tc_wgrad_launch(const float* H, int ldh, const float* G, int ldg, float* partials, int rows, int Mw,
                            int N, int rows_per_slice, int* error, cudaStream_t stream) {
    TcGemmArgs a;
    memset(&a, 0, sizeof(a));
    a.A = H;
    a.B = G;
    a.C = partials;
    a.M = Mw;
    a.N = N;
    a.K = rows;
    a.lda = ldh;
    a.ldb = ldg;
    a.ldc = N;
    a.k_slice = rows_per_slice;
    a.error = error;
    cudaError_t e = configure<true>(N);
    if (e != cudaSuccess) return e;
    const int slices = (rows + rows_per_slice - 1) / rows_per_slice;
    tc_gemm_kernel<true><<<dim3(slices, Mw / TC_BM), TC_THREADS, smem_bytes(N), stream>>>(a);
    return cudaGetLastError();
}

}  // namespace qb
