// Launchers of the tcgen05 float32 GEMMs (tc_gemm.cuh).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace qb {

// Shapes the tensor-core kernels accept.
bool tc_rows_ok(int N, int K);     // C[M][N] = A[M][K] * W: N % 64 == 0, 64 <= N <= 256, K % 32 == 0
bool tc_wgrad_ok(int Mw, int N);   // P = H^T G with H [rows][Mw], G [rows][N]: Mw % 128 == 0, N as above
bool tc_enabled();                 // QB200_TC=0 switches the tensor-core GEMMs off

// Words of the four pre-split image planes of a weight [K][N].
size_t tc_image_words(int K, int N);
cudaError_t tc_prep_launch(const float* w, int K, int N, uint32_t* image, cudaStream_t stream);

// C[M][N] = A[M][K] * B (+ bias on the first bias_rows rows); backward selects the image
// planes that make B = W^T (then K is W's N and N is W's K).
cudaError_t tc_rows_launch(const float* A, int lda, const uint32_t* image, bool backward, int wK, int wN, float* C,
                           int ldc, const float* bias, int bias_rows, int M, int* error, cudaStream_t stream);

// partials[z][m][n] = sum over rows of slice z of H[r][m] * G[r][n]; returns the slice count.
cudaError_t tc_wgrad_launch(const float* H, int ldh, const float* G, int ldg, float* partials, int rows, int Mw,
                            int N, int rows_per_slice, int* error, cudaStream_t stream);

// Second generation (tc_tma_gemm.cuh): operands by TMA tensor maps, no pre-split images.
// 0: tensor-core GEMMs off (QB200_TC=0); 1: first generation (QB200_TC=1, or no driver entry point
// for tensor maps); 2: TMA kernels.
int tc_generation();
// wt[n][k] = w[k][n]: the K-major operand of the forward GEMM.
cudaError_t tc2_transpose_launch(const float* w, int K, int N, float* wt, cudaStream_t stream);
// One pass over W [K][N]: wt = W^T [N][K], wt_lo = the lo plane of W^T, w_lo = the lo plane of W (each K*N floats).
cudaError_t tc2_prepare_launch(const float* w, int K, int N, float* wt, float* wt_lo, float* w_lo, cudaStream_t stream);
// C[M][N] = A[M][K] * Bt^T (+ bias on the first bias_rows rows), Bt row-major [N][K].  Bt_lo, when
// given, is Bt's lo plane (tc2_prepare_launch): the kernel loads it instead of computing it per tile.
cudaError_t tc2_rows_launch(const float* A, int lda, const float* Bt, const float* Bt_lo, int ldb, float* C, int ldc,
                            const float* bias, int bias_rows, int M, int N, int K, int* error, cudaStream_t stream);
cudaError_t tc2_wgrad_launch(const float* H, int ldh, const float* G, int ldg, float* partials, int rows, int Mw, int N,
                             int rows_per_slice, int* error, cudaStream_t stream);

}  // namespace qb
