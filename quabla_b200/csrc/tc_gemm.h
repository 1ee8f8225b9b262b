// Launchers of the tcgen05 float32 GEMMs (tc_tma_gemm.cuh).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace qb {

// Shapes the tensor-core kernels accept.
bool tc_rows_ok(int N, int K);     // C[M][N] = A[M][K] * W: N % 64 == 0, 64 <= N <= 256, K % 32 == 0
bool tc_wgrad_ok(int Mw, int N);   // P = H^T G with H [rows][Mw], G [rows][N]: Mw % 128 == 0, N as above
// Whether the tensor-core GEMMs can run: QB200_TC=0 switches them off, and the driver must provide the
// tensor-map encoder (operands arrive by TMA tensor maps).
bool tc_available();
// Scheme of the forward and data-gradient GEMMs for a launch of `rows` rows: true = hi parts rounded to tf32 and
// the correction products as bfloat16 instructions (launches of 65,536 rows and more), false = three tf32 products
// on truncated hi parts.  QB200_TC_COR=tf32|bf16 forces one; tc_cor_mode() is 0 / 1 for those and 2 otherwise.
bool tc_cor16_for(long long rows);
int tc_cor_mode();

// float32 words of the per-layer weight image of a weight [K][N] (tc2_prepare_launch), four parts of K*N words:
// [W^T | lo(W^T) | lo(W) | unused], or with bfloat16 corrections
// [tf32(W^T) | pair matrix of W^T | pair matrix of W | tf32(W)]; a pair matrix holds per row and per 32 contraction
// elements 32 x bf16(v) then 32 x bf16(v - tf32(v)), i.e. 128-byte rows that one tensor-map box brings per k-tile.
size_t tc_image_words(int K, int N);

// One pass over W [K][N]: wt = W^T [N][K], wt_lo = the lo plane of W^T, w_lo = the lo plane of W (each K*N floats;
// w_hi is not written).  With bfloat16 corrections: wt = W^T rounded to tf32, w_hi = W rounded to tf32, and wt_lo
// and w_lo each receive the bfloat16 pair matrix described above.
cudaError_t tc2_prepare_launch(const float* w, int K, int N, float* wt, float* wt_lo, float* w_lo, float* w_hi,
                               bool cor16, cudaStream_t stream);
// C[M][N] = A[M][K] * Bt^T (+ bias on the first bias_rows rows), Bt row-major [N][K].  Bt_lo (required)
// is what tc2_prepare_launch wrote for Bt (its lo plane; or its bfloat16 pair matrix, and Bt is then
// the tf32-rounded matrix written with it; ldb must equal K): the kernel loads it instead of computing a lo plane per tile.
cudaError_t tc2_rows_launch(const float* A, int lda, const float* Bt, const float* Bt_lo, int ldb, float* C, int ldc,
                            const float* bias, int bias_rows, int M, int N, int K, bool cor16, int* error,
                            cudaStream_t stream);
cudaError_t tc2_wgrad_launch(const float* H, int ldh, const float* G, int ldg, float* partials, int rows, int Mw, int N,
                             int rows_per_slice, int* error, cudaStream_t stream);

}  // namespace qb
