// Host side of the tcgen05 float32 GEMMs.
#include "tc_gemm.h"

#include <cstdlib>
#include <cstring>

#include "tc_tma_gemm.cuh"

namespace qb {

static bool tc_switch_on() {
    const char* env = getenv("QB200_TC");
    return !(env != nullptr && strcmp(env, "0") == 0);
}

// Correction products of the forward and data-gradient GEMMs: bfloat16 instructions on tf32-rounded hi parts, or
// tf32 instructions on truncated hi parts (the plain 3xTF32 scheme).  The bfloat16 scheme is about 9 % faster per
// GEMM and leaves a random error of 6.7e-7 per output against ~1e-7 (its systematic part is smaller); in sums over
// the rows of a launch (bias gradients above all) random errors shrink with the square root of the row count, so
// it is used for launches of at least TC_COR16_MIN_ROWS rows, where it stays below what a plain float32 FMA product
// leaves on a few hundred rows.  QB200_TC_COR=tf32 or =bf16 (read at every call) forces one scheme.
constexpr long long TC_COR16_MIN_ROWS = 65536;

int tc_cor_mode() {
    const char* env = getenv("QB200_TC_COR");
    if (env != nullptr && strcmp(env, "tf32") == 0) return 0;
    if (env != nullptr && strcmp(env, "bf16") == 0) return 1;
    return 2;
}

bool tc_cor16_for(long long rows) {
    const int mode = tc_cor_mode();
    return mode == 1 || (mode == 2 && rows >= TC_COR16_MIN_ROWS);
}

bool tc_rows_ok(int N, int K) { return N % 64 == 0 && N >= 64 && N <= 256 && K % TC_BK == 0 && K >= TC_BK; }

bool tc_wgrad_ok(int Mw, int N) { return Mw % TC_BM == 0 && N % 64 == 0 && N >= 64 && N <= 256; }

size_t tc_image_words(int K, int N) { return (size_t)4 * K * N; }  // one image; a plan keeps one per scheme

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &status) != cudaSuccess ||
            status != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

bool tc_available() {
    static const bool available = tc_switch_on() && encode_tiled() != nullptr;
    return available;
}

// Row-major float32 matrix [rows][cols] with leading dimension ld, boxes of box_cols x box_rows,
// the given 128-byte swizzle, zero fill outside the matrix.
static bool make_map(CUtensorMap* map, const float* base, long long rows, int cols, int ld, int box_cols, int box_rows,
                     CUtensorMapSwizzle swizzle) {
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return encode_tiled()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// bfloat16 pair matrix of tc2_prepare_launch: [rows][2 * inner] halves, boxes of 64 halves (128 bytes) x box_rows under
// the 128-byte swizzle.
static bool make_map16(CUtensorMap* map, const void* base, long long rows, int inner, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)(2 * inner), (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)(2 * inner) * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return encode_tiled()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

cudaError_t tc2_prepare_launch(const float* w, int K, int N, float* wt, float* wt_lo, float* w_lo, float* w_hi,
                               bool cor16, cudaStream_t stream) {
    if (cor16) {
        t2_prepare16_kernel<<<dim3((N + 31) / 32, (K + 31) / 32), dim3(32, 8), 0, stream>>>(
            w, K, N, wt, reinterpret_cast<uint16_t*>(wt_lo), reinterpret_cast<uint16_t*>(w_lo), w_hi);
        return cudaGetLastError();
    }
    t2_prepare_kernel<<<dim3((N + 31) / 32, (K + 31) / 32), dim3(32, 8), 0, stream>>>(
        w, K, N, wt, reinterpret_cast<uint32_t*>(wt_lo), reinterpret_cast<uint32_t*>(w_lo));
    return cudaGetLastError();
}

template <bool WGRAD, int BN, bool PRELO, bool C16 = false>
static cudaError_t launch2(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mblo, const CUtensorMap& mc,
                           const TcTmaArgs& a, dim3 grid, cudaStream_t stream) {
    typedef T2Geom<WGRAD, BN, PRELO, C16> G;
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(tc_tma_gemm_kernel<WGRAD, BN, PRELO, C16>),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    tc_tma_gemm_kernel<WGRAD, BN, PRELO, C16><<<grid, T2_THREADS_TOTAL, G::SMEM_BYTES, stream>>>(ma, mb, mblo, mc, a);
    return cudaGetLastError();
}

cudaError_t tc2_rows_launch(const float* A, int lda, const float* Bt, const float* Bt_lo, int ldb, float* C, int ldc,
                            const float* bias, int bias_rows, int M, int N, int K, bool cor16, int* error,
                            cudaStream_t stream) {
    const int BN = N % 128 == 0 ? 128 : 64;
    CUtensorMap ma, mb, mblo, mc;
    if (Bt_lo == nullptr) return cudaErrorInvalidValue;
    const bool c16 = cor16;  // Bt_lo is then the bfloat16 pair matrix, N rows of 2 K halves (dense: ldb == K)
    if (!make_map(&ma, A, M, K, lda, T2_BK, T2_BM, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map(&mb, Bt, N, K, ldb, T2_BK, BN, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !(c16 ? make_map16(&mblo, Bt_lo, N, K, BN)
              : make_map(&mblo, Bt_lo, N, K, ldb, T2_BK, BN, CU_TENSOR_MAP_SWIZZLE_128B)) ||
        !make_map(&mc, C, M, N, ldc, 32, T2_BM, CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorInvalidValue;
    TcTmaArgs a;
    memset(&a, 0, sizeof(a));
    a.C = C;
    a.bias = bias;
    a.M = M;
    a.N = N;
    a.K = K;
    a.ldc = ldc;
    a.bias_rows = bias_rows;
    a.units = ((M + T2_BM - 1) / T2_BM) * (N / BN);
    a.error = error;
    const dim3 grid(a.units < 148 ? a.units : 148);
    if (c16)
        return BN == 128 ? launch2<false, 128, true, true>(ma, mb, mblo, mc, a, grid, stream)
                         : launch2<false, 64, true, true>(ma, mb, mblo, mc, a, grid, stream);
    return BN == 128 ? launch2<false, 128, true>(ma, mb, mblo, mc, a, grid, stream)
                     : launch2<false, 64, true>(ma, mb, mblo, mc, a, grid, stream);
}

cudaError_t tc2_wgrad_launch(const float* H, int ldh, const float* G, int ldg, float* partials, int rows, int Mw, int N,
                             int rows_per_slice, int* error, cudaStream_t stream) {
    const int BN = N % 128 == 0 ? 128 : 64;
    const int slices = (rows + rows_per_slice - 1) / rows_per_slice;
    CUtensorMap ma, mb, mc;
    if (!make_map(&ma, H, rows, Mw, ldh, 32, T2_BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B) ||
        !make_map(&mb, G, rows, N, ldg, 32, T2_BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B) ||
        !make_map(&mc, partials, (long long)slices * Mw, N, N, 32, T2_BM, CU_TENSOR_MAP_SWIZZLE_128B))
        return cudaErrorInvalidValue;
    TcTmaArgs a;
    memset(&a, 0, sizeof(a));
    a.C = partials;
    a.M = Mw;
    a.N = N;
    a.K = rows;
    a.ldc = N;
    a.k_slice = rows_per_slice;
    a.error = error;
    const dim3 grid(Mw / T2_BM, N / BN, slices);  // the tiles of one slice run together and share its rows in L2
    return BN == 128 ? launch2<true, 128, false>(ma, mb, mb, mc, a, grid, stream)
                     : launch2<true, 64, false>(ma, mb, mb, mc, a, grid, stream);
}

}  // namespace qb
