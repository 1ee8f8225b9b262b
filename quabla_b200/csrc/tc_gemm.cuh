// float32 GEMMs of the layer-wise engine on the 5th-generation tensor cores:
// tcgen05.mma (kind::tf32) with the accumulator in tensor memory, operands in
// shared memory described by matrix descriptors, completion tracked by
// mbarriers.  float32 accuracy comes from the 3xTF32 split: every operand is
// hi + lo (two tf32 numbers) and a product is A_lo.B_hi + A_hi.B_lo + A_hi.B_hi.
//
// These kernels take over the wide-network contractions that the reference
// issues as cuBLAS strided-batched calls with batch = B, M = 1
// (crates/quabla-core/src/tensor_ir/cuda.rs:4936-5035) and as a materialised
// [B, in, out] product for every weight gradient (op/vjp.rs:176-209).
//
// Shapes.  A CTA of 256 threads computes a 128 x N tile (N <= 256, N % 64 == 0)
// over K in steps of 32:
//   ROWS  C[m][n] = sum_k A[m][k] * Bimg[n][k] (+ bias[n] on the first bias_rows rows)
//         A float32 row-major (split in registers on the way to shared memory),
//         Bimg a pre-split weight image [n][k] (hi and lo planes);
//   WGRAD P[z][m][n] = sum_{r in slice z} H[r][m] * G[r][n]
//         both operands float32 row-major with the contraction index r outermost;
//         they are transposed on the way to shared memory.
//
// Shared-memory operand layout (no swizzle, K-major): 8 rows x 16 bytes form a
// contiguous 128-byte core matrix; core matrices adjacent in k are 128 bytes
// apart (leading byte offset), 8-row groups are 8 * 128 bytes apart (stride
// byte offset).  One tcgen05.mma consumes k = 8 (two core matrices).
#pragma once
#include <cstdint>

#include "fused_mma_kernel.cuh"  // split_tf32, mbarrier and cp.async helpers

namespace qb {

constexpr int TC_BM = 128;
constexpr int TC_BK = 32;
constexpr int TC_THREADS = 256;
constexpr int TC_CHUNKS = TC_BK / 4;  // 16-byte chunks per row of a k-step

struct TcGemmArgs {
    const float* A;         // ROWS: [M][lda];   WGRAD: H [rows][lda]
    const float* B;         // WGRAD only: G [rows][ldb]
    const uint32_t* Bhi;    // ROWS only: weight image planes [N][K]
    const uint32_t* Blo;
    float* C;               // ROWS: [M][ldc];   WGRAD: partials [slices][Mw][N]
    const float* bias;
    int M, N, K;            // ROWS: M rows, K inner;  WGRAD: M = width of H (tile index blockIdx.y), K = rows
    int lda, ldb, ldc;
    int bias_rows;
    int k_slice;            // WGRAD: rows per slice (multiple of TC_BK)
    int* error;
};

// Shared-memory matrix descriptor, K-major, no swizzle: start address, leading byte offset
// (next core matrix in k) and stride byte offset (next 8-row group) in 16-byte units,
// descriptor version 1 in bits 46-47.
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
    d |= (uint64_t)(128 >> 4) << 16;
    d |= (uint64_t)((TC_CHUNKS * 128) >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

// Instruction descriptor: float32 accumulator, tf32 operands, both K-major, M = 128.
__device__ __forceinline__ uint32_t tc_idesc(int N) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

// Arrives on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 32 lanes x 32 consecutive columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tc_load32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Byte offset of element (row, k) inside an operand tile of the layout above.
__device__ __forceinline__ int tc_offset(int row, int k) {
    return ((row >> 3) * TC_CHUNKS + (k >> 2)) * 128 + (row & 7) * 16 + (k & 3) * 4;
}

__device__ __forceinline__ void tc_store_split4(unsigned char* hi, unsigned char* lo, int offset, const float (&v)[4]) {
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) split_tf32(v[i], h[i], l[i]);
    *reinterpret_cast<uint4*>(hi + offset) = make_uint4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<uint4*>(lo + offset) = make_uint4(l[0], l[1], l[2], l[3]);
}

// Dynamic shared memory: 2 stages x {A hi, A lo, B hi, B lo}, then 2 mbarriers and the TMEM address.
//
// Accuracy.  The tensor core adds into its accumulator with truncation; a chain of K/8 * 3
// instructions on one accumulator biases the result by several 1e-6 relative, which the
// derivative streams amplify.  So every k-tile (32 k = 12 instructions) accumulates from zero
// into one of two tensor-memory buffers, and the threads drain that partial into float32
// registers with round-to-nearest adds while the next k-tile's instructions run.
// Thread (half, row): rows = accumulator lanes, half selects N/2 of the columns.
template <bool WGRAD>
__global__ void __launch_bounds__(TC_THREADS, 1) tc_gemm_kernel(TcGemmArgs a) {
    extern __shared__ __align__(128) unsigned char tc_smem[];
    const int tid = threadIdx.x, warp = tid >> 5;
    const int half = tid >> 7, trow = tid & 127;
    const int N = a.N, NH = N >> 1;  // N % 64 == 0: NH is a multiple of 32
    const int a_bytes = TC_BM * TC_BK * 4, b_bytes = N * TC_BK * 4;
    const int stage_bytes = 2 * a_bytes + 2 * b_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tc_smem + 2 * stage_bytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);

    int buf_cols = 64;
    while (buf_cols < N) buf_cols <<= 1;
    const int tmem_cols = 2 * buf_cols;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0) {
        mbar_init(bars, 1);
        mbar_init(bars + 1, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t idesc = tc_idesc(N);
    // This thread's window of an accumulator buffer: its lane quarter, its half of the columns.
    const uint32_t my_tmem = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(half * NH);

    int m0, k_begin, k_end;
    if (WGRAD) {
        m0 = blockIdx.y * TC_BM;
        k_begin = blockIdx.x * a.k_slice;
        k_end = min(a.K, k_begin + a.k_slice);
    } else {
        m0 = blockIdx.x * TC_BM;
        k_begin = 0;
        k_end = a.K;
    }
    const int k_tiles = (k_end - k_begin + TC_BK - 1) / TC_BK;

    float acc[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
    auto drain = [&](int kt) {
        // Partial of k-tile kt: wait for its instructions, add its buffer into the registers.
        mbar_wait(bars + (kt & 1), (uint32_t)((kt >> 1) & 1), a.error);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t src = my_tmem + (uint32_t)((kt & 1) * buf_cols);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (c * 32 < NH) {
                float v[32];
                tc_load32(src + c * 32, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[c * 32 + i] += v[i];
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    };

    for (int kt = 0; kt < k_tiles; ++kt) {
        const int s = kt & 1;
        unsigned char* a_hi = tc_smem + s * stage_bytes;
        unsigned char* a_lo = a_hi + a_bytes;
        unsigned char* b_hi = a_lo + a_bytes;
        unsigned char* b_lo = b_hi + b_bytes;
        // Stage s and buffer s are free: k-tile kt-2 was drained in the previous iteration.
        const int k0 = k_begin + kt * TC_BK;
        if (!WGRAD) {
            // A: 128 rows x 8 chunks of 4 floats, split in registers.
#pragma unroll
            for (int i = 0; i < TC_BM * TC_CHUNKS / TC_THREADS; ++i) {
                const int idx = tid + i * TC_THREADS;
                const int r = idx >> 3, c = idx & 7;
                float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                if (m0 + r < a.M) {
                    const float4 q = *reinterpret_cast<const float4*>(a.A + (size_t)(m0 + r) * a.lda + k0 + 4 * c);
                    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
                }
                tc_store_split4(a_hi, a_lo, tc_offset(r, 4 * c), v);
            }
            // B: pre-split image rows [n][k0 .. k0+31], 16-byte asynchronous copies.
            for (int idx = tid; idx < N * TC_CHUNKS; idx += TC_THREADS) {
                const int n = idx >> 3, c = idx & 7;
                const size_t src = (size_t)n * a.K + k0 + 4 * c;
                cp_async16(b_hi + tc_offset(n, 4 * c), a.Bhi + src);
                cp_async16(b_lo + tc_offset(n, 4 * c), a.Blo + src);
            }
            cp_async_commit();
            cp_async_wait_all();
        } else {
            // A(m, k) = H[k0 + k][m0 + m]: thread = (m, half of the chunks), four consecutive k per store.
#pragma unroll
            for (int cc = 0; cc < TC_CHUNKS / 2; ++cc) {
                const int c = half * (TC_CHUNKS / 2) + cc;
                float v[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int r = k0 + 4 * c + q;
                    v[q] = (r < k_end && m0 + trow < a.M) ? a.A[(size_t)r * a.lda + m0 + trow] : 0.0f;
                }
                tc_store_split4(a_hi, a_lo, tc_offset(trow, 4 * c), v);
            }
            // B(n, k) = G[k0 + k][n].
            for (int n = tid; n < N; n += TC_THREADS) {
#pragma unroll
                for (int c = 0; c < TC_CHUNKS; ++c) {
                    float v[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int r = k0 + 4 * c + q;
                        v[q] = r < k_end ? a.B[(size_t)r * a.ldb + n] : 0.0f;
                    }
                    tc_store_split4(b_hi, b_lo, tc_offset(n, 4 * c), v);
                }
            }
        }
        // Make the generic-proxy writes visible to the tensor core, then let one thread issue.
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t ah = smem_u32(a_hi), al = smem_u32(a_lo), bh = smem_u32(b_hi), bl = smem_u32(b_lo);
            const uint32_t dst = tmem_base + (uint32_t)(s * buf_cols);
            // The small correction products first (they add onto a small accumulator without
            // loss), the four full-magnitude products last: four significant truncations per tile.
#pragma unroll
            for (int kb = 0; kb < TC_BK / 8; ++kb) {
                const uint32_t step = kb * 2 * 128;  // two core matrices per k = 8
                tc_mma(dst, tc_desc(al + step), tc_desc(bh + step), idesc, kb == 0 ? 0u : 1u);
                tc_mma(dst, tc_desc(ah + step), tc_desc(bl + step), idesc, 1u);
            }
#pragma unroll
            for (int kb = 0; kb < TC_BK / 8; ++kb) {
                const uint32_t step = kb * 2 * 128;
                tc_mma(dst, tc_desc(ah + step), tc_desc(bh + step), idesc, 1u);
            }
            tc_commit(bars + s);
        }
        if (kt >= 1) drain(kt - 1);  // overlaps with the instructions just issued
    }
    if (k_tiles > 0) drain(k_tiles - 1);

    // Epilogue from registers: thread = (row, half of the columns).
    const int row = m0 + trow;
    if (row < a.M) {
        float* out = WGRAD ? a.C + ((size_t)blockIdx.x * a.M + row) * a.ldc : a.C + (size_t)row * a.ldc;
        out += half * NH;
        const bool biased = !WGRAD && a.bias != nullptr && row < a.bias_rows;
        const float* bias = a.bias + half * NH;
#pragma unroll
        for (int i = 0; i < 128; i += 4) {
            if (i < NH) {
                float4 q = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
                if (biased) {
                    q.x += bias[i];
                    q.y += bias[i + 1];
                    q.z += bias[i + 2];
                    q.w += bias[i + 3];
                }
                *reinterpret_cast<float4*>(out + i) = q;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols));
    }
}

// Pre-split weight images of one weight W[K][N] (row-major):
//   planes 0, 1: forward image  [n][k] = W[k][n]   (hi, lo)   -> Z = H W
//   planes 2, 3: backward image [k][n] = W[k][n]   (hi, lo)   -> G' = G W^T, read as [n' = k][k' = n]
__global__ void tc_prep_weight_kernel(const float* __restrict__ w, int K, int N, uint32_t* __restrict__ img) {
    const size_t plane = (size_t)K * N;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < K * N; e += gridDim.x * blockDim.x) {
        const int k = e / N, n = e % N;
        uint32_t hi, lo;
        split_tf32(w[e], hi, lo);
        img[0 * plane + (size_t)n * K + k] = hi;
        img[1 * plane + (size_t)n * K + k] = lo;
        img[2 * plane + e] = hi;
        img[3 * plane + e] = lo;
    }
}

}  // namespace qb
