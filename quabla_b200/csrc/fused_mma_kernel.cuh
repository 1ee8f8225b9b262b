// Fused engine, float32, hidden width 64, weight contractions on the tensor
// cores with the 3xTF32 split: every float32 operand x is written as
// hi + lo with hi = tf32(x), lo = tf32(x - hi), and a product A.B is
// accumulated in float32 as A_lo.B_hi + A_hi.B_lo + A_hi.B_hi, which keeps
// float32 accuracy (the dropped A_lo.B_lo term is ~2^-22 relative).
//
// Same structure as fused_step_kernel (fused_kernel.cuh): one persistent CTA
// per SM walks tiles of 32 points, runs forward / residual / reverse sweep per
// tile, keeps the saved jets in an L2-resident per-CTA scratch and accumulates
// weight gradients per CTA.  What changes is who owns what:
//
//   warp w: point group pg = w & 1 (16 points), column group cg = w >> 1 (16 units);
//   for every stream s the warp owns the 16 x 16 tile (points x units) as two
//   m16n8k8 accumulator fragments, so thread (g = lane / 4, t = lane % 4) holds
//   points {g, g + 8} x units {2t, 2t + 1} of both fragments for ALL streams,
//   and the tanh-jet composition stays register-only.
//
// Replaces, like the SIMT variant, the reference's per-node plan execution
// (crates/quabla-core/src/tensor_ir/cuda.rs:1792-2972) and its cuBLAS
// strided-batched GEMV-shaped calls (cuda.rs:4936-5035).
#pragma once
#include <cstdint>
#include <cstdio>

#include "fused_kernel.cuh"

namespace qb {

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

// hi = x with the 13 low mantissa bits cleared (a valid tf32; the remainder x - hi is exact),
// lo = that remainder ROUNDED to tf32.  Rounding matters: truncating lo leaves a one-sided
// error of up to 2^-21 |x| that accumulates linearly over the contraction.  The tensor core
// ignores the 13 low bits of an operand, so adding half a tf32 ulp (bit 12) to the remainder's
// bit pattern rounds it to nearest with one integer add instead of a cvt.rna.tf32.
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
    hi = __float_as_uint(x) & 0xffffe000u;
#ifdef QB_SPLIT_CVT
    lo = to_tf32(x - __uint_as_float(hi));
#else
    lo = __float_as_uint(x - __uint_as_float(hi)) + 0x1000u;
#endif
}

// Four 8x8 matrices of 16-bit pairs = four 8x4 tiles of 32-bit words: thread (g, t) of the
// warp receives word t of row g of each tile, which is exactly the m16n8k8 tf32 fragment
// layout when rows are contiguous in the fragment's k index.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* row_ptr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(row_ptr)));
}

// d += a (16x8, row) * b (8x8, col), tf32 operands, float32 accumulate.
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    // Not volatile: the accumulator operands carry the dependencies, the compiler may interleave
    // independent chains.
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---- asynchronous staging: bulk copies (TMA engine, no multicast) and cp.async ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bulk copy global -> shared of `bytes` (multiple of 16, both addresses 16-byte aligned),
// completion counted on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Waits for phase `parity` of `bar`; gives up after a bounded number of polls and
// reports through *error (the kernel then finishes with wrong numbers, flagged).
__device__ __forceinline__ void mbar_wait_limited(uint64_t* bar, uint32_t parity, int* error, int limit) {
    uint32_t done = 0;
    for (int spin = 0; spin < limit && !done; ++spin) {
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(done)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
    }
    if (!done) *error = 1;
}
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, int* error) {
    mbar_wait_limited(bar, parity, error, 1 << 22);
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Weight images written by prep_weights_kernel, one per hidden-to-hidden layer:
// [4][64][WIMG_LDH] tf32 words = {forward hi, forward lo, transposed hi, transposed lo}.
// An image is the B operand stored [n][k] (k contiguous, rows padded), exactly as it sits
// in shared memory: forward B(k, n) = W[k][n], transposed B(k, n) = W[n][k].
constexpr int WIMG_LDH = 68;
constexpr int WIMG_PLANE = 64 * WIMG_LDH;            // words per plane
constexpr int WIMG_PAIR_BYTES = 2 * WIMG_PLANE * 4;  // hi + lo of one orientation

struct PrepArgs {
    int layers;                       // hidden-to-hidden layers
    int w_off[FUSED_MAX_LAYERS + 1];  // parameter offset of network layer 1 + i
};

static __global__ void prep_weights_kernel(const float* __restrict__ params, PrepArgs p, uint32_t* __restrict__ images) {
    const int layer = blockIdx.y;  // hidden-to-hidden layer index 0..layers-1 (network layer index - 1)
    if (layer >= p.layers) return;
    const float* w = params + p.w_off[layer];
    uint32_t* img = images + (size_t)layer * 4 * WIMG_PLANE;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < 64 * 64; e += gridDim.x * blockDim.x) {
        const int k = e >> 6, n = e & 63;
        uint32_t hi, lo;
        split_tf32(w[e], hi, lo);
        img[0 * WIMG_PLANE + n * WIMG_LDH + k] = hi;
        img[1 * WIMG_PLANE + n * WIMG_LDH + k] = lo;
        img[2 * WIMG_PLANE + k * WIMG_LDH + n] = hi;
        img[3 * WIMG_PLANE + k * WIMG_LDH + n] = lo;
    }
}

// PG = point groups of 16 per tile.  PG = 2: 256 threads, 32 points, two weight buffers, one CTA per
// SM.  PG = 1: 128 threads, 16 points, one weight buffer; half the shared memory, so two CTAs share
// an SM and one's GEMM phases overlap the other's epilogues and residual program.
template <int CODE, int PG>
struct MmaGeom {
    typedef Sig<CODE> sig;
    static constexpr int W = 64;
    static constexpr int S = sig::S;
    static constexpr int THREADS = 128 * PG;
    static constexpr int NBUF = PG;  // weight-image buffers
    static constexpr int TP = 16 * PG;
    static constexpr int ROWS = S * TP;
    // Every operand row is 16-byte aligned and its stride is 4 (mod 32) words, so the eight
    // row addresses of an ldmatrix tile fall into distinct bank groups.
    static constexpr int LDA = 68;        // activations / cotangents, row-major [row][unit]
    static constexpr int LDT = ROWS + 4;  // transposed operands of the weight gradient, [unit][row]
    static constexpr int OFF_ACT = 0;                       // [ROWS][LDA]
    static constexpr int LDH = 72;        // previous layer's jets [row][unit], read k-major: stride 8 (mod 32)
    static constexpr int OFF_HT = OFF_ACT + ROWS * LDA;     // [ROWS][LDH] previous layer's jets
    static constexpr int OFF_ZT = OFF_HT + ROWS * LDH;      // [64][LDT] pre-activation cotangents, transposed
    static constexpr int OFF_WB = OFF_ZT + W * LDT;         // NBUF buffers x {hi, lo} x [64][WIMG_LDH]
    static constexpr int OFF_RED = OFF_WB + NBUF * 2 * WIMG_PLANE;  // [5][PG][64] column reductions / [4][S][TP] head partials
    static constexpr int RED = (5 * PG * W > 4 * ROWS) ? 5 * PG * W : 4 * ROWS;
    static constexpr int OFF_U = OFF_RED + RED;             // [S][TP]
    static constexpr int OFF_UH = OFF_U + ROWS;             // [S][TP]
    static constexpr int OFF_BAR = OFF_UH + ROWS;           // NBUF mbarriers (4 words reserved)
    static constexpr int TOTAL = OFF_BAR + 4;
    static constexpr size_t SMEM_BASE_BYTES = ((size_t)TOTAL * sizeof(float) + 15) / 16 * 16;
    // Saved jets keep the row stride of the shared-memory operand (LDA), so that one bulk copy saves a layer.
    static constexpr size_t SCRATCH_PER_CTA = (size_t)S * TP * LDA;
};

// acc[s][j] += A[rows of stream s][64] * B[64][16 columns of this warp], 3xTF32.
// A: activations [ROWS][LDA] float32 (split here); B: pre-split weight image [n][k].
template <int S, int TP, int LDA>
__device__ __forceinline__ void warp_gemm_3xtf32(const float* __restrict__ A, const uint32_t* __restrict__ Bhi,
                                                 const uint32_t* __restrict__ Blo, int row0, int col0, int lane,
                                                 float (&acc)[S][2][4]) {
#pragma unroll
    for (int s = 0; s < S; ++s)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[s][j][c] = 0.0f;
    const int mi = lane >> 3, rr = lane & 7;
    // A tiles: (rows 0-7, k 0-3), (rows 8-15, k 0-3), (rows 0-7, k 4-7), (rows 8-15, k 4-7).
    const float* a_lane = A + (row0 + rr + (mi & 1) * 8) * LDA + (mi >> 1) * 4;
    // B tiles: (n 0-7, k 0-3), (n 0-7, k 4-7), (n 8-15, k 0-3), (n 8-15, k 4-7).
    const int b_lane = (col0 + (mi >> 1) * 8 + rr) * WIMG_LDH + (mi & 1) * 4;
#pragma unroll 2
    for (int kb = 0; kb < 8; ++kb) {
        uint32_t bhi[4], blo[4];
        ldmatrix_x4(bhi, Bhi + b_lane + kb * 8);
        ldmatrix_x4(blo, Blo + b_lane + kb * 8);
        // The tensor core adds into its accumulator with truncation, which biases a long chain
        // (measured: 5e-6 relative on the gradients against 1e-6 with this scheme).  So the three
        // products of one k-block chain from zero, and the block's partial is added to the running
        // sum with a round-to-nearest float add.
#pragma unroll
        for (int s = 0; s < S; ++s) {
            uint32_t raw[4], ahi[4], alo[4];
            ldmatrix_x4(raw, a_lane + s * TP * LDA + kb * 8);
#pragma unroll
            for (int q = 0; q < 4; ++q) split_tf32(__uint_as_float(raw[q]), ahi[q], alo[q]);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                mma_tf32(part, alo, bhi[2 * j], bhi[2 * j + 1]);
                mma_tf32(part, ahi, blo[2 * j], blo[2 * j + 1]);
                mma_tf32(part, ahi, bhi[2 * j], bhi[2 * j + 1]);
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[s][j][c] += part[c];
            }
        }
    }
}

// Sum v[4] (this thread's 4 units, already summed over its points) over the 8
// point rows of the warp; lanes with g == 0 store the warp's totals.
__device__ __forceinline__ void reduce_units_over_points(float (&v)[4], float* dst, int lane, int col0, int t) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        v[c] += __shfl_xor_sync(0xffffffffu, v[c], 4);
        v[c] += __shfl_xor_sync(0xffffffffu, v[c], 8);
        v[c] += __shfl_xor_sync(0xffffffffu, v[c], 16);
    }
    if (lane < 4) {
        dst[col0 + 2 * t] = v[0];
        dst[col0 + 2 * t + 1] = v[1];
        dst[col0 + 8 + 2 * t] = v[2];
        dst[col0 + 8 + 2 * t + 1] = v[3];
    }
}


// Optional per-phase cycle counters of CTA 0 (compile with -DQB_PHASE_TIMING), printed once per launch.
#ifdef QB_PHASE_TIMING
#define QB_PHASE(i)                                      \
    do {                                                 \
        if (tid == 0) {                                  \
            const long long now_ = clock64();            \
            phase_[i] += now_ - last_;                   \
            last_ = now_;                                \
        }                                                \
    } while (0)
#else
#define QB_PHASE(i)
#endif

template <int CODE, int PG, int ACT>
__global__ void __launch_bounds__(128 * PG, 3 - PG) fused_mma_kernel(FusedArgs<float> a) {
    typedef MmaGeom<CODE, PG> G;
    constexpr int THREADS = G::THREADS, NBUF = G::NBUF;
    typedef Sig<CODE> SG;
    constexpr int S = G::S, TP = G::TP, W = G::W, LDA = G::LDA, LDT = G::LDT, LDH = G::LDH, ROWS = G::ROWS;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* smem = reinterpret_cast<float*>(smem_raw);
    float* act = smem + G::OFF_ACT;
    float* ht = smem + G::OFF_HT;
    float* zt = smem + G::OFF_ZT;
    uint32_t* wbuf = reinterpret_cast<uint32_t*>(smem + G::OFF_WB);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + G::OFF_BAR);
    float* red = smem + G::OFF_RED;
    float* us = smem + G::OFF_U;
    float* uh = smem + G::OFF_UH;
    int4* code = reinterpret_cast<int4*>(smem_raw + G::SMEM_BASE_BYTES);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#ifdef QB_PHASE_TIMING
    long long phase_[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    long long last_ = clock64();
#endif
    const int g = lane >> 2, t = lane & 3;
    const int pg = PG == 2 ? (warp & 1) : 0, cg = PG == 2 ? (warp >> 1) : warp;
    const int row0 = pg * 16;   // first point of the warp inside the tile
    const int col0 = cg * 16;   // first unit of the warp
    const int L = a.L, d0 = a.d0;
    const bool backward = a.forward_only == 0;
    float* my_grad = a.grad_cta + (size_t)blockIdx.x * a.P;
    float* sz = a.scratch_z + (size_t)blockIdx.x * L * G::SCRATCH_PER_CTA;
    float* sh = a.scratch_h + (size_t)blockIdx.x * L * G::SCRATCH_PER_CTA;

    for (int i = tid; i < a.prog.n_instr; i += THREADS) code[i] = a.prog.code[i];
    if (backward)
        for (int i = tid; i < a.P; i += THREADS) my_grad[i] = 0.0f;
    double loss_sum = 0.0;
    const float seed = a.cotangent[0] * a.weight * a.extra;
    if (tid == 0) {
#pragma unroll
        for (int b = 0; b < NBUF; ++b) mbar_init(bars + b, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // Unit of accumulator element (j, c) and its point index (0: row g, 1: row g + 8).
    auto unit_of = [&](int j, int c) { return col0 + j * 8 + 2 * t + (c & 1); };

    const long long n_tiles = (a.n_points + TP - 1) / TP;
    // Weight pipeline: the split weight images are bulk-copied into NBUF shared buffers in
    // the fixed order a tile uses them (forward layers 1..L-1, then the transposed images
    // of layers L-1..1), NBUF uses ahead of the GEMM that consumes them.
    const int HL = L - 1;
    const int uses_per_tile = backward ? 2 * HL : HL;
    const long long my_tiles = blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const long long total_uses = my_tiles * uses_per_tile;
    const uint32_t* images = static_cast<const uint32_t*>(a.weight_images);
    long long use = 0;
    auto issue = [&](long long q) {
        if (tid == 0 && q < total_uses) {
            const int idx = (int)(q % uses_per_tile);
            const int layer = idx < HL ? idx : 2 * HL - 1 - idx;
            const int plane = idx < HL ? 0 : 2;
            uint64_t* bar = bars + (q % NBUF);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(bar, WIMG_PAIR_BYTES);
            bulk_load(wbuf + (q % NBUF) * 2 * WIMG_PLANE, images + ((size_t)layer * 4 + plane) * WIMG_PLANE,
                      WIMG_PAIR_BYTES, bar);
        }
    };
#pragma unroll
    for (int q = 0; q < NBUF; ++q) issue(q);
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const long long p0 = tile * TP;
        float acc[S][2][4];
        float x[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const long long p = min(p0 + row0 + g + 8 * i, a.n_points - 1);
#pragma unroll
            for (int k = 0; k < 4; ++k) x[i][k] = k < d0 ? a.table[p * a.ncols + k] : 0.0f;
        }

        // ------------------------------ forward ------------------------------
        for (int l = 0; l < L; ++l) {
            if (l == 0) {
                const float* w0 = a.params + a.w_off[0];
#pragma unroll
                for (int s = 0; s < S; ++s)
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int c = 0; c < 4; ++c) acc[s][j][c] = 0.0f;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (k < d0) {
#pragma unroll
                        for (int j = 0; j < 2; ++j)
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                const float w = w0[k * W + unit_of(j, c)];
                                acc[0][j][c] += x[c >> 1][k] * w;
#pragma unroll
                                for (int dj = 0; dj < SG::ndirs; ++dj) acc[SG::base(dj)][j][c] += a.dirs[dj * d0 + k] * w;
                            }
                    }
                }
            } else {
                const uint32_t* whi = wbuf + (use % NBUF) * 2 * WIMG_PLANE;
                mbar_wait(bars + (use % NBUF), (uint32_t)((use / NBUF) & 1), a.error);
                __syncthreads();  // the previous epilogue's activations are in place
                if (backward && tid == 0) {
                    // Save layer l-1's jets for the reverse sweep: the operand tile as it sits in shared memory,
                    // one bulk copy (TMA engine) instead of 8-byte stores from every thread.
                    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                                     sh + (size_t)(l - 1) * G::SCRATCH_PER_CTA),
                                 "r"(smem_u32(act)), "r"((uint32_t)(ROWS * LDA * sizeof(float)))
                                 : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                QB_PHASE(0);      // wait for the weight image
                warp_gemm_3xtf32<S, TP, LDA>(act, whi, whi + WIMG_PLANE, row0, col0, lane, acc);
                // The epilogue overwrites the operand: the bulk copy must have read it.
                if (backward && tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                __syncthreads();
                issue(use + NBUF);
                ++use;
                QB_PHASE(1);  // forward GEMM
            }
            if (a.b_off[l] >= 0) {
                const float* bl = a.params + a.b_off[l];
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[0][j][c] += bl[unit_of(j, c)];
            }
            float* zl = sz + (size_t)l * G::SCRATCH_PER_CTA;
            if (backward) {
#pragma unroll
                for (int s = 0; s < S; ++s)
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int i = 0; i < 2; ++i)
                            st2(zl + ((size_t)s * TP + row0 + g + 8 * i) * W + col0 + j * 8 + 2 * t, acc[s][j][2 * i],
                                acc[s][j][2 * i + 1]);
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float v[S];
#pragma unroll
                    for (int s = 0; s < S; ++s) v[s] = acc[s][j][c];
                    jet_apply<float, SG, ACT>(v, a.merge_w);
#pragma unroll
                    for (int s = 0; s < S; ++s) acc[s][j][c] = v[s];
                }
            if (l + 1 < L) {
#pragma unroll
                for (int s = 0; s < S; ++s)
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int i = 0; i < 2; ++i)
                            st2(act + (s * TP + row0 + g + 8 * i) * LDA + col0 + j * 8 + 2 * t, acc[s][j][2 * i],
                                acc[s][j][2 * i + 1]);
                // The next iteration saves this tile with a bulk copy: make the writes visible to that proxy.
                if (backward) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
        }

        QB_PHASE(2);  // forward epilogues (bias, saves, tanh jets, staging of the next operand)
        // ------------------------- head and residual -------------------------
        float wh[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) wh[j][c] = a.params[a.w_off[L] + unit_of(j, c)];
#pragma unroll
        for (int s = 0; s < S; ++s)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                float dot = 0.0f;
#pragma unroll
                for (int j = 0; j < 2; ++j) dot += acc[s][j][2 * i] * wh[j][2 * i] + acc[s][j][2 * i + 1] * wh[j][2 * i + 1];
                dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                dot += __shfl_xor_sync(0xffffffffu, dot, 2);
                if (t == 0) red[(cg * S + s) * TP + row0 + g + 8 * i] = dot;
            }
        __syncthreads();
        if (tid < TP) {
            const long long p = p0 + tid;
            const bool valid = p < a.n_points;
            const long long pc = valid ? p : a.n_points - 1;
#pragma unroll
            for (int s = 0; s < S; ++s) {
                float u = red[(0 * S + s) * TP + tid];
#pragma unroll
                for (int q = 1; q < 4; ++q) u += red[(q * S + s) * TP + tid];
                if (s == 0 && a.b_off[L] >= 0) u += a.params[a.b_off[L]];
                us[s * TP + tid] = u;
            }
            float r[MAX_REGS];
            run_program<float>(code, a.prog.n_instr, static_cast<const float*>(a.prog.consts), a.table + pc * a.ncols,
                               us + tid, TP, r);
            if (valid) loss_sum += (double)r[a.prog.value_reg];
#pragma unroll
            for (int s = 0; s < S; ++s) {
                const int reg = a.prog.grad_regs[s];
                uh[s * TP + tid] = (valid && reg >= 0) ? seed * r[reg] : 0.0f;
            }
        }
        __syncthreads();
        QB_PHASE(3);  // head and residual program
        if (!backward) continue;
        // The saved jets are read back below (cp.async): the bulk stores must have completed.  The
        // barriers of the head phase separate this wait from the first prefetch.
        if (tid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");

        // ------------------------------ backward ------------------------------
        {
            // Head: dW = sum h * uhat, db = sum uhat(primal), G = uhat (x) w.
            float ug[S][2];
#pragma unroll
            for (int s = 0; s < S; ++s) {
                ug[s][0] = uh[s * TP + row0 + g];
                ug[s][1] = uh[s * TP + row0 + g + 8];
            }
            float pw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int s = 0; s < S; ++s)
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        pw[2 * j + (c & 1)] += acc[s][j][c] * ug[s][c >> 1];
                        acc[s][j][c] = ug[s][c >> 1] * wh[j][c];
                    }
            reduce_units_over_points(pw, red + pg * W, lane, col0, t);
            __syncthreads();
            if (tid < W) my_grad[a.w_off[L] + tid] += PG == 2 ? red[tid] + red[W + tid] : red[tid];
            if (tid == 0 && a.b_off[L] >= 0) {
                float total = 0.0f;
                for (int p = 0; p < TP; ++p) total += uh[p];
                my_grad[a.b_off[L]] += total;
            }
            __syncthreads();
        }
        for (int l = L - 1; l >= 0; --l) {
            const float* zl = sz + (size_t)l * G::SCRATCH_PER_CTA;
            if (l > 0) {
                // Prefetch the previous layer's saved jets (weight-gradient operand) while the
                // transposed jets are computed.
                const float* hp = sh + (size_t)(l - 1) * G::SCRATCH_PER_CTA;
                for (int e = tid; e < ROWS * 16; e += THREADS)
                    cp_async16(ht + (e >> 4) * LDH + 4 * (e & 15), hp + (size_t)(e >> 4) * LDA + 4 * (e & 15));
                cp_async_commit();
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    float z0[S], z1[S];
#pragma unroll
                    for (int s = 0; s < S; ++s)
                        ld2(zl + ((size_t)s * TP + row0 + g + 8 * i) * W + col0 + j * 8 + 2 * t, z0[s], z1[s]);
                    float g0[S], g1[S];
#pragma unroll
                    for (int s = 0; s < S; ++s) {
                        g0[s] = acc[s][j][2 * i];
                        g1[s] = acc[s][j][2 * i + 1];
                    }
                    jet_apply_transposed<float, SG, ACT>(z0, g0, a.merge_w);
                    jet_apply_transposed<float, SG, ACT>(z1, g1, a.merge_w);
#pragma unroll
                    for (int s = 0; s < S; ++s) {
                        acc[s][j][2 * i] = g0[s];
                        acc[s][j][2 * i + 1] = g1[s];
                    }
                }
            {
                float pb[4];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    pb[2 * j] = acc[0][j][0] + acc[0][j][2];
                    pb[2 * j + 1] = acc[0][j][1] + acc[0][j][3];
                }
                reduce_units_over_points(pb, red + pg * W, lane, col0, t);
            }
            if (l == 0) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (k < d0) {
                        float pw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                        for (int j = 0; j < 2; ++j)
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                float v = x[c >> 1][k] * acc[0][j][c];
#pragma unroll
                                for (int dj = 0; dj < SG::ndirs; ++dj) v += a.dirs[dj * d0 + k] * acc[SG::base(dj)][j][c];
                                pw[2 * j + (c & 1)] += v;
                            }
                        reduce_units_over_points(pw, red + ((1 + k) * PG + pg) * W, lane, col0, t);
                    }
                }
                __syncthreads();
                for (int e = tid; e < (1 + d0) * W; e += THREADS) {
                    const int which = e / W, n = e % W;
                    const float total = PG == 2 ? red[(which * 2) * W + n] + red[(which * 2 + 1) * W + n] : red[which * W + n];
                    if (which == 0) {
                        if (a.b_off[0] >= 0) my_grad[a.b_off[0] + n] += total;
                    } else {
                        my_grad[a.w_off[0] + (which - 1) * W + n] += total;
                    }
                }
                __syncthreads();
                break;
            }
            QB_PHASE(4);  // transposed jets (reload of z, tanh, bias partials)
            // Stage: cotangents as the dgrad A operand / wgrad B operand, the previous layer's
            // jets for the weight gradient, the transposed split weights for dgrad.
#pragma unroll
            for (int s = 0; s < S; ++s)
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 2; ++i)
                        st2(act + (s * TP + row0 + g + 8 * i) * LDA + col0 + j * 8 + 2 * t, acc[s][j][2 * i],
                            acc[s][j][2 * i + 1]);
#pragma unroll
            for (int s = 0; s < S; ++s)
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) zt[unit_of(j, c) * LDT + s * TP + row0 + g + 8 * (c >> 1)] = acc[s][j][c];
            cp_async_wait_all();
            __syncthreads();
            QB_PHASE(5);  // backward staging
            if (tid < W && a.b_off[l] >= 0) my_grad[a.b_off[l] + tid] += PG == 2 ? red[tid] + red[W + tid] : red[tid];
            // Weight gradient: dW[k][n] += sum_rows H[row][k] * Zhat[row][n]; warp: 16 k x 64/PG n,
            // the cotangents read from their transposed copy.
            {
                constexpr int NJJ = 4 / PG;  // 16-column groups of this warp's (64 / PG) columns
                const int k0 = (warp / PG) * 16, n0 = (warp % PG) * (W / PG);
                float* gw = my_grad + a.w_off[l];
                // Starts from the running per-CTA sums, loaded before the loop so that the latency of
                // the read-modify-write hides behind the contraction.
                float dw[2 * NJJ][4];
#pragma unroll
                for (int j = 0; j < 2 * NJJ; ++j)
#pragma unroll
                    for (int i = 0; i < 2; ++i)
                        ld2(gw + (k0 + g + 8 * i) * W + n0 + j * 8 + 2 * t, dw[j][2 * i], dw[j][2 * i + 1]);
                const int mi = lane >> 3, rr = lane & 7;
                const float* b_lane = zt + (n0 + (mi >> 1) * 8 + rr) * LDT + (mi & 1) * 4;
#pragma unroll 2
                for (int kb = 0; kb < ROWS / 8; ++kb) {
                    // A(m = unit, k = row) from the row-major jets: element (g, t) = H[kb*8 + t][k0 + g].
                    const float* ha = ht + (kb * 8 + t) * LDH + k0 + g;
                    uint32_t ahi[4], alo[4];
                    split_tf32(ha[0], ahi[0], alo[0]);
                    split_tf32(ha[8], ahi[1], alo[1]);
                    split_tf32(ha[4 * LDH], ahi[2], alo[2]);
                    split_tf32(ha[4 * LDH + 8], ahi[3], alo[3]);
#pragma unroll
                    for (int jj = 0; jj < NJJ; ++jj) {
                        uint32_t braw[4], bhi[4], blo[4];
                        ldmatrix_x4(braw, b_lane + jj * 16 * LDT + kb * 8);
#pragma unroll
                        for (int q = 0; q < 4; ++q) split_tf32(__uint_as_float(braw[q]), bhi[q], blo[q]);
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                            mma_tf32(part, alo, bhi[2 * h], bhi[2 * h + 1]);
                            mma_tf32(part, ahi, blo[2 * h], blo[2 * h + 1]);
                            mma_tf32(part, ahi, bhi[2 * h], bhi[2 * h + 1]);
#pragma unroll
                            for (int c = 0; c < 4; ++c) dw[2 * jj + h][c] += part[c];
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < 2 * NJJ; ++j)
#pragma unroll
                    for (int i = 0; i < 2; ++i)
                        st2(gw + (k0 + g + 8 * i) * W + n0 + j * 8 + 2 * t, dw[j][2 * i], dw[j][2 * i + 1]);
            }
            QB_PHASE(6);  // weight gradient
            // Cotangents of layer l-1's jets: G = Zhat W^T.
            {
                const uint32_t* whi = wbuf + (use % NBUF) * 2 * WIMG_PLANE;
                mbar_wait(bars + (use % NBUF), (uint32_t)((use / NBUF) & 1), a.error);
                warp_gemm_3xtf32<S, TP, LDA>(act, whi, whi + WIMG_PLANE, row0, col0, lane, acc);
            }
            __syncthreads();
            issue(use + NBUF);
            ++use;
            QB_PHASE(7);  // dgrad
        }
    }
#ifdef QB_PHASE_TIMING
    if (tid == 0 && blockIdx.x == 0) {
        printf("phases S=%d:", S);
        for (int i = 0; i < 8; ++i) printf(" %lld", phase_[i]);
        printf("\n");
    }
#endif

    double* lred = reinterpret_cast<double*>(ht);
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
