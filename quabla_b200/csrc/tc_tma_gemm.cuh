// float32 GEMMs of the layer-wise engine: operands arrive by TMA tensor-map loads (cp.async.bulk.tensor,
// swizzled, no multicast) into a ring of shared-memory stages, the products run on tcgen05.mma with
// accumulators in tensor memory, and completion is tracked by mbarriers with bounded waits.
//
// Split float32.  x = hi + lo and a product is lo_a.hi_b + hi_a.lo_b + hi_a.hi_b.  The tensor core reads the
// upper 19 bits of a float32 operand, so a tile as loaded IS a hi operand (hi = x & 0xffffe000) and lo =
// tf32(x - hi) is computed element by element (the weight gradient); the forward and data-gradient products
// round hi to the nearest tf32 instead and run the two correction products as bfloat16 instructions (C16, below).
//
// The first operand of every product lives in TENSOR MEMORY, hi and lo, written there by the consumer warps, so the
// MMAs read one operand from shared memory: these kernels are bound by the bytes that cross shared memory per
// k-tile (loads written, MMA operands read, tiles moved by the consumers), not by the tensor pipe.
//
// Accuracy.  The tensor core adds into its accumulator with truncation, so a k-tile of 32
// accumulates from zero into one of two tensor-memory buffers and the threads add that partial to
// float32 registers with round-to-nearest adds while the next k-tile's instructions run.
//
// Work of one CTA (eight consumer warps, a loading warp and an issuing warp): 128 x BN output tiles, k-tiles of
// 32 floats (one 128-byte swizzle span).
//   ROWS   C[m][n] = sum_k A[m][k] * Bt[n][k] (+ bias[n] on rows < bias_rows).  Both operands are
//          K-major: a stage holds A [128 rows][128 B], Bt [BN rows][128 B] and Bt's prepared second matrix.  The
//          consumers copy their row of A into tensor memory.  The CTA is persistent over output tiles (tile =
//          blockIdx.x + i * gridDim.x, n-tile fastest), and the stage ring runs ahead across tile boundaries.
//   WGRAD  P[z][m][n] = sum over the rows r of slice z of H[r][m] * G[r][n].  Both operands are loaded
//          MN-major: a stage holds 4 atoms [32 r][32 m] of H and BN/32 atoms [32 r][32 n] of G, each 4 KB,
//          exactly as a tensor-map box of the row-major matrices lands them.  The consumers transpose H into
//          tensor memory (lane = m, column = r) and write G's lo plane beside the stage ring.
#pragma once
#include <cuda.h>

#include <cstdint>

#include "fused_mma_kernel.cuh"  // split_tf32, mbarrier helpers
#include "tc_gemm.cuh"           // tc_commit, tile constants

namespace qb {

// -DQB_T2_TIMING: consumer thread 0 of CTA 0 sums the cycles it spends in each phase of an item and prints them.
#ifdef QB_T2_TIMING
#define QB_T2_PHASE(i)                         \
    do {                                       \
        const long long now_ = clock64();      \
        t2_phase[i] += now_ - t2_last;         \
        t2_last = now_;                        \
    } while (0)
#else
#define QB_T2_PHASE(i)
#endif

constexpr int T2_BM = 128;
constexpr int T2_BK = 32;
constexpr int T2_THREADS = 256;                    // consumer threads
constexpr int T2_THREADS_TOTAL = T2_THREADS + 64;  // + the loading warp and the issuing warp
constexpr int T2_STAGES = 4;
constexpr int T2_A_BYTES = T2_BM * T2_BK * 4;  // 16 KB

struct TcTmaArgs {
    float* C;           // ROWS: [M][ldc];  WGRAD: partials [slices][Mw][N]
    const float* bias;
    int M, N, K;        // ROWS: M rows, K inner;  WGRAD: M = width of H, K = rows
    int ldc;
    int bias_rows;
    int k_slice;        // WGRAD: rows per slice (multiple of T2_BK)
    int units;          // ROWS: output tiles in total
    int* error;
};

// PRELO (ROWS, always): the lo plane of the weight operand is not computed per tile but loaded from a
// second matrix written once per step (tc2_prepare_launch); a stage then holds A, Bt and Bt_lo, the
// ring has three stages, and the consumers convert the activation tile only.
//
// C16 (with PRELO): the two correction products run as bfloat16 instructions (kind::f16, k = 16 per
// instruction, half the tensor-pipe time of two tf32 instructions).  Here hi is x rounded to nearest
// tf32 (not the truncation the tensor core would apply), so |lo| = |x - hi| <= 2^-12 of x's binade, and a
// correction product multiplies such a lo by a full-size value: rounding either factor to bfloat16
// (relative error <= 2^-8) leaves an error of the order of 2^-20 of a term (measured: 6.7e-7 relative rms on a
// 64- to 256-long product; three tf32 products on truncated hi parts: 2.2e-7; torch's float32 matmul: 1.5-2.9e-7).
// The weight operand comes prepared: Bt already rounded to tf32, and a bfloat16 pair matrix whose 128-byte rows
// hold [bf16(Bt) | bf16(lo(Bt))] of one k-tile (BN rows per stage, 128-byte swizzle).  The consumers write
// the activation tile's tf32(x), bf16(x) and bf16(lo(x)) to tensor memory.
template <bool WGRAD, int BN, bool PRELO = false, bool C16 = false>
struct T2Geom {
    static_assert(WGRAD != PRELO, "ROWS loads the prepared weight planes; the weight gradient has no weight operand");
    static_assert(PRELO || !C16, "bfloat16 corrections need the prepared weight planes");
    static constexpr int STAGES = PRELO ? 3 : T2_STAGES;
    static constexpr int B_BYTES = BN * T2_BK * 4;
    static constexpr int STAGE_BYTES = T2_A_BYTES + B_BYTES + (PRELO ? B_BYTES : 0);  // multiple of 1024
    static constexpr int LO_OFFSET = STAGES * STAGE_BYTES;
    // The first operand's hi and lo parts live in tensor memory, so only the second operand has a lo plane here
    // (and in ROWS with PRELO that one is loaded with the stage).
    static constexpr int LO_BYTES = PRELO ? 0 : B_BYTES;
    // Output staging for the tensor-map store: BN/32 boxes of [128 rows][128 bytes].  WGRAD writes
    // once, after its last MMA, and reuses the stage ring; ROWS overlaps the store with the next tile.
    static constexpr int OUT_BYTES = T2_BM * BN * 4;
    static constexpr int OUT_OFFSET = WGRAD ? 0 : LO_OFFSET + 2 * LO_BYTES;
    static constexpr int BAR_OFFSET = LO_OFFSET + 2 * LO_BYTES + (WGRAD ? 0 : OUT_BYTES);
    static constexpr int SMEM_BYTES = BAR_OFFSET + 128 + 1024;          // barriers, TMEM slot, alignment slack
    static constexpr int VECTORS = STAGE_BYTES / 16;                    // 16-byte vectors per stage
    static_assert(!WGRAD || OUT_BYTES <= LO_OFFSET, "the output staging must fit in the stage ring");
};

// Matrix descriptors for 128-byte-swizzled operand tiles (descriptor version 1, layout type 2).
// K-major: rows of 128 bytes, 8-row groups 1024 bytes apart (stride byte offset); the leading
// byte offset is fixed to 1 by the format.  MN-major tf32 operands exist only in the "128-byte
// swizzle with 32-byte atoms" layout (type 1; the tensor map uses SWIZZLE_128B_ATOM_32B): rows of
// 128 bytes along M/N, 4-k-row groups 512 bytes apart (stride), atoms of 32 elements along M/N
// 4096 bytes apart (leading).
__device__ __forceinline__ uint64_t t2_desc_kmajor(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3fff) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint64_t t2_desc_mnmajor(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3fff) | ((uint64_t)(4096 >> 4) << 16) | ((uint64_t)(512 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)1 << 61);
}

// Instruction descriptor: float32 accumulator, tf32 operands, M = 128, N = BN; bits 15 and 16
// select MN-major A and B.
__device__ __forceinline__ uint32_t t2_idesc(int N, bool mn_major) {
    uint32_t d = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(T2_BM >> 4) << 24);
    if (mn_major) d |= (1u << 15) | (1u << 16);
    return d;
}

// The same with bfloat16 operands (kind::f16), K-major.
__device__ __forceinline__ uint32_t t2_idesc16(int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(T2_BM >> 4) << 24);
}

// One box of a 2-D tensor map into shared memory; completion is counted in bytes on `bar`.
__device__ __forceinline__ void t2_tma_load(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// lo operand of x: x - (x & 0xffffe000) is exact in float32; adding half a tf32 ulp to its bit
// pattern makes the tensor core's truncation of the low 13 bits a round-to-nearest.  Three
// full-rate ALU instructions per element (cvt.rna.tf32 issues at a fraction of that rate).
__device__ __forceinline__ uint32_t t2_lo_bits(uint32_t x) {
    const float d = __uint_as_float(x) - __uint_as_float(x & 0xffffe000u);
    return __float_as_uint(d) + 0x1000u;
}

// x rounded to the nearest tf32 (ties away from zero), as float32 bits with the low 13 bits clear.
__device__ __forceinline__ uint32_t t2_round_tf32(uint32_t x) { return (x + 0x1000u) & 0xffffe000u; }

// 32 lanes x 32 consecutive columns into registers; the caller waits (tcgen05.wait::ld) once for
// all loads it issued.
__device__ __forceinline__ void t2_load32_nowait(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

// 32 lanes x 16 consecutive columns from registers into tensor memory (thread i writes lane base + i).
__device__ __forceinline__ void t2_store16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// 32 lanes x 8 consecutive columns from registers into tensor memory.
__device__ __forceinline__ void t2_store8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

// Two float32 values rounded to bfloat16 and packed, `first` in the low half (the lower k index).
__device__ __forceinline__ uint32_t t2_pack_bf16(float first, float second) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(second), "f"(first));
    return d;
}

// D (+)= A * B with bfloat16 operands: A [128 lanes][8 columns, two k per column] in tensor memory, k = 16.
__device__ __forceinline__ void t2_mma16_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

// D (+)= A * B with A [128 lanes][8 columns] in tensor memory and B described in shared memory.
__device__ __forceinline__ void t2_mma_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void t2_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Warp roles: warps 0-7 (256 threads) are consumers: they compute the lo planes, drain the
// accumulator partials and write the output; warp 8 issues the tensor-map loads; warp 9 owns
// tensor memory and issues the MMAs.  Hand-offs per item (one k-tile of one output tile), all
// through mbarriers with bounded waits:
//   full[stage]   loads landed                     producer's TMA  -> consumers
//   ready[buf]    lo plane written                 consumers (256) -> issuer
//   done[buf]     the item's MMAs completed        tcgen05.commit  -> consumers (drain)
//   empty[stage]  the item's MMAs completed        tcgen05.commit  -> producer (stage reusable)
// A consumer arrives on ready[buf] of item i only after it drained item i-2, so that arrival
// also tells the issuer that accumulator buffer `buf` is free.
template <bool WGRAD, int BN, bool PRELO, bool C16>
__global__ void __launch_bounds__(T2_THREADS_TOTAL, 1)
    tc_tma_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_blo, const __grid_constant__ CUtensorMap map_c,
                       TcTmaArgs a) {
    typedef T2Geom<WGRAD, BN, PRELO, C16> G;
    constexpr int STAGES = G::STAGES;
    extern __shared__ unsigned char t2_smem_raw[];
    // Swizzled tiles need 1024-byte alignment.
    unsigned char* const smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(t2_smem_raw) + 1023) &
                                                                 ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint64_t* const full = reinterpret_cast<uint64_t*>(smem + G::BAR_OFFSET);  // [T2_STAGES]
    uint64_t* const empty = full + T2_STAGES;                                  // [T2_STAGES]
    uint64_t* const ready = empty + T2_STAGES;                                 // [2]
    uint64_t* const done = ready + 2;                                          // [2]
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(done + 2);
    // The first operand (hi and lo, 32 columns each, two buffers) sits in tensor memory behind the two accumulator
    // buffers, written there by the consumer warps, so an MMA reads only the second operand from shared memory:
    // both kernels are bound by shared-memory bandwidth (loads written, operands read by the MMAs, tiles moved by
    // the consumers).  ROWS: the activation rows.  WGRAD: H transposed, lane = m, column = row r of the k-tile.
    constexpr int A_COL0 = 2 * BN;                         // first column of the operand buffers
    constexpr int TMEM_COLS = BN == 128 ? 512 : 256;       // 2 BN + 128, rounded up to a power of two
    constexpr int NH = BN / 2;         // columns drained by one consumer thread
    constexpr int ISSUE_WARP = T2_THREADS / 32 + 1, LOAD_WARP = T2_THREADS / 32;

    if (warp == ISSUE_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < T2_STAGES; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            mbar_init(ready + b, T2_THREADS);
            mbar_init(done + b, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // Work list of this CTA.
    const int n_tiles = a.N / BN;
    int units, k_tiles, k_begin = 0;
    if (WGRAD) {
        units = 1;
        k_begin = blockIdx.z * a.k_slice;
        const int k_end = min(a.K, k_begin + a.k_slice);
        k_tiles = (k_end - k_begin + T2_BK - 1) / T2_BK;
    } else {
        units = ((int)blockIdx.x < a.units) ? (a.units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
        k_tiles = a.K / T2_BK;
    }
    const int items = units * k_tiles;
    // Tile coordinates of unit u of this CTA.
    auto unit_m0 = [&](int u) { return WGRAD ? (int)blockIdx.x * T2_BM : (((int)blockIdx.x + u * (int)gridDim.x) / n_tiles) * T2_BM; };
    auto unit_n0 = [&](int u) { return WGRAD ? (int)blockIdx.y * BN : (((int)blockIdx.x + u * (int)gridDim.x) % n_tiles) * BN; };

    if (warp == LOAD_WARP) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
            if (PRELO) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_blo) : "memory");
            int u = 0, kt = 0, m0 = unit_m0(0), n0 = unit_n0(0);
            for (int p = 0; p < items; ++p) {
                const int s = p % STAGES;
                if (p >= STAGES) mbar_wait(empty + s, (uint32_t)((p / STAGES - 1) & 1), a.error);
                unsigned char* stage = smem + s * G::STAGE_BYTES;
                const int k0 = k_begin + kt * T2_BK;
                mbar_expect_tx(full + s, G::STAGE_BYTES);
                if (!WGRAD) {
                    t2_tma_load(stage, &map_a, k0, m0, full + s);               // box {32 k, 128 rows}
                    t2_tma_load(stage + T2_A_BYTES, &map_b, k0, n0, full + s);  // box {32 k, BN rows}
                    if (PRELO && !C16) t2_tma_load(stage + T2_A_BYTES + G::B_BYTES, &map_blo, k0, n0, full + s);
                    // C16: 64 halves per row of the pair matrix, [bf16(Bt) | bf16(lo(Bt))] of this k-tile
                    if (C16) t2_tma_load(stage + T2_A_BYTES + G::B_BYTES, &map_blo, 2 * k0, n0, full + s);
                } else {
#pragma unroll
                    for (int j = 0; j < T2_BM / 32; ++j) t2_tma_load(stage + j * 4096, &map_a, m0 + 32 * j, k0, full + s);
#pragma unroll
                    for (int j = 0; j < BN / 32; ++j)
                        t2_tma_load(stage + T2_A_BYTES + j * 4096, &map_b, n0 + 32 * j, k0, full + s);
                }
                if (++kt == k_tiles) {
                    kt = 0;
                    ++u;
                    m0 = unit_m0(u);
                    n0 = unit_n0(u);
                }
            }
        }
    } else if (warp == ISSUE_WARP) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            // The first operand comes from tensor memory (K-major by construction); WGRAD's second is MN-major.
            const uint32_t idesc = t2_idesc(BN, false) | (WGRAD ? (1u << 16) : 0u);
            for (int it = 0; it < items; ++it) {
                const int s = it % STAGES, b = it & 1;
                mbar_wait(ready + b, (uint32_t)((it >> 1) & 1), a.error);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t ah = smem_u32(smem + s * G::STAGE_BYTES);
                const uint32_t al = smem_u32(smem + G::LO_OFFSET + b * G::LO_BYTES);  // without PRELO: lo of the second operand
                const uint32_t bh = ah + T2_A_BYTES, bl = PRELO ? bh + G::B_BYTES : al;
                const uint32_t dst = tmem_base + (uint32_t)(b * BN);
                // k = 8 per instruction: 32 bytes along a K-major row, two 4-row groups (1024 bytes)
                // of an MN-major atom.  The small correction products go first (they add onto a
                // small accumulator without loss), the full-magnitude products last.
                constexpr uint32_t STEP = WGRAD ? 1024 : 32;
                if (C16) {
                    // Operand buffer b: x in columns 0-31, bf16(x) in 32-47, bf16(lo(x)) in 48-63; sixteen k
                    // (32 bytes of a weight-plane row) per instruction.
                    const uint32_t idesc16 = t2_idesc16(BN);
                    // Rows of 128 bytes under the 128-byte swizzle: bf16(Bt) in bytes 0-63, bf16(lo(Bt)) in 64-127.
                    const uint32_t b16h = bh + G::B_BYTES, b16l = b16h + 64;
#pragma unroll
                    for (int kc = 0; kc < T2_BK / 16; ++kc) {
                        const uint32_t ta = tmem_base + (uint32_t)(A_COL0 + b * 64 + 32 + kc * 8);
                        t2_mma16_tmem_a(dst, ta + 16, t2_desc_kmajor(b16h + kc * 32), idesc16, kc == 0 ? 0u : 1u);
                        t2_mma16_tmem_a(dst, ta, t2_desc_kmajor(b16l + kc * 32), idesc16, 1u);
                    }
                }
#pragma unroll
                for (int kb = 0; kb < (C16 ? 0 : T2_BK / 8); ++kb) {
                    const uint32_t o = kb * STEP;
                    const uint32_t ta = tmem_base + (uint32_t)(A_COL0 + b * 64 + kb * 8);  // hi; lo is 32 columns on
                    if (WGRAD) {
                        t2_mma_tmem_a(dst, ta + 32, t2_desc_mnmajor(bh + o), idesc, kb == 0 ? 0u : 1u);
                        t2_mma_tmem_a(dst, ta, t2_desc_mnmajor(bl + o), idesc, 1u);
                    } else {
                        t2_mma_tmem_a(dst, ta + 32, t2_desc_kmajor(bh + o), idesc, kb == 0 ? 0u : 1u);
                        t2_mma_tmem_a(dst, ta, t2_desc_kmajor(bl + o), idesc, 1u);
                    }
                }
#pragma unroll
                for (int kb = 0; kb < T2_BK / 8; ++kb) {
                    const uint32_t o = kb * STEP;
                    t2_mma_tmem_a(dst, tmem_base + (uint32_t)(A_COL0 + b * 64 + kb * 8),
                                  WGRAD ? t2_desc_mnmajor(bh + o) : t2_desc_kmajor(bh + o), idesc, 1u);
                }
                tc_commit(done + b);
                tc_commit(empty + s);
            }
        }
    } else {
        // ------------------------------ consumers ------------------------------
        const int half = warp >> 2;  // which BN/2 columns this thread drains
        const uint32_t my_tmem = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(half * NH);
        const int trow = (warp & 3) * 32 + lane;  // accumulator lane = output row within the tile
        float acc[NH];
#pragma unroll
        for (int i = 0; i < NH; ++i) acc[i] = 0.0f;

#ifdef QB_T2_TIMING
        long long t2_phase[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}, t2_last = clock64();
#endif
        // Partial of item q: wait for its instructions, add its buffer into the registers.
        auto drain = [&](int q) {
            mbar_wait(done + (q & 1), (uint32_t)((q >> 1) & 1), a.error);
            QB_T2_PHASE(4);  // wait for the MMAs
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t src = my_tmem + (uint32_t)((q & 1) * BN);
            uint32_t v[NH];
#pragma unroll
            for (int c = 0; c < NH / 32; ++c) t2_load32_nowait(src + c * 32, v + c * 32);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            QB_T2_PHASE(5);  // tensor-memory loads
#pragma unroll
            for (int i = 0; i < NH; ++i) acc[i] += __uint_as_float(v[i]);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        };
        // Output of unit u: registers -> staging in shared memory (boxes of [128 rows][32 columns],
        // 128-byte swizzle: chunk c of row r at c ^ (r & 7), conflict-free for a warp's 32 rows) ->
        // one tensor-map store per box, issued by one thread and left in flight while the next
        // unit's k-tiles run.  Rows outside the matrix are clipped by the store.
        unsigned char* const staging = smem + G::OUT_OFFSET;
        auto write_out = [&](int u) {
            if (tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // staging is free again
            asm volatile("bar.sync 1, %0;" ::"n"(T2_THREADS) : "memory");
            QB_T2_PHASE(8);  // staging free, every warp here
            const int m0 = unit_m0(u), n0 = unit_n0(u);
            const bool biased = !WGRAD && a.bias != nullptr && m0 + trow < a.bias_rows;
#pragma unroll
            for (int j = 0; j < NH / 32; ++j) {
                unsigned char* box = staging + (half * (NH / 32) + j) * (T2_BM * 128) + trow * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    float4 v = make_float4(acc[j * 32 + 4 * c], acc[j * 32 + 4 * c + 1], acc[j * 32 + 4 * c + 2],
                                           acc[j * 32 + 4 * c + 3]);
                    if (biased) {
                        const float4 bv = *reinterpret_cast<const float4*>(a.bias + n0 + half * NH + j * 32 + 4 * c);
                        v.x += bv.x;
                        v.y += bv.y;
                        v.z += bv.z;
                        v.w += bv.w;
                    }
                    *reinterpret_cast<float4*>(box + ((c ^ (trow & 7)) << 4)) = v;
                }
            }
#pragma unroll
            for (int i = 0; i < NH; ++i) acc[i] = 0.0f;
            QB_T2_PHASE(9);  // staging written
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync 1, %0;" ::"n"(T2_THREADS) : "memory");
            QB_T2_PHASE(10);  // every warp's part written
            if (tid == 0) {
                const int y = WGRAD ? (int)blockIdx.z * a.M + m0 : m0;
#pragma unroll
                for (int j = 0; j < BN / 32; ++j)
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&map_c),
                                 "r"(n0 + 32 * j), "r"(y), "r"(smem_u32(staging + j * (T2_BM * 128)))
                                 : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        };

        int drained = 0, unit_done = 0;
        for (int it = 0; it < items; ++it) {
            const int s = it % STAGES, b = it & 1;
            const unsigned char* hi = smem + s * G::STAGE_BYTES;
            unsigned char* lo = smem + G::LO_OFFSET + b * G::LO_BYTES;
            mbar_wait(full + s, (uint32_t)((it / STAGES) & 1), a.error);
            QB_T2_PHASE(0);  // wait for the loads
            // The lo buffer b was last read by item it-2, which this thread has drained.
            if (!WGRAD) {
                // Activation tile: this thread's row (its accumulator lane), 16 of the 32 k (by column
                // half), read through the 128-byte swizzle (chunk c of row r sits at c ^ (r & 7)) and
                // written, hi and lo, to the operand buffer b in tensor memory.
                uint32_t xh[16], xl[16];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int chunk = (half * 4 + c) ^ (trow & 7);
                    const uint4 x = *reinterpret_cast<const uint4*>(hi + trow * 128 + chunk * 16);
                    xh[4 * c + 0] = x.x; xh[4 * c + 1] = x.y; xh[4 * c + 2] = x.z; xh[4 * c + 3] = x.w;
                }
                const uint32_t ta = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(A_COL0 + b * 64 + half * 16);
                if (C16) {
                    uint32_t h16[8], l16[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float x0 = __uint_as_float(xh[2 * i]), x1 = __uint_as_float(xh[2 * i + 1]);
                        xh[2 * i] = t2_round_tf32(xh[2 * i]);
                        xh[2 * i + 1] = t2_round_tf32(xh[2 * i + 1]);
                        h16[i] = t2_pack_bf16(x0, x1);
                        l16[i] = t2_pack_bf16(x0 - __uint_as_float(xh[2 * i]), x1 - __uint_as_float(xh[2 * i + 1]));
                    }
                    t2_store16(ta, xh);
                    const uint32_t t16 = ta - (uint32_t)(half * 16) + 32 + (uint32_t)(half * 8);
                    t2_store8(t16, h16);
                    t2_store8(t16 + 16, l16);
                } else {
                    t2_store16(ta, xh);
#pragma unroll
                    for (int i = 0; i < 16; ++i) xl[i] = t2_lo_bits(xh[i]);
                    t2_store16(ta + 32, xl);
                }
                QB_T2_PHASE(1);  // read, convert, issue the tensor-memory stores
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                QB_T2_PHASE(2);  // stores complete
            } else {
                // H tile, transposed into tensor memory: this thread's m (its accumulator lane) and 16 of the 32 rows
                // (by column half).  The tile is four atoms [32 r][32 m] whose 32-byte unit u of row r sits at
                // u ^ (r & 3); a warp reads the 128 bytes of one row of its atom per load.
                uint32_t xh[16], xl[16];
                const unsigned char* column = hi + (warp & 3) * 4096 + (lane & 7) * 4;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int r = half * 16 + i;
                    xh[i] = *reinterpret_cast<const uint32_t*>(column + r * 128 + (((lane >> 3) ^ (r & 3)) << 5));
                    xl[i] = t2_lo_bits(xh[i]);
                }
                const uint32_t ta = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(A_COL0 + b * 64 + half * 16);
                t2_store16(ta, xh);
                t2_store16(ta + 32, xl);
                // G tile: lo plane in shared memory at the same offsets.
#pragma unroll
                for (int i = 0; i < (G::B_BYTES / 16) / T2_THREADS; ++i) {
                    const int v = tid + i * T2_THREADS;
                    const uint4 x = *reinterpret_cast<const uint4*>(hi + T2_A_BYTES + 16 * v);
                    *reinterpret_cast<uint4*>(lo + 16 * v) =
                        make_uint4(t2_lo_bits(x.x), t2_lo_bits(x.y), t2_lo_bits(x.z), t2_lo_bits(x.w));
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            // Generic-proxy writes must be visible to the tensor core (async proxy) before the
            // issuer is told; the tcgen05 fence orders the drain of item it-2 before that too.
            // (With the lo plane loaded, the consumers wrote tensor memory only.)
            if (!PRELO) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            t2_arrive(ready + b);
            QB_T2_PHASE(3);  // fences, arrive
            if (it >= 1) {
                drain(it - 1);
                QB_T2_PHASE(6);
                if (++drained == k_tiles) {  // item it-1 closed a unit (counters: no integer division in this loop)
                    drained = 0;
                    write_out(unit_done++);
                }
                QB_T2_PHASE(7);
            }
        }
#ifdef QB_T2_TIMING
        if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && items > 100)
            printf("t2 phases WGRAD=%d C16=%d items=%d: full %lld conv %lld wait_st %lld arrive %lld done %lld ld %lld adds %lld out %lld (per unit: sync %lld stage %lld sync %lld)\n",
                   (int)WGRAD, (int)C16, items, t2_phase[0] / items, t2_phase[1] / items, t2_phase[2] / items, t2_phase[3] / items,
                   t2_phase[4] / items, t2_phase[5] / items, t2_phase[6] / items, t2_phase[7] / items, t2_phase[8] / units, t2_phase[9] / units,
                   t2_phase[10] / units);
#endif
        if (items > 0) {
            drain(items - 1);
            write_out(units - 1);
        }
        if (tid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // stores complete before exit
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == ISSUE_WARP) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
    }
}

// One pass over a weight W [K][N] for the PRELO kernels: wt[n][k] = W[k][n] (the K-major forward
// operand), wt_lo = its lo plane, w_lo[k][n] = the lo plane of W itself (the data gradient's operand).
__global__ void t2_prepare_kernel(const float* __restrict__ w, int K, int N, float* __restrict__ wt,
                                  uint32_t* __restrict__ wt_lo, uint32_t* __restrict__ w_lo) {
    __shared__ float tile[32][33];
    const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int k = k0 + r, n = n0 + threadIdx.x;
        const float v = (k < K && n < N) ? w[(size_t)k * N + n] : 0.0f;
        tile[r][threadIdx.x] = v;
        if (k < K && n < N) w_lo[(size_t)k * N + n] = t2_lo_bits(__float_as_uint(v));
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int n = n0 + r, k = k0 + threadIdx.x;
        if (n < N && k < K) {
            const float v = tile[threadIdx.x][r];
            wt[(size_t)n * K + k] = v;
            wt_lo[(size_t)n * K + k] = t2_lo_bits(__float_as_uint(v));
        }
    }
}

// The same pass for the C16 kernels, with hi(x) = x rounded to the nearest tf32 and lo(x) = x - hi(x):
// wt = hi(W^T) and w_hi = hi(W) in float32, then the bfloat16 pair matrices wt16 (of W^T) and w16 (of W), 2*K*N
// halves each: a row holds, per 32 contraction elements, 32 x bf16(v) followed by 32 x bf16(lo(v)), so that one
// tensor-map box of 128-byte rows brings both planes of a k-tile.
__global__ void t2_prepare16_kernel(const float* __restrict__ w, int K, int N, float* __restrict__ wt,
                                    uint16_t* __restrict__ wt16, uint16_t* __restrict__ w16, float* __restrict__ w_hi) {
    __shared__ float tile[32][33];
    const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
    // Row r of a pair matrix with `inner` contraction elements: per 32 of them, 64 halves [32 x bf16(v) | 32 x bf16(lo(v))].
    auto split = [](float v, float* hi32, uint16_t* pair, size_t row, int inner, int c) {
        const float rounded = __uint_as_float(t2_round_tf32(__float_as_uint(v)));
        const uint32_t packed = t2_pack_bf16(v, v - rounded);
        *hi32 = rounded;
        uint16_t* at = pair + row * (2 * (size_t)inner) + (size_t)(c >> 5) * 64 + (c & 31);
        at[0] = (uint16_t)(packed & 0xffffu);
        at[32] = (uint16_t)(packed >> 16);
    };
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int k = k0 + r, n = n0 + threadIdx.x;
        const float v = (k < K && n < N) ? w[(size_t)k * N + n] : 0.0f;
        tile[r][threadIdx.x] = v;
        if (k < K && n < N) split(v, w_hi + (size_t)k * N + n, w16, (size_t)k, N, n);
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int n = n0 + r, k = k0 + threadIdx.x;
        if (n < N && k < K) split(tile[threadIdx.x][r], wt + (size_t)n * K + k, wt16, (size_t)n, K, k);
    }
}

}  // namespace qb
