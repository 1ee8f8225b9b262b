// tcgen05 primitives shared by the float32 GEMMs of the layer-wise engine (tc_tma_gemm.cuh): tile constants and
// the commit that arrives on an mbarrier when the issued MMAs have completed.
//
// These kernels take over the wide-network contractions that the reference issues as cuBLAS strided-batched
// calls with batch = B, M = 1 (crates/quabla-core/src/tensor_ir/cuda.rs:4936-5035) and as a materialised
// [B, in, out] product for every weight gradient (op/vjp.rs:176-209).
#pragma once
#include <cstdint>

#include "fused_mma_kernel.cuh"  // mbarrier helpers, smem_u32

namespace qb {

constexpr int TC_BM = 128;  // rows of an output tile (tensor-memory lanes)
constexpr int TC_BK = 32;   // contraction elements per k-tile (one 128-byte swizzle span of float32)

// Arrives on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

}  // namespace qb
