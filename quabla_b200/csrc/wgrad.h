// The stand-alone batch-reduced weight gradient, shared by its two entry points
// (qb200_weight_gradient takes the split scratch from the stream-ordered pool,
// qb200_weight_gradient_static from an array built into the library), so that both
// run the same kernels on the same split and return the same bits.
#pragma once
#include "common.h"

namespace qb {

// Most row slices one call may have (the slice index is the grid's z extent).
constexpr int64_t WGRAD_MAX_SLICES = 65535;

// Bytes of scratch a call needs: one [d_in][d_out] partial per slice of 4096 rows,
// then one int (the tensor-core kernel's bounded-wait flag) on a 16-byte boundary.
size_t weight_gradient_scratch_bytes(int dtype, int64_t rows, int d_in, int d_out);

// Argument checks common to both entry points; `who` names the caller in messages.
qb200_status weight_gradient_check(const char* who, int dtype, const void* acts, const void* cots, const void* grad,
                                   int64_t rows, int d_in, int d_out);

// Enqueues the contraction and the fixed-order reduction on `stream`; `scratch` holds
// weight_gradient_scratch_bytes().  Allocates nothing.
qb200_status weight_gradient_into(int dtype, const void* acts, const void* cots, int64_t rows, int d_in, int d_out,
                                  void* grad, void* scratch, cudaStream_t stream);

}  // namespace qb
