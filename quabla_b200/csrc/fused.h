// Lookup of the fused-engine kernel instantiations (see fused_kernel.cuh).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

namespace qb {

template <typename T> struct FusedArgs;

template <typename T>
struct FusedEntry {
    void (*kernel)(FusedArgs<T>);
    int streams;                  // S
    int tile_points;              // TP
    size_t smem_bytes;            // dynamic shared memory per CTA, without the residual program
    size_t scratch_per_layer;     // saved-jet elements per CTA per hidden layer (each of Z and H)
    bool tensor_core;             // 3xTF32 variant: needs the pre-split weight images
    int threads;                  // threads per CTA
    int ctas_per_sm;              // CTAs the kernel is sized to co-reside on one SM
};

constexpr size_t FUSED_MAX_SMEM = 227 * 1024;

// Dynamic shared memory of a launch: the regions plus the staged residual program.
template <typename T>
inline size_t fused_smem_bytes(const FusedEntry<T>& entry, int n_instr) {
    return entry.smem_bytes + (size_t)n_instr * 16 + 16;
}

// True when a kernel exists for this dtype, hidden width, derivative signature code (sum over
// directions j of order_j * 5^j) and activation (ACT_TANH or ACT_SIN).
template <typename T>
bool fused_lookup(int width, int code, int act, FusedEntry<T>* out);

// Launches entry.kernel; sets the shared-memory attribute on first use.
template <typename T>
cudaError_t fused_launch(const FusedEntry<T>& entry, int grid, cudaStream_t stream, const FusedArgs<T>& args);

// Bytes of the pre-split weight images of `hidden_to_hidden` layers of width 64.
size_t fused_weight_image_bytes(int hidden_to_hidden);
// Writes the images from the flat float32 parameters; w_off[i] is the offset of network layer 1 + i.
cudaError_t fused_prep_launch(const float* params, const int* w_off, int hidden_to_hidden, void* images,
                              cudaStream_t stream);
// One thread's bounded wait on a barrier that is never completed: raises *error when it gives up.
cudaError_t unarmed_wait_launch(int* error, cudaStream_t stream);

}  // namespace qb
