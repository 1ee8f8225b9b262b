// qb200_weight_gradient_static: the batch-reduced weight gradient for callers
// that must not allocate.
//
// Some hosts embed this library where device allocation is off limits once
// they are running: a plugin inside a runtime that owns the whole memory pool
// and forbids cudaMalloc from guests, a real-time control loop that may not
// take the allocator's lock, or code that runs after the application has
// deliberately filled the device.  qb200_weight_gradient takes its split
// scratch from the stream-ordered allocator on every call, so those hosts
// cannot use it.  This variant keeps the scratch in a fixed array that is part
// of the library image: the caller passes inputs and the output, nothing else.
//
// The array costs kStaticScratchBytes of device memory on every GPU that loads
// the library, until the process exits.
#include <mutex>

#include "common.h"
#include "layer_kernels.cuh"
#include "wgrad.h"

namespace {

constexpr size_t kStaticScratchBytes = (size_t)16 << 20;  // 16 MiB
constexpr int kMaxDevices = 64;

// Device-side storage.  In host code this name is only a handle for the
// runtime; the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char qb_static_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
void* g_scratch_address[kMaxDevices] = {nullptr};

// The scratch address on the current device, looked up once per device with
// that device current.
qb200_status scratch_for_current_device(void** out) {
    int device = -1;
    QB_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return qb::fail(QB200_INVALID, "device ordinal %d is outside 0..%d", device, kMaxDevices - 1);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
        void* address = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&address, qb_static_scratch);
        if (e != cudaSuccess || address == nullptr)
            return qb::fail(QB200_CUDA_ERROR, "cudaGetSymbolAddress for the static scratch failed on device %d: %s", device, cudaGetErrorString(e));
        g_scratch_address[device] = address;
    }
    *out = g_scratch_address[device];
    return QB200_OK;
}

}  // namespace

extern "C" qb200_status qb200_weight_gradient_static(int32_t dtype, const void* d_acts, const void* d_cots,
                                                     int64_t rows, int32_t d_in, int32_t d_out, void* d_grad,
                                                     void* cuda_stream) {
    QB_TRY(qb::weight_gradient_check("weight_gradient_static", dtype, d_acts, d_cots, d_grad, rows, d_in, d_out));
    const size_t needed = qb::weight_gradient_scratch_bytes(dtype, rows, d_in, d_out);
    if (needed > kStaticScratchBytes)
        return qb::fail(QB200_TOO_LARGE,
                        "weight_gradient_static needs %zu bytes of split scratch (ceil(rows/%d) x d_in x d_out elements "
                        "and a 16-byte flag) but the built-in array holds %zu; use qb200_weight_gradient or fewer rows "
                        "per call",
                        needed, qb::WGRAD_ROWS_PER_SLICE, kStaticScratchBytes);
    void* scratch = nullptr;
    QB_TRY(scratch_for_current_device(&scratch));
    // The same dispatch as qb200_weight_gradient (tensor cores for eligible float32 shapes, FP64 MMA or
    // the SIMT kernel otherwise), on the built-in array instead of pool memory.
    return qb::weight_gradient_into(dtype, d_acts, d_cots, rows, d_in, d_out, d_grad, scratch,
                                    static_cast<cudaStream_t>(cuda_stream));
}
