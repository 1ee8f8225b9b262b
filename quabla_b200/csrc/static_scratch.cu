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

template <typename T>
qb200_status run(const void* acts, const void* cots, int64_t rows, int d_in, int d_out, void* grad, void* scratch,
                 cudaStream_t stream) {
    const int slices = (int)((rows + qb::WGRAD_ROWS_PER_SLICE - 1) / qb::WGRAD_ROWS_PER_SLICE);
    const size_t count = (size_t)d_in * d_out;
    qb::GemmArgs<T> g;
    g.A = static_cast<const T*>(acts);
    g.B = static_cast<const T*>(cots);
    g.C = static_cast<T*>(scratch);
    g.bias = nullptr;
    g.sam = 1;
    g.sak = d_in;
    g.sbk = d_out;
    g.sbn = 1;
    g.M = d_in;
    g.N = d_out;
    g.K = (int)rows;
    g.ldc = d_out;
    g.bias_rows = 0;
    g.k_chunk = qb::WGRAD_ROWS_PER_SLICE;
    dim3 grid((d_out + qb::GEMM_BN - 1) / qb::GEMM_BN, (d_in + qb::GEMM_BM - 1) / qb::GEMM_BM, slices);
    // Every slice writes all d_in*d_out entries of its partial, and the
    // reduction reads exactly the slices of this call, so nothing in the
    // scratch has to start at zero and stale contents of an earlier, larger
    // call are never read.
    qb::gemm_kernel<T, false, true><<<grid, 256, 0, stream>>>(g);
    qb::reduce_partials_kernel<T><<<((int)count + 255) / 256, 256, 0, stream>>>(static_cast<const T*>(scratch),
                                                                               static_cast<T*>(grad), (int)count, slices);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return qb::fail(QB200_CUDA_ERROR, "weight gradient launch failed: %s", cudaGetErrorString(e));
    return QB200_OK;
}

}  // namespace

extern "C" qb200_status qb200_weight_gradient_static(int32_t dtype, const void* d_acts, const void* d_cots,
                                                     int64_t rows, int32_t d_in, int32_t d_out, void* d_grad,
                                                     void* cuda_stream) {
    if (d_acts == nullptr || d_cots == nullptr || d_grad == nullptr) return qb::fail(QB200_INVALID, "weight_gradient_static needs three device arrays");
    if (dtype != QB200_F32 && dtype != QB200_F64) return qb::fail(QB200_INVALID, "unknown dtype %d", dtype);
    if (rows < 1 || rows > (int64_t)1 << 30 || d_in < 1 || d_out < 1 || d_in > 65536 || d_out > 65536)
        return qb::fail(QB200_INVALID, "weight_gradient_static: rows %lld, d_in %d, d_out %d out of range", (long long)rows, d_in, d_out);
    const size_t element = dtype == QB200_F32 ? sizeof(float) : sizeof(double);
    const size_t slices = (size_t)((rows + qb::WGRAD_ROWS_PER_SLICE - 1) / qb::WGRAD_ROWS_PER_SLICE);
    const size_t needed = slices * (size_t)d_in * (size_t)d_out * element;
    if (needed > kStaticScratchBytes)
        return qb::fail(QB200_TOO_LARGE,
                        "weight_gradient_static needs %zu bytes of split scratch (ceil(rows/%d) x d_in x d_out elements) "
                        "but the built-in array holds %zu; use qb200_weight_gradient or fewer rows per call",
                        needed, qb::WGRAD_ROWS_PER_SLICE, kStaticScratchBytes);
    void* scratch = nullptr;
    QB_TRY(scratch_for_current_device(&scratch));
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    if (dtype == QB200_F32) return run<float>(d_acts, d_cots, rows, d_in, d_out, d_grad, scratch, stream);
    return run<double>(d_acts, d_cots, rows, d_in, d_out, d_grad, scratch, stream);
}
