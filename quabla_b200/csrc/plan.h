// The plan executor: owns the device state of one compiled PINN training plan
// and drives the kernels.  It stands in for the reference's per-node executor
// (crates/quabla-core/src/tensor_ir/cuda.rs:1792-2972) and its buffer pool and
// retained-input bookkeeping (cuda.rs:191-284, 1699-1790).
#pragma once
#include <map>
#include <memory>

#include "common.h"
#include "jet_math.cuh"

struct qb200_plan {
    virtual ~qb200_plan() {}
    virtual qb200_status bind(const char* name, const void* host, size_t nbytes) = 0;
    virtual qb200_status execute_local() = 0;   // forward + reverse, no collective
    virtual qb200_status all_reduce() = 0;       // the plan's own communicator, if attached
    virtual qb200_status read_output(int index, void* host, size_t nbytes) = 0;
    virtual qb200_status optimizer_step(const qb200_opt_config* config) = 0;
    virtual qb200_status loss(void* host_scalar) = 0;
    virtual qb200_status read_input(const char* name, void* host, size_t nbytes) = 0;
    virtual qb200_status sample_uniform(const char* name, int column, uint64_t key, double minval, double maxval) = 0;
    virtual qb200_status read_moments(int which, void* host, size_t nbytes) = 0;
    virtual qb200_status write_moments(int which, const void* host, size_t nbytes, int64_t step_count) = 0;
    virtual qb200_status query(int key, int64_t* out) = 0;
    virtual qb200_status synchronize() = 0;
    virtual qb200_status attach_comm(const void* id, int rank, int world, int reduction) = 0;
    virtual qb200_status detach_comm() = 0;
    virtual qb200_status set_option(int key, int64_t value) = 0;
    virtual qb200_status inject_wait_timeout() = 0;  // test seam: a bounded wait that gives up

    // Used by the single-process data-parallel plan.
    virtual void* flat_device_ptr() = 0;
    virtual size_t flat_count() const = 0;
    virtual cudaStream_t stream() const = 0;
    virtual void set_dp_scale(double inv_world) = 0;
    virtual int device() const = 0;
    virtual int dtype() const = 0;
    virtual int64_t input_shard_bytes(const char* name) const = 0;  // -1 when unknown
    // Element offset and count of output `index` (0: loss, 1..: gradients) inside the flat buffer.
    virtual qb200_status output_span(int index, size_t* offset, size_t* count) const = 0;
    virtual size_t element_bytes() const = 0;
};

namespace qb {
qb200_status validate_desc(const qb200_desc& desc);
qb200_status validate_opt_config(const qb200_opt_config* config);
qb200_status make_plan(const qb200_desc& desc, int device, qb200_plan** out);
}  // namespace qb
