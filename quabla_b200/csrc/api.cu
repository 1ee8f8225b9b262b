// extern "C" surface of libqb200 (include/qb200.h): description builder, plan
// entry points, the single-process data-parallel plan and the stand-alone
// optimizer.
#include <dlfcn.h>

#include <chrono>
#include <cmath>
#include <cstring>
#include <memory>
#include <mutex>
#include <set>
#include <type_traits>

#include "dmma_gemm.cuh"
#include "layer_kernels.cuh"
#include "plan.h"
#include "tc_gemm.h"
#include "point_kernels.cuh"
#include "wgrad.h"

namespace qb {

static thread_local std::string g_error;

void set_error(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_error = buf;
}

qb200_status fail(qb200_status status, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_error = buf;
    return status;
}

const NcclApi* nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    static std::string why;
    std::call_once(once, [] {
        // A library already mapped into the process under this soname (for
        // example by an importing framework) is reused by dlopen.
        void* h = nullptr;
        const char* names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char* n : names) {
            h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (h != nullptr) break;
        }
        if (h == nullptr) {
            why = std::string("NCCL library is unavailable: ") + (dlerror() ? dlerror() : "dlopen failed");
            return;
        }
        bool ok = true;
        auto sym = [&](const char* n) {
            void* p = dlsym(h, n);
            if (p == nullptr) {
                ok = false;
                why = std::string("NCCL library lacks ") + n;
            }
            return p;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommInitAll = reinterpret_cast<decltype(api.CommInitAll)>(sym("ncclCommInitAll"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        api.loaded = ok;
    });
    if (!api.loaded) {
        set_error("%s", why.c_str());
        return nullptr;
    }
    return &api;
}

}  // namespace qb

using qb::fail;

// Single-process data-parallel plan: replicas on distinct devices driven by one
// host thread (crates/quabla-core/src/tensor_ir/cuda.rs:116-170, 621-866).
struct qb200_dp {
    std::vector<std::unique_ptr<qb200_plan>> replicas;
    std::vector<int> ordinals;
    std::vector<ncclComm_t> comms;  // empty: dropped, recreated by the next step
    std::mutex mutex;               // serialises collective invocations (cuda.rs:693-703)
    int inject_failure_rank = -1;
    int comm_generation = 0;
    // Rank 0's flat [loss, gradients...] buffer as the last step left it, read back inside the step
    // (the reference's execute_replicas returns host outputs, cuda.rs:741-749).
    std::vector<char> host_outputs;
    bool host_outputs_valid = false;
};

namespace {

qb200_status dp_ensure_comms(qb200_dp* dp) {
    if (!dp->comms.empty() || dp->replicas.size() == 1) return QB200_OK;
    const qb::NcclApi* api = qb::nccl_api();
    if (api == nullptr) return QB200_NCCL_ERROR;
    dp->comms.assign(dp->replicas.size(), nullptr);
    ncclResult_t r = api->CommInitAll(dp->comms.data(), (int)dp->ordinals.size(), dp->ordinals.data());
    if (r != ncclSuccess) {
        dp->comms.clear();
        return fail(QB200_NCCL_ERROR, "ncclCommInitAll failed: %s", api->GetErrorString(r));
    }
    ++dp->comm_generation;
    return QB200_OK;
}

void dp_drop_comms(qb200_dp* dp) {
    const qb::NcclApi* api = qb::nccl_api();
    if (api != nullptr)
        for (ncclComm_t c : dp->comms)
            if (c != nullptr) api->CommAbort(c);
    dp->comms.clear();
}

double seconds_since(std::chrono::steady_clock::time_point t0) {
    return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}

}  // namespace

template <typename T>
static qb200_status optimizer_apply_typed(void* p, const void* g, void* m, void* v, int64_t count,
                                          const qb200_opt_config* c, int64_t step, cudaStream_t stream) {
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((count + 255) / 256, 148 * 16));
    if (c->rule == QB200_SGD) {
        qb::sgd_kernel<T><<<grid, 256, 0, stream>>>(static_cast<T*>(p), static_cast<const T*>(g), (T)c->learning_rate,
                                                    nullptr, count);
    } else {
        qb::AdamCoeffs<T> k;
        k.learning_rate = (T)c->learning_rate;
        k.beta1 = (T)c->beta1;
        k.beta2 = (T)c->beta2;
        k.one_minus_beta1 = (T)(1.0 - c->beta1);
        k.one_minus_beta2 = (T)(1.0 - c->beta2);
        k.epsilon = (T)c->epsilon;
        k.correction1 = (T)(1.0 - std::pow(c->beta1, (double)step));
        k.correction2 = (T)(1.0 - std::pow(c->beta2, (double)step));
        k.weight_decay = (T)c->weight_decay;
        qb::adam_kernel<T><<<grid, 256, 0, stream>>>(static_cast<T*>(p), static_cast<const T*>(g), static_cast<T*>(m),
                                                     static_cast<T*>(v), k, nullptr, count);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(QB200_CUDA_ERROR, "optimizer launch failed: %s", cudaGetErrorString(e));
    return QB200_OK;
}

template <typename T>
static qb200_status weight_gradient_typed(const void* acts, const void* cots, int64_t rows, int d_in, int d_out,
                                          void* grad, void* scratch, cudaStream_t stream) {
    const int slices = (int)((rows + qb::WGRAD_ROWS_PER_SLICE - 1) / qb::WGRAD_ROWS_PER_SLICE);
    const size_t count = (size_t)d_in * d_out;
    cudaError_t e;
    if (std::is_same<T, float>::value && qb::tc_available() && qb::tc_wgrad_ok(d_in, d_out)) {
        // Tensor-core contraction (tcgen05, 3xTF32); same slices, same reduction.
        const size_t flag_offset = ((size_t)slices * count * sizeof(T) + 15) / 16 * 16;
        int* flag = reinterpret_cast<int*>(static_cast<char*>(scratch) + flag_offset);
        e = cudaMemsetAsync(flag, 0, sizeof(int), stream);
        if (e == cudaSuccess)
            e = qb::tc2_wgrad_launch(static_cast<const float*>(acts), d_in, static_cast<const float*>(cots), d_out,
                                     static_cast<float*>(scratch), (int)rows, d_in, d_out, qb::WGRAD_ROWS_PER_SLICE, flag,
                                     stream);
    } else {
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
        e = qb::gemm_launch<T, false, true>(g, slices, stream);  // FP64 tensor-core kernel for eligible float64 shapes
        if (e == cudaSuccess) e = cudaGetLastError();
    }
    // A failed contraction leaves the scratch as it was: the reduction must not run on it.
    if (e != cudaSuccess) return fail(QB200_CUDA_ERROR, "weight gradient launch failed: %s", cudaGetErrorString(e));
    // Every slice writes all d_in * d_out entries of its partial and the reduction reads exactly the
    // slices of this call, so nothing in the scratch has to start at zero.
    qb::reduce_partials_kernel<T><<<((int)count + 255) / 256, 256, 0, stream>>>(static_cast<const T*>(scratch),
                                                                               static_cast<T*>(grad), (int)count, slices);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(QB200_CUDA_ERROR, "weight gradient reduction launch failed: %s", cudaGetErrorString(e));
    return QB200_OK;
}

namespace qb {

size_t weight_gradient_scratch_bytes(int dtype, int64_t rows, int d_in, int d_out) {
    const size_t element = dtype == QB200_F32 ? sizeof(float) : sizeof(double);
    const size_t slices = (size_t)((rows + WGRAD_ROWS_PER_SLICE - 1) / WGRAD_ROWS_PER_SLICE);
    return (slices * (size_t)d_in * (size_t)d_out * element + 15) / 16 * 16 + 16;
}

qb200_status weight_gradient_check(const char* who, int dtype, const void* acts, const void* cots, const void* grad,
                                   int64_t rows, int d_in, int d_out) {
    if (acts == nullptr || cots == nullptr || grad == nullptr) return fail(QB200_INVALID, "%s needs three device arrays", who);
    if (dtype != QB200_F32 && dtype != QB200_F64) return fail(QB200_INVALID, "unknown dtype %d", dtype);
    if (rows < 1 || rows > (int64_t)1 << 30 || d_in < 1 || d_out < 1 || d_in > 65536 || d_out > 65536)
        return fail(QB200_INVALID, "%s: rows %lld, d_in %d, d_out %d out of range", who, (long long)rows, d_in, d_out);
    if ((rows + WGRAD_ROWS_PER_SLICE - 1) / WGRAD_ROWS_PER_SLICE > WGRAD_MAX_SLICES)
        return fail(QB200_TOO_LARGE, "%s: %lld rows exceed the %lld rows one call can split (%lld slices of %d rows); "
                                     "call once per block of rows and add the results",
                    who, (long long)rows, (long long)(WGRAD_MAX_SLICES * WGRAD_ROWS_PER_SLICE),
                    (long long)WGRAD_MAX_SLICES, WGRAD_ROWS_PER_SLICE);
    return QB200_OK;
}

qb200_status weight_gradient_into(int dtype, const void* acts, const void* cots, int64_t rows, int d_in, int d_out,
                                  void* grad, void* scratch, cudaStream_t stream) {
    if (dtype == QB200_F32) return weight_gradient_typed<float>(acts, cots, rows, d_in, d_out, grad, scratch, stream);
    return weight_gradient_typed<double>(acts, cots, rows, d_in, d_out, grad, scratch, stream);
}

}  // namespace qb

extern "C" {

const char* qb200_last_error(void) { return qb::g_error.c_str(); }
const char* qb200_version(void) { return "qb200 0.1.0 (sm_100a)"; }

int32_t qb200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

qb200_status qb200_desc_create(int32_t dtype, qb200_desc** out) {
    if (out == nullptr) return fail(QB200_INVALID, "desc_create needs an output");
    if (dtype != QB200_F32 && dtype != QB200_F64)
        return fail(QB200_INVALID, "a plan has one floating dtype, float32 or float64; got %d", dtype);
    *out = new qb200_desc();
    (*out)->dtype = dtype;
    return QB200_OK;
}

void qb200_desc_destroy(qb200_desc* desc) { delete desc; }

qb200_status qb200_desc_set_network(qb200_desc* desc, const int32_t* sizes, int32_t n_sizes) {
    if (desc == nullptr || sizes == nullptr || n_sizes < 2) return fail(QB200_INVALID, "set_network needs at least two sizes");
    desc->sizes.assign(sizes, sizes + n_sizes);
    return QB200_OK;
}

qb200_status qb200_desc_set_activation(qb200_desc* desc, int32_t activation) {
    if (desc == nullptr) return fail(QB200_INVALID, "set_activation needs a description");
    if (activation < QB200_ACT_TANH || activation > QB200_ACT_GELU)
        return fail(QB200_UNSUPPORTED, "activation %d is not supported: tanh (0), sin (1), sigmoid (2), softplus (3), "
                                       "silu (4) or gelu (5)", activation);
    desc->activation = activation;
    return QB200_OK;
}

qb200_status qb200_desc_add_parameter(qb200_desc* desc, const char* name, int32_t layer, int32_t kind) {
    if (desc == nullptr || name == nullptr) return fail(QB200_INVALID, "add_parameter needs a description and a name");
    desc->params.push_back({name, layer, kind});
    return QB200_OK;
}

qb200_status qb200_desc_add_input(qb200_desc* desc, const char* name, int64_t rows, int64_t cols, int32_t retained,
                                  int32_t* out_index) {
    if (desc == nullptr || name == nullptr) return fail(QB200_INVALID, "add_input needs a description and a name");
    desc->inputs.push_back({name, rows, cols, retained != 0});
    if (out_index != nullptr) *out_index = (int32_t)desc->inputs.size() - 1;
    return QB200_OK;
}

qb200_status qb200_desc_add_set(qb200_desc* desc, int64_t n_points, double weight, int32_t* out_set) {
    if (desc == nullptr) return fail(QB200_INVALID, "add_set needs a description");
    qb200_desc::Set s;
    s.n = n_points;
    s.weight = weight;
    desc->sets.push_back(s);
    if (out_set != nullptr) *out_set = (int32_t)desc->sets.size() - 1;
    return QB200_OK;
}

static qb200_status set_of(qb200_desc* desc, int32_t set, qb200_desc::Set** out) {
    if (desc == nullptr) return fail(QB200_INVALID, "null description");
    if (set < 0 || set >= (int32_t)desc->sets.size()) return fail(QB200_INVALID, "set %d of %zu", set, desc->sets.size());
    *out = &desc->sets[set];
    return QB200_OK;
}

qb200_status qb200_desc_set_add_column(qb200_desc* desc, int32_t set, int32_t input_index, int32_t column) {
    qb200_desc::Set* s;
    QB_TRY(set_of(desc, set, &s));
    s->cols.push_back({input_index, column});
    return QB200_OK;
}

qb200_status qb200_desc_set_add_direction(qb200_desc* desc, int32_t set, const double* vec, int32_t order) {
    qb200_desc::Set* s;
    QB_TRY(set_of(desc, set, &s));
    if (vec == nullptr) return fail(QB200_INVALID, "direction vector is null");
    if (desc->sizes.empty()) return fail(QB200_INVALID, "call set_network before add_direction");
    s->dirs.emplace_back(vec, vec + desc->sizes[0]);
    s->orders.push_back(order);
    return QB200_OK;
}

qb200_status qb200_desc_set_merge_second_order(qb200_desc* desc, int32_t set, const double* weights, int32_t n_weights) {
    qb200_desc::Set* s;
    QB_TRY(set_of(desc, set, &s));
    if (weights == nullptr || n_weights < 1) return fail(QB200_INVALID, "merge weights are missing");
    if (n_weights != (int32_t)s->dirs.size())
        return fail(QB200_INVALID, "%d merge weights for %zu directions", n_weights, s->dirs.size());
    if (s->has_program) return fail(QB200_INVALID, "declare the merged stream before the program");
    for (int32_t j = 0; j < n_weights; ++j)
        if (!std::isfinite(weights[j])) return fail(QB200_INVALID, "merge weight %d is not finite", j);
    s->merge_w.assign(weights, weights + n_weights);
    return QB200_OK;
}

qb200_status qb200_desc_set_program(qb200_desc* desc, int32_t set, const int32_t* code, int32_t n_instr,
                                    const double* consts, int32_t n_consts, int32_t n_regs, int32_t value_reg,
                                    const int32_t* grad_regs, int32_t n_grad_regs) {
    qb200_desc::Set* s;
    QB_TRY(set_of(desc, set, &s));
    if (code == nullptr || n_instr < 1) return fail(QB200_INVALID, "program is empty");
    if (n_consts < 0 || (n_consts > 0 && consts == nullptr)) return fail(QB200_INVALID, "program constants are missing");
    if (n_grad_regs < 0 || (n_grad_regs > 0 && grad_regs == nullptr)) return fail(QB200_INVALID, "gradient registers are missing");
    s->code.assign(code, code + 4 * (size_t)n_instr);
    s->consts.assign(consts, consts + n_consts);
    s->n_regs = n_regs;
    s->value_reg = value_reg;
    s->grad_regs.assign(grad_regs, grad_regs + n_grad_regs);
    s->has_program = true;
    return QB200_OK;
}

qb200_status qb200_plan_create(const qb200_desc* desc, int32_t device_ordinal, qb200_plan** out) {
    if (desc == nullptr || out == nullptr) return fail(QB200_INVALID, "plan_create needs a description and an output");
    *out = nullptr;
    return qb::make_plan(*desc, device_ordinal, out);
}

void qb200_plan_destroy(qb200_plan* plan) { delete plan; }

#define QB_PLAN(plan) \
    if ((plan) == nullptr) return fail(QB200_INVALID, "null plan")

qb200_status qb200_plan_bind(qb200_plan* plan, const char* name, const void* host, size_t nbytes) {
    QB_PLAN(plan);
    return plan->bind(name, host, nbytes);
}

qb200_status qb200_plan_execute(qb200_plan* plan) {
    QB_PLAN(plan);
    QB_TRY(plan->execute_local());
    return plan->all_reduce();
}

qb200_status qb200_plan_read_output(qb200_plan* plan, int32_t index, void* host, size_t nbytes) {
    QB_PLAN(plan);
    if (host == nullptr) return fail(QB200_INVALID, "read_output needs a host buffer");
    return plan->read_output(index, host, nbytes);
}

qb200_status qb200_plan_optimizer_step(qb200_plan* plan, const qb200_opt_config* config) {
    QB_PLAN(plan);
    return plan->optimizer_step(config);
}

qb200_status qb200_plan_loss(qb200_plan* plan, void* host_scalar) {
    QB_PLAN(plan);
    return plan->loss(host_scalar);
}

qb200_status qb200_plan_read_input(qb200_plan* plan, const char* name, void* host, size_t nbytes) {
    QB_PLAN(plan);
    return plan->read_input(name, host, nbytes);
}

qb200_status qb200_plan_sample_uniform(qb200_plan* plan, const char* name, int32_t column, uint64_t key, double minval,
                                       double maxval) {
    QB_PLAN(plan);
    return plan->sample_uniform(name, column, key, minval, maxval);
}

qb200_status qb200_plan_read_moments(qb200_plan* plan, int32_t which, void* host, size_t nbytes) {
    QB_PLAN(plan);
    if (host == nullptr) return fail(QB200_INVALID, "read_moments needs a host buffer");
    return plan->read_moments(which, host, nbytes);
}

qb200_status qb200_plan_write_moments(qb200_plan* plan, int32_t which, const void* host, size_t nbytes,
                                      int64_t step_count) {
    QB_PLAN(plan);
    if (host == nullptr) return fail(QB200_INVALID, "write_moments needs a host buffer");
    return plan->write_moments(which, host, nbytes, step_count);
}

qb200_status qb200_plan_query(qb200_plan* plan, int32_t key, int64_t* out) {
    QB_PLAN(plan);
    return plan->query(key, out);
}

qb200_status qb200_plan_synchronize(qb200_plan* plan) {
    QB_PLAN(plan);
    return plan->synchronize();
}

qb200_status qb200_plan_set_option(qb200_plan* plan, int32_t key, int64_t value) {
    QB_PLAN(plan);
    return plan->set_option(key, value);
}

qb200_status qb200_plan_inject_wait_timeout(qb200_plan* plan) {
    QB_PLAN(plan);
    return plan->inject_wait_timeout();
}

qb200_status qb200_nccl_unique_id(void* out_128_bytes) {
    if (out_128_bytes == nullptr) return fail(QB200_INVALID, "unique_id needs a 128-byte buffer");
    const qb::NcclApi* api = qb::nccl_api();
    if (api == nullptr) return QB200_NCCL_ERROR;
    ncclUniqueId id;
    ncclResult_t r = api->GetUniqueId(&id);
    if (r != ncclSuccess) return fail(QB200_NCCL_ERROR, "ncclGetUniqueId failed: %s", api->GetErrorString(r));
    memcpy(out_128_bytes, &id, sizeof(id));
    return QB200_OK;
}

qb200_status qb200_plan_attach_comm(qb200_plan* plan, const void* id, int32_t rank, int32_t world,
                                    int32_t reduction) {
    QB_PLAN(plan);
    return plan->attach_comm(id, rank, world, reduction);
}

qb200_status qb200_plan_detach_comm(qb200_plan* plan) {
    QB_PLAN(plan);
    return plan->detach_comm();
}

/* ---- single-process data parallel ------------------------------------- */

qb200_status qb200_dp_create(const qb200_desc* shard_desc, const int32_t* ordinals, int32_t n, qb200_dp** out) {
    if (shard_desc == nullptr || ordinals == nullptr || out == nullptr) return fail(QB200_INVALID, "dp_create needs a description, ordinals and an output");
    *out = nullptr;
    if (n < 1) return fail(QB200_INVALID, "data-parallel plan needs at least one device");
    const int count = qb200_device_count();
    std::set<int> seen;
    for (int i = 0; i < n; ++i) {
        if (ordinals[i] < 0 || ordinals[i] >= count)
            return fail(QB200_INVALID, "data-parallel device ordinal %d is outside the %d visible devices", ordinals[i], count);
        if (!seen.insert(ordinals[i]).second) return fail(QB200_INVALID, "data-parallel device ordinals must be unique");
    }
    if (n > 1 && qb::nccl_api() == nullptr) return QB200_NCCL_ERROR;
    std::unique_ptr<qb200_dp> dp(new qb200_dp());
    for (int i = 0; i < n; ++i) {
        qb200_plan* p = nullptr;
        QB_TRY(qb::make_plan(*shard_desc, ordinals[i], &p));
        dp->replicas.emplace_back(p);
        dp->ordinals.push_back(ordinals[i]);
    }
    QB_TRY(dp_ensure_comms(dp.get()));
    *out = dp.release();
    return QB200_OK;
}

void qb200_dp_destroy(qb200_dp* dp) {
    if (dp == nullptr) return;
    for (auto& r : dp->replicas) r->synchronize();
    const qb::NcclApi* api = qb::nccl_api();
    if (api != nullptr)
        for (ncclComm_t c : dp->comms)
            if (c != nullptr) api->CommDestroy(c);
    dp->comms.clear();
    delete dp;
}

qb200_status qb200_dp_bind_sharded(qb200_dp* dp, const char* name, const void* host, size_t nbytes) {
    if (dp == nullptr || name == nullptr || host == nullptr) return fail(QB200_INVALID, "dp_bind_sharded needs a plan, a name and a buffer");
    const int64_t shard = dp->replicas[0]->input_shard_bytes(name);
    if (shard < 0) return fail(QB200_INVALID, "the plan has no input named '%s'", name);
    if (nbytes != (size_t)shard * dp->replicas.size())
        return fail(QB200_INVALID, "input '%s' needs %zu replicas x %lld bytes, got %zu", name, dp->replicas.size(), (long long)shard, nbytes);
    for (size_t r = 0; r < dp->replicas.size(); ++r)
        QB_TRY(dp->replicas[r]->bind(name, static_cast<const char*>(host) + r * (size_t)shard, (size_t)shard));
    return QB200_OK;
}

qb200_status qb200_dp_bind_replicated(qb200_dp* dp, const char* name, const void* host, size_t nbytes) {
    if (dp == nullptr || name == nullptr || host == nullptr) return fail(QB200_INVALID, "dp_bind_replicated needs a plan, a name and a buffer");
    for (auto& r : dp->replicas) QB_TRY(r->bind(name, host, nbytes));
    return QB200_OK;
}

qb200_status qb200_dp_step(qb200_dp* dp, int32_t reduction, qb200_dp_timing* timing) {
    if (dp == nullptr) return fail(QB200_INVALID, "null data-parallel plan");
    if (reduction != QB200_REDUCE_SUM && reduction != QB200_REDUCE_MEAN) return fail(QB200_INVALID, "reduction must be sum or mean");
    std::lock_guard<std::mutex> lock(dp->mutex);
    const size_t n = dp->replicas.size();
    qb200_status st = dp_ensure_comms(dp);
    if (st != QB200_OK) return st;
    auto failed = [&](qb200_status code) {
        // Any error after the lock drops the communicators
        // (crates/quabla-core/src/tensor_ir/cuda.rs:699-716).
        const std::string message = qb::g_error;
        for (auto& r : dp->replicas) r->synchronize();
        dp_drop_comms(dp);
        return fail(code, "%s; the communicators were aborted, the next call recreates them", message.c_str());
    };
    dp->host_outputs_valid = false;
    auto t0 = std::chrono::steady_clock::now();
    const double scale = reduction == QB200_REDUCE_MEAN ? 1.0 / (double)n : 1.0;
    for (size_t r = 0; r < n; ++r) {
        if ((int)r == dp->inject_failure_rank) {
            dp->inject_failure_rank = -1;
            qb::set_error("replica %zu: injected host failure before enqueue", r);
            return failed(QB200_INVALID);
        }
        dp->replicas[r]->set_dp_scale(scale);
        st = dp->replicas[r]->execute_local();
        if (st != QB200_OK) return failed(st);
    }
    const double enqueue = seconds_since(t0);
    t0 = std::chrono::steady_clock::now();
    if (n > 1) {
        const qb::NcclApi* api = qb::nccl_api();
        ncclResult_t r = api->GroupStart();
        for (size_t i = 0; i < n && r == ncclSuccess; ++i) {
            qb200_plan* p = dp->replicas[i].get();
            cudaSetDevice(p->device());
            r = api->AllReduce(p->flat_device_ptr(), p->flat_device_ptr(), p->flat_count(),
                               p->dtype() == QB200_F32 ? ncclFloat32 : ncclFloat64, ncclSum, dp->comms[i], p->stream());
        }
        ncclResult_t e = api->GroupEnd();
        if (r == ncclSuccess) r = e;
        if (r != ncclSuccess) {
            qb::set_error("grouped ncclAllReduce failed: %s", api->GetErrorString(r));
            return failed(QB200_NCCL_ERROR);
        }
    }
    for (auto& r : dp->replicas) {
        st = r->synchronize();
        if (st != QB200_OK) return failed(st);
    }
    const double collective = seconds_since(t0);
    t0 = std::chrono::steady_clock::now();
    {
        qb200_plan* p = dp->replicas[0].get();
        const size_t bytes = p->flat_count() * p->element_bytes();
        dp->host_outputs.resize(bytes);
        cudaError_t e = cudaSetDevice(p->device());
        if (e == cudaSuccess) e = cudaMemcpyAsync(dp->host_outputs.data(), p->flat_device_ptr(), bytes, cudaMemcpyDeviceToHost, p->stream());
        if (e == cudaSuccess) e = cudaStreamSynchronize(p->stream());
        if (e != cudaSuccess) {
            qb::set_error("reading rank 0's outputs failed: %s", cudaGetErrorString(e));
            return failed(QB200_CUDA_ERROR);
        }
        dp->host_outputs_valid = true;
    }
    if (timing != nullptr) {
        timing->replica_enqueue = enqueue;
        timing->collective = collective;
        timing->output_readback = seconds_since(t0);
    }
    return QB200_OK;
}

qb200_status qb200_dp_read_output(qb200_dp* dp, int32_t index, void* host, size_t nbytes) {
    if (dp == nullptr || host == nullptr) return fail(QB200_INVALID, "dp_read_output needs a plan and a buffer");
    std::lock_guard<std::mutex> lock(dp->mutex);
    if (!dp->host_outputs_valid) return dp->replicas[0]->read_output(index, host, nbytes);  // reports "before execute"
    qb200_plan* p = dp->replicas[0].get();
    size_t offset = 0, count = 0;
    QB_TRY(p->output_span(index, &offset, &count));
    const size_t element = p->element_bytes();
    if (nbytes != count * element) return fail(QB200_INVALID, "output %d has %zu bytes, got a buffer of %zu", index, count * element, nbytes);
    memcpy(host, dp->host_outputs.data() + offset * element, nbytes);
    return QB200_OK;
}

qb200_status qb200_dp_optimizer_step(qb200_dp* dp, const qb200_opt_config* config) {
    if (dp == nullptr) return fail(QB200_INVALID, "null data-parallel plan");
    QB_TRY(qb::validate_opt_config(config));
    for (auto& r : dp->replicas) QB_TRY(r->optimizer_step(config));
    return QB200_OK;
}

qb200_plan* qb200_dp_replica(qb200_dp* dp, int32_t rank) {
    if (dp == nullptr || rank < 0 || rank >= (int32_t)dp->replicas.size()) return nullptr;
    return dp->replicas[rank].get();
}

int32_t qb200_dp_replica_count(const qb200_dp* dp) { return dp == nullptr ? 0 : (int32_t)dp->replicas.size(); }

qb200_status qb200_dp_inject_host_failure(qb200_dp* dp, int32_t rank) {
    if (dp == nullptr) return fail(QB200_INVALID, "null data-parallel plan");
    if (rank < 0 || rank >= (int32_t)dp->replicas.size()) return fail(QB200_INVALID, "rank %d of %zu", rank, dp->replicas.size());
    dp->inject_failure_rank = rank;
    return QB200_OK;
}

/* ---- stand-alone optimizer -------------------------------------------- */

qb200_status qb200_optimizer_apply(int32_t dtype, void* d_param, const void* d_grad, void* d_m, void* d_v,
                                   int64_t count, const qb200_opt_config* config, int64_t step, void* cuda_stream) {
    QB_TRY(qb::validate_opt_config(config));
    if (config->has_clip) return fail(QB200_UNSUPPORTED, "optimizer_apply does not clip; use a plan's optimizer_step");
    if (d_param == nullptr || d_grad == nullptr || count < 0) return fail(QB200_INVALID, "optimizer_apply needs parameter and gradient arrays");
    if (config->rule == QB200_ADAM && (d_m == nullptr || d_v == nullptr)) return fail(QB200_INVALID, "Adam needs both moment arrays");
    if (step < 1) return fail(QB200_INVALID, "step counts updates from 1");
    if (count == 0) return QB200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    if (dtype == QB200_F32) return optimizer_apply_typed<float>(d_param, d_grad, d_m, d_v, count, config, step, s);
    if (dtype == QB200_F64) return optimizer_apply_typed<double>(d_param, d_grad, d_m, d_v, count, config, step, s);
    return fail(QB200_INVALID, "unknown dtype %d", dtype);
}

qb200_status qb200_weight_gradient(int32_t dtype, const void* d_acts, const void* d_cots, int64_t rows, int32_t d_in,
                                   int32_t d_out, void* d_grad, void* cuda_stream) {
    QB_TRY(qb::weight_gradient_check("weight_gradient", dtype, d_acts, d_cots, d_grad, rows, d_in, d_out));
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    void* scratch = nullptr;
    QB_CUDA(cudaMallocAsync(&scratch, qb::weight_gradient_scratch_bytes(dtype, rows, d_in, d_out), s));
    const qb200_status status = qb::weight_gradient_into(dtype, d_acts, d_cots, rows, d_in, d_out, d_grad, scratch, s);
    cudaFreeAsync(scratch, s);
    return status;
}

qb200_status qb200_matmul_3xtf32(const void* d_a, const void* d_w, const void* d_bias, void* d_c, int64_t M,
                                 int32_t N, int32_t K, int64_t bias_rows, void* cuda_stream) {
    if (d_a == nullptr || d_w == nullptr || d_c == nullptr) return fail(QB200_INVALID, "matmul_3xtf32 needs A, W and C");
    if (M < 1 || M > (int64_t)1 << 30) return fail(QB200_INVALID, "matmul_3xtf32: M = %lld out of range", (long long)M);
    if (!qb::tc_available())
        return fail(QB200_UNSUPPORTED, "matmul_3xtf32 needs the driver's tensor-map encoder (and QB200_TC not set to 0)");
    if (!qb::tc_rows_ok(N, K))
        return fail(QB200_UNSUPPORTED, "matmul_3xtf32 needs N %% 64 == 0, 64 <= N <= 256 and K %% 32 == 0; got N = %d, K = %d", N, K);
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    uint32_t* image = nullptr;
    QB_CUDA(cudaMallocAsync(reinterpret_cast<void**>(&image), (qb::tc_image_words(K, N) + 4) * sizeof(uint32_t), s));
    int* flag = reinterpret_cast<int*>(image + qb::tc_image_words(K, N));
    QB_CUDA(cudaMemsetAsync(flag, 0, sizeof(int), s));
    // The K-major operand is W transposed, unsplit; its lo plane is written beside it.
    float* wt = reinterpret_cast<float*>(image);
    const bool cor16 = qb::tc_cor16_for(M);
    cudaError_t e = qb::tc2_prepare_launch(static_cast<const float*>(d_w), K, N, wt, wt + (size_t)K * N,
                                           wt + 2 * (size_t)K * N, wt + 3 * (size_t)K * N, cor16, s);
    if (e == cudaSuccess)
        e = qb::tc2_rows_launch(static_cast<const float*>(d_a), K, wt, wt + (size_t)K * N, K, static_cast<float*>(d_c), N,
                                static_cast<const float*>(d_bias), (int)std::min<int64_t>(bias_rows, M), (int)M, N, K,
                                cor16, flag, s);
    int host_flag = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&host_flag, flag, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaFreeAsync(image, s);
    if (e != cudaSuccess) return fail(QB200_CUDA_ERROR, "matmul_3xtf32 failed: %s", cudaGetErrorString(e));
    if (host_flag != 0) return fail(QB200_CUDA_ERROR, "matmul_3xtf32: a bounded wait inside the kernel gave up");
    return QB200_OK;
}

}  // extern "C"
