// Plan executor and optimizer state (see plan.h).
#include "plan.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <mutex>

#include "fused.h"
#include "fused_kernel.cuh"
#include "jet_kernels.cuh"
#include "dmma_gemm.cuh"
#include "layer_kernels.cuh"
#include "point_kernels.cuh"
#include "tc_gemm.h"

namespace qb {

static const char* kCotangentName = "__quabla_loss_cotangent";

qb200_status validate_opt_config(const qb200_opt_config* c) {
    // Ranges of DeviceOptimizerConfig::validate
    // (crates/quabla-core/src/tensor_ir/device_optimizer.rs:65-95).
    if (c == nullptr) return fail(QB200_INVALID, "optimizer config is null");
    if (c->rule != QB200_SGD && c->rule != QB200_ADAM) return fail(QB200_INVALID, "unknown optimizer rule %d", c->rule);
    if (!(std::isfinite(c->learning_rate) && c->learning_rate >= 0.0))
        return fail(QB200_INVALID, "device optimizer learning_rate must be finite and nonnegative");
    if (c->has_clip && !(std::isfinite(c->clip_norm) && c->clip_norm > 0.0))
        return fail(QB200_INVALID, "device optimizer clip_norm must be positive and finite");
    if (c->rule == QB200_ADAM) {
        if (!(c->beta1 >= 0.0 && c->beta1 < 1.0 && c->beta2 >= 0.0 && c->beta2 < 1.0))
            return fail(QB200_INVALID, "device Adam beta1 and beta2 must be in [0, 1)");
        if (!(std::isfinite(c->epsilon) && c->epsilon > 0.0))
            return fail(QB200_INVALID, "device Adam epsilon must be positive and finite");
        if (!(std::isfinite(c->weight_decay) && c->weight_decay >= 0.0))
            return fail(QB200_INVALID, "device AdamW weight_decay must be finite and nonnegative");
    }
    return QB200_OK;
}

qb200_status validate_desc(const qb200_desc& d) {
    if (d.dtype != QB200_F32 && d.dtype != QB200_F64) return fail(QB200_INVALID, "unknown dtype %d", d.dtype);
    const int L = (int)d.sizes.size() - 1;
    if (L < 1) return fail(QB200_INVALID, "the network needs at least one layer");
    for (int s : d.sizes)
        if (s <= 0) return fail(QB200_INVALID, "layer sizes must be positive");
    if (d.sizes.back() != 1)
        return fail(QB200_UNSUPPORTED, "the network output must be one scalar per point, got width %d", d.sizes.back());
    if (d.sizes[0] > MAX_COLS) return fail(QB200_UNSUPPORTED, "network input width %d exceeds %d", d.sizes[0], MAX_COLS);
    std::vector<int> weights(L, 0), biases(L, 0);
    for (size_t i = 0; i < d.params.size(); ++i) {
        const auto& p = d.params[i];
        if (p.layer < 0 || p.layer >= L) return fail(QB200_INVALID, "parameter '%s' names layer %d of %d", p.name.c_str(), p.layer, L);
        if (p.kind != QB200_WEIGHT && p.kind != QB200_BIAS) return fail(QB200_INVALID, "parameter '%s' has unknown kind", p.name.c_str());
        (p.kind == QB200_WEIGHT ? weights : biases)[p.layer]++;
        for (size_t j = 0; j < i; ++j)
            if (d.params[j].name == p.name) return fail(QB200_INVALID, "duplicate parameter name '%s'", p.name.c_str());
        for (const auto& in : d.inputs)
            if (in.name == p.name) return fail(QB200_INVALID, "name '%s' is both a parameter and an input", p.name.c_str());
        if (p.name == kCotangentName) return fail(QB200_INVALID, "'%s' is reserved", kCotangentName);
    }
    for (int l = 0; l < L; ++l) {
        if (weights[l] != 1) return fail(QB200_INVALID, "layer %d needs exactly one weight parameter, got %d", l, weights[l]);
        if (biases[l] > 1) return fail(QB200_INVALID, "layer %d has %d bias parameters", l, biases[l]);
    }
    for (size_t i = 0; i < d.inputs.size(); ++i) {
        const auto& in = d.inputs[i];
        if (in.rows <= 0 || in.cols <= 0) return fail(QB200_INVALID, "input '%s' has an empty shape", in.name.c_str());
        for (size_t j = 0; j < i; ++j)
            if (d.inputs[j].name == in.name) return fail(QB200_INVALID, "duplicate input name '%s'", in.name.c_str());
    }
    if (d.sets.empty()) return fail(QB200_INVALID, "the plan has no point set");
    if ((int)d.sets.size() > MAX_SETS) return fail(QB200_UNSUPPORTED, "more than %d point sets", MAX_SETS);
    const int d0 = d.sizes[0];
    for (size_t si = 0; si < d.sets.size(); ++si) {
        const auto& s = d.sets[si];
        if (s.n <= 0 || s.n > (int64_t)1 << 31) return fail(QB200_INVALID, "set %zu: point count out of range", si);
        if (!std::isfinite(s.weight)) return fail(QB200_INVALID, "set %zu: weight must be finite", si);
        if ((int)s.cols.size() < d0) return fail(QB200_INVALID, "set %zu: %zu columns for %d network inputs", si, s.cols.size(), d0);
        if ((int)s.cols.size() > MAX_COLS) return fail(QB200_UNSUPPORTED, "set %zu: more than %d columns", si, MAX_COLS);
        for (const auto& c : s.cols) {
            if (c.first < 0 || c.first >= (int)d.inputs.size()) return fail(QB200_INVALID, "set %zu: column names input %d", si, c.first);
            const auto& in = d.inputs[c.first];
            if (in.rows != s.n) return fail(QB200_INVALID, "set %zu: input '%s' has %lld rows for %lld points", si, in.name.c_str(), (long long)in.rows, (long long)s.n);
            if (c.second < 0 || c.second >= in.cols) return fail(QB200_INVALID, "set %zu: column %d of input '%s'", si, c.second, in.name.c_str());
        }
        if ((int)s.dirs.size() > MAX_DIRS) return fail(QB200_UNSUPPORTED, "set %zu: more than %d derivative directions", si, MAX_DIRS);
        for (size_t j = 0; j < s.dirs.size(); ++j) {
            if ((int)s.dirs[j].size() != d0) return fail(QB200_INVALID, "set %zu: direction %zu has the wrong length", si, j);
            if (s.orders[j] < 1 || s.orders[j] > MAX_ORDER) return fail(QB200_UNSUPPORTED, "set %zu: derivative order %d (1..%d supported)", si, s.orders[j], MAX_ORDER);
        }
        const int S = s.streams();
        if (S > MAX_STREAMS) return fail(QB200_UNSUPPORTED, "set %zu: %d streams exceed %d", si, S, MAX_STREAMS);
        if (!s.has_program) return fail(QB200_INVALID, "set %zu has no residual program", si);
        const int n_instr = (int)s.code.size() / 4;
        if (n_instr < 1 || n_instr > MAX_INSTR) return fail(QB200_UNSUPPORTED, "set %zu: program of %d instructions (1..%d)", si, n_instr, MAX_INSTR);
        if (s.n_regs < 1 || s.n_regs > MAX_REGS) return fail(QB200_UNSUPPORTED, "set %zu: %d registers (1..%d)", si, s.n_regs, MAX_REGS);
        std::vector<char> written(s.n_regs, 0);
        for (int pc = 0; pc < n_instr; ++pc) {
            const int op = s.code[4 * pc], dst = s.code[4 * pc + 1], a = s.code[4 * pc + 2], b = s.code[4 * pc + 3];
            if (dst < 0 || dst >= s.n_regs) return fail(QB200_INVALID, "set %zu: instruction %d writes register %d", si, pc, dst);
            auto reg_ok = [&](int r) { return r >= 0 && r < s.n_regs && written[r]; };
            bool ok = true;
            switch (op) {
                case OP_CONST: ok = a >= 0 && a < (int)s.consts.size(); break;
                case OP_COL: ok = a >= 0 && a < (int)s.cols.size(); break;
                case OP_JET: ok = a >= 0 && a < S; break;
                case OP_ADD: case OP_SUB: case OP_MUL: case OP_DIV: ok = reg_ok(a) && reg_ok(b); break;
                case OP_NEG: case OP_SIN: case OP_COS: case OP_EXP: case OP_TANH: case OP_SQRT: case OP_LOG:
                case OP_LOG1P: case OP_EXPM1: case OP_ERF: case OP_ERFC: case OP_TAN:
                case OP_POWI: ok = reg_ok(a); break;
                default: return fail(QB200_UNSUPPORTED, "set %zu: instruction %d has unknown opcode %d", si, pc, op);
            }
            if (!ok) return fail(QB200_INVALID, "set %zu: instruction %d has an operand out of range or read before it is written", si, pc);
            written[dst] = 1;
        }
        if (s.value_reg < 0 || s.value_reg >= s.n_regs || !written[s.value_reg]) return fail(QB200_INVALID, "set %zu: value register is never written", si);
        if ((int)s.grad_regs.size() != S) return fail(QB200_INVALID, "set %zu: %zu gradient registers for %d streams", si, s.grad_regs.size(), S);
        for (int r : s.grad_regs)
            if (r < -1 || r >= s.n_regs || (r >= 0 && !written[r])) return fail(QB200_INVALID, "set %zu: a gradient register is never written", si);
    }
    return QB200_OK;
}

namespace {

template <typename T> struct DTypeOf;
template <> struct DTypeOf<float> { static constexpr int value = QB200_F32; static constexpr ncclDataType_t nccl = ncclFloat32; };
template <> struct DTypeOf<double> { static constexpr int value = QB200_F64; static constexpr ncclDataType_t nccl = ncclFloat64; };

inline int grid_for(long long total, int block, int cap = 148 * 16) {
    long long g = (total + block - 1) / block;
    return (int)std::max<long long>(1, std::min<long long>(g, cap));
}

template <typename T>
class Plan final : public qb200_plan {
  public:
    Plan(const qb200_desc& d, int device) : desc_(d), device_(device) {}
    ~Plan() override { release(); }

    qb200_status init();

    qb200_status bind(const char* name, const void* host, size_t nbytes) override;
    qb200_status execute_local() override;
    qb200_status all_reduce() override;
    qb200_status read_output(int index, void* host, size_t nbytes) override;
    qb200_status optimizer_step(const qb200_opt_config* config) override;
    qb200_status loss(void* host_scalar) override;
    qb200_status read_input(const char* name, void* host, size_t nbytes) override;
    qb200_status sample_uniform(const char* name, int column, uint64_t key, double minval, double maxval) override;
    qb200_status read_moments(int which, void* host, size_t nbytes) override;
    qb200_status write_moments(int which, const void* host, size_t nbytes, int64_t step_count) override;
    qb200_status query(int key, int64_t* out) override;
    qb200_status synchronize() override;
    qb200_status attach_comm(const void* id, int rank, int world, int reduction) override;
    qb200_status detach_comm() override;
    qb200_status set_option(int key, int64_t value) override;
    qb200_status inject_wait_timeout() override;

    void* flat_device_ptr() override { return d_flat_; }
    // [loss, gradients..., flag]: the last element carries the device error flag through the all-reduce.
    size_t flat_count() const override { return 2 + n_params_; }
    cudaStream_t stream() const override { return stream_; }
    void set_dp_scale(double inv_world) override { dp_scale_ = inv_world; }
    int device() const override { return device_; }
    int dtype() const override { return DTypeOf<T>::value; }
    int64_t input_shard_bytes(const char* name) const override;
    qb200_status output_span(int index, size_t* offset, size_t* count) const override {
        if (index < 0 || index > (int)leaves_.size()) return fail(QB200_INVALID, "output index %d of %zu", index, leaves_.size() + 1);
        *offset = index == 0 ? 0 : 1 + leaves_[index - 1].offset;
        *count = index == 0 ? 1 : leaves_[index - 1].count;
        return QB200_OK;
    }
    size_t element_bytes() const override { return sizeof(T); }

  private:
    struct Leaf {
        size_t offset, count;
        bool bound = false;
    };
    struct InputState {
        T* dev = nullptr;
        bool bound = false;
    };
    struct SetState {
        JetSpec spec;
        MergeW<T> merge_w;         // spec.merge_w in the plan dtype
        int sig_code = 0;          // sum of order_j * 5^j (-1: more than 8 digits would overflow)
        int ncols = 0;
        T* table = nullptr;
        T* dirs = nullptr;
        int4* code = nullptr;
        T* consts = nullptr;
        ProgramRef prog;
        int chunk = 0;             // points per chunk
        int partial_offset = 0;    // first loss partial of this set
        int partial_count = 0;
        bool table_dirty = true;
    };

    template <typename P> qb200_status dev_alloc(P** ptr, size_t count) {
        void* raw = nullptr;
        QB_CUDA(cudaMalloc(&raw, std::max<size_t>(count, 1) * sizeof(P)));
        *ptr = static_cast<P*>(raw);
        buffers_.push_back(raw);
        return QB200_OK;
    }
    void release();
    qb200_status use_device() const {
        QB_CUDA(cudaSetDevice(device_));
        return QB200_OK;
    }
    qb200_status check_bound() const;
    qb200_status refresh_tables();
    qb200_status run(bool forward_only);
    qb200_status run_chunk(int si, long long point0, int C, int partial_slot, bool forward_only);
    qb200_status run_fused(int si, bool forward_only);
    qb200_status prepare_weight_images();
    qb200_status tc_setup();
    qb200_status tc_prepare();
    // Each returns true when the tensor-core path took the launch.
    bool tc_forward(int layer, const T* A, T* C, long long rows, int bias_rows, qb200_status* st);
    bool tc_dgrad(int layer, const T* G, T* Gprev, long long rows, qb200_status* st);
    bool tc_wgrad(int layer, const T* H, const T* G, long long rows, int rows_per_slice, qb200_status* st);
    qb200_status check_device_error();
    bool choose_fused();
    bool tc_fwd_ok(int layer) const { return !tc_fwd_.empty() && tc_fwd_[layer]; }
    bool tc_bwd_ok(int layer) const { return !tc_bwd_.empty() && tc_bwd_[layer]; }
    // Tensor-pipe passes of a forward or data-gradient product at the bfloat16 rate (QB200_Q_GEMM_PIPE_FLOPS).
    static double tc_rows_weight(long long rows) { return tc_cor16_for(rows) ? 4.0 : 6.0; }
    bool tc_wgrad_ok_layer(int layer) const { return !tc_wgrad_.empty() && tc_wgrad_[layer]; }
    StepStatus<T> step_status(bool with_flat_flag) const {
        StepStatus<T> s;
        s.error = d_error_;
        s.flat_flag = with_flat_flag ? d_flat_ + 1 + n_params_ : nullptr;
        s.host_status = d_status_;
        return s;
    }
    // Device time of the tensor-core GEMM launches (option QB200_OPT_KERNEL_TIMERS): an event pair
    // around each one, summed by query().
    void timer_begin(double flops, double pipe_weight = 0.0) {
        if (!timers_) return;
        if (timer_events_.size() < 2 * (timer_used_ + 1)) {
            cudaEvent_t a = nullptr, b = nullptr;
            if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) {
                timers_ = false;
                return;
            }
            timer_events_.push_back(a);
            timer_events_.push_back(b);
        }
        cudaEventRecord(timer_events_[2 * timer_used_], cs_);
        timer_flops_ += flops;
        timer_pipe_flops_ += flops * pipe_weight;
    }
    void timer_end() {
        if (!timers_) return;
        cudaEventRecord(timer_events_[2 * timer_used_ + 1], cs_);
        ++timer_used_;
    }
    qb200_status launched(const char* what) {
        ++launches_;
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return fail(QB200_CUDA_ERROR, "launch of %s failed: %s", what, cudaGetErrorString(e));
        return QB200_OK;
    }
    const T* weight(int layer) const { return d_params_ + leaves_[w_leaf_[layer]].offset; }
    const T* bias(int layer) const { return b_leaf_[layer] >= 0 ? d_params_ + leaves_[b_leaf_[layer]].offset : nullptr; }

    qb200_desc desc_;
    int device_;
    cudaStream_t stream_ = nullptr;
    std::vector<void*> buffers_;
    int L_ = 0;  // layers (hidden + head)
    size_t n_params_ = 0;
    std::vector<Leaf> leaves_;
    std::vector<int> w_leaf_, b_leaf_;
    std::vector<InputState> inputs_;
    std::vector<SetState> sets_;
    T* d_params_ = nullptr;
    T* d_flat_ = nullptr;      // [loss, gradients...]
    double* d_acc_ = nullptr;  // gradient accumulators
    T* d_m_ = nullptr;
    T* d_v_ = nullptr;
    T* d_ct_ = nullptr;
    T* d_loss_only_ = nullptr;
    double* d_partials_ = nullptr;
    double* d_clip_ = nullptr;
    int total_partials_ = 0;
    // Chunk scratch.  The layer-wise engine keeps two complete sets ("lanes"), each with a stream of its own,
    // and sends consecutive chunks down alternate lanes: the HBM-bound jet kernels of one chunk then run beside the
    // tensor-bound GEMMs of the other (a jet block of 128 threads fits on an SM next to a GEMM CTA).  The members
    // below are the lane in use; select_lane() swaps them on the host between chunks.
    struct Lane {
        cudaStream_t stream = nullptr;
        std::vector<T*> H, Z;
        T* G[2] = {nullptr, nullptr};
        T* U = nullptr;
        T* Uhat = nullptr;
        T* wpartial = nullptr;
        double* acc = nullptr;     // gradient accumulators of the chunks that went down this lane
        cudaEvent_t done = nullptr;
    };
    std::vector<Lane> lanes_;
    cudaStream_t cs_ = nullptr;    // stream of the lane in use
    bool single_lane_ = false;     // option QB200_OPT_SINGLE_LANE: every chunk down lane 0 (for per-kernel timing)
    cudaEvent_t ev_lanes_ = nullptr;
    void select_lane(int k) {
        const Lane& ln = lanes_[k];
        H_ = ln.H;
        Z_ = ln.Z;
        G_[0] = ln.G[0];
        G_[1] = ln.G[1];
        U_ = ln.U;
        Uhat_ = ln.Uhat;
        wpartial_ = ln.wpartial;
        d_acc_ = ln.acc;
        cs_ = ln.stream;
    }
    std::vector<T*> H_, Z_;
    T* G_[2] = {nullptr, nullptr};
    T* U_ = nullptr;
    T* Uhat_ = nullptr;
    T* wpartial_ = nullptr;
    size_t scratch_bytes_ = 0;
    // fused engine (narrow networks): see fused_kernel.cuh
    bool fused_ = false;
    int fused_width_ = 0;
    std::vector<FusedEntry<T>> fused_entries_;  // per set
    std::vector<int> fused_grid_;               // per set
    // Every set has its own saved-jet scratch and gradient rows, so that the small sets run beside
    // the first one on a second stream; rows of all sets are consecutive for the final reduction.
    std::vector<size_t> fused_jet0_, fused_row0_;  // per set: first scratch element, first gradient row
    size_t fused_rows_ = 0;
    cudaStream_t side_stream_ = nullptr;        // lower priority: fills the tail of the first set's kernel
    cudaEvent_t ev_fork_ = nullptr, ev_join_ = nullptr;
    T* fused_z_ = nullptr;
    T* fused_h_ = nullptr;
    T* fused_grad_ = nullptr;
    void* fused_images_ = nullptr;   // tensor-core variant: pre-split weight images
    int* d_error_ = nullptr;         // device flag set by a bounded wait that gave up
    int* h_status_ = nullptr;        // mapped host words: [0] a wait gave up, [1] an optimizer update was skipped
    int* d_status_ = nullptr;        // the same words as the device sees them
    std::recursive_mutex mutex_;     // one caller at a time, as the reference's per-plan state mutex (cuda.rs:86)
    bool timers_ = false;
    std::vector<cudaEvent_t> timer_events_;
    size_t timer_used_ = 0;
    double timer_flops_ = 0.0, timer_pipe_flops_ = 0.0;

    bool fused_tensor_core_ = false;
    // layer-wise engine, float32: tcgen05 GEMMs for the layers whose shapes allow it
    std::vector<uint32_t*> tc_image_;   // per layer: pre-split weight images (null: not eligible)
    std::vector<char> tc_fwd_, tc_bwd_, tc_wgrad_;
    bool tc_any_ = false;
    cudaEvent_t ev_begin_ = nullptr, ev_end_ = nullptr;  // around the kernels of point set 0
    cudaEvent_t ev_ar0_ = nullptr, ev_ar1_ = nullptr;    // around the gradient all-reduce
    bool ev_valid_ = false, ev_ar_valid_ = false;
    int64_t launches_ = 0;
    int64_t steps_ = 0;
    bool executed_ = false;
    bool moments_ready_ = false;
    size_t wpartial_elems_ = 0;  // capacity of wpartial_ in elements
    double dp_scale_ = 1.0;
    ncclComm_t comm_ = nullptr;
    int world_ = 1;
};

constexpr int K_CHUNK_ROWS = WGRAD_ROWS_PER_SLICE;
constexpr int SM_COUNT = 148;
// Rows per split-K slice of a weight gradient over `rows` rows whose output has `tiles` CTA tiles:
// at most K_CHUNK_ROWS (the bound on sums carried in the plan dtype), and few enough that the grid
// fills whole waves of SM_COUNT CTAs.  A function of the sizes only, so the sum order is fixed.
static int slice_rows(long long rows, int tiles, int granule) {
    const long long by_precision = (rows + K_CHUNK_ROWS - 1) / K_CHUNK_ROWS;
    const long long waves = std::max<long long>(1, (by_precision * tiles + SM_COUNT - 1) / SM_COUNT);
    const long long slices = std::max(by_precision, (waves * SM_COUNT + tiles - 1) / tiles);
    long long chunk = (rows + slices - 1) / slices;
    chunk = std::max<long long>(256, (chunk + granule - 1) / granule * granule);
    return (int)std::min<long long>(chunk, K_CHUNK_ROWS);
}
constexpr int BIAS_SLICES = 512;  // upper bound on the row slices of one bias-gradient column sum

template <typename T>
void Plan<T>::release() {
    cudaSetDevice(device_);
    if (comm_ != nullptr) {
        const NcclApi* api = nccl_api();
        if (api != nullptr) api->CommDestroy(comm_);
        comm_ = nullptr;
    }
    if (stream_ != nullptr) cudaStreamSynchronize(stream_);
    for (void* p : buffers_) cudaFree(p);
    buffers_.clear();
    if (h_status_ != nullptr) cudaFreeHost(h_status_);
    h_status_ = d_status_ = nullptr;
    for (cudaEvent_t e : timer_events_) cudaEventDestroy(e);
    timer_events_.clear();
    if (ev_begin_ != nullptr) cudaEventDestroy(ev_begin_);
    if (ev_end_ != nullptr) cudaEventDestroy(ev_end_);
    if (ev_ar0_ != nullptr) cudaEventDestroy(ev_ar0_);
    if (ev_ar1_ != nullptr) cudaEventDestroy(ev_ar1_);
    ev_begin_ = ev_end_ = ev_ar0_ = ev_ar1_ = nullptr;
    for (size_t k = 0; k < lanes_.size(); ++k) {
        if (lanes_[k].done != nullptr) cudaEventDestroy(lanes_[k].done);
        if (k > 0 && lanes_[k].stream != nullptr) {
            cudaStreamSynchronize(lanes_[k].stream);
            cudaStreamDestroy(lanes_[k].stream);
        }
    }
    lanes_.clear();
    if (ev_lanes_ != nullptr) cudaEventDestroy(ev_lanes_);
    ev_lanes_ = nullptr;
    if (ev_fork_ != nullptr) cudaEventDestroy(ev_fork_);
    if (ev_join_ != nullptr) cudaEventDestroy(ev_join_);
    ev_fork_ = ev_join_ = nullptr;
    if (side_stream_ != nullptr) {
        cudaStreamSynchronize(side_stream_);
        cudaStreamDestroy(side_stream_);
    }
    side_stream_ = nullptr;
    if (stream_ != nullptr) cudaStreamDestroy(stream_);
    stream_ = nullptr;
}

template <typename T>
qb200_status Plan<T>::init() {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0)
        return fail(QB200_CUDA_ERROR, "no CUDA device is available: the qb200 backend has no CPU fallback");
    if (device_ < 0 || device_ >= count) return fail(QB200_INVALID, "device ordinal %d of %d", device_, count);
    QB_TRY(use_device());
    QB_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    QB_CUDA(cudaEventCreate(&ev_begin_));
    QB_CUDA(cudaEventCreate(&ev_end_));
    QB_CUDA(cudaEventCreate(&ev_ar0_));
    QB_CUDA(cudaEventCreate(&ev_ar1_));

    L_ = (int)desc_.sizes.size() - 1;
    w_leaf_.assign(L_, -1);
    b_leaf_.assign(L_, -1);
    size_t offset = 0;
    for (size_t i = 0; i < desc_.params.size(); ++i) {
        const auto& p = desc_.params[i];
        Leaf leaf;
        leaf.offset = offset;
        leaf.count = p.kind == QB200_WEIGHT ? (size_t)desc_.sizes[p.layer] * desc_.sizes[p.layer + 1] : (size_t)desc_.sizes[p.layer + 1];
        // Leaves start on 4-element boundaries so that kernels may use vector loads; the
        // padding stays zero (zero gradient, zero parameter, zero moments).
        offset += (leaf.count + 3) / 4 * 4;
        leaves_.push_back(leaf);
        (p.kind == QB200_WEIGHT ? w_leaf_ : b_leaf_)[p.layer] = (int)i;
    }
    n_params_ = offset;
    QB_TRY(dev_alloc(&d_params_, n_params_));
    QB_TRY(dev_alloc(&d_flat_, 2 + n_params_));
    QB_TRY(dev_alloc(&d_ct_, 1));
    QB_TRY(dev_alloc(&d_loss_only_, 1));
    QB_TRY(dev_alloc(&d_clip_, 3));
    QB_TRY(dev_alloc(&d_error_, 1));
    QB_CUDA(cudaMemsetAsync(d_error_, 0, sizeof(int), stream_));
    QB_CUDA(cudaMemsetAsync(d_flat_, 0, (2 + n_params_) * sizeof(T), stream_));
    {
        void* raw = nullptr;
        QB_CUDA(cudaHostAlloc(&raw, 2 * sizeof(int), cudaHostAllocMapped));
        h_status_ = static_cast<int*>(raw);
        h_status_[0] = h_status_[1] = 0;
        void* mapped = nullptr;
        QB_CUDA(cudaHostGetDevicePointer(&mapped, raw, 0));
        d_status_ = static_cast<int*>(mapped);
    }
    QB_CUDA(cudaMemsetAsync(d_params_, 0, n_params_ * sizeof(T), stream_));
    QB_CUDA(cudaMemsetAsync(d_clip_, 0, 3 * sizeof(double), stream_));
    const T one = T(1);
    QB_CUDA(cudaMemcpyAsync(d_ct_, &one, sizeof(T), cudaMemcpyHostToDevice, stream_));
    QB_CUDA(cudaStreamSynchronize(stream_));

    inputs_.resize(desc_.inputs.size());
    for (size_t i = 0; i < desc_.inputs.size(); ++i)
        QB_TRY(dev_alloc(&inputs_[i].dev, (size_t)(desc_.inputs[i].rows * desc_.inputs[i].cols)));

    fused_ = choose_fused();
    // Saved-jet scratch: sized per set from a byte budget, then the maximum over sets.
    const int d0 = desc_.sizes[0];
    int dmax = 0;
    size_t sum_h = 0, sum_z = 0, wmax = 0;
    for (int l = 0; l < L_; ++l) {
        sum_h += desc_.sizes[l];
        if (l >= 1) {
            sum_z += desc_.sizes[l];
            dmax = std::max(dmax, desc_.sizes[l]);
        }
        wmax = std::max(wmax, (size_t)desc_.sizes[l] * desc_.sizes[l + 1]);
    }
    dmax = std::max(dmax, d0);
    // 16 GB of the 180: the 3-D heat step (1,048,576 points, 86 KB of saved jets per point) then runs in six
    // chunks of 175 K points; it measured 115.8 ms with chunks of 65,536 points, 113.5-113.8 with 131,072 and 112.7
    // with 174,592, and 126.6 / 139.5 / 176.0 with 18,944 / 9,472 / 4,608 (chunks small enough for a layer's planes
    // to stay in L2 between the kernel that writes them and the one that reads them lose more to the short
    // launches than they gain).
    size_t budget = (size_t)16 << 30;
    if (const char* env = getenv("QB200_SCRATCH_BYTES")) {
        const long long v = atoll(env);
        if (v > 0) budget = (size_t)v;
    }
    int chunk_cap = 1 << 20;
    if (const char* env = getenv("QB200_CHUNK_POINTS")) {
        const long long v = atoll(env);
        if (v > 0) chunk_cap = (int)std::min<long long>(v, 1 << 24);
    }
    // Two lanes (see Lane) for float64 plans when some point set is large enough to be cut into chunks worth
    // overlapping; the scratch budget is shared between them.  float32 plans keep one lane: their tcgen05 GEMMs
    // hold the GPU at its power limit, where running the jet kernels beside them only lowers the clock (measured:
    // 3-D heat step 125.4 ms with one lane, 127.8 ms with two; Burgers 35.4 ms and 33.4 ms).  QB200_LANES=1 or 2
    // overrides.
    int n_lanes = 1;
    if (!fused_) {
        long long largest = 0;
        for (const auto& s : desc_.sets) largest = std::max<long long>(largest, s.n);
        const char* env = getenv("QB200_LANES");
        const int asked = env != nullptr ? atoi(env) : 0;
        if (largest >= 16384 && (asked == 2 || (asked != 1 && sizeof(T) == 8))) n_lanes = 2;
    }
    budget /= (size_t)n_lanes;
    size_t max_rows = 0, max_chunk = 0;
    std::vector<size_t> h_elems(L_, 0), z_elems(L_, 0);
    size_t g_elems = 0;
    sets_.resize(desc_.sets.size());
    for (size_t si = 0; si < desc_.sets.size(); ++si) {
        const auto& s = desc_.sets[si];
        SetState& st = sets_[si];
        st.spec.S = s.streams();
        st.spec.ndirs = (int)s.dirs.size();
        {
            long long code = 0, scale = 1;
            for (int k : s.orders) {
                code += k * scale;
                scale *= 5;
            }
            st.sig_code = code < SIG_MERGED ? (int)code : -1;
            if (!s.merge_w.empty() && st.sig_code >= 0) st.sig_code += SIG_MERGED;
        }
        int base = 1;
        st.spec.merged = s.merge_w.empty() ? 0 : 1;
        for (int j = 0; j < MAX_DIRS; ++j) {
            st.spec.order[j] = j < st.spec.ndirs ? s.orders[j] : 0;
            st.spec.base[j] = base;
            base += st.spec.order[j];
            st.spec.merge_w[j] = j < (int)s.merge_w.size() ? s.merge_w[j] : 0.0;
            st.merge_w.w[j] = (T)st.spec.merge_w[j];
        }
        st.ncols = (int)s.cols.size();
        const size_t S = st.spec.S;
        const size_t per_point = S * (sum_h + sum_z + 2 * (size_t)dmax + 2) * sizeof(T);
        long long chunk = (long long)std::min<size_t>(budget / per_point, (size_t)chunk_cap);
        // Bound the split-K slices of a weight gradient (512: the 3-D heat step then runs in six chunks).
        chunk = std::min<long long>(chunk, (long long)K_CHUNK_ROWS * 512 / (long long)S);
        // With two lanes a set is cut into at least two chunks.
        if (n_lanes > 1 && s.n >= 16384) chunk = std::min<long long>(chunk, ((s.n + 1) / 2 + 255) / 256 * 256);
        if (chunk >= s.n) {
            chunk = s.n;
        } else {
            chunk = std::max<long long>(256, chunk / 256 * 256);
            // Equal chunks instead of full ones and a short tail: the same count, each rounded up to 256 points.
            const long long count = (s.n + chunk - 1) / chunk;
            chunk = std::min(chunk, ((s.n + count - 1) / count + 255) / 256 * 256);
        }
        st.chunk = (int)chunk;
        max_chunk = std::max(max_chunk, (size_t)chunk);
        max_rows = std::max(max_rows, S * (size_t)chunk);
        for (int l = 0; l < L_; ++l) {
            h_elems[l] = std::max(h_elems[l], S * (size_t)chunk * desc_.sizes[l]);
            if (l >= 1) z_elems[l] = std::max(z_elems[l], S * (size_t)chunk * desc_.sizes[l]);
        }
        g_elems = std::max(g_elems, S * (size_t)chunk * dmax);

        QB_TRY(dev_alloc(&st.table, (size_t)s.n * st.ncols));
        std::vector<T> dirs(std::max<size_t>(1, s.dirs.size() * d0));
        for (size_t j = 0; j < s.dirs.size(); ++j)
            for (int k = 0; k < d0; ++k) dirs[j * d0 + k] = (T)s.dirs[j][k];
        QB_TRY(dev_alloc(&st.dirs, dirs.size()));
        QB_CUDA(cudaMemcpy(st.dirs, dirs.data(), dirs.size() * sizeof(T), cudaMemcpyHostToDevice));
        const int n_instr = (int)s.code.size() / 4;
        QB_TRY(dev_alloc(&st.code, (size_t)n_instr));
        QB_CUDA(cudaMemcpy(st.code, s.code.data(), (size_t)n_instr * sizeof(int4), cudaMemcpyHostToDevice));
        // Constants are rounded once to the plan dtype, as plan compilation folds a
        // weak Python scalar into the strong dtype (tensor_ir.rs:6995-7004, 6278-6283).
        std::vector<T> consts(std::max<size_t>(1, s.consts.size()));
        for (size_t i = 0; i < s.consts.size(); ++i) consts[i] = (T)s.consts[i];
        QB_TRY(dev_alloc(&st.consts, consts.size()));
        QB_CUDA(cudaMemcpy(st.consts, consts.data(), consts.size() * sizeof(T), cudaMemcpyHostToDevice));
        st.prog.code = st.code;
        st.prog.consts = st.consts;
        st.prog.n_instr = n_instr;
        st.prog.value_reg = s.value_reg;
        for (int k = 0; k < MAX_STREAMS; ++k) st.prog.grad_regs[k] = k < (int)s.grad_regs.size() ? s.grad_regs[k] : -1;
        const int chunks = (int)((s.n + chunk - 1) / chunk);
        st.partial_offset = total_partials_;
        st.partial_count = fused_ ? fused_grid_[si] : chunks * (int)((chunk + 255) / 256);
        total_partials_ += st.partial_count;
    }
    QB_TRY(dev_alloc(&d_partials_, (size_t)total_partials_));
    if (fused_) {
        // Per-CTA saved jets (rewritten every tile, so they stay in L2) and per-CTA
        // gradient rows; the layer-wise scratch is not needed.
        size_t jets = 0, rows = 0;
        const int hidden = L_ - 1;
        fused_jet0_.assign(sets_.size(), 0);
        fused_row0_.assign(sets_.size(), 0);
        for (size_t si = 0; si < sets_.size(); ++si) {
            fused_jet0_[si] = jets;
            fused_row0_[si] = rows;
            jets += (size_t)fused_grid_[si] * hidden * fused_entries_[si].scratch_per_layer;
            rows += (size_t)fused_grid_[si];
        }
        fused_rows_ = rows;
        if (sets_.size() > 1) {
            int least = 0, greatest = 0;
            QB_CUDA(cudaDeviceGetStreamPriorityRange(&least, &greatest));
            QB_CUDA(cudaStreamCreateWithPriority(&side_stream_, cudaStreamNonBlocking, least));
            QB_CUDA(cudaEventCreateWithFlags(&ev_fork_, cudaEventDisableTiming));
            QB_CUDA(cudaEventCreateWithFlags(&ev_join_, cudaEventDisableTiming));
        }
        QB_TRY(dev_alloc(&fused_z_, jets));
        QB_TRY(dev_alloc(&fused_h_, jets));
        QB_TRY(dev_alloc(&fused_grad_, rows * n_params_));
        scratch_bytes_ = (2 * jets + rows * n_params_) * sizeof(T);
        for (const auto& e : fused_entries_) fused_tensor_core_ = fused_tensor_core_ || e.tensor_core;
        if (fused_tensor_core_) {
            unsigned char* raw = nullptr;
            QB_TRY(dev_alloc(&raw, fused_weight_image_bytes(hidden - 1)));
            fused_images_ = raw;
        }
        return QB200_OK;
    }
    QB_TRY(tc_setup());
    const size_t slices = (max_rows + K_CHUNK_ROWS - 1) / K_CHUNK_ROWS + SM_COUNT + 1;  // see slice_rows()
    // Weight-gradient slices, or the (at most BIAS_SLICES) row slices of a bias gradient.
    const size_t partial_elems = std::max(slices * std::max<size_t>(wmax, (size_t)dmax), (size_t)BIAS_SLICES * dmax);
    wpartial_elems_ = partial_elems;
    scratch_bytes_ = 0;
    lanes_.resize(n_lanes);
    QB_CUDA(cudaEventCreateWithFlags(&ev_lanes_, cudaEventDisableTiming));
    for (int k = 0; k < n_lanes; ++k) {
        Lane& ln = lanes_[k];
        if (k == 0)
            ln.stream = stream_;
        else
            QB_CUDA(cudaStreamCreateWithFlags(&ln.stream, cudaStreamNonBlocking));
        QB_CUDA(cudaEventCreateWithFlags(&ln.done, cudaEventDisableTiming));
        ln.H.assign(L_, nullptr);
        ln.Z.assign(L_, nullptr);
        for (int l = 0; l < L_; ++l) {
            QB_TRY(dev_alloc(&ln.H[l], h_elems[l]));
            scratch_bytes_ += h_elems[l] * sizeof(T);
            if (l >= 1) {
                QB_TRY(dev_alloc(&ln.Z[l], z_elems[l]));
                scratch_bytes_ += z_elems[l] * sizeof(T);
            }
        }
        QB_TRY(dev_alloc(&ln.G[0], g_elems));
        QB_TRY(dev_alloc(&ln.G[1], g_elems));
        QB_TRY(dev_alloc(&ln.U, max_rows));
        QB_TRY(dev_alloc(&ln.Uhat, max_rows));
        QB_TRY(dev_alloc(&ln.wpartial, partial_elems));
        QB_TRY(dev_alloc(&ln.acc, n_params_));
        scratch_bytes_ += (2 * g_elems + 2 * max_rows + partial_elems) * sizeof(T);
    }
    select_lane(0);
    return QB200_OK;
}

template <typename T>
int64_t Plan<T>::input_shard_bytes(const char* name) const {
    for (size_t i = 0; i < desc_.inputs.size(); ++i)
        if (desc_.inputs[i].name == name) return (int64_t)(desc_.inputs[i].rows * desc_.inputs[i].cols * sizeof(T));
    for (size_t i = 0; i < desc_.params.size(); ++i)
        if (desc_.params[i].name == name) return (int64_t)(leaves_[i].count * sizeof(T));
    if (kCotangentName == std::string(name)) return (int64_t)sizeof(T);
    return -1;
}

template <typename T>
qb200_status Plan<T>::bind(const char* name, const void* host, size_t nbytes) {
    if (name == nullptr || host == nullptr) return fail(QB200_INVALID, "bind needs a name and a host buffer");
    std::lock_guard<std::recursive_mutex> lock(mutex_);
    QB_TRY(use_device());
    const std::string key(name);
    if (key == kCotangentName) {
        if (nbytes != sizeof(T)) return fail(QB200_INVALID, "input '%s' is one scalar of %zu bytes, got %zu", name, sizeof(T), nbytes);
        QB_CUDA(cudaMemcpyAsync(d_ct_, host, nbytes, cudaMemcpyHostToDevice, stream_));
        QB_CUDA(cudaStreamSynchronize(stream_));
        return QB200_OK;
    }
    for (size_t i = 0; i < desc_.params.size(); ++i) {
        if (desc_.params[i].name != key) continue;
        const size_t want = leaves_[i].count * sizeof(T);
        if (nbytes != want) return fail(QB200_INVALID, "parameter '%s' needs %zu bytes, got %zu", name, want, nbytes);
        QB_CUDA(cudaMemcpyAsync(d_params_ + leaves_[i].offset, host, nbytes, cudaMemcpyHostToDevice, stream_));
        QB_CUDA(cudaStreamSynchronize(stream_));
        leaves_[i].bound = true;
        return QB200_OK;
    }
    for (size_t i = 0; i < desc_.inputs.size(); ++i) {
        if (desc_.inputs[i].name != key) continue;
        const size_t want = (size_t)(desc_.inputs[i].rows * desc_.inputs[i].cols) * sizeof(T);
        if (nbytes != want) return fail(QB200_INVALID, "input '%s' needs %zu bytes, got %zu", name, want, nbytes);
        QB_CUDA(cudaMemcpyAsync(inputs_[i].dev, host, nbytes, cudaMemcpyHostToDevice, stream_));
        // The host buffer may be pageable and reused by the caller right away.
        QB_CUDA(cudaStreamSynchronize(stream_));
        inputs_[i].bound = true;
        for (size_t si = 0; si < desc_.sets.size(); ++si)
            for (const auto& c : desc_.sets[si].cols)
                if (c.first == (int)i) sets_[si].table_dirty = true;
        return QB200_OK;
    }
    return fail(QB200_INVALID, "the plan has no input named '%s'", name);
}

template <typename T>
qb200_status Plan<T>::sample_uniform(const char* name, int column, uint64_t key, double minval, double maxval) {
    if (name == nullptr) return fail(QB200_INVALID, "sample_uniform needs an input name");
    const double width = maxval - minval;
    if (!(minval < maxval) || !std::isfinite(width))
        return fail(QB200_INVALID, "random_uniform requires finite minval < maxval, got [%g, %g)", minval, maxval);
    // Clip bounds in the plan dtype: the smallest representable value >= minval and the largest < maxval.
    double low, high;
    if (sizeof(T) == 8) {
        low = minval;
        high = std::nextafter(maxval, -std::numeric_limits<double>::infinity());
    } else {
        float low32 = (float)minval, high32 = (float)maxval;
        if ((double)low32 < minval) low32 = std::nextafter(low32, std::numeric_limits<float>::infinity());
        if ((double)high32 >= maxval) high32 = std::nextafter(high32, -std::numeric_limits<float>::infinity());
        if (low32 > high32) return fail(QB200_INVALID, "no float32 value lies in [%g, %g)", minval, maxval);
        low = low32;
        high = high32;
    }
    QB_TRY(use_device());
    const std::string wanted(name);
    for (size_t i = 0; i < desc_.inputs.size(); ++i) {
        if (desc_.inputs[i].name != wanted) continue;
        const long long rows = desc_.inputs[i].rows;
        const int cols = (int)desc_.inputs[i].cols;
        if (column < 0 || column >= cols) return fail(QB200_INVALID, "input '%s' has %d columns, got column %d", name, cols, column);
        if (!inputs_[i].bound && cols > 1) {
            // The other columns must come from somewhere: zero the array on first use.
            QB_CUDA(cudaMemsetAsync(inputs_[i].dev, 0, (size_t)rows * cols * sizeof(T), stream_));
        }
        const int grid = (int)std::min<long long>((rows + 255) / 256, 148 * 8);
        sample_uniform_kernel<T><<<std::max(grid, 1), 256, 0, stream_>>>(inputs_[i].dev + column, rows, cols,
                                                                        (unsigned long long)key, minval, width, low, high);
        QB_TRY(launched("sample_uniform_kernel"));
        inputs_[i].bound = true;
        for (size_t si = 0; si < desc_.sets.size(); ++si)
            for (const auto& c : desc_.sets[si].cols)
                if (c.first == (int)i) sets_[si].table_dirty = true;
        return QB200_OK;
    }
    return fail(QB200_INVALID, "the plan has no data input named '%s'", name);
}

template <typename T>
qb200_status Plan<T>::check_bound() const {
    for (size_t i = 0; i < desc_.params.size(); ++i)
        if (!leaves_[i].bound) return fail(QB200_NOT_BOUND, "parameter '%s' was never bound", desc_.params[i].name.c_str());
    for (size_t i = 0; i < desc_.inputs.size(); ++i)
        if (!inputs_[i].bound) return fail(QB200_NOT_BOUND, "input '%s' was never bound", desc_.inputs[i].name.c_str());
    return QB200_OK;
}

template <typename T>
qb200_status Plan<T>::refresh_tables() {
    for (size_t si = 0; si < sets_.size(); ++si) {
        SetState& st = sets_[si];
        if (!st.table_dirty) continue;
        GatherArgs a;
        a.ncols = st.ncols;
        for (int c = 0; c < st.ncols; ++c) {
            const auto& col = desc_.sets[si].cols[c];
            a.src[c] = inputs_[col.first].dev;
            a.stride[c] = (int)desc_.inputs[col.first].cols;
            a.column[c] = col.second;
        }
        const long long n = desc_.sets[si].n;
        gather_table_kernel<T><<<grid_for(n * st.ncols, 256), 256, 0, stream_>>>(a, st.table, n);
        QB_TRY(launched("gather_table_kernel"));
        st.table_dirty = false;
    }
    return QB200_OK;
}

template <typename T>
bool Plan<T>::choose_fused() {
    if (const char* env = getenv("QB200_ENGINE"))
        if (std::string(env) == "layerwise") return false;
    // The fused kernels carry tanh and sin; the composite activations run on the layer-wise engine.
    if (desc_.activation != QB200_ACT_TANH && desc_.activation != QB200_ACT_SIN) return false;
    const int hidden = L_ - 1;
    if (hidden < 1 || hidden > FUSED_MAX_LAYERS || desc_.sizes[0] > 4) return false;
    const int W = desc_.sizes[1];
    for (int l = 1; l <= hidden; ++l)
        if (desc_.sizes[l] != W) return false;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device_);
    fused_entries_.resize(desc_.sets.size());
    fused_grid_.resize(desc_.sets.size());
    for (size_t si = 0; si < desc_.sets.size(); ++si) {
        const auto& s = desc_.sets[si];
        int code = 0, scale = 1;
        for (int k : s.orders) {
            code += k * scale;
            scale *= 5;
        }
        if (!s.merge_w.empty()) code += SIG_MERGED;
        if (!fused_lookup<T>(W, code, desc_.activation, &fused_entries_[si])) return false;
        if (fused_smem_bytes(fused_entries_[si], (int)s.code.size() / 4) > FUSED_MAX_SMEM) return false;
        const long long tiles = (s.n + fused_entries_[si].tile_points - 1) / fused_entries_[si].tile_points;
        fused_grid_[si] = (int)std::min<long long>(tiles, (long long)sms * fused_entries_[si].ctas_per_sm);
    }
    fused_width_ = W;
    return true;
}

template <typename T>
qb200_status Plan<T>::prepare_weight_images() {
    return fail(QB200_UNSUPPORTED, "the tensor-core fused engine is float32 only");
}

template <>
qb200_status Plan<float>::prepare_weight_images() {
    const int hidden_to_hidden = L_ - 2;
    if (hidden_to_hidden < 1) return QB200_OK;
    int w_off[FUSED_MAX_LAYERS + 1];
    for (int i = 0; i < hidden_to_hidden; ++i) w_off[i] = (int)leaves_[w_leaf_[1 + i]].offset;
    cudaError_t e = fused_prep_launch(d_params_, w_off, hidden_to_hidden, fused_images_, stream_);
    ++launches_;
    if (e != cudaSuccess) return fail(QB200_CUDA_ERROR, "launch of prep_weights_kernel failed: %s", cudaGetErrorString(e));
    return QB200_OK;
}

// Called after a stream synchronisation: the mapped host words say whether a bounded wait gave up
// during a step (locally: word 0) or an optimizer update was left out because some rank's did
// (word 1).  Reports once and clears, so that the next step starts clean.
template <typename T>
qb200_status Plan<T>::check_device_error() {
    if (h_status_ == nullptr) return QB200_OK;
    const int gave_up = h_status_[0], skipped = h_status_[1];
    if (gave_up == 0 && skipped == 0) return QB200_OK;
    h_status_[0] = h_status_[1] = 0;
    steps_ = std::max<int64_t>(0, steps_ - skipped);  // skipped updates do not count (bias corrections)
    QB_CUDA(cudaMemsetAsync(d_error_, 0, sizeof(int), stream_));
    QB_CUDA(cudaStreamSynchronize(stream_));
    if (gave_up != 0)
        return fail(QB200_CUDA_ERROR, "a staged copy inside a kernel did not complete within its wait limit; the results "
                                      "of that step are invalid%s", skipped ? " and its optimizer update was skipped" : "");
    return fail(QB200_CUDA_ERROR, "another rank's step was invalid (a bounded wait gave up there); the optimizer update "
                                  "of that step was skipped on every rank");
}

template <typename T>
qb200_status Plan<T>::run_fused(int si, bool forward_only) {
    SetState& st = sets_[si];
    const auto& s = desc_.sets[si];
    FusedArgs<T> a;
    a.L = L_ - 1;
    a.d0 = desc_.sizes[0];
    a.P = (int)n_params_;
    a.params = d_params_;
    for (int l = 0; l <= FUSED_MAX_LAYERS; ++l) {
        a.w_off[l] = l < L_ ? (int)leaves_[w_leaf_[l]].offset : 0;
        a.b_off[l] = (l < L_ && b_leaf_[l] >= 0) ? (int)leaves_[b_leaf_[l]].offset : -1;
    }
    a.table = st.table;
    a.ncols = st.ncols;
    a.n_points = s.n;
    for (int i = 0; i < MAX_DIRS * 4; ++i) a.dirs[i] = T(0);
    for (int j = 0; j < MAX_DIRS; ++j) a.merge_w[j] = sets_[si].merge_w.w[j];
    for (size_t j = 0; j < s.dirs.size(); ++j)
        for (int k = 0; k < a.d0; ++k) a.dirs[j * a.d0 + k] = (T)s.dirs[j][k];
    a.prog = st.prog;
    a.cotangent = d_ct_;
    a.weight = (T)s.weight;
    a.extra = (T)dp_scale_;
    a.scratch_z = fused_z_ + fused_jet0_[si];
    a.scratch_h = fused_h_ + fused_jet0_[si];
    a.grad_cta = fused_grad_ + fused_row0_[si] * n_params_;
    a.loss_cta = d_partials_ + st.partial_offset;
    a.forward_only = forward_only ? 1 : 0;
    a.weight_images = fused_images_;
    a.error = d_error_;
    // Sets after the first run on the side stream, between the fork and join events of run().
    cudaStream_t stream = (si > 0 && side_stream_ != nullptr) ? side_stream_ : stream_;
    cudaError_t e = fused_launch<T>(fused_entries_[si], fused_grid_[si], stream, a);
    ++launches_;
    if (e != cudaSuccess) return fail(QB200_CUDA_ERROR, "launch of fused_step_kernel failed: %s", cudaGetErrorString(e));
    return QB200_OK;
}

// ---- tcgen05 GEMMs in the layer-wise engine (float32 plans only) -----------------------
template <typename T> qb200_status Plan<T>::tc_setup() { return QB200_OK; }
template <typename T> qb200_status Plan<T>::tc_prepare() { return QB200_OK; }
template <typename T> bool Plan<T>::tc_forward(int, const T*, T*, long long, int, qb200_status*) { return false; }
template <typename T> bool Plan<T>::tc_dgrad(int, const T*, T*, long long, qb200_status*) { return false; }
template <typename T> bool Plan<T>::tc_wgrad(int, const T*, const T*, long long, int, qb200_status*) { return false; }

template <>
qb200_status Plan<float>::tc_setup() {
    tc_image_.assign(L_, nullptr);
    tc_fwd_.assign(L_, 0);
    tc_bwd_.assign(L_, 0);
    tc_wgrad_.assign(L_, 0);
    if (!tc_available()) return QB200_OK;
    for (int l = 0; l < L_; ++l) {
        const int K = desc_.sizes[l], N = desc_.sizes[l + 1];
        tc_fwd_[l] = tc_rows_ok(N, K);
        tc_bwd_[l] = l > 0 && tc_rows_ok(K, N);
        tc_wgrad_[l] = tc_wgrad_ok(K, N);
        if (tc_fwd_[l] || tc_bwd_[l]) QB_TRY(dev_alloc(&tc_image_[l], 2 * tc_image_words(K, N)));  // one image per scheme
        tc_any_ = tc_any_ || tc_fwd_[l] || tc_bwd_[l] || tc_wgrad_[l];
    }
    return QB200_OK;
}

template <>
qb200_status Plan<float>::tc_prepare() {
    for (int l = 0; l < L_; ++l) {
        if (tc_image_[l] == nullptr) continue;
        // TMA kernels take the weight unsplit plus its lo plane: W itself for the data gradient, W^T for the
        // forward product.  Image: four parts of K*N words (tc_image_words).
        // The first image serves launches with bfloat16 corrections, the second those with tf32 corrections; which
        // of the two a launch takes depends on its rows (tc_cor16_for), so both are written unless one is forced.
        const size_t kn = (size_t)desc_.sizes[l] * desc_.sizes[l + 1];
        const int mode = tc_cor_mode();
        for (int scheme = 0; scheme < 2; ++scheme) {
            const bool cor16 = scheme == 0;
            if ((mode == 0 && cor16) || (mode == 1 && !cor16)) continue;
            float* image = reinterpret_cast<float*>(tc_image_[l]) + (cor16 ? 0 : 4 * kn);
            cudaError_t e = tc2_prepare_launch(weight(l), desc_.sizes[l], desc_.sizes[l + 1], image, image + kn, image + 2 * kn,
                                               image + 3 * kn, cor16, stream_);
            ++launches_;
            if (e != cudaSuccess)
                return fail(QB200_CUDA_ERROR, "launch of tc_prep_weight_kernel failed: %s", cudaGetErrorString(e));
        }
    }
    return QB200_OK;
}

template <>
bool Plan<float>::tc_forward(int layer, const float* A, float* C, long long rows, int bias_rows, qb200_status* st) {
    if (!tc_fwd_[layer]) return false;
    const int K = desc_.sizes[layer], N = desc_.sizes[layer + 1];
    const bool cor16 = tc_cor16_for(rows);
    const float* image = reinterpret_cast<const float*>(tc_image_[layer]) + (cor16 ? 0 : 4 * (size_t)K * N);
    cudaError_t e = tc2_rows_launch(A, K, image, image + (size_t)K * N, K, C, N, bias(layer), bias_rows, (int)rows, N, K, cor16,
                                    d_error_, cs_);
    ++launches_;
    *st = e == cudaSuccess ? QB200_OK : fail(QB200_CUDA_ERROR, "launch of tc_gemm_kernel(forward) failed: %s", cudaGetErrorString(e));
    return true;
}

template <>
bool Plan<float>::tc_dgrad(int layer, const float* G, float* Gprev, long long rows, qb200_status* st) {
    if (!tc_bwd_[layer]) return false;
    const int K = desc_.sizes[layer], N = desc_.sizes[layer + 1];
    // The weight itself is the K-major operand here (its tf32-rounded copy when the corrections run in bfloat16).
    const bool cor16 = tc_cor16_for(rows);
    const float* image = reinterpret_cast<const float*>(tc_image_[layer]) + (cor16 ? 0 : 4 * (size_t)K * N);
    cudaError_t e = tc2_rows_launch(G, N, cor16 ? image + 3 * (size_t)K * N : weight(layer), image + 2 * (size_t)K * N, N, Gprev,
                                    K, nullptr, 0, (int)rows, K, N, cor16, d_error_, cs_);
    ++launches_;
    *st = e == cudaSuccess ? QB200_OK : fail(QB200_CUDA_ERROR, "launch of tc_gemm_kernel(dgrad) failed: %s", cudaGetErrorString(e));
    return true;
}

template <>
bool Plan<float>::tc_wgrad(int layer, const float* H, const float* G, long long rows, int rows_per_slice,
                           qb200_status* st) {
    if (layer < 0 || layer >= L_ || !tc_wgrad_[layer]) return false;
    const int K = desc_.sizes[layer], N = desc_.sizes[layer + 1];
    cudaError_t e = tc2_wgrad_launch(H, K, G, N, wpartial_, (int)rows, K, N, rows_per_slice, d_error_, cs_);
    ++launches_;
    *st = e == cudaSuccess ? QB200_OK : fail(QB200_CUDA_ERROR, "launch of tc_gemm_kernel(wgrad) failed: %s", cudaGetErrorString(e));
    return true;
}

template <typename T>
qb200_status Plan<T>::run_chunk(int si, long long point0, int C, int partial_slot, bool forward_only) {
    SetState& st = sets_[si];
    const JetSpec& spec = st.spec;
    const int S = spec.S;
    const long long rows = (long long)S * C;
    const std::vector<int>& sz = desc_.sizes;
    const int head = L_ - 1;  // index of the linear output layer

    seed_input_kernel<T><<<grid_for(rows * sz[0], 256), 256, 0, cs_>>>(st.table, st.ncols, point0, C, sz[0], spec,
                                                                           st.dirs, H_[0]);
    QB_TRY(launched("seed_input_kernel"));
    // The first hidden layer's product is formed inside the jet kernels (FirstLayer in jet_kernels.cuh) when the
    // network has few inputs and layer 1 is not also the last hidden layer; QB200_FIRST_FUSED=0 keeps it apart.
    const int first_grid = jet_sig_grid((long long)C * sz[1] / JetVec<T>::V);
    static const bool first_switch = [] {
        const char* env = getenv("QB200_FIRST_FUSED");
        return !(env != nullptr && strcmp(env, "0") == 0);
    }();
    const bool first_fused = first_switch && head >= 2 && jet_first_inputs_ok(sz[0]) && jet_bias_fusable<T>(sz[1]) &&
                             jet_sig_eligible<T>(st.sig_code, (long long)C * sz[1], H_[1], G_[0], G_[1]) &&
                             (reinterpret_cast<uintptr_t>(H_[0]) & 15) == 0 &&
                             (size_t)first_grid * (sz[0] + 1) * sz[1] <= wpartial_elems_;
    FirstLayer<T> first;
    first.X = H_[0];
    first.W = weight(0);
    first.b = bias(0);
    first.wpartial = wpartial_ + (size_t)first_grid * sz[1];
    first.C = C;
    first.d = sz[1];
    static const bool head_switch = [] {
        const char* env = getenv("QB200_HEAD_FUSED");
        return !(env != nullptr && strcmp(env, "0") == 0);
    }();
    bool head_dotted = false;
    for (int l = 1; l <= head; ++l) {
        if (l == 1 && first_fused) {
            jet_forward_first_launch<T>(st.sig_code, H_[1], (long long)C * sz[1], desc_.activation, st.merge_w, sz[0], first, cs_);
            QB_TRY(launched("jet_forward_kernel(first layer)"));
            continue;
        }
        // Z_l = H_{l-1} W_{l-1} (+ bias on the primal rows), H_l = tanh-jet(Z_l).
        GemmArgs<T> g;
        g.A = H_[l - 1];
        g.B = weight(l - 1);
        g.C = Z_[l];
        g.bias = bias(l - 1);
        g.sam = sz[l - 1];
        g.sak = 1;
        g.sbk = sz[l];
        g.sbn = 1;
        g.M = (int)rows;
        g.N = sz[l];
        g.K = sz[l - 1];
        g.ldc = sz[l];
        g.bias_rows = C;
        g.k_chunk = g.K;
        qb200_status tc_status = QB200_OK;
        const bool narrow = g.K <= 4 && g.N % 4 == 0 && g.N >= 32 && 256 % (g.N / 4) == 0;
        if (tc_fwd_ok(l - 1) || !narrow) timer_begin(2.0 * (double)rows * g.N * g.K, tc_fwd_ok(l - 1) ? tc_rows_weight(rows) : 0.0);
        if (tc_forward(l - 1, H_[l - 1], Z_[l], rows, C, &tc_status)) {
            QB_TRY(tc_status);
            timer_end();
        } else if (g.K <= 4 && g.N % 4 == 0 && g.N >= 32 && 256 % (g.N / 4) == 0) {
            // Narrow contraction (the first layer): stream the output once.
            const int rows_per_block = 256 / (g.N / 4);
            const int grid = (int)std::min<long long>((rows + rows_per_block - 1) / rows_per_block, 148 * 16);
            switch (g.K) {
                case 1: skinny_forward_kernel<T, 1><<<grid, 256, 0, cs_>>>(g.A, g.B, g.bias, g.C, rows, g.N, C); break;
                case 2: skinny_forward_kernel<T, 2><<<grid, 256, 0, cs_>>>(g.A, g.B, g.bias, g.C, rows, g.N, C); break;
                case 3: skinny_forward_kernel<T, 3><<<grid, 256, 0, cs_>>>(g.A, g.B, g.bias, g.C, rows, g.N, C); break;
                default: skinny_forward_kernel<T, 4><<<grid, 256, 0, cs_>>>(g.A, g.B, g.bias, g.C, rows, g.N, C); break;
            }
            QB_TRY(launched("skinny_forward_kernel"));
        } else {
            const cudaError_t e = gemm_launch<T, true, true>(g, 1, cs_);
            (void)e;  // launched() reads the launch status
            QB_TRY(launched("gemm_kernel(forward)"));
            timer_end();
        }
        const long long plane = (long long)C * sz[l];
        if (jet_sig_eligible<T>(st.sig_code, plane, Z_[l], H_[l], nullptr)) {
            // The last hidden layer's kernel also leaves the output layer's product as per-warp partials.
            HeadDot<T> dot = HeadDot<T>();
            if (l == head && head_switch && head_dot_fusable<T>(sz[l]) && jet_bias_fusable<T>(sz[l]) &&
                (size_t)rows * (sz[l] / (32 * JetVec<T>::V)) <= wpartial_elems_) {
                dot.w = weight(head);
                dot.partial = wpartial_;
                dot.C = C;
                dot.d = sz[l];
                head_dotted = true;
            }
            jet_forward_sig_launch<T>(st.sig_code, Z_[l], H_[l], plane, desc_.activation, st.merge_w, cs_, dot);
        }
        else
            jet_forward_kernel<T><<<grid_for(plane, 256), 256, 0, cs_>>>(Z_[l], H_[l], plane, spec, desc_.activation);
        QB_TRY(launched("jet_forward_kernel"));
    }
    if (head_dotted) {
        head_combine_kernel<T><<<grid_for(rows, 256), 256, 0, cs_>>>(wpartial_, bias(head), U_, rows,
                                                                       sz[head] / (32 * JetVec<T>::V), C);
        QB_TRY(launched("head_combine_kernel"));
    } else {
        head_forward_kernel<T><<<grid_for(rows * 32, 256), 256, 0, cs_>>>(H_[head], weight(head), bias(head), U_, rows,
                                                                              sz[head], C);
        QB_TRY(launched("head_forward_kernel"));
    }
    const T w = (T)desc_.sets[si].weight;
    residual_kernel<T><<<(C + 255) / 256, 256, 0, cs_>>>(st.table, st.ncols, point0, C, S, U_,
                                                             forward_only ? nullptr : Uhat_, st.prog, d_ct_, w,
                                                             (T)dp_scale_, d_partials_ + partial_slot);
    QB_TRY(launched("residual_kernel"));
    if (forward_only) return QB200_OK;

    auto wgrad = [&](const T* Hprev, const T* Gz, int d_in, int d_out, int leaf, int layer) -> qb200_status {
        {
            qb200_status tc_status = QB200_OK;
            // Output tiles of the tensor-core kernel: 128 rows of dW by 128 or 64 columns.
            const int tc_col_tiles = d_out / (d_out % 128 == 0 ? 128 : 64);
            const int tc_chunk = slice_rows(rows, std::max(1, d_in / 128) * std::max(1, tc_col_tiles), 32);
            const bool tc_takes = layer >= 0 && layer < L_ && tc_wgrad_ok_layer(layer);
            if (tc_takes) timer_begin(2.0 * (double)rows * d_in * d_out, 6.0);
            if (tc_wgrad(layer, Hprev, Gz, rows, tc_chunk, &tc_status)) {
                QB_TRY(tc_status);
                timer_end();
                const int count = d_in * d_out;
                const int slices = (int)((rows + tc_chunk - 1) / tc_chunk);
                accumulate_partials_launch<T>(wpartial_, d_acc_ + leaves_[leaf].offset, count, slices, cs_);
                return launched("accumulate_partials_kernel");
            }
        }
        if ((d_in <= 4 && d_out >= 32) || (d_out == 1 && d_in >= 32)) {
            // One narrow side: stream the wide matrix once (HBM-bound) instead of a 64 x 64 tile GEMM.
            const int count = d_in * d_out;
            long long chunk = (rows + 8 * SM_COUNT - 1) / (8 * SM_COUNT);
            chunk = std::min<long long>(K_CHUNK_ROWS, std::max<long long>(64, (chunk + 7) / 8 * 8));
            const long long room = (long long)(wpartial_elems_ / (size_t)count);
            if ((rows + chunk - 1) / chunk > room) chunk = ((rows + room - 1) / room + 7) / 8 * 8;
            const int slices = (int)((rows + chunk - 1) / chunk);
            if (chunk <= K_CHUNK_ROWS) {
                const dim3 grid((std::max(d_in, d_out) + 255) / 256, slices);
                if (d_out == 1)
                    skinny_wgrad_kernel<T, 1, false><<<grid, 256, 0, cs_>>>(Hprev, Gz, wpartial_, rows, d_in, d_out, (int)chunk);
                else if (d_in == 1)
                    skinny_wgrad_kernel<T, 1, true><<<grid, 256, 0, cs_>>>(Hprev, Gz, wpartial_, rows, d_in, d_out, (int)chunk);
                else if (d_in == 2)
                    skinny_wgrad_kernel<T, 2, true><<<grid, 256, 0, cs_>>>(Hprev, Gz, wpartial_, rows, d_in, d_out, (int)chunk);
                else if (d_in == 3)
                    skinny_wgrad_kernel<T, 3, true><<<grid, 256, 0, cs_>>>(Hprev, Gz, wpartial_, rows, d_in, d_out, (int)chunk);
                else
                    skinny_wgrad_kernel<T, 4, true><<<grid, 256, 0, cs_>>>(Hprev, Gz, wpartial_, rows, d_in, d_out, (int)chunk);
                QB_TRY(launched("skinny_wgrad_kernel"));
                accumulate_partials_launch<T>(wpartial_, d_acc_ + leaves_[leaf].offset, count, slices, cs_);
                return launched("accumulate_partials_kernel");
            }
        }
        GemmArgs<T> g;
        g.A = Hprev;
        g.B = Gz;
        g.C = wpartial_;
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
        const bool fp64_tensor = sizeof(T) == 8 && d_in >= 32 && d_out >= 32;  // the kernel gemm_launch will pick
        g.k_chunk = slice_rows(rows, gemm_output_tiles(d_in, d_out, fp64_tensor), GEMM_BK);
        const int slices = (int)((rows + g.k_chunk - 1) / g.k_chunk);
        timer_begin(2.0 * (double)rows * d_in * d_out);
        const cudaError_t e = gemm_launch<T, false, true>(g, slices, cs_);
        (void)e;
        QB_TRY(launched("gemm_kernel(wgrad)"));
        timer_end();
        const int count = d_in * d_out;
        accumulate_partials_launch<T>(wpartial_, d_acc_ + leaves_[leaf].offset,
                                                                                count, slices, cs_);
        return launched("accumulate_partials_kernel");
    };
    auto bgrad = [&](const T* Gz, int d_out, int leaf) -> qb200_status {
        if (leaf < 0) return QB200_OK;
        // About eight CTAs per SM over (column blocks x row slices); a slice never drops below
        // 256 rows, so the slice count depends on the sizes only and the sum order is fixed.
        const int col_blocks = (d_out + 31) / 32;
        const int want = std::min(BIAS_SLICES, std::max(1, (8 * 148 + col_blocks - 1) / col_blocks));
        const int row_chunk = std::max(256, ((C + want - 1) / want + 7) / 8 * 8);
        const int slices = (C + row_chunk - 1) / row_chunk;
        dim3 grid(col_blocks, slices);
        colsum_kernel<T><<<grid, 256, 0, cs_>>>(Gz, wpartial_, C, d_out, row_chunk);
        QB_TRY(launched("colsum_kernel"));
        accumulate_partials_launch<T>(wpartial_, d_acc_ + leaves_[leaf].offset,
                                                                                d_out, slices, cs_);
        return launched("accumulate_partials_kernel");
    };

    // Head: dW = H^T Uhat, db = sum of the primal cotangents, G = Uhat (x) w.
    int cur = 0;
    // The head's data gradient G = Uhat (x) w is formed inside the last hidden layer's jet kernel when
    // that kernel has a compile-time signature; otherwise it is materialised here.
    const bool head_fused = head >= 1 && sz[head] % JetVec<T>::V == 0 &&
                            jet_sig_eligible<T>(st.sig_code, (long long)C * sz[head], Z_[head], H_[head], G_[cur]) &&
                            (reinterpret_cast<uintptr_t>(weight(head)) & 15) == 0;
    // ... and dW of the head in the same kernel (jet_kernels.cuh), when its per-block partials fit beside the bias partials.
    const int head_grid = head >= 1 ? jet_sig_grid((long long)C * sz[head] / JetVec<T>::V) : 0;
    const bool head_w_fused = head_fused && head_switch && jet_bias_fusable<T>(sz[head]) &&
                              2 * (size_t)head_grid * sz[head] <= wpartial_elems_;
    if (!head_w_fused) QB_TRY(wgrad(H_[head], Uhat_, sz[head], 1, w_leaf_[head], head));
    QB_TRY(bgrad(Uhat_, 1, b_leaf_[head]));
    if (!head_fused) {
        head_backward_kernel<T><<<grid_for(rows * sz[head], 256), 256, 0, cs_>>>(Uhat_, weight(head), G_[cur], rows,
                                                                                     sz[head]);
        QB_TRY(launched("head_backward_kernel"));
    }
    for (int l = head; l >= 1; --l) {
        const long long plane = (long long)C * sz[l];
        // The vectorised kernel can form the bias-gradient partials (one row of sz[l] per block) on its way.
        if (l == 1 && first_fused) {
            // Cotangents of H_1 in, bias- and weight-gradient partials out; nothing of layer 1 is written back.
            T* bias_partial = b_leaf_[0] >= 0 ? wpartial_ : nullptr;
            jet_backward_first_launch<T>(st.sig_code, H_[1], G_[cur], plane, sz[1], desc_.activation, bias_partial, st.merge_w,
                                         sz[0], first, cs_);
            QB_TRY(launched("jet_backward_kernel(first layer)"));
            if (bias_partial != nullptr) {
                accumulate_partials_launch<T>(wpartial_, d_acc_ + leaves_[b_leaf_[0]].offset, sz[1], first_grid, cs_);
                QB_TRY(launched("accumulate_partials_kernel"));
            }
            accumulate_partials_launch<T>(first.wpartial, d_acc_ + leaves_[w_leaf_[0]].offset, sz[0] * sz[1], first_grid, cs_);
            QB_TRY(launched("accumulate_partials_kernel"));
            break;
        }
        const bool sig = (l == head && head_fused) || jet_sig_eligible<T>(st.sig_code, plane, Z_[l], H_[l], G_[cur]);
        const int jet_grid = jet_sig_grid(plane / JetVec<T>::V);
        const bool bias_fused = sig && b_leaf_[l - 1] >= 0 && jet_bias_fusable<T>(sz[l]) &&
                                (size_t)jet_grid * sz[l] <= wpartial_elems_;
        T* bias_partial = bias_fused ? wpartial_ : nullptr;
        if (l == head && head_fused)
            jet_backward_head_launch<T>(st.sig_code, Z_[l], H_[l], G_[cur], plane, Uhat_, weight(head), sz[head], C,
                                        desc_.activation, bias_partial, st.merge_w, cs_,
                                        head_w_fused ? wpartial_ + (size_t)head_grid * sz[head] : nullptr);
        else if (sig)
            jet_backward_sig_launch<T>(st.sig_code, Z_[l], H_[l], G_[cur], plane, sz[l], desc_.activation, bias_partial,
                                       st.merge_w, cs_);
        else
            jet_backward_kernel<T><<<grid_for(plane, 256), 256, 0, cs_>>>(Z_[l], H_[l], G_[cur], plane, spec, desc_.activation);
        QB_TRY(launched("jet_backward_kernel"));
        if (bias_fused) {
            accumulate_partials_launch<T>(wpartial_, d_acc_ + leaves_[b_leaf_[l - 1]].offset, sz[l], jet_grid, cs_);
            QB_TRY(launched("accumulate_partials_kernel"));
        }
        if (l == head && head_w_fused) {
            accumulate_partials_launch<T>(wpartial_ + (size_t)head_grid * sz[head], d_acc_ + leaves_[w_leaf_[head]].offset,
                                          sz[head], head_grid, cs_);
            QB_TRY(launched("accumulate_partials_kernel"));
        }
        QB_TRY(wgrad(H_[l - 1], G_[cur], sz[l - 1], sz[l], w_leaf_[l - 1], l - 1));
        if (!bias_fused) QB_TRY(bgrad(G_[cur], sz[l], b_leaf_[l - 1]));
        if (l > 1) {
            GemmArgs<T> g;
            g.A = G_[cur];
            g.B = weight(l - 1);
            g.C = G_[cur ^ 1];
            g.bias = nullptr;
            g.sam = sz[l];
            g.sak = 1;
            g.sbk = 1;
            g.sbn = sz[l];
            g.M = (int)rows;
            g.N = sz[l - 1];
            g.K = sz[l];
            g.ldc = sz[l - 1];
            g.bias_rows = 0;
            g.k_chunk = g.K;
            qb200_status tc_status = QB200_OK;
            timer_begin(2.0 * (double)rows * g.N * g.K, tc_bwd_ok(l - 1) ? tc_rows_weight(rows) : 0.0);
            if (tc_dgrad(l - 1, G_[cur], G_[cur ^ 1], rows, &tc_status)) {
                QB_TRY(tc_status);
            } else {
                const cudaError_t e = gemm_launch<T, true, false>(g, 1, cs_);
                (void)e;
                QB_TRY(launched("gemm_kernel(dgrad)"));
            }
            timer_end();
            cur ^= 1;
        }
    }
    return QB200_OK;
}

template <typename T>
qb200_status Plan<T>::run(bool forward_only) {
    QB_TRY(use_device());
    QB_TRY(check_bound());
    QB_TRY(refresh_tables());
    if (!forward_only) {
        timer_used_ = 0;
        timer_flops_ = 0.0;
        timer_pipe_flops_ = 0.0;
    }
    if (!forward_only && !fused_)
        for (const Lane& ln : lanes_) QB_CUDA(cudaMemsetAsync(ln.acc, 0, n_params_ * sizeof(double), stream_));
    if (fused_ && fused_tensor_core_) QB_TRY(prepare_weight_images());
    const bool side = fused_ && side_stream_ != nullptr;
    if (side) {
        // Tables and weight images are ready on the main stream before the side stream starts.
        QB_CUDA(cudaEventRecord(ev_fork_, stream_));
        QB_CUDA(cudaStreamWaitEvent(side_stream_, ev_fork_, 0));
    }
    if (!fused_ && tc_any_) QB_TRY(tc_prepare());
    if (!fused_ && lanes_.size() > 1) {
        // Tables, weight images and cleared accumulators are ready on the main stream before the other lane starts.
        QB_CUDA(cudaEventRecord(ev_lanes_, stream_));
        for (size_t k = 1; k < lanes_.size(); ++k) QB_CUDA(cudaStreamWaitEvent(lanes_[k].stream, ev_lanes_, 0));
    }
    int next_lane = 0;
    LossArgs la;
    la.n_sets = (int)sets_.size();
    for (size_t si = 0; si < sets_.size(); ++si) {
        SetState& st = sets_[si];
        const long long n = desc_.sets[si].n;
        int slot = st.partial_offset;
        if (si == 0 && !forward_only) QB_CUDA(cudaEventRecord(ev_begin_, stream_));
        if (fused_) {
            QB_TRY(run_fused((int)si, forward_only));
            if (si == 0 && !forward_only) {
                QB_CUDA(cudaEventRecord(ev_end_, stream_));
                ev_valid_ = true;
            }
            la.offset[si] = st.partial_offset;
            la.count[si] = fused_grid_[si];
            la.weight[si] = desc_.sets[si].weight;
            continue;
        }
        for (long long p0 = 0; p0 < n; p0 += st.chunk) {
            const int C = (int)std::min<long long>(st.chunk, n - p0);
            select_lane(next_lane);
            next_lane = single_lane_ ? 0 : (next_lane + 1) % (int)lanes_.size();
            QB_TRY(run_chunk((int)si, p0, C, slot, forward_only));
            slot += (C + 255) / 256;
        }
        select_lane(0);
        if (si == 0 && !forward_only) {
            QB_CUDA(cudaEventRecord(ev_end_, stream_));
            ev_valid_ = true;
        }
        la.offset[si] = st.partial_offset;
        la.count[si] = slot - st.partial_offset;
        la.weight[si] = desc_.sets[si].weight;
    }
    if (side) {
        QB_CUDA(cudaEventRecord(ev_join_, side_stream_));
        QB_CUDA(cudaStreamWaitEvent(stream_, ev_join_, 0));
    }
    if (!fused_)
        for (size_t k = 1; k < lanes_.size(); ++k) {
            QB_CUDA(cudaEventRecord(lanes_[k].done, lanes_[k].stream));
            QB_CUDA(cudaStreamWaitEvent(stream_, lanes_[k].done, 0));
        }
    T* loss_out = forward_only ? d_loss_only_ : d_flat_;
    if (fused_ && !forward_only) {
        const int P = (int)n_params_;
        fused_finalize_kernel<T><<<(P + 31) / 32 + 1, 256, 0, stream_>>>(fused_grad_, P, (int)fused_rows_, d_flat_ + 1,
                                                                       d_partials_, la, (T)dp_scale_, loss_out,
                                                                       step_status(true));
        QB_TRY(launched("fused_finalize_kernel"));
        executed_ = true;
        return QB200_OK;
    }
    loss_finalize_kernel<T><<<1, 256, 0, stream_>>>(d_partials_, la, forward_only ? T(1) : (T)dp_scale_, loss_out,
                                                    step_status(!forward_only));
    QB_TRY(launched("loss_finalize_kernel"));
    if (!forward_only) {
        // The lanes' accumulators are added in lane order: the result does not depend on how the lanes overlapped.
        finalize_gradients_kernel<T><<<((int)n_params_ + 255) / 256, 256, 0, stream_>>>(
            lanes_[0].acc, lanes_.size() > 1 ? lanes_[1].acc : nullptr, d_flat_ + 1, (int)n_params_);
        QB_TRY(launched("finalize_gradients_kernel"));
        executed_ = true;
    }
    return QB200_OK;
}

template <typename T>
qb200_status Plan<T>::execute_local() {
    std::lock_guard<std::recursive_mutex> lock(mutex_);
    return run(false);
}

template <typename T>
qb200_status Plan<T>::all_reduce() {
    std::lock_guard<std::recursive_mutex> lock(mutex_);
    if (comm_ == nullptr) return QB200_OK;
    const NcclApi* api = nccl_api();
    if (api == nullptr) return QB200_NCCL_ERROR;
    cudaEventRecord(ev_ar0_, stream_);
    ncclResult_t r = api->AllReduce(d_flat_, d_flat_, 2 + n_params_, DTypeOf<T>::nccl, ncclSum, comm_, stream_);
    cudaEventRecord(ev_ar1_, stream_);
    ev_ar_valid_ = r == ncclSuccess;
    if (r != ncclSuccess) {
        // Failure contract: drop the communicator, the caller re-attaches
        // (crates/quabla-core/src/tensor_ir/cuda.rs:132-145, 699-716).
        api->CommAbort(comm_);
        comm_ = nullptr;
        dp_scale_ = 1.0;
        return fail(QB200_NCCL_ERROR, "ncclAllReduce failed: %s; the communicator was aborted, attach a new one", api->GetErrorString(r));
    }
    return QB200_OK;
}

template <typename T>
qb200_status Plan<T>::read_output(int index, void* host, size_t nbytes) {
    std::lock_guard<std::recursive_mutex> lock(mutex_);
    QB_TRY(use_device());
    if (!executed_) return fail(QB200_INVALID, "read_output before execute");
    if (index < 0 || index > (int)leaves_.size()) return fail(QB200_INVALID, "output index %d of %zu", index, leaves_.size() + 1);
    const size_t offset = index == 0 ? 0 : 1 + leaves_[index - 1].offset;
    const size_t count = index == 0 ? 1 : leaves_[index - 1].count;
    if (nbytes != count * sizeof(T)) return fail(QB200_INVALID, "output %d has %zu bytes, got a buffer of %zu", index, count * sizeof(T), nbytes);
    QB_CUDA(cudaMemcpyAsync(host, d_flat_ + offset, nbytes, cudaMemcpyDeviceToHost, stream_));
    QB_CUDA(cudaStreamSynchronize(stream_));
    return check_device_error();
}

template <typename T>
qb200_status Plan<T>::optimizer_step(const qb200_opt_config* c) {
    QB_TRY(validate_opt_config(c));  // before any device work (cuda_optimizer.rs:207-212)
    std::lock_guard<std::recursive_mutex> lock(mutex_);
    QB_TRY(use_device());
    if (!executed_) return fail(QB200_INVALID, "optimizer_step before execute: there are no gradients");
    if (!moments_ready_ && c->rule == QB200_ADAM) {
        QB_TRY(dev_alloc(&d_m_, n_params_));
        QB_TRY(dev_alloc(&d_v_, n_params_));
        QB_CUDA(cudaMemsetAsync(d_m_, 0, n_params_ * sizeof(T), stream_));
        QB_CUDA(cudaMemsetAsync(d_v_, 0, n_params_ * sizeof(T), stream_));
        moments_ready_ = true;
    }
    // The flag slot behind the gradients: non-zero after the all-reduce when any rank's step raised the
    // device error flag; the kernels below then leave parameters and moments as they are.
    const T* skip = d_flat_ + 1 + n_params_;
    const double* clip = nullptr;
    if (c->has_clip) {
        global_norm_kernel<T><<<1, 1024, 0, stream_>>>(d_flat_ + 1, (long long)n_params_, c->clip_norm, d_clip_, skip);
        QB_TRY(launched("global_norm_kernel"));
        clip = d_clip_;
    }
    ++steps_;
    const int grid = grid_for((long long)n_params_, 256);
    if (c->rule == QB200_SGD) {
        sgd_kernel<T><<<grid, 256, 0, stream_>>>(d_params_, d_flat_ + 1, (T)c->learning_rate, clip, (long long)n_params_,
                                                 skip, d_status_);
        return launched("sgd_kernel");
    }
    // Coefficients in double, rounded once (AdamCoefficients::new(..).map(T::from_f64),
    // device_optimizer.rs:97-101, 129-150; cuda_optimizer.rs:340-359).
    AdamCoeffs<T> k;
    k.learning_rate = (T)c->learning_rate;
    k.beta1 = (T)c->beta1;
    k.beta2 = (T)c->beta2;
    k.one_minus_beta1 = (T)(1.0 - c->beta1);
    k.one_minus_beta2 = (T)(1.0 - c->beta2);
    k.epsilon = (T)c->epsilon;
    k.correction1 = (T)(1.0 - std::pow(c->beta1, (double)steps_));
    k.correction2 = (T)(1.0 - std::pow(c->beta2, (double)steps_));
    k.weight_decay = (T)c->weight_decay;
    adam_kernel<T><<<grid, 256, 0, stream_>>>(d_params_, d_flat_ + 1, d_m_, d_v_, k, clip, (long long)n_params_, skip,
                                              d_status_);
    return launched("adam_kernel");
}

template <typename T>
qb200_status Plan<T>::loss(void* host_scalar) {
    if (host_scalar == nullptr) return fail(QB200_INVALID, "loss needs a host scalar");
    std::lock_guard<std::recursive_mutex> lock(mutex_);
    QB_TRY(run(true));
    QB_CUDA(cudaMemcpyAsync(host_scalar, d_loss_only_, sizeof(T), cudaMemcpyDeviceToHost, stream_));
    QB_CUDA(cudaStreamSynchronize(stream_));
    return check_device_error();
}

template <typename T>
qb200_status Plan<T>::read_input(const char* name, void* host, size_t nbytes) {
    if (name == nullptr || host == nullptr) return fail(QB200_INVALID, "read_input needs a name and a host buffer");
    std::lock_guard<std::recursive_mutex> lock(mutex_);
    QB_TRY(use_device());
    const std::string key(name);
    const T* src = nullptr;
    size_t count = 0;
    if (key == kCotangentName) {
        src = d_ct_;
        count = 1;
    }
    for (size_t i = 0; i < desc_.params.size() && src == nullptr; ++i)
        if (desc_.params[i].name == key) {
            if (!leaves_[i].bound) return fail(QB200_NOT_BOUND, "parameter '%s' was never bound", name);
            src = d_params_ + leaves_[i].offset;
            count = leaves_[i].count;
        }
    for (size_t i = 0; i < desc_.inputs.size() && src == nullptr; ++i)
        if (desc_.inputs[i].name == key) {
            if (!inputs_[i].bound) return fail(QB200_NOT_BOUND, "input '%s' was never bound", name);
            src = inputs_[i].dev;
            count = (size_t)(desc_.inputs[i].rows * desc_.inputs[i].cols);
        }
    if (src == nullptr) return fail(QB200_INVALID, "the plan has no input named '%s'", name);
    if (nbytes != count * sizeof(T)) return fail(QB200_INVALID, "input '%s' has %zu bytes, got a buffer of %zu", name, count * sizeof(T), nbytes);
    QB_CUDA(cudaMemcpyAsync(host, src, nbytes, cudaMemcpyDeviceToHost, stream_));
    QB_CUDA(cudaStreamSynchronize(stream_));
    return check_device_error();
}

template <typename T>
qb200_status Plan<T>::read_moments(int which, void* host, size_t nbytes) {
    QB_TRY(use_device());
    if (which != 0 && which != 1) return fail(QB200_INVALID, "moment selector must be 0 or 1");
    if (nbytes != n_params_ * sizeof(T)) return fail(QB200_INVALID, "moments are %zu bytes, got a buffer of %zu", n_params_ * sizeof(T), nbytes);
    if (!moments_ready_) {
        memset(host, 0, nbytes);
        return QB200_OK;
    }
    QB_CUDA(cudaMemcpyAsync(host, which == 0 ? d_m_ : d_v_, nbytes, cudaMemcpyDeviceToHost, stream_));
    QB_CUDA(cudaStreamSynchronize(stream_));
    return QB200_OK;
}

template <typename T>
qb200_status Plan<T>::write_moments(int which, const void* host, size_t nbytes, int64_t step_count) {
    QB_TRY(use_device());
    if (which != 0 && which != 1) return fail(QB200_INVALID, "moment selector must be 0 or 1");
    if (nbytes != n_params_ * sizeof(T)) return fail(QB200_INVALID, "moments are %zu bytes, got a buffer of %zu", n_params_ * sizeof(T), nbytes);
    if (step_count < 0) return fail(QB200_INVALID, "step count must be nonnegative");
    if (!moments_ready_) {
        QB_TRY(dev_alloc(&d_m_, n_params_));
        QB_TRY(dev_alloc(&d_v_, n_params_));
        QB_CUDA(cudaMemsetAsync(d_m_, 0, n_params_ * sizeof(T), stream_));
        QB_CUDA(cudaMemsetAsync(d_v_, 0, n_params_ * sizeof(T), stream_));
        moments_ready_ = true;
    }
    QB_CUDA(cudaMemcpyAsync(which == 0 ? d_m_ : d_v_, host, nbytes, cudaMemcpyHostToDevice, stream_));
    QB_CUDA(cudaStreamSynchronize(stream_));
    steps_ = step_count;
    return QB200_OK;
}

template <typename T>
qb200_status Plan<T>::query(int key, int64_t* out) {
    if (out == nullptr) return fail(QB200_INVALID, "query needs an output");
    switch (key) {
        case QB200_Q_DEVICE_BUFFER_COUNT: *out = (int64_t)buffers_.size(); return QB200_OK;
        case QB200_Q_NONFINITE_CLIP_SEEN: {
            QB_TRY(use_device());
            double s[3];
            QB_CUDA(cudaMemcpyAsync(s, d_clip_, sizeof(s), cudaMemcpyDeviceToHost, stream_));
            QB_CUDA(cudaStreamSynchronize(stream_));
            *out = s[2] != 0.0;
            return QB200_OK;
        }
        case QB200_Q_STREAM: *out = (int64_t)(intptr_t)stream_; return QB200_OK;
        case QB200_Q_PARAMETER_COUNT: *out = (int64_t)n_params_; return QB200_OK;
        case QB200_Q_OUTPUT_COUNT: *out = (int64_t)leaves_.size() + 1; return QB200_OK;
        case QB200_Q_KERNEL_LAUNCHES: *out = launches_; return QB200_OK;
        case QB200_Q_FLAT_DEVICE_PTR: *out = (int64_t)(intptr_t)d_flat_; return QB200_OK;
        case QB200_Q_SCRATCH_BYTES: *out = (int64_t)scratch_bytes_; return QB200_OK;
        case QB200_Q_STEP_COUNT: *out = steps_; return QB200_OK;
        case QB200_Q_ENGINE: *out = fused_ ? (fused_tensor_core_ ? 2 : 1) : (tc_any_ ? 3 : 0); return QB200_OK;
        case QB200_Q_ALLREDUCE_NANOSECONDS: {
            if (!ev_ar_valid_) {
                *out = 0;  // no communicator attached, or no execute yet
                return QB200_OK;
            }
            float ms = 0.0f;
            QB_CUDA(cudaEventSynchronize(ev_ar1_));
            QB_CUDA(cudaEventElapsedTime(&ms, ev_ar0_, ev_ar1_));
            *out = (int64_t)((double)ms * 1e6);
            return QB200_OK;
        }
        case QB200_Q_GEMM_NANOSECONDS: {
            if (timer_used_ == 0) {
                *out = 0;
                return QB200_OK;
            }
            QB_TRY(use_device());
            QB_CUDA(cudaEventSynchronize(timer_events_[2 * timer_used_ - 1]));
            double total_ms = 0.0;
            for (size_t i = 0; i < timer_used_; ++i) {
                float ms = 0.0f;
                QB_CUDA(cudaEventElapsedTime(&ms, timer_events_[2 * i], timer_events_[2 * i + 1]));
                total_ms += ms;
            }
            *out = (int64_t)(total_ms * 1e6);
            return QB200_OK;
        }
        case QB200_Q_GEMM_LAUNCHES: *out = (int64_t)timer_used_; return QB200_OK;
        case QB200_Q_LANES: *out = (int64_t)std::max<size_t>(1, lanes_.size()); return QB200_OK;
        case QB200_Q_GEMM_FLOPS: *out = (int64_t)timer_flops_; return QB200_OK;
        case QB200_Q_GEMM_PIPE_FLOPS: *out = (int64_t)timer_pipe_flops_; return QB200_OK;
        case QB200_Q_SET0_NANOSECONDS: {
            if (!ev_valid_) return fail(QB200_INVALID, "no execute has run yet");
            QB_TRY(use_device());
            QB_CUDA(cudaEventSynchronize(ev_end_));
            float ms = 0.0f;
            QB_CUDA(cudaEventElapsedTime(&ms, ev_begin_, ev_end_));
            *out = (int64_t)(ms * 1e6);
            return QB200_OK;
        }
        default: return fail(QB200_INVALID, "unknown query key %d", key);
    }
}

template <typename T>
qb200_status Plan<T>::synchronize() {
    std::lock_guard<std::recursive_mutex> lock(mutex_);
    QB_TRY(use_device());
    QB_CUDA(cudaStreamSynchronize(stream_));
    return check_device_error();
}

template <typename T>
qb200_status Plan<T>::set_option(int key, int64_t value) {
    std::lock_guard<std::recursive_mutex> lock(mutex_);
    switch (key) {
        case QB200_OPT_KERNEL_TIMERS: timers_ = value != 0; return QB200_OK;
        case QB200_OPT_SINGLE_LANE: single_lane_ = value != 0; return QB200_OK;
        default: return fail(QB200_INVALID, "unknown option key %d", key);
    }
}

template <typename T>
qb200_status Plan<T>::inject_wait_timeout() {
    std::lock_guard<std::recursive_mutex> lock(mutex_);
    QB_TRY(use_device());
    const cudaError_t e = unarmed_wait_launch(d_error_, stream_);
    ++launches_;
    if (e != cudaSuccess) return fail(QB200_CUDA_ERROR, "launch of unarmed_wait_kernel failed: %s", cudaGetErrorString(e));
    return QB200_OK;
}

template <typename T>
qb200_status Plan<T>::attach_comm(const void* id, int rank, int world, int reduction) {
    if (id == nullptr) return fail(QB200_INVALID, "attach_comm needs the 128-byte NCCL id");
    if (world < 1 || rank < 0 || rank >= world) return fail(QB200_INVALID, "rank %d of world %d", rank, world);
    if (reduction != QB200_REDUCE_SUM && reduction != QB200_REDUCE_MEAN) return fail(QB200_INVALID, "reduction must be sum or mean");
    if (comm_ != nullptr) return fail(QB200_INVALID, "a communicator is already attached");
    const NcclApi* api = nccl_api();
    if (api == nullptr) return QB200_NCCL_ERROR;
    QB_TRY(use_device());
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof(uid));
    ncclResult_t r = api->CommInitRank(&comm_, world, uid, rank);
    if (r != ncclSuccess) {
        comm_ = nullptr;
        return fail(QB200_NCCL_ERROR, "ncclCommInitRank failed: %s", api->GetErrorString(r));
    }
    world_ = world;
    dp_scale_ = reduction == QB200_REDUCE_MEAN ? 1.0 / world : 1.0;
    return QB200_OK;
}

template <typename T>
qb200_status Plan<T>::detach_comm() {
    if (comm_ == nullptr) return QB200_OK;
    const NcclApi* api = nccl_api();
    if (api != nullptr) {
        use_device();
        cudaStreamSynchronize(stream_);
        // A clean detach destroys the communicator; a failed all-reduce has aborted and dropped it
        // already (all_reduce above; cuda.rs:132-145).
        api->CommDestroy(comm_);
    }
    comm_ = nullptr;
    world_ = 1;
    dp_scale_ = 1.0;
    return QB200_OK;
}

}  // namespace

qb200_status make_plan(const qb200_desc& desc, int device, qb200_plan** out) {
    QB_TRY(validate_desc(desc));
    qb200_status st;
    if (desc.dtype == QB200_F32) {
        auto* p = new Plan<float>(desc, device);
        st = p->init();
        if (st != QB200_OK) {
            delete p;
            return st;
        }
        *out = p;
    } else {
        auto* p = new Plan<double>(desc, device);
        st = p->init();
        if (st != QB200_OK) {
            delete p;
            return st;
        }
        *out = p;
    }
    return QB200_OK;
}

}  // namespace qb
