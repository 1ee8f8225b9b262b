/*
 * qb200 — C ABI of the B200-native backend for Quabla's PINN training step.
 *
 * The reference (latteine1217/quabla) has no C ABI: its CUDA backend is a Rust
 * module (crates/quabla-core/src/tensor_ir/cuda.rs) selected by
 * compiler::lower (crates/quabla-core/src/compiler.rs:483-499).  Every entry
 * point below names the reference method it stands in for, so that a Rust
 * `extern "C"` block (or the ctypes binding in quabla_b200/_lib.py) can bind
 * it where the reference calls that method today.
 *
 * Conventions
 *  - plain pointers and sizes only; all functions return a qb200_status;
 *  - every failing call leaves a message readable with qb200_last_error()
 *    (the reference returns Result<_, String>);
 *  - validation errors precede any device work
 *    (cuda_optimizer.rs:207-212, cuda.rs:3349-3368);
 *  - a plan owns all of its device memory (parameters, optimizer moments,
 *    saved activations); host buffers are copied, never aliased;
 *  - one CUDA stream per plan (QB200_Q_STREAM) carries every kernel of a step; plans with several
 *    point sets on the fused engines also own a lower-priority side stream on which the small
 *    sets' kernels run between a fork and a join event of the main stream, so work enqueued on
 *    the main stream after a step is still ordered after all of it;
 *  - calls on one plan are serialised by a per-plan mutex (the reference keeps its plan state
 *    behind one, cuda.rs:86);
 *  - there is no CPU fallback: a description the backend does not recognise
 *    returns QB200_UNSUPPORTED (docs/guide/13-architecture.md:392-393,
 *    "no silent fallback").
 */
#ifndef QB200_H
#define QB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum qb200_status {
    QB200_OK = 0,
    QB200_INVALID = 1,      /* bad argument, failed validation */
    QB200_UNSUPPORTED = 2,  /* outside the recognised PINN family */
    QB200_CUDA_ERROR = 3,   /* a CUDA runtime call failed */
    QB200_NCCL_ERROR = 4,   /* NCCL missing or a collective failed */
    QB200_NOT_BOUND = 5,    /* execute before every input was bound */
    QB200_TOO_LARGE = 6     /* a fixed-capacity entry point was given too much */
} qb200_status;

/* One floating dtype per plan; mixed programs are rejected
 * (cuda.rs:998-1030, cuda_real.rs:151-210). */
typedef enum qb200_dtype { QB200_F32 = 0, QB200_F64 = 1 } qb200_dtype;

typedef enum qb200_param_kind { QB200_WEIGHT = 0, QB200_BIAS = 1 } qb200_param_kind;

/* Update rule of the device optimizer (device_optimizer.rs:17-34). */
typedef enum qb200_rule { QB200_SGD = 0, QB200_ADAM = 1 } qb200_rule;

/* DeviceOptimizerConfig (device_optimizer.rs:37-45); validated with the rules of
 * device_optimizer.rs:65-95: learning_rate finite and >= 0 (zero is valid),
 * betas in [0,1), epsilon > 0, weight_decay >= 0, clip_norm > 0 when has_clip. */
typedef struct qb200_opt_config {
    int32_t rule;          /* qb200_rule */
    int32_t has_clip;      /* 0: no global-norm clipping */
    double learning_rate;
    double beta1;
    double beta2;
    double epsilon;
    double weight_decay;   /* non-zero selects AdamW's decoupled decay */
    double clip_norm;
} qb200_opt_config;

/* Reduction of a data-parallel step (cuda.rs:786-789: ncclSum / ncclAvg). */
typedef enum qb200_reduction { QB200_REDUCE_SUM = 0, QB200_REDUCE_MEAN = 1 } qb200_reduction;

/* CudaDataParallelTiming (cuda.rs:154-170), host wall clock in seconds. */
typedef struct qb200_dp_timing {
    double replica_enqueue;
    double collective;
    double output_readback;
} qb200_dp_timing;

/* Keys of qb200_plan_query. */
typedef enum qb200_query {
    QB200_Q_DEVICE_BUFFER_COUNT = 0, /* CudaExecutionPlan::device_buffer_count, cuda.rs:1146-1173 */
    QB200_Q_NONFINITE_CLIP_SEEN = 1, /* nonfinite_clip_seen, cuda_optimizer.rs:405-420 */
    QB200_Q_STREAM = 2,              /* the plan's cudaStream_t, for event timing by the caller */
    QB200_Q_PARAMETER_COUNT = 3,     /* elements of the flat parameter buffer (leaves padded to 4 elements) */
    QB200_Q_OUTPUT_COUNT = 4,        /* 1 (loss) + number of parameter leaves */
    QB200_Q_KERNEL_LAUNCHES = 5,     /* kernels of this library launched by the plan so far */
    QB200_Q_FLAT_DEVICE_PTR = 6,     /* device address of the flat [loss, gradients...] buffer */
    QB200_Q_SCRATCH_BYTES = 7,       /* bytes of saved-jet scratch the plan holds */
    QB200_Q_STEP_COUNT = 8,          /* optimizer updates applied so far */
    QB200_Q_ENGINE = 9,              /* 0: layer-wise (FP pipe), 1: fused (FP32 pipe), 2: fused (mma 3xTF32), 3: layer-wise with tcgen05 GEMMs */
    QB200_Q_SET0_NANOSECONDS = 10,   /* device time of the last execute's kernels for point set 0 (events) */
    QB200_Q_ALLREDUCE_NANOSECONDS = 11, /* device time of the last execute's gradient all-reduce, waits for peers included */
    QB200_Q_GEMM_NANOSECONDS = 12,   /* with QB200_OPT_KERNEL_TIMERS: summed device time of the last execute's layer GEMM launches
                                        (tcgen05 / FP64-MMA / SIMT products of the layer-wise engine; 0 on the fused engines) */
    QB200_Q_GEMM_LAUNCHES = 13,      /* ... how many launches that sum covers */
    QB200_Q_GEMM_FLOPS = 14,         /* ... and their 2*M*N*K in total */
    QB200_Q_LANES = 15,              /* streams over which the layer-wise engine spreads consecutive chunks (1 or 2) */
    QB200_Q_GEMM_PIPE_FLOPS = 16     /* ... the tensor-pipe work of those launches in FLOPs at the bfloat16 rate: 2*M*N*K times 6 where the
                                        three products of an element are tf32 instructions (tf32 runs at half the bfloat16 rate), times 4
                                        where the two correction products are bfloat16 instructions; 0 for float64 and SIMT launches */
} qb200_query;

/* Keys of qb200_plan_set_option. */
typedef enum qb200_option {
    QB200_OPT_KERNEL_TIMERS = 0,     /* non-zero: record a CUDA event pair around every layer GEMM launch */
    QB200_OPT_SINGLE_LANE = 1        /* non-zero: every chunk on the plan's main stream, so that kernels do not overlap
                                        and the event pairs of QB200_OPT_KERNEL_TIMERS time one kernel each */
} qb200_option;

/* Opcodes of the per-point residual program (see qb200_desc_set_program). */
typedef enum qb200_op {
    QB200_OP_CONST = 0, /* r[dst] = consts[a] */
    QB200_OP_COL = 1,   /* r[dst] = column a of the point (coordinates first, then aux) */
    QB200_OP_JET = 2,   /* r[dst] = network output stream a (0 = u, then the derivative streams) */
    QB200_OP_ADD = 3,
    QB200_OP_SUB = 4,
    QB200_OP_MUL = 5,
    QB200_OP_DIV = 6,
    QB200_OP_NEG = 7,
    QB200_OP_SIN = 8,
    QB200_OP_COS = 9,
    QB200_OP_EXP = 10,
    QB200_OP_TANH = 11,
    QB200_OP_POWI = 12, /* r[dst] = r[a] ** b, b an integer literal */
    QB200_OP_SQRT = 13,
    QB200_OP_LOG = 14,
    QB200_OP_LOG1P = 15, /* UnaryMath kinds of the reference (elementwise.rs:400-450) */
    QB200_OP_EXPM1 = 16,
    QB200_OP_ERF = 17,
    QB200_OP_ERFC = 18,
    QB200_OP_TAN = 19
} qb200_op;

typedef struct qb200_desc qb200_desc;
typedef struct qb200_plan qb200_plan;
typedef struct qb200_dp qb200_dp;

/* Message of the last failing call on this thread. */
const char* qb200_last_error(void);
/* Library version string. */
const char* qb200_version(void);
/* Number of visible CUDA devices (0 when the driver is absent). */
int32_t qb200_device_count(void);

/* ------------------------------------------------------------------------
 * Plan description: what the reference hands its backend as a frozen
 * TensorExecutionPlan (CudaBackend::compile(plan), cuda.rs:464-481), restated
 * as the structure the fusion pass recognises in a PINN value-and-gradient
 * plan: a tanh MLP, the parameter leaves in gradient-output order, the data
 * inputs, and per point set the derivative streams and the residual program.
 * ------------------------------------------------------------------------ */
qb200_status qb200_desc_create(int32_t dtype, qb200_desc** out);
void qb200_desc_destroy(qb200_desc* desc);

/* sizes[0] = input width, sizes[n-1] = 1; hidden layers are Linear+tanh
 * (a1/a2: tensor_ir.rs:4968-4972, elementwise.rs:400-407), the last is Linear. */
qb200_status qb200_desc_set_network(qb200_desc* desc, const int32_t* sizes, int32_t n_sizes);

/* Activation of the hidden layers: tanh (the default), sin, or one of the reference's composites: sigmoid and
 * softplus (crates/quabla-python/src/composite.rs:178-209), silu = x sigmoid(x) and the tanh-approximated gelu
 * written through sigmoid (python/quabla/_ops.py:475-505); derivative chains of elementwise.rs:400-468.  The jets
 * of every activation are composed to the order the derivative signature needs (up to 4, plus one for the
 * reverse sweep).  tanh and sin networks use every engine; the composite activations run on the layer-wise
 * engine. */
typedef enum {
    QB200_ACT_TANH = 0,
    QB200_ACT_SIN = 1,
    QB200_ACT_SIGMOID = 2,
    QB200_ACT_SOFTPLUS = 3,
    QB200_ACT_SILU = 4,
    QB200_ACT_GELU = 5
} qb200_activation;
qb200_status qb200_desc_set_activation(qb200_desc* desc, int32_t activation);

/* A parameter leaf, named as the reference names inputs (pytree path,
 * _transforms.py:363-377).  Gradient outputs follow the order of these calls
 * (tensor_trace.rs:4562-4573).  layer counts from 0; a weight is
 * [sizes[layer], sizes[layer+1]] row-major, a bias [sizes[layer+1]]. */
qb200_status qb200_desc_add_parameter(qb200_desc* desc, const char* name, int32_t layer, int32_t kind);

/* A data input [rows, cols] row-major in the plan dtype.  retained != 0: bound
 * once and kept on the device (cuda.rs:1928-1930); otherwise re-uploaded by
 * every qb200_plan_bind (per-step batch, cuda.rs:1902-1934). */
qb200_status qb200_desc_add_input(qb200_desc* desc, const char* name, int64_t rows, int64_t cols,
                                  int32_t retained, int32_t* out_index);

/* A point set contributes  weight * sum_i e(point_i)  to the loss (a `Mean`
 * is weight = 1/n_points, a11/a12: tensor_ir.rs:2061-2063, op/vjp.rs:292-298). */
qb200_status qb200_desc_add_set(qb200_desc* desc, int64_t n_points, double weight, int32_t* out_set);
/* Next column of the set's point table: the first sizes[0] are the network's
 * inputs, later ones are auxiliary per-point data (forcing, targets). */
qb200_status qb200_desc_set_add_column(qb200_desc* desc, int32_t set, int32_t input_index, int32_t column);
/* A derivative direction v (length sizes[0]) carried to `order` (1..4): adds
 * `order` streams d^m u / dv^m after the streams declared so far. */
qb200_status qb200_desc_set_add_direction(qb200_desc* desc, int32_t set, const double* vec, int32_t order);
/* Declares one more stream after all directions' streams: M = sum_j weights[j] * d^2 u / dv_j^2 over
 * the set's directions (n_weights = number of directions declared; 0 leaves a direction out).  The
 * directions themselves then need first order only: the kernels carry M through every layer as
 *   M_out = f'(z) M_in + f''(z) sum_j weights[j] (dz/dv_j)^2,
 * the forward-Laplacian recurrence, instead of one second-order stream per direction.  For a residual
 * that uses the second derivatives only through that sum (u_xx + u_yy, a heat or wave operator) this
 * is the reference's value and gradient (hessian + trace, python/quabla/_transforms.py:1780-1995)
 * with fewer streams.  Call after the last add_direction and before set_program; the program
 * addresses M as the last stream. */
qb200_status qb200_desc_set_merge_second_order(qb200_desc* desc, int32_t set, const double* weights, int32_t n_weights);
/* Register program evaluated once per point: code is n_instr x {op, dst, a, b}.
 * value_reg holds e; grad_regs[s] holds de/d(stream s) or is -1 when zero. */
qb200_status qb200_desc_set_program(qb200_desc* desc, int32_t set, const int32_t* code, int32_t n_instr,
                                    const double* consts, int32_t n_consts, int32_t n_regs,
                                    int32_t value_reg, const int32_t* grad_regs, int32_t n_grad_regs);

/* ------------------------------------------------------------------------
 * Single-device plan: CudaExecutionPlan<T> (cuda.rs:76-96).
 * ------------------------------------------------------------------------ */
/* CudaBackend::compile / compile_float64 (cuda.rs:464-481). */
qb200_status qb200_plan_create(const qb200_desc* desc, int32_t device_ordinal, qb200_plan** out);
void qb200_plan_destroy(qb200_plan* plan);

/* Upload a named input (parameter, data, or "__quabla_loss_cotangent",
 * tensor_trace.rs:5365-5378) from host memory; nbytes must match exactly
 * (input validation of execute_many, cuda.rs:1190-1220, 1699-1721). */
qb200_status qb200_plan_bind(qb200_plan* plan, const char* name, const void* host, size_t nbytes);

/* execute_retaining_without_output (cuda.rs:1233-1240): forward, residual,
 * reverse pass; leaves [loss, gradients...] on the device (all-reduced when a
 * communicator is attached). */
qb200_status qb200_plan_execute(qb200_plan* plan);

/* One output of execute_many in program order: index 0 is the loss, 1.. are
 * the gradients in parameter order (cuda.rs:1190-1220, 2961-2971). */
qb200_status qb200_plan_read_output(qb200_plan* plan, int32_t index, void* host, size_t nbytes);

/* optimizer_step (cuda_optimizer.rs:207-398) with the element rule of
 * device_optimizer.rs:241-285, bias corrections formed in double on the host
 * and rounded once to the plan dtype (cuda_optimizer.rs:340-359). */
qb200_status qb200_plan_optimizer_step(qb200_plan* plan, const qb200_opt_config* config);

/* execute_primary_retaining (cuda.rs:1245-1314): loss at the current
 * parameters, forward only; host_scalar receives one element of the plan dtype. */
qb200_status qb200_plan_loss(qb200_plan* plan, void* host_scalar);

/* retained_input_to_host (cuda.rs:1451-1489). */
qb200_status qb200_plan_read_input(qb200_plan* plan, const char* name, void* host, size_t nbytes);

/* Resamples column `column` of the data input `name` on the device, without a host copy:
 * element i becomes the i-th value of random_uniform([rows], key, minval, maxval, plan dtype)
 * (crates/quabla-python/src/tensor.rs:1482-1534 on the SplitMix64 stream of tensor.rs:327-333;
 * python/quabla/random.py:119-129), bit for bit.  Stands where a training loop re-draws its
 * collocation batch on the host and uploads it (batch_argnums of optim.Trainer,
 * python/quabla/optim.py:458-487).  Counts as binding the input; other columns keep their
 * values (zero if the input was never bound). */
qb200_status qb200_plan_sample_uniform(qb200_plan* plan, const char* name, int32_t column, uint64_t key,
                                       double minval, double maxval);

/* Optimizer moments, which the reference keeps private to the device trainer:
 * which = 0 first moment, 1 second moment; all leaves flat in parameter order, every leaf starting on
 * a 4-element boundary (QB200_Q_PARAMETER_COUNT elements in all; the padding is zero). */
qb200_status qb200_plan_read_moments(qb200_plan* plan, int32_t which, void* host, size_t nbytes);
qb200_status qb200_plan_write_moments(qb200_plan* plan, int32_t which, const void* host, size_t nbytes,
                                      int64_t step_count);

qb200_status qb200_plan_query(qb200_plan* plan, int32_t key, int64_t* out);
/* Measurement switches (qb200_option); no counterpart in the reference, whose timing is host wall clock
 * (CudaDataParallelTiming, cuda.rs:154-170). */
qb200_status qb200_plan_set_option(qb200_plan* plan, int32_t key, int64_t value);
/* CudaExecutionPlan::synchronize (cuda.rs:1174-1180).  Like every call that waits for the stream
 * (read_output, read_input, loss) it returns QB200_CUDA_ERROR when a bounded wait inside a kernel
 * gave up during a step since the last report; the optimizer update of such a step is skipped on
 * the device (on every rank of a data-parallel run: the flag travels with the gradient all-reduce),
 * so parameters and moments never absorb invalid gradients. */
qb200_status qb200_plan_synchronize(qb200_plan* plan);
/* Test seam for that error path: enqueues one thread's short bounded wait on a barrier that nothing
 * completes; the wait gives up and raises the plan's device error flag exactly as a staged copy that
 * never lands would.  Nothing faults, traps or spins for long.  The reference reaches the same state
 * only through a failing CUDA call (cuda.rs:1386-1447 propagates the driver error). */
qb200_status qb200_plan_inject_wait_timeout(qb200_plan* plan);

/* Multi-process data parallelism (one process per GPU): rank 0 obtains an id,
 * the caller ships the 128 bytes to the other ranks, every rank attaches.
 * After that qb200_plan_execute ends with ONE all-reduce of the flat
 * [loss, gradients...] buffer (replaces the per-output collectives of
 * cuda.rs:780-814).  reduction MEAN pre-scales the local cotangent by 1/world
 * (tensor_ir.rs:11683-11706). */
qb200_status qb200_nccl_unique_id(void* out_128_bytes);
qb200_status qb200_plan_attach_comm(qb200_plan* plan, const void* id_128_bytes, int32_t rank,
                                    int32_t world, int32_t reduction);
/* Drops (aborts) the communicator; the failure contract of cuda.rs:132-145, 699-716. */
qb200_status qb200_plan_detach_comm(qb200_plan* plan);

/* ------------------------------------------------------------------------
 * Single-process data-parallel plan: CudaDataParallelExecutionPlan
 * (cuda.rs:116-170, 381-445, 621-866).  One host thread drives all replicas;
 * set descriptions carry the per-replica (shard) point counts, as the
 * reference traces the loss at shard shape (tensor_trace.rs:4688-4710).
 * ------------------------------------------------------------------------ */
/* compile_data_parallel (cuda.rs:388-406); requirements of cuda.rs:1033-1068
 * except that n = 1 is allowed. */
qb200_status qb200_dp_create(const qb200_desc* shard_desc, const int32_t* ordinals, int32_t n,
                             qb200_dp** out);
void qb200_dp_destroy(qb200_dp* dp);
/* Axis-0 equal shards in rank order (tensor_trace.rs:4772-4775): host holds
 * n * shard rows. */
qb200_status qb200_dp_bind_sharded(qb200_dp* dp, const char* name, const void* host, size_t nbytes);
/* The same host buffer to every replica (parameters, cotangent). */
qb200_status qb200_dp_bind_replicated(qb200_dp* dp, const char* name, const void* host, size_t nbytes);
/* execute_replicas (cuda.rs:642-665, 721-760): enqueue every replica, one
 * grouped all-reduce, synchronise.  A failure aborts the communicators and the
 * next call recreates them (cuda.rs:699-716). */
qb200_status qb200_dp_step(qb200_dp* dp, int32_t reduction, qb200_dp_timing* timing);
/* Outputs are read from rank 0 (cuda.rs:741-749). */
qb200_status qb200_dp_read_output(qb200_dp* dp, int32_t index, void* host, size_t nbytes);
/* The same optimizer step on every replica from the reduced gradients. */
qb200_status qb200_dp_optimizer_step(qb200_dp* dp, const qb200_opt_config* config);
/* The replica plan of a rank, for reads and queries; owned by dp. */
qb200_plan* qb200_dp_replica(qb200_dp* dp, int32_t rank);
int32_t qb200_dp_replica_count(const qb200_dp* dp);
/* Test seam for the failure contract: the next qb200_dp_step fails on the host,
 * after replica `rank - 1` was enqueued and before `rank`, as a missing input
 * does in the reference's tests (crates/quabla-core/tests/tensor_ir.rs:5127-5145). */
qb200_status qb200_dp_inject_host_failure(qb200_dp* dp, int32_t rank);

/* ------------------------------------------------------------------------
 * Stand-alone device optimizer over caller-owned device arrays, the kernels of
 * cuda_optimizer.rs:126-165 (quabla_device_adam / quabla_device_sgd) as one
 * launch over a flat buffer.  `step` counts updates from 1.
 * ------------------------------------------------------------------------ */
qb200_status qb200_optimizer_apply(int32_t dtype, void* d_param, const void* d_grad, void* d_m, void* d_v,
                                   int64_t count, const qb200_opt_config* config, int64_t step,
                                   void* cuda_stream);

/* ------------------------------------------------------------------------
 * Stand-alone batch-reduced weight gradient over caller-owned device arrays:
 *   grad[d_in][d_out] = sum over rows of acts[row][d_in]^T cots[row][d_out],
 * the contraction the reference reaches as a materialised [B, in, out] product
 * followed by a sum over the batch axis (op/vjp.rs:176-209,
 * tensor_ir.rs:9324-9353, cuda.rs:8202-8247).  Rows are summed in the array
 * dtype per slice of 4096 rows, the slices then in double in ascending order,
 * so the result is bit-reproducible.  Allocates its split scratch from the
 * stream-ordered pool for the duration of the call.
 * ------------------------------------------------------------------------ */
qb200_status qb200_weight_gradient(int32_t dtype, const void* d_acts, const void* d_cots, int64_t rows,
                                   int32_t d_in, int32_t d_out, void* d_grad, void* cuda_stream);

/* ------------------------------------------------------------------------
 * Stand-alone float32 matrix product on the tensor cores (tcgen05, split operands):
 *   C[M][N] = A[M][K] * W[K][N]  (+ bias[N] on the first bias_rows rows),
 * the layer contraction h @ W (+ b) of the hot path (a1/a2: tensor_ir.rs:4968-4972,
 * op/batch.rs:58-79) for all streams at once.  N % 64 == 0, 64 <= N <= 256,
 * K % 32 == 0, all arrays row-major float32 on the device.  Synchronises the stream.
 * Each element is split as x = hi + lo.  M >= 65536: hi = x rounded to tf32, hi.hi runs
 * as tf32 instructions and the two correction products lo.x and x.lo as bfloat16
 * instructions; error against a float64 product, K = 64..256: 7e-7 relative rms, random.
 * M < 65536: hi = x truncated to tf32 and all three products as tf32 instructions: 2e-7,
 * most of it a common scale factor (a float32 FMA product: 1.5e-7 to 3e-7).
 * QB200_TC_COR=tf32 or =bf16 in the environment forces one scheme for every M.
 * ------------------------------------------------------------------------ */
qb200_status qb200_matmul_3xtf32(const void* d_a, const void* d_w, const void* d_bias, void* d_c, int64_t M,
                                 int32_t N, int32_t K, int64_t bias_rows, void* cuda_stream);

/* ------------------------------------------------------------------------
 * qb200_weight_gradient for callers that cannot allocate device memory.
 * No counterpart in the reference: its backend allocates freely from a pool.
 *
 * Meant for hosts where device allocation is not available at call time: a
 * plugin inside a runtime that owns the memory pool, a latency-bound loop that
 * may not take the allocator lock, a process that has already handed every
 * free byte to something else.  Same arguments and, for every shape, the same
 * result bit for bit as qb200_weight_gradient: both entry points run one
 * shared dispatch (tcgen05 contraction for float32 with d_in % 128 == 0 and
 * d_out % 64 == 0, d_out <= 256; FP64 tensor-core or plain kernel otherwise)
 * on the same split.  The split scratch is a 16 MiB array built into the
 * library (held on every GPU that loads the library until the process exits)
 * and no cudaMalloc/cudaFree or other allocating call is made.
 *
 *  - Limit: ceil(rows / 4096) * d_in * d_out * sizeof(element), rounded up to
 *    16 bytes, + 16 bytes <= 16 MiB, otherwise QB200_TOO_LARGE and nothing is
 *    launched.  (Both entry points also refuse more than 65535 slices, that is
 *    rows > 268,431,360, with QB200_TOO_LARGE.)
 *  - The first call on each device looks up the array's device address (with
 *    that device current); make that first call before starting any stream
 *    capture.
 *  - All calls on a device share the one array: two calls whose kernels can
 *    overlap on the GPU (different streams, no ordering) race; order them.
 *    The array keeps the previous call's contents, which this function never
 *    reads.
 * ------------------------------------------------------------------------ */
qb200_status qb200_weight_gradient_static(int32_t dtype, const void* d_acts, const void* d_cots, int64_t rows,
                                          int32_t d_in, int32_t d_out, void* d_grad, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* QB200_H */
