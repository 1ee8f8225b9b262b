// Per-point and per-parameter kernels: point-table gather, the residual
// program, the loss reduction, gradient finalisation, global-norm clipping and
// the flat optimizer update.
#pragma once
#include "jet_math.cuh"

namespace qb {

constexpr int MAX_REGS = 64;     // registers of a residual program
constexpr int MAX_INSTR = 1024;  // instructions of a residual program
constexpr int MAX_SETS = 16;     // point sets of a plan
constexpr int MAX_COLS = 16;     // columns of a point table

// Opcodes; numbering fixed by include/qb200.h (qb200_op).
enum : int {
    OP_CONST = 0, OP_COL, OP_JET, OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_NEG, OP_SIN, OP_COS, OP_EXP, OP_TANH,
    OP_POWI, OP_SQRT, OP_LOG, OP_LOG1P, OP_EXPM1, OP_ERF, OP_ERFC, OP_TAN
};

struct ProgramRef {
    const int4* code;    // {op, dst, a, b}
    const void* consts;  // plan dtype
    int n_instr;
    int value_reg;
    int grad_regs[MAX_STREAMS];
};

template <typename T> __device__ __forceinline__ T qb_sin(T x);
template <> __device__ __forceinline__ float qb_sin<float>(float x) { return sinf(x); }
template <> __device__ __forceinline__ double qb_sin<double>(double x) { return sin(x); }
template <typename T> __device__ __forceinline__ T qb_cos(T x);
template <> __device__ __forceinline__ float qb_cos<float>(float x) { return cosf(x); }
template <> __device__ __forceinline__ double qb_cos<double>(double x) { return cos(x); }
template <typename T> __device__ __forceinline__ T qb_exp(T x);
template <> __device__ __forceinline__ float qb_exp<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ double qb_exp<double>(double x) { return exp(x); }
template <typename T> __device__ __forceinline__ T qb_log(T x);
template <> __device__ __forceinline__ float qb_log<float>(float x) { return logf(x); }
template <> __device__ __forceinline__ double qb_log<double>(double x) { return log(x); }
template <typename T> __device__ __forceinline__ T qb_log1p(T x);
template <> __device__ __forceinline__ float qb_log1p<float>(float x) { return log1pf(x); }
template <> __device__ __forceinline__ double qb_log1p<double>(double x) { return log1p(x); }
template <typename T> __device__ __forceinline__ T qb_expm1(T x);
template <> __device__ __forceinline__ float qb_expm1<float>(float x) { return expm1f(x); }
template <> __device__ __forceinline__ double qb_expm1<double>(double x) { return expm1(x); }
template <typename T> __device__ __forceinline__ T qb_erf(T x);
template <> __device__ __forceinline__ float qb_erf<float>(float x) { return erff(x); }
template <> __device__ __forceinline__ double qb_erf<double>(double x) { return erf(x); }
template <typename T> __device__ __forceinline__ T qb_erfc(T x);
template <> __device__ __forceinline__ float qb_erfc<float>(float x) { return erfcf(x); }
template <> __device__ __forceinline__ double qb_erfc<double>(double x) { return erfc(x); }
template <typename T> __device__ __forceinline__ T qb_tan(T x);
template <> __device__ __forceinline__ float qb_tan<float>(float x) { return tanf(x); }
template <> __device__ __forceinline__ double qb_tan<double>(double x) { return tan(x); }
template <typename T> __device__ __forceinline__ T qb_sqrt(T x);
template <> __device__ __forceinline__ float qb_sqrt<float>(float x) { return sqrtf(x); }
template <> __device__ __forceinline__ double qb_sqrt<double>(double x) { return sqrt(x); }

// Integer power by repeated squaring, the rule of the reference's quabla_powi
// helper (crates/quabla-core/src/tensor_ir/cuda.rs:7894-7899).
template <typename T>
__device__ __forceinline__ T qb_powi(T x, int n) {
    const bool inv = n < 0;
    unsigned e = inv ? (unsigned)(-(long long)n) : (unsigned)n;
    T r = T(1);
    while (e) {
        if (e & 1u) r *= x;
        x *= x;
        e >>= 1;
    }
    return inv ? T(1) / r : r;
}

// Runs the register program of one point.  `cols` are the point's table
// columns, `jets[s * jet_stride]` the network output streams.
template <typename T>
__device__ __forceinline__ void run_program(const int4* code, int n_instr, const T* consts, const T* cols,
                                            const T* jets, long long jet_stride, T* r) {
    for (int pc = 0; pc < n_instr; ++pc) {
        const int4 in = code[pc];
        T v;
        switch (in.x) {
            case OP_CONST: v = consts[in.z]; break;
            case OP_COL: v = cols[in.z]; break;
            case OP_JET: v = jets[in.z * jet_stride]; break;
            case OP_ADD: v = r[in.z] + r[in.w]; break;
            case OP_SUB: v = r[in.z] - r[in.w]; break;
            case OP_MUL: v = r[in.z] * r[in.w]; break;
            case OP_DIV: v = r[in.z] / r[in.w]; break;
            case OP_NEG: v = -r[in.z]; break;
            case OP_SIN: v = qb_sin<T>(r[in.z]); break;
            case OP_COS: v = qb_cos<T>(r[in.z]); break;
            case OP_EXP: v = qb_exp<T>(r[in.z]); break;
            case OP_TANH: v = qb_tanh<T>(r[in.z]); break;
            case OP_POWI: v = qb_powi<T>(r[in.z], in.w); break;
            case OP_SQRT: v = qb_sqrt<T>(r[in.z]); break;
            case OP_LOG: v = qb_log<T>(r[in.z]); break;
            case OP_LOG1P: v = qb_log1p<T>(r[in.z]); break;
            case OP_EXPM1: v = qb_expm1<T>(r[in.z]); break;
            case OP_ERF: v = qb_erf<T>(r[in.z]); break;
            case OP_ERFC: v = qb_erfc<T>(r[in.z]); break;
            case OP_TAN: v = qb_tan<T>(r[in.z]); break;
            default: v = T(0); break;
        }
        r[in.y] = v;
    }
}

// Sum of one double per thread over a 256-thread block, fixed order.
__device__ __forceinline__ double block_sum_256(double v, double* smem /* [8] */) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    double total = 0.0;
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) total += smem[i];
    }
    return total;  // valid on thread 0
}

// Point table of a set: table[i][c] = input_c[i * stride_c + column_c].
struct GatherArgs {
    const void* src[MAX_COLS];
    int stride[MAX_COLS];
    int column[MAX_COLS];
    int ncols;
};
template <typename T>
__global__ void gather_table_kernel(GatherArgs a, T* __restrict__ table, long long n) {
    const long long total = n * a.ncols;
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total;
         e += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(e % a.ncols);
        const long long i = e / a.ncols;
        table[e] = static_cast<const T*>(a.src[c])[i * a.stride[c] + a.column[c]];
    }
}

// One thread per point of the chunk: e = program(point), block partial of e in
// double, and (unless forward only) the output-stream cotangents
//   Uhat[s][c] = cotangent * weight * extra * de/dU_s.
template <typename T>
__global__ void __launch_bounds__(256) residual_kernel(const T* __restrict__ table, int table_cols, long long point0,
                                                       int C, int S, const T* __restrict__ U, T* __restrict__ Uhat,
                                                       ProgramRef prog, const T* __restrict__ cotangent, T weight,
                                                       T extra, double* __restrict__ block_partials) {
    __shared__ int4 code[MAX_INSTR];
    __shared__ double red[8];
    for (int i = threadIdx.x; i < prog.n_instr; i += blockDim.x) code[i] = prog.code[i];
    __syncthreads();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    double e = 0.0;
    if (c < C) {
        T r[MAX_REGS];
        run_program<T>(code, prog.n_instr, static_cast<const T*>(prog.consts), table + (point0 + c) * table_cols,
                       U + c, C, r);
        e = (double)r[prog.value_reg];
        if (Uhat != nullptr) {
            const T seed = cotangent[0] * weight * extra;
            for (int s = 0; s < S; ++s) {
                const int reg = prog.grad_regs[s];
                Uhat[(long long)s * C + c] = reg >= 0 ? seed * r[reg] : T(0);
            }
        }
    }
    const double total = block_sum_256(e, red);
    if (threadIdx.x == 0) block_partials[blockIdx.x] = total;
}

// loss = sum over sets of round(weight_s * sum of that set's partials), added
// in set order in the plan dtype (each Mean is one node rounded to the plan
// dtype, then an Add: crates/quabla-core/src/tensor_ir.rs:2061-2063, 7794-7797).
struct LossArgs {
    int n_sets;
    int offset[MAX_SETS];
    int count[MAX_SETS];
    double weight[MAX_SETS];
};
// Weighted sum of the per-block loss partials of every point set, in a fixed order; whole block.
// `step` (may be null) closes a step: the device error flag that a bounded wait raises when it gives up
// is copied into the slot behind the gradients, so that one all-reduce tells every rank, and the
// optimizer kernels skip an update whose gradients are not to be trusted.
template <typename T>
struct StepStatus {
    const int* error;  // device flag of the plan
    T* flat_flag;      // slot behind the gradients in the flat [loss, gradients..., flag] buffer
    int* host_status;  // mapped host words: [0] a wait gave up, [1] optimizer updates skipped since the last report
};

template <typename T>
__device__ __forceinline__ void loss_finalize_block(const double* __restrict__ partials, const LossArgs& a, T extra,
                                                    T* __restrict__ out, double* red,
                                                    const StepStatus<T>* step = nullptr) {
    if (step != nullptr && threadIdx.x == 0) {
        const int e = *step->error;
        if (step->flat_flag != nullptr) step->flat_flag[0] = e != 0 ? T(1) : T(0);
        if (e != 0) step->host_status[0] = 1;
    }
    T loss = T(0);
    for (int s = 0; s < a.n_sets; ++s) {
        double v = 0.0;
        for (int i = threadIdx.x; i < a.count[s]; i += 256) v += partials[a.offset[s] + i];
        const double total = block_sum_256(v, red);
        if (threadIdx.x == 0) loss += (T)(total * a.weight[s]);
        __syncthreads();
    }
    if (threadIdx.x == 0) out[0] = loss * extra;
}

template <typename T>
__global__ void __launch_bounds__(256) loss_finalize_kernel(const double* __restrict__ partials, LossArgs a, T extra,
                                                            T* __restrict__ out, StepStatus<T> step) {
    __shared__ double red[8];
    loss_finalize_block<T>(partials, a, extra, out, red, &step);
}

// End of a step of the fused engines, one launch: grads[i] = sum over the per-CTA gradient rows of
// every point set (rows are consecutive, set after set) in double, in a fixed order, and the loss
// from the per-CTA partials.  Blocks 0 .. gridDim.x - 2 own 32 consecutive elements each; thread
// (x, y) sums the rows y, y + 8, ... of element x (coalesced along x), then the eight partial sums
// are added in y order.  The last block forms the loss.
template <typename T>
__global__ void __launch_bounds__(256) fused_finalize_kernel(const T* __restrict__ grad_rows, int P, int rows,
                                                             T* __restrict__ grads,
                                                             const double* __restrict__ partials, LossArgs a, T extra,
                                                             T* __restrict__ loss_out, StepStatus<T> step) {
    __shared__ double part[8][33];
    if (blockIdx.x == gridDim.x - 1) {
        loss_finalize_block<T>(partials, a, extra, loss_out, &part[0][0], &step);
        return;
    }
    const int x = threadIdx.x & 31, y = threadIdx.x >> 5;
    const int i = blockIdx.x * 32 + x;
    double s = 0.0;
    if (i < P) {
#pragma unroll 4
        for (int c = y; c < rows; c += 8) s += (double)grad_rows[(size_t)c * P + i];
    }
    part[y][x] = s;
    __syncthreads();
    if (y == 0 && i < P) {
        double total = part[0][x];
#pragma unroll
        for (int k = 1; k < 8; ++k) total += part[k][x];
        grads[i] = (T)total;
    }
}

template <typename T>
__global__ void finalize_gradients_kernel(const double* __restrict__ acc, const double* __restrict__ acc_b,
                                          T* __restrict__ grads, int count) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) grads[i] = (T)(acc_b != nullptr ? acc[i] + acc_b[i] : acc[i]);
}

// Round-to-nearest primitives without FMA contraction, so that the update is
// the reference's expression one rounded operation at a time
// (crates/quabla-core/src/tensor_ir/device_optimizer.rs:241-285).
template <typename T> struct Rn;
template <> struct Rn<float> {
    static __device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
    static __device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
    static __device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
    static __device__ __forceinline__ float div(float a, float b) { return __fdiv_rn(a, b); }
    static __device__ __forceinline__ float sqrt(float a) { return __fsqrt_rn(a); }
};
template <> struct Rn<double> {
    static __device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }
    static __device__ __forceinline__ double sub(double a, double b) { return __dsub_rn(a, b); }
    static __device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
    static __device__ __forceinline__ double div(double a, double b) { return __ddiv_rn(a, b); }
    static __device__ __forceinline__ double sqrt(double a) { return __dsqrt_rn(a); }
};

template <typename T>
struct AdamCoeffs {
    T learning_rate, beta1, beta2, one_minus_beta1, one_minus_beta2, epsilon, correction1, correction2, weight_decay;
};

// m' = m*b1 + g*(1-b1); v' = v*b2 + (g*g)*(1-b2);
// d = (m'/c1) / (sqrt(v'/c2) + eps); if wd != 0: d += wd*p; p' = p - d*lr.
// clip_scalars (may be null): [peak, factor, sticky flag]; the gradient is
// scaled in double and rounded once (cuda_optimizer.rs:150-163).
// skip (may be null): the flag slot of the flat gradient buffer; non-zero means that some rank's
// step raised the device error flag, and the update is left out on every rank alike.
template <typename T>
__device__ __forceinline__ bool update_skipped(const T* __restrict__ skip, int* __restrict__ host_status) {
    if (skip == nullptr || skip[0] == T(0)) return false;
    if (blockIdx.x == 0 && threadIdx.x == 0 && host_status != nullptr) host_status[1] += 1;  // updates skipped since the last report
    return true;
}

template <typename T>
__global__ void adam_kernel(T* __restrict__ p, const T* __restrict__ g, T* __restrict__ m, T* __restrict__ v,
                            AdamCoeffs<T> k, const double* __restrict__ clip_scalars, long long count,
                            const T* __restrict__ skip = nullptr, int* __restrict__ host_status = nullptr) {
    typedef Rn<T> R;
    if (update_skipped(skip, host_status)) return;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
         i += (long long)gridDim.x * blockDim.x) {
        T grad = g[i];
        if (clip_scalars != nullptr) grad = (T)((double)grad * clip_scalars[1]);
        const T param = p[i];
        const T first = R::add(R::mul(m[i], k.beta1), R::mul(grad, k.one_minus_beta1));
        const T second = R::add(R::mul(v[i], k.beta2), R::mul(R::mul(grad, grad), k.one_minus_beta2));
        const T numerator = R::div(first, k.correction1);
        const T denominator = R::add(R::sqrt(R::div(second, k.correction2)), k.epsilon);
        T delta = R::div(numerator, denominator);
        if (k.weight_decay != T(0)) delta = R::add(delta, R::mul(k.weight_decay, param));
        p[i] = R::sub(param, R::mul(delta, k.learning_rate));
        m[i] = first;
        v[i] = second;
    }
}

template <typename T>
__global__ void sgd_kernel(T* __restrict__ p, const T* __restrict__ g, T learning_rate,
                           const double* __restrict__ clip_scalars, long long count,
                           const T* __restrict__ skip = nullptr, int* __restrict__ host_status = nullptr) {
    typedef Rn<T> R;
    if (update_skipped(skip, host_status)) return;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
         i += (long long)gridDim.x * blockDim.x) {
        T grad = g[i];
        if (clip_scalars != nullptr) grad = (T)((double)grad * clip_scalars[1]);
        p[i] = R::sub(p[i], R::mul(grad, learning_rate));
    }
}

// Global L2 norm of the flat gradient as m * sqrt(sum((g/m)^2)) with m the
// largest |g|, in double; writes scalars = [peak, clip factor, sticky
// non-finite flag] (python/quabla/optim.py:83-123, cuda_optimizer.rs:39-109).
// One block: the flat gradient is at most a few hundred thousand elements.
template <typename T>
__global__ void __launch_bounds__(1024) global_norm_kernel(const T* __restrict__ g, long long count, double max_norm,
                                                           double* __restrict__ scalars,
                                                           const T* __restrict__ skip = nullptr) {
    __shared__ double red[1024];
    __shared__ int any_nan;
    if (skip != nullptr && skip[0] != T(0)) return;  // the update is skipped: leave the sticky flag alone
    if (threadIdx.x == 0) any_nan = 0;
    __syncthreads();
    double peak = 0.0;
    bool nan_seen = false;
    for (long long i = threadIdx.x; i < count; i += 1024) {
        const double a = fabs((double)g[i]);
        if (a != a) nan_seen = true;
        peak = fmax(peak, a);  // fmax drops NaN; tracked separately
    }
    if (nan_seen) atomicOr(&any_nan, 1);
    red[threadIdx.x] = peak;
    __syncthreads();
    for (int o = 512; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] = fmax(red[threadIdx.x], red[threadIdx.x + o]);
        __syncthreads();
    }
    peak = any_nan ? nan("") : red[0];
    __syncthreads();
    const double scale = (isfinite(peak) && peak > 0.0) ? peak : 1.0;
    double sum = 0.0;
    for (long long i = threadIdx.x; i < count; i += 1024) {
        const double q = (double)g[i] / scale;
        sum += q * q;
    }
    red[threadIdx.x] = sum;
    __syncthreads();
    for (int o = 512; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const double root = sqrt(red[0]);
        const double norm = scale * root;
        double factor;
        if (norm <= max_norm) {
            factor = 1.0;
        } else if (isfinite(norm)) {
            factor = max_norm / norm;
        } else if (isfinite(peak)) {
            factor = (max_norm / scale) / root;
        } else {
            factor = nan("");
        }
        scalars[0] = peak;
        scalars[1] = factor;
        // Sticky: set by a NaN or infinite gradient entry (then root is not finite either), not by a
        // norm that merely overflowed while peak and root stayed finite (cuda_optimizer.rs:98-103).
        if (!(isfinite(peak) && isfinite(root))) scalars[2] = 1.0;
    }
}

// ---------------------------------------------------------------------------
// Device-side resampling of a collocation column with the reference's generator, so that a
// training loop can draw a fresh batch without a host copy.  Element i of the column is
//   clip(round_to_dtype(minval + width * ((splitmix64_output(key, i) >> 11) / 2^53)), low, high),
// the arithmetic of random_uniform (crates/quabla-python/src/tensor.rs:1482-1534) on the i-th
// output of the SplitMix64 stream seeded by key (tensor.rs:327-333): state = key + (i + 1) * gamma,
// then the two multiply-xorshift rounds.  The stream is counter-based, so every element is
// independent; multiply and add are kept separate (no FMA) as on the host.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void sample_uniform_kernel(T* __restrict__ column, long long rows, int stride, unsigned long long key,
                                      double minval, double width, double low, double high) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < rows; i += (long long)gridDim.x * blockDim.x) {
        unsigned long long z = key + (unsigned long long)(i + 1) * 0x9e3779b97f4a7c15ull;
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
        z = z ^ (z >> 31);
        const double unit = (double)(z >> 11) * (1.0 / 9007199254740992.0);  // exact: 53 bits, power-of-two scale
        double value = __dadd_rn(minval, __dmul_rn(width, unit));
        if (sizeof(T) == 4) value = (double)(float)value;  // one rounding to float32, as astype does
        value = fmin(fmax(value, low), high);
        column[i * stride] = (T)value;
    }
}

}  // namespace qb
