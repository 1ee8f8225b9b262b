/*
 * TEST INFRASTRUCTURE — CPU oracle, "contracted" form.  Not part of the
 * product: only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline
 * legs may build, load or call this file.
 *
 * What it restates.  The reference evaluates a PINN loss and its parameter
 * gradients by running the traced value-and-gradient plan on its CPU
 * interpreter, in float64, node by node
 * (crates/quabla-core/src/tensor_ir.rs:7107-7818: f64 compute, :1639-1656
 * matmul with f64 accumulation in increasing k, :1838-1840 sequential sums,
 * :2061-2063 mean = sum * (1/n)).  In exact arithmetic that plan computes, per
 * collocation point, the network output and its input derivatives
 * (reverse-over-reverse `grad(grad(u))` or forward-over-reverse `hessian`,
 * python/quabla/_transforms.py:825-950, 1812-2036, 2173-2179), the residual, the
 * mean of its square, and the derivative of that scalar with respect to every
 * weight (matmul VJP: crates/quabla-core/src/tensor_ir/op/vjp.rs:176-209, tanh
 * chain rule: elementwise.rs:416-468).
 *
 * This file computes the same quantities in float64 with the derivative
 * streams carried forward as Taylor jets and one reverse sweep, and with the
 * weight gradients contracted over the batch on the fly instead of being
 * materialised as [B, in, out] (which the literal plan does, vjp.rs:176-209 +
 * tensor_ir.rs:9324-9353, and which makes it unusable at the benchmark sizes).
 * The literal restatement (oracle/literal, NumPy) follows the reference's graph
 * transforms rule by rule; tests pin this file against it at small sizes and
 * against the reference's closed-form known answers.
 *
 * Difference from the reference's numbers: summation order only (points are
 * added in index order, as the reference's sequential sum does, but the batch
 * contraction of a weight gradient is fused).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

#define QBO_MAX_DIRS 8
#define QBO_MAX_ORDER 4
#define QBO_MAX_STREAMS 17
#define QBO_MAX_REGS 64

enum {
    OP_CONST = 0, OP_COL, OP_JET, OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_NEG, OP_SIN, OP_COS, OP_EXP, OP_TANH, OP_POWI,
    OP_SQRT, OP_LOG, OP_LOG1P, OP_EXPM1, OP_ERF, OP_ERFC, OP_TAN
};

typedef struct {
    int n_layers;            /* linear layers, the last one without tanh */
    const int* sizes;        /* n_layers + 1 */
    const double* const* W;  /* W[l]: [sizes[l]][sizes[l+1]] row-major */
    const double* const* b;  /* b[l]: [sizes[l+1]] or NULL */
    int activation;          /* of the hidden layers: 0 tanh, 1 sin, 2 sigmoid, 3 softplus, 4 silu, 5 gelu */
} qbo_net;

typedef struct {
    int64_t n;
    int ncols;
    const double* table; /* [n][ncols], network inputs first */
    int ndirs;
    const double* dirs; /* [ndirs][sizes[0]] */
    const int* orders;
    const int32_t* code; /* n_instr x {op, dst, a, b} */
    int n_instr;
    const double* consts;
    int value_reg;
    const int32_t* grad_regs; /* per stream, -1 = zero */
    double weight;
} qbo_set;

static double powi(double x, int n) { /* f64::powi, tensor_ir.rs:2072-2079 */
    int neg = n < 0;
    unsigned e = neg ? (unsigned)(-(long long)n) : (unsigned)n;
    double r = 1.0;
    while (e) {
        if (e & 1u) r *= x;
        x *= x;
        e >>= 1;
    }
    return neg ? 1.0 / r : r;
}

static void run_program(const qbo_set* s, const double* cols, const double* jets, double* r) {
    for (int pc = 0; pc < s->n_instr; ++pc) {
        const int32_t* in = s->code + 4 * pc;
        double v;
        switch (in[0]) {
            case OP_CONST: v = s->consts[in[2]]; break;
            case OP_COL: v = cols[in[2]]; break;
            case OP_JET: v = jets[in[2]]; break;
            case OP_ADD: v = r[in[2]] + r[in[3]]; break;
            case OP_SUB: v = r[in[2]] - r[in[3]]; break;
            case OP_MUL: v = r[in[2]] * r[in[3]]; break;
            case OP_DIV: v = r[in[2]] / r[in[3]]; break;
            case OP_NEG: v = -r[in[2]]; break;
            case OP_SIN: v = sin(r[in[2]]); break;
            case OP_COS: v = cos(r[in[2]]); break;
            case OP_EXP: v = exp(r[in[2]]); break;
            case OP_TANH: v = tanh(r[in[2]]); break;
            case OP_POWI: v = powi(r[in[2]], in[3]); break;
            case OP_SQRT: v = sqrt(r[in[2]]); break;
            case OP_LOG: v = log(r[in[2]]); break;
            case OP_LOG1P: v = log1p(r[in[2]]); break;
            case OP_EXPM1: v = expm1(r[in[2]]); break;
            case OP_ERF: v = erf(r[in[2]]); break;
            case OP_ERFC: v = erfc(r[in[2]]); break;
            case OP_TAN: v = tan(r[in[2]]); break;
            default: v = 0.0; break;
        }
        r[in[1]] = v;
    }
}

/* tanh derivatives through t: t' = 1 - t^2 (elementwise.rs:427-432) and its
 * successive derivatives. */
static void tanh_derivs(double t, double* d /* [6]: d[k] = k-th derivative */) {
    d[0] = t;
    d[1] = 1.0 - t * t;
    d[2] = -2.0 * t * d[1];
    d[3] = -2.0 * (d[1] * d[1] + t * d[2]);
    d[4] = -2.0 * (3.0 * d[1] * d[2] + t * d[3]);
    d[5] = -2.0 * (3.0 * d[2] * d[2] + 4.0 * d[1] * d[3] + t * d[4]);
}

/* sin and its derivatives: cos, -sin, -cos, sin, cos (chain rules of elementwise.rs:416-468). */
static void sin_derivs(double z, double* d) {
    const double sn = sin(z), cs = cos(z);
    d[0] = sn;
    d[1] = cs;
    d[2] = -sn;
    d[3] = -cs;
    d[4] = sn;
    d[5] = cs;
}

/* The logistic function as the reference composes it (crates/quabla-python/src/composite.rs:178-199:
 * where(z > 0, 1/(1+e), e/(1+e)), e = exp(-|z|)) and its derivatives by repeated differentiation of
 * ds/dz = s - s^2: every derivative is a polynomial in s, built here coefficient by coefficient. */
static void logistic_derivs(double z, double* d /* [6] */) {
    const double e = exp(-fabs(z));
    const double s = z > 0.0 ? 1.0 / (1.0 + e) : e / (1.0 + e);
    double poly[8] = {0.0, 1.0, 0, 0, 0, 0, 0, 0}; /* k-th derivative = sum_i poly[i] s^i; starts as s itself */
    int degree = 1;
    for (int k = 0; k < 6; ++k) {
        double value = 0.0;
        for (int i = degree; i >= 0; --i) value = value * s + poly[i];
        d[k] = value;
        /* d/dz of sum c_i s^i = sum i c_i s^(i-1) (s - s^2) = sum i c_i (s^i - s^(i+1)) */
        double next[8] = {0};
        for (int i = 1; i <= degree; ++i) {
            next[i] += i * poly[i];
            next[i + 1] -= i * poly[i];
        }
        for (int i = 0; i < 8; ++i) poly[i] = next[i];
        degree += 1;
    }
}

/* Derivatives of x * g(x) from those of g (Leibniz). */
static void times_x(double x, const double* g, double* d) {
    d[0] = x * g[0];
    for (int k = 1; k < 6; ++k) d[k] = x * g[k] + k * g[k - 1];
}

/* gelu, tanh approximation written through the logistic function: x s(c (x + a x^3)), c = 2 sqrt(2/pi)
 * (python/quabla/_ops.py:481-505); |x| > 40 returns x or -0 with a constant derivative.  The derivatives of
 * s(v(x)) come from the Taylor coefficients of the composition, computed by truncated series arithmetic. */
static void gelu_derivs(double x, double* d) {
    if (fabs(x) > 40.0) {
        d[0] = x > 0.0 ? x : -0.0;
        d[1] = x > 0.0 ? 1.0 : 0.0;
        d[2] = d[3] = d[4] = d[5] = 0.0;
        return;
    }
    const double c = 2.0 * sqrt(2.0 / 3.14159265358979323846), a = 0.044715;
    double ds[6];
    logistic_derivs(c * (x + a * x * x * x), ds);
    /* v(x + h) - v(x) as a series in h: coefficients u[1..3] */
    double u[6] = {0.0, c * (1.0 + 3.0 * a * x * x), c * 3.0 * a * x, c * a, 0.0, 0.0};
    /* g(x + h) = sum_k ds[k]/k! * (u(h))^k, truncated at h^5 */
    double series[6] = {ds[0], 0, 0, 0, 0, 0};
    double power[6] = {1.0, 0, 0, 0, 0, 0}; /* u^k */
    double factorial = 1.0;
    for (int k = 1; k < 6; ++k) {
        double next[6] = {0};
        for (int i = 0; i < 6; ++i)
            for (int j = 1; i + j < 6; ++j) next[i + j] += power[i] * u[j];
        for (int i = 0; i < 6; ++i) power[i] = next[i];
        factorial *= k;
        for (int i = 0; i < 6; ++i) series[i] += ds[k] / factorial * power[i];
    }
    double g[6];
    factorial = 1.0;
    for (int k = 0; k < 6; ++k) {
        if (k > 0) factorial *= k;
        g[k] = series[k] * factorial;
    }
    times_x(x, g, d);
}

/* Activation value and derivatives at the pre-activation z:
 * 0 tanh, 1 sin, 2 sigmoid, 3 softplus, 4 silu, 5 gelu. */
static void activation_derivs(int activation, double z, double* d) {
    double s[6];
    switch (activation) {
        case 1: sin_derivs(z, d); break;
        case 2: logistic_derivs(z, d); break;
        case 3: /* relu(z) + log1p(exp(-|z|)) (composite.rs:201-209); derivative: the logistic function */
            logistic_derivs(z, s);
            d[0] = (z > 0.0 ? z : 0.0) + log1p(exp(-fabs(z)));
            for (int k = 1; k < 6; ++k) d[k] = s[k - 1];
            break;
        case 4: /* z * sigmoid(z) (python/quabla/_ops.py:475-478) */
            logistic_derivs(z, s);
            times_x(z, s, d);
            break;
        case 5: gelu_derivs(z, d); break;
        default: tanh_derivs(tanh(z), d); break;
    }
}

/* Faa di Bruno: h_m = d^m tanh(z(s))/ds^m, m = 1..K, from z[m-1] = d^m z/ds^m. */
static void compose(const double* d, const double* z, int K, double* h) {
    double z1 = z[0];
    h[0] = d[1] * z1;
    if (K >= 2) h[1] = d[2] * z1 * z1 + d[1] * z[1];
    if (K >= 3) h[2] = d[3] * z1 * z1 * z1 + 3.0 * d[2] * z1 * z[1] + d[1] * z[2];
    if (K >= 4)
        h[3] = d[4] * z1 * z1 * z1 * z1 + 6.0 * d[3] * z1 * z1 * z[1] + d[2] * (3.0 * z[1] * z[1] + 4.0 * z1 * z[2]) +
               d[1] * z[3];
}

/* Transposed Jacobian of compose: gz = cotangents of z[0..K-1]; returns the
 * contribution to the cotangent of the primal pre-activation. */
static double compose_t(const double* d, const double* z, const double* g, int K, double* gz) {
    double z1 = z[0];
    double jz[QBO_MAX_ORDER][QBO_MAX_ORDER]; /* jz[m][q] = d h_{m+1} / d z_{q+1} */
    double j0[QBO_MAX_ORDER];                /* d h_{m+1} / d z_0 */
    memset(jz, 0, sizeof(jz));
    j0[0] = d[2] * z1;
    jz[0][0] = d[1];
    if (K >= 2) {
        j0[1] = d[3] * z1 * z1 + d[2] * z[1];
        jz[1][0] = 2.0 * d[2] * z1;
        jz[1][1] = d[1];
    }
    if (K >= 3) {
        j0[2] = d[4] * z1 * z1 * z1 + 3.0 * d[3] * z1 * z[1] + d[2] * z[2];
        jz[2][0] = 3.0 * d[3] * z1 * z1 + 3.0 * d[2] * z[1];
        jz[2][1] = 3.0 * d[2] * z1;
        jz[2][2] = d[1];
    }
    if (K >= 4) {
        j0[3] = d[5] * z1 * z1 * z1 * z1 + 6.0 * d[4] * z1 * z1 * z[1] + d[3] * (3.0 * z[1] * z[1] + 4.0 * z1 * z[2]) +
                d[2] * z[3];
        jz[3][0] = 4.0 * d[4] * z1 * z1 * z1 + 12.0 * d[3] * z1 * z[1] + 4.0 * d[2] * z[2];
        jz[3][1] = 6.0 * d[3] * z1 * z1 + 6.0 * d[2] * z[1];
        jz[3][2] = 4.0 * d[2] * z1;
        jz[3][3] = d[1];
    }
    double z0bar = 0.0;
    for (int q = 0; q < K; ++q) gz[q] = 0.0;
    for (int m = 0; m < K; ++m) {
        z0bar += j0[m] * g[m];
        for (int q = 0; q <= m; ++q) gz[q] += jz[m][q] * g[m];
    }
    return z0bar;
}

typedef struct {
    int S;
    int base[QBO_MAX_DIRS];
    size_t act_off[64]; /* offset of layer l's activations in the workspace */
    size_t pre_off[64];
    size_t total;
    int dmax;
} qbo_layout;

static void make_layout(const qbo_net* net, const qbo_set* s, qbo_layout* L) {
    L->S = 1;
    for (int j = 0; j < s->ndirs; ++j) {
        L->base[j] = L->S;
        L->S += s->orders[j];
    }
    size_t off = 0;
    L->dmax = 0;
    for (int l = 0; l <= net->n_layers; ++l) {
        L->act_off[l] = off;
        off += (size_t)L->S * net->sizes[l];
        L->pre_off[l] = off;
        off += (size_t)L->S * net->sizes[l];
        if (net->sizes[l] > L->dmax) L->dmax = net->sizes[l];
    }
    L->total = off;
}

/* One point: forward jets, residual, and (unless forward_only) the reverse
 * sweep adding this point's weight-gradient contribution into gW/gb. */
static double point_eval(const qbo_net* net, const qbo_set* s, const qbo_layout* L, const double* cols, double seed,
                         double* work, double* ga, double* gb_buf, double* const* gW, double* const* gb,
                         int forward_only) {
    const int S = L->S, nl = net->n_layers, d0 = net->sizes[0];
    double* h0 = work + L->act_off[0];
    for (int k = 0; k < d0; ++k) h0[k] = cols[k];
    for (int st = 1; st < S; ++st)
        for (int k = 0; k < d0; ++k) h0[st * d0 + k] = 0.0;
    for (int j = 0; j < s->ndirs; ++j)
        for (int k = 0; k < d0; ++k) h0[L->base[j] * d0 + k] = s->dirs[j * d0 + k];

    for (int l = 0; l < nl; ++l) {
        const int din = net->sizes[l], dout = net->sizes[l + 1];
        const double* hin = work + L->act_off[l];
        double* z = work + L->pre_off[l + 1];
        double* hout = work + L->act_off[l + 1];
        const double* W = net->W[l];
        for (int st = 0; st < S; ++st) {
            double* zs = z + (size_t)st * dout;
            for (int n = 0; n < dout; ++n) zs[n] = 0.0;
            /* i-k-j order, f64 accumulate, increasing k (tensor_ir.rs:1639-1656). */
            for (int k = 0; k < din; ++k) {
                const double a = hin[(size_t)st * din + k];
                const double* wr = W + (size_t)k * dout;
                for (int n = 0; n < dout; ++n) zs[n] += a * wr[n];
            }
            if (st == 0 && net->b[l] != NULL)
                for (int n = 0; n < dout; ++n) zs[n] += net->b[l][n];
        }
        if (l == nl - 1) {
            memcpy(hout, z, sizeof(double) * (size_t)S * dout);
            break;
        }
        for (int n = 0; n < dout; ++n) {
            double d[6];
            activation_derivs(net->activation, z[n], d);
            hout[n] = d[0];
            for (int j = 0; j < s->ndirs; ++j) {
                double zz[QBO_MAX_ORDER], hh[QBO_MAX_ORDER];
                const int K = s->orders[j];
                for (int m = 0; m < K; ++m) zz[m] = z[(size_t)(L->base[j] + m) * dout + n];
                compose(d, zz, K, hh);
                for (int m = 0; m < K; ++m) hout[(size_t)(L->base[j] + m) * dout + n] = hh[m];
            }
        }
    }
    const double* U = work + L->act_off[nl]; /* [S][1] */
    double r[QBO_MAX_REGS];
    run_program(s, cols, U, r);
    const double e = r[s->value_reg];
    if (forward_only) return e;

    /* Reverse sweep.  ga = cotangent of the current layer's output streams. */
    for (int st = 0; st < S; ++st) ga[st] = s->grad_regs[st] >= 0 ? seed * r[s->grad_regs[st]] : 0.0;
    for (int l = nl - 1; l >= 0; --l) {
        const int din = net->sizes[l], dout = net->sizes[l + 1];
        const double* hin = work + L->act_off[l];
        const double* z = work + L->pre_off[l + 1];
        /* ga holds cotangents of the layer's output jets [S][dout]; turn them into cotangents of z. */
        if (l != nl - 1) {
            for (int n = 0; n < dout; ++n) {
                double d[6];
                activation_derivs(net->activation, z[n], d);  /* z[n]: the primal pre-activation */
                double z0bar = d[1] * ga[n];
                for (int j = 0; j < s->ndirs; ++j) {
                    double zz[QBO_MAX_ORDER], gg[QBO_MAX_ORDER], gz[QBO_MAX_ORDER];
                    const int K = s->orders[j];
                    for (int m = 0; m < K; ++m) {
                        zz[m] = z[(size_t)(L->base[j] + m) * dout + n];
                        gg[m] = ga[(size_t)(L->base[j] + m) * dout + n];
                    }
                    z0bar += compose_t(d, zz, gg, K, gz);
                    for (int m = 0; m < K; ++m) ga[(size_t)(L->base[j] + m) * dout + n] = gz[m];
                }
                ga[n] = z0bar;
            }
        }
        /* dW += sum over streams of hin^T gz ; db += gz of the primal stream. */
        double* dW = gW[l];
        for (int st = 0; st < S; ++st)
            for (int k = 0; k < din; ++k) {
                const double a = hin[(size_t)st * din + k];
                if (a == 0.0) continue;
                double* row = dW + (size_t)k * dout;
                const double* g = ga + (size_t)st * dout;
                for (int n = 0; n < dout; ++n) row[n] += a * g[n];
            }
        if (gb[l] != NULL)
            for (int n = 0; n < dout; ++n) gb[l][n] += ga[n];
        if (l > 0) {
            const double* W = net->W[l];
            for (int st = 0; st < S; ++st)
                for (int k = 0; k < din; ++k) {
                    double acc = 0.0;
                    const double* wr = W + (size_t)k * dout;
                    const double* g = ga + (size_t)st * dout;
                    for (int n = 0; n < dout; ++n) acc += g[n] * wr[n];
                    gb_buf[(size_t)st * din + k] = acc;
                }
            memcpy(ga, gb_buf, sizeof(double) * (size_t)S * din);
        }
    }
    return e;
}

typedef struct {
    const qbo_net* net;
    const qbo_set* set;
    const qbo_layout* layout;
    double seed;
    int forward_only;
    int64_t lo, hi;
    double* const* gW; /* where this worker accumulates */
    double* const* gb;
    double loss_sum;
    int failed;
} qbo_job;

static void* run_job(void* arg) {
    qbo_job* job = (qbo_job*)arg;
    const qbo_layout* L = job->layout;
    double* work = (double*)malloc(sizeof(double) * L->total);
    double* ga = (double*)malloc(sizeof(double) * (size_t)L->S * L->dmax);
    double* gbuf = (double*)malloc(sizeof(double) * (size_t)L->S * L->dmax);
    if (!work || !ga || !gbuf) {
        job->failed = 1;
    } else {
        double sum = 0.0;
        for (int64_t i = job->lo; i < job->hi; ++i)
            sum += point_eval(job->net, job->set, L, job->set->table + (size_t)i * job->set->ncols, job->seed, work, ga,
                              gbuf, job->gW, job->gb, job->forward_only);
        job->loss_sum = sum;
    }
    free(work);
    free(ga);
    free(gbuf);
    return NULL;
}

/*
 * Adds  weight * sum_i e_i  to *loss and the matching gradients to gW / gb.
 * cotangent is the loss cotangent (the Trainer binds 1.0,
 * crates/quabla-python/src/tensor_trace.rs:5365-5378).  threads <= 1 runs the
 * points in index order on one thread, as the reference interpreter does;
 * threads > 1 splits the points into contiguous blocks (one POSIX thread each)
 * and adds the per-thread partial sums in block order.
 * Returns 0, or -1 on an invalid description or a failed allocation.
 */
int qbo_set_value_and_grad(const qbo_net* net, const qbo_set* s, double cotangent, double* loss, double* const* gW,
                           double* const* gb, int forward_only, int threads) {
    if (net->n_layers < 1 || net->n_layers > 62 || s->ndirs > QBO_MAX_DIRS) return -1;
    qbo_layout L;
    make_layout(net, s, &L);
    if (L.S > QBO_MAX_STREAMS) return -1;
    const int nl = net->n_layers;
    int nt = threads > 1 ? threads : 1;
    if (nt > 256) nt = 256;
    if ((int64_t)nt > s->n) nt = (int)s->n;
    size_t n_params = 0;
    for (int l = 0; l < nl; ++l) n_params += (size_t)net->sizes[l] * net->sizes[l + 1] + net->sizes[l + 1];
    qbo_job* jobs = (qbo_job*)calloc((size_t)nt, sizeof(qbo_job));
    pthread_t* tids = (pthread_t*)calloc((size_t)nt, sizeof(pthread_t));
    double* partial = nt > 1 && !forward_only ? (double*)calloc((size_t)nt * n_params, sizeof(double)) : NULL;
    double** ptrs = (double**)calloc((size_t)nt * 2 * nl, sizeof(double*));
    int failed = (!jobs || !tids || !ptrs || (nt > 1 && !forward_only && !partial));
    for (int t = 0; t < nt && !failed; ++t) {
        qbo_job* job = &jobs[t];
        job->net = net;
        job->set = s;
        job->layout = &L;
        job->seed = cotangent * s->weight;
        job->forward_only = forward_only;
        job->lo = s->n * t / nt;
        job->hi = s->n * (t + 1) / nt;
        double** tW = ptrs + (size_t)t * 2 * nl;
        double** tb = tW + nl;
        if (partial != NULL) {
            double* p = partial + (size_t)t * n_params;
            for (int l = 0; l < nl; ++l) {
                tW[l] = p;
                p += (size_t)net->sizes[l] * net->sizes[l + 1];
                tb[l] = gb[l] != NULL ? p : NULL;
                p += net->sizes[l + 1];
            }
        } else {
            for (int l = 0; l < nl; ++l) {
                tW[l] = gW ? gW[l] : NULL;
                tb[l] = gb ? gb[l] : NULL;
            }
        }
        job->gW = tW;
        job->gb = tb;
    }
    if (!failed) {
        if (nt == 1) {
            run_job(&jobs[0]);
        } else {
            int started = 0;
            for (int t = 0; t < nt; ++t) {
                if (pthread_create(&tids[t], NULL, run_job, &jobs[t]) != 0) {
                    failed = 1;
                    break;
                }
                ++started;
            }
            for (int t = 0; t < started; ++t) pthread_join(tids[t], NULL);
        }
    }
    if (!failed) {
        double total = 0.0;
        for (int t = 0; t < nt; ++t) {
            total += jobs[t].loss_sum;
            failed |= jobs[t].failed;
        }
        *loss += total * s->weight;
        if (partial != NULL) {
            for (int t = 0; t < nt; ++t) {
                const double* p = partial + (size_t)t * n_params;
                for (int l = 0; l < nl; ++l) {
                    const size_t nw = (size_t)net->sizes[l] * net->sizes[l + 1];
                    for (size_t i = 0; i < nw; ++i) gW[l][i] += p[i];
                    p += nw;
                    if (gb[l] != NULL)
                        for (int i = 0; i < net->sizes[l + 1]; ++i) gb[l][i] += p[i];
                    p += net->sizes[l + 1];
                }
            }
        }
    }
    free(jobs);
    free(tids);
    free(partial);
    free(ptrs);
    return failed ? -1 : 0;
}

/* Network output streams of one point (for stream-by-stream checks of the
 * forward kernels): out[S]. */
int qbo_point_jets(const qbo_net* net, const qbo_set* s, const double* cols, double* out) {
    qbo_layout L;
    make_layout(net, s, &L);
    double* work = (double*)malloc(sizeof(double) * L.total);
    double* ga = (double*)malloc(sizeof(double) * (size_t)L.S * L.dmax);
    if (!work || !ga) return -1;
    point_eval(net, s, &L, cols, 0.0, work, ga, ga, NULL, NULL, 1);
    for (int st = 0; st < L.S; ++st) out[st] = work[L.act_off[net->n_layers] + st];
    free(work);
    free(ga);
    return 0;
}

int qbo_max_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}
