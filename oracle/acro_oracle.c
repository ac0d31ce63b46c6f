/*
 * TEST INFRASTRUCTURE — not part of the product.
 *
 * Plain-C restatement of the reference's interpreted CPU path for string
 * tensor contractions (LLNL/acrotensor), used only as a checker by tests/,
 * the smoke check and bench.py's CPU-baseline leg.  The product library never
 * links, loads or calls this file.
 *
 * Parity status: PINNED.  The restatement is compared bit for bit against the
 * reference's own code (the unmodified sources compiled into
 * oracle/_ref/libacro_ref.so) by tests/test_oracle.py, and against the
 * committed fixtures in tests/golden/ that were produced by that library.
 *
 * What is restated, and where it lives in the reference:
 *   grammar            kernel/TensorKernel.cpp:26-139
 *   index bookkeeping  kernel/TensorKernel.cpp:45-63   (output indices first, then
 *                                                       contraction indices in
 *                                                       first-appearance order)
 *   loop extents       kernel/TensorKernel.cpp:375-403
 *   loop order         kernel/DimensionedMultiKernel.cpp:67-135 (non-contracted loops
 *                                                       outermost, largest first,
 *                                                       ties by name)
 *   dense strides      kernel/DimensionedKernel.cpp:133-145
 *   arithmetic         exec/CPUInterpretedExecutor.cpp:59-91 and
 *                      exec/CPUInterpretedExecutor.hpp:58-77:
 *                        "=" zero-fills the output, then for every loop tuple
 *                        out[..] += ((in0 * in1) * in2) * ...   (left to right)
 *                      "+=" and "-=" both accumulate with "+" (the reference's
 *                      CPU executor never subtracts).
 *   multi-kernel       exec/KernelExecutor.cpp:86-103 (sub-kernels run in order)
 *
 * Compile with floating-point contraction off so that a*b+c is never fused:
 * the reference's x86-64 build has no FMA.
 */
#include <ctype.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define MAX_VARS 17   /* output + 16 inputs */
#define MAX_RANK 16
#define MAX_LOOPS 32
#define MAX_NAME 32

#define API __attribute__((visibility("default")))

static __thread char g_err[512];

API const char *acro_oracle_last_error(void) { return g_err; }

static int fail(const char *msg, const char *detail)
{
    snprintf(g_err, sizeof g_err, "%s%s%s", msg, detail ? ": " : "", detail ? detail : "");
    return -1;
}

typedef struct {
    char name[MAX_NAME];
    int rank;
    char idx[MAX_RANK][MAX_NAME];
} var_t;

typedef struct {
    var_t out;
    int op; /* 0 "=", 1 "+=", 2 "-=" */
    int n_in;
    var_t in[MAX_VARS - 1];
    int n_all, n_contr;
    char all[MAX_LOOPS][MAX_NAME];   /* output indices, then contraction indices */
    char contr[MAX_LOOPS][MAX_NAME];
} kernel_t;

/* <var> := <Upper><alnum>* ( '_' <lower|digit>+ )+        kernel/TensorKernel.cpp:69-117 */
static int parse_var(const char **pp, var_t *v)
{
    const char *p = *pp;
    size_t n = 0;
    memset(v, 0, sizeof *v);
    if (!isupper((unsigned char)*p)) return -1;
    while (isalnum((unsigned char)*p)) {
        if (n + 1 >= MAX_NAME) return -1;
        v->name[n++] = *p++;
    }
    if (*p != '_') return -1;
    while (*p == '_') {
        ++p;
        if (!(islower((unsigned char)*p) || isdigit((unsigned char)*p))) return -1;
        if (v->rank >= MAX_RANK) return -1;
        n = 0;
        while (islower((unsigned char)*p) || isdigit((unsigned char)*p)) {
            if (n + 1 >= MAX_NAME) return -1;
            v->idx[v->rank][n++] = *p++;
        }
        v->rank++;
    }
    *pp = p;
    return 0;
}

static int find_name(char names[][MAX_NAME], int n, const char *s)
{
    for (int i = 0; i < n; ++i)
        if (strcmp(names[i], s) == 0) return i;
    return -1;
}

static int parse_kernel(const char *text, kernel_t *k)
{
    char buf[1024];
    size_t n = 0;
    for (const char *c = text; *c; ++c) {
        if (isspace((unsigned char)*c)) continue;      /* whitespace is stripped first, :31 */
        if (n + 1 >= sizeof buf) return fail("kernel string too long", text);
        buf[n++] = *c;
    }
    buf[n] = 0;
    memset(k, 0, sizeof *k);
    const char *p = buf;
    if (parse_var(&p, &k->out)) return fail("bad output variable in kernel", text);
    if (p[0] == '=') { k->op = 0; p += 1; }
    else if (p[0] == '+' && p[1] == '=') { k->op = 1; p += 2; }
    else if (p[0] == '-' && p[1] == '=') { k->op = 2; p += 2; }
    else return fail("bad assignment operator in kernel", text);
    do {
        if (k->n_in >= MAX_VARS - 1) return fail("too many inputs in kernel", text);
        if (parse_var(&p, &k->in[k->n_in])) return fail("bad input variable in kernel", text);
        k->n_in++;
    } while (*p);
    for (int d = 0; d < k->out.rank; ++d)
        if (find_name(k->all, k->n_all, k->out.idx[d]) < 0)
            strcpy(k->all[k->n_all++], k->out.idx[d]);
    for (int v = 0; v < k->n_in; ++v)
        for (int d = 0; d < k->in[v].rank; ++d)
            if (find_name(k->all, k->n_all, k->in[v].idx[d]) < 0) {
                if (k->n_all >= MAX_LOOPS) return fail("too many indices in kernel", text);
                strcpy(k->contr[k->n_contr++], k->in[v].idx[d]);
                strcpy(k->all[k->n_all++], k->in[v].idx[d]);
            }
    return 0;
}

typedef struct {
    double *data;
    int rank;
    const int *dims;
} tensor_t;

static int run_kernel(const char *text, tensor_t *out, tensor_t *const *ins, int n_in_given)
{
    kernel_t k;
    if (parse_kernel(text, &k)) return -1;
    if (n_in_given != k.n_in) return fail("input count does not match kernel", text);
    if (out->rank != k.out.rank) return fail("output rank does not match kernel", text);
    for (int v = 0; v < k.n_in; ++v)
        if (ins[v]->rank != k.in[v].rank) return fail("input rank does not match kernel", text);

    /* extents: output dims first, inputs override, inputs must agree (:375-403) */
    int ext_by_name[MAX_LOOPS];
    for (int i = 0; i < k.n_all; ++i) ext_by_name[i] = 1;
    for (int d = 0; d < out->rank; ++d) ext_by_name[find_name(k.all, k.n_all, k.out.idx[d])] = out->dims[d];
    for (int v = 0; v < k.n_in; ++v)
        for (int d = 0; d < ins[v]->rank; ++d)
            ext_by_name[find_name(k.all, k.n_all, k.in[v].idx[d])] = ins[v]->dims[d];
    for (int v = 0; v < k.n_in; ++v)
        for (int d = 0; d < ins[v]->rank; ++d)
            if (ext_by_name[find_name(k.all, k.n_all, k.in[v].idx[d])] != ins[v]->dims[d])
                return fail("Incompatible tensor dimensions for kernel", text);
    /* The reference never checks the output's extents against the inputs'; a mismatch
       there is an out-of-bounds write upstream, so the restatement refuses it. */
    for (int d = 0; d < out->rank; ++d)
        if (ext_by_name[find_name(k.all, k.n_all, k.out.idx[d])] != out->dims[d])
            return fail("output extent disagrees with an input extent", text);

    /* loop order: non-contracted loops, largest first (ties by name), then the
       contraction loops in first-appearance order. */
    int n_outer = k.n_all - k.n_contr, order[MAX_LOOPS], used[MAX_LOOPS] = {0};
    for (int i = 0; i < n_outer; ++i) {
        int best = -1;
        for (int j = 0; j < n_outer; ++j) {
            if (used[j]) continue;
            if (best < 0 || ext_by_name[j] > ext_by_name[best] ||
                (ext_by_name[j] == ext_by_name[best] && strcmp(k.all[j], k.all[best]) < 0))
                best = j;
        }
        used[best] = 1;
        order[i] = best;
    }
    for (int i = n_outer; i < k.n_all; ++i) order[i] = i;

    int nl = k.n_all;
    int64_t ext[MAX_LOOPS];
    for (int l = 0; l < nl; ++l) ext[l] = ext_by_name[order[l]];

    /* per-variable stride with respect to every loop (an index used twice in one
       variable, e.g. B_i_i, contributes both of its dimension strides) */
    int nv = k.n_in + 1;
    int64_t step[MAX_VARS][MAX_LOOPS];
    memset(step, 0, sizeof step);
    for (int v = 0; v < nv; ++v) {
        const var_t *var = v == 0 ? &k.out : &k.in[v - 1];
        const tensor_t *t = v == 0 ? out : ins[v - 1];
        int64_t s = 1;
        for (int d = var->rank - 1; d >= 0; --d) {
            int name_id = find_name(k.all, k.n_all, var->idx[d]);
            for (int l = 0; l < nl; ++l)
                if (order[l] == name_id) step[v][l] += s;
            s *= t->dims[d];
        }
    }

    int64_t out_size = 1;
    for (int d = 0; d < out->rank; ++d) out_size *= out->dims[d];
    if (k.op == 0)
        for (int64_t i = 0; i < out_size; ++i) out->data[i] = 0.0;

    int64_t total = 1;
    for (int l = 0; l < nl; ++l) total *= ext[l];
    int64_t I[MAX_LOOPS] = {0}, off[MAX_VARS] = {0};
    double *o = out->data;
    for (int64_t it = 0; it < total; ++it) {
        double rhs = ins[0]->data[off[1]];
        for (int v = 1; v < k.n_in; ++v) rhs *= ins[v]->data[off[v + 1]];
        o[off[0]] += rhs;
        /* odometer step, innermost loop fastest */
        for (int l = nl - 1; l >= 0; --l) {
            if (++I[l] < ext[l]) {
                for (int v = 0; v < nv; ++v) off[v] += step[v][l];
                break;
            }
            I[l] = 0;
            for (int v = 0; v < nv; ++v) off[v] -= step[v][l] * (ext[l] - 1);
        }
    }
    return 0;
}

/*
 * Run a program of contraction strings over a table of host tensors
 * (same calling convention as the reference shim's acro_ref_run).
 * Kernels run one after another; wrapping them in a multi-kernel launch does
 * not change the reference's CPU results, so the flag is accepted and ignored.
 */
API int acro_oracle_run(int n_tensors, double *const *data, const int *ranks, const int *dims_flat,
                        int n_kernels, const char *const *kernels, const int *out_idx,
                        const int *n_in, const int *in_idx_flat, int as_multi_launch)
{
    (void)as_multi_launch;
    tensor_t *tab = (tensor_t *)calloc((size_t)n_tensors, sizeof *tab);
    if (!tab) return fail("out of memory", NULL);
    const int *d = dims_flat;
    for (int i = 0; i < n_tensors; ++i) {
        tab[i].data = data[i];
        tab[i].rank = ranks[i];
        tab[i].dims = d;
        for (int r = 0; r < ranks[i]; ++r)
            if (d[r] <= 0) { free(tab); return fail("non-positive tensor dimension", NULL); }
        d += ranks[i];
    }
    const int *ii = in_idx_flat;
    int rc = 0;
    for (int kx = 0; kx < n_kernels && rc == 0; ++kx) {
        tensor_t *ins[MAX_VARS];
        if (n_in[kx] > MAX_VARS - 1) { rc = fail("too many inputs", kernels[kx]); break; }
        for (int j = 0; j < n_in[kx]; ++j) ins[j] = &tab[ii[j]];
        rc = run_kernel(kernels[kx], &tab[out_idx[kx]], ins, n_in[kx]);
        ii += n_in[kx];
    }
    free(tab);
    return rc;
}

/*
 * Batched inverse / determinant of 1x1, 2x2, 3x3 matrices: ops/NativeCPUOps.hpp:38-86 and
 * ops/NativeCPUOps.cpp:11-120, operation by operation.  ainv or adet may be NULL.  The
 * reference's 3x3 formula stores entry (r,c) of the true inverse at position (c,r).
 */
API int acro_oracle_batch_inv_det(const double *a, double *ainv, double *adet, int64_t count, int dim)
{
    if (dim < 1 || dim > 3 || count < 1 || !a) return fail("bad arguments to batch_inv_det", NULL);
    const int blk = dim * dim;
    for (int64_t m = 0; m < count; ++m) {
        double A[9], inv[9], det;
        for (int i = 0; i < blk; ++i) A[i] = a[m * blk + i];
        if (dim == 1) det = A[0];
        else if (dim == 2) det = (A[0] * A[3] - A[1] * A[2]);
        else det = (A[0] * A[4] * A[8] + A[1] * A[5] * A[6] + A[2] * A[3] * A[7]
                    - A[6] * A[4] * A[2] - A[7] * A[5] * A[0] - A[8] * A[3] * A[1]);
        if (adet) adet[m] = det;
        if (!ainv) continue;
        double invdet = 1.0 / det;
        if (dim == 1) inv[0] = 1.0 / det;
        else if (dim == 2) {
            inv[0] = invdet * A[3];
            inv[1] = -invdet * A[1];
            inv[2] = -invdet * A[2];
            inv[3] = invdet * A[0];
        } else {
            inv[0] = invdet * (A[4] * A[8] - A[5] * A[7]);
            inv[1] = invdet * (A[5] * A[6] - A[3] * A[8]);
            inv[2] = invdet * (A[3] * A[7] - A[4] * A[6]);
            inv[3] = invdet * (A[2] * A[7] - A[1] * A[8]);
            inv[4] = invdet * (A[0] * A[8] - A[2] * A[6]);
            inv[5] = invdet * (A[1] * A[6] - A[0] * A[7]);
            inv[6] = invdet * (A[1] * A[5] - A[2] * A[4]);
            inv[7] = invdet * (A[2] * A[3] - A[0] * A[5]);
            inv[8] = invdet * (A[0] * A[4] - A[1] * A[3]);
        }
        for (int i = 0; i < blk; ++i) ainv[m * blk + i] = inv[i];
    }
    return 0;
}

/* Aout[i] = Ain[M[i]]   (ops/NativeCPUOps.cpp:123-130) */
API int acro_oracle_flat_scatter(double *aout, const double *ain, const int *map, int64_t range)
{
    for (int64_t i = 0; i < range; ++i) aout[i] = ain[map[i]];
    return 0;
}

/* Aout = 0; Aout[M[i]] += Ain[i] in ascending i   (ops/NativeCPUOps.cpp:133-144) */
API int acro_oracle_flat_sum_gather(double *aout, const double *ain, const int *map, int64_t domain, int64_t range)
{
    for (int64_t d = 0; d < domain; ++d) aout[d] = 0.0;
    for (int64_t i = 0; i < range; ++i) aout[map[i]] += ain[i];
    return 0;
}

/* Grammar check only: 0 when the string parses, -1 otherwise. */
API int acro_oracle_parses(const char *kernel)
{
    kernel_t k;
    return parse_kernel(kernel, &k);
}
