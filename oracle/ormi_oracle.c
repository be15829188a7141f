/*
 * TEST INFRASTRUCTURE — a CPU restatement of the reference's realize path, used only as the checker
 * (tests/, the smoke test, and the cpu_baseline leg of the benchmark).  The product never links,
 * loads or calls it.
 *
 * Parity status: PINNED.  tests/test_oracle.py checks this file against every known-answer test the
 * reference holds for the path (ormi-core/csrc/tests/backend/cpu/test_jit.cpp,
 * .../kernels/reduce/test_sum.cpp, .../kernels/blas/test_matmul.cpp, csrc/tests/core/test_ops.cpp,
 * csrc/tests/backend/test_runtime.cpp, ormi-core/tests/test_tensor.py) and, bit for bit on the
 * pointwise and sum paths, against the unmodified reference compiled into oracle/_ref/.
 *
 * What is restated (one function each, in the reference's evaluation order):
 *   ormi::execute_graph          ormi-core/csrc/backend/runtime.cpp:13-39     -> oracle_port_run
 *   cpu::execute_jit             ormi-core/csrc/backend/cpu/jit.cpp:12-85      -> eval_pointwise
 *   CPU lowerings                ormi-core/csrc/backend/cpu/lowerings/pointwise.cpp:5-15
 *   cpu::sum                     ormi-core/csrc/backend/cpu/kernels/reduce/sum.cpp:8-51 -> eval_sum
 *   cpu::matmul                  ormi-core/csrc/backend/cpu/kernels/blas/matmul.cpp:10-77 -> eval_matmul
 * The SGEMM arithmetic itself lives in OpenBLAS (un-pinned system package in the reference build,
 * 0.3.15 in this image); it is restated from its definition C = A*B with fp32 accumulation over k in
 * ascending order, so matmul parity with the reference is to rounding, not bit-exact.
 *
 * EXTENSION, parity unpinned: ORMI_OP_MAXIMUM, ORMI_OP_GE and ORMI_OP_MAX have no counterpart in the reference, so
 * nothing of the reference can pin them.  They are evaluated in the same style (one node at a time over realized
 * parents; MAX walks the input exactly like eval_sum and keeps the larger value) and tests/test_oracle.py checks
 * them against compositions the reference CAN run (max(a,b) = (a + b + sqrt((a-b)^2)) / 2 to rounding).
 *
 * Because the reference realizes every parent before a node (runtime.cpp:16-18), each pointwise node
 * is evaluated on its own over realized parents; results are rounded to fp32 after every op, exactly
 * like the register file of the reference's interpreter.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "ormi_b200.h"

static char g_err[256];
const char* oracle_port_last_error(void) { return g_err; }

typedef struct {
    float*  ptr;      /* realized buffer (owned unless alias/leaf) */
    int64_t elems;    /* elements in the buffer */
    int     owned;
} slot_t;

static int64_t numel(const ormi_b200_node* n) {
    int64_t e = 1;
    for (int d = 0; d < n->ndim; ++d) e *= n->shape[d];
    return e;
}

static int is_view(int op) { return op == ORMI_OP_TRANSPOSE || op == ORMI_OP_RESHAPE || op == ORMI_OP_EXPAND; }

static float apply(int op, float a, float b) {
    switch (op) {
        case ORMI_OP_ADD: return a + b;
        case ORMI_OP_SUB: return a - b;
        case ORMI_OP_MUL: return a * b;
        case ORMI_OP_DIV: return a / b;
        case ORMI_OP_POW: return powf(a, b);
        case ORMI_OP_NEG: return -a;
        case ORMI_OP_EXP: return expf(a);
        case ORMI_OP_LOG: return logf(a);
        case ORMI_OP_SIN: return sinf(a);
        case ORMI_OP_COS: return cosf(a);
        case ORMI_OP_MAXIMUM: return a >= b ? a : b;            /* extension */
        case ORMI_OP_GE: return a >= b ? 1.0f : 0.0f;           /* extension */
    }
    return NAN;
}

/* Strides of a realized operand against the output shape: jit.cpp:31-46.  An operand that is rank 0
 * or whose buffer holds one float is read at [0] (jit.cpp:24). */
static void operand_strides(const ormi_b200_node* leaf, const slot_t* s, int out_ndim, int* ls, int* scalar) {
    *scalar = (leaf->ndim == 0) || (s->elems == 1);
    for (int d = 0; d < out_ndim; ++d) ls[d] = 0;
    if (*scalar) return;
    int off = out_ndim - leaf->ndim;
    for (int d = 0; d < out_ndim; ++d) {
        int od = d - off;
        if (od >= 0 && leaf->shape[od] != 1) ls[d] = leaf->strides[od];
    }
}

static int eval_pointwise(const ormi_b200_node* nodes, slot_t* slots, int i) {
    const ormi_b200_node* n = &nodes[i];
    int64_t total = numel(n);
    float* out = (float*)malloc((size_t)(total > 0 ? total : 1) * sizeof(float));
    if (!out) { snprintf(g_err, sizeof g_err, "out of memory"); return 1; }
    int ndim = n->ndim;
    int ostr[ORMI_B200_MAX_DIMS];
    for (int d = ndim - 1, acc = 1; d >= 0; --d) { ostr[d] = acc; acc *= n->shape[d]; }
    const float* src[2] = {0, 0};
    int ls[2][ORMI_B200_MAX_DIMS];
    int scalar[2] = {1, 1};
    for (int p = 0; p < n->n_parents; ++p) {
        int pi = n->parents[p];
        src[p] = slots[pi].ptr;
        operand_strides(&nodes[pi], &slots[pi], ndim, ls[p], &scalar[p]);
    }
    for (int64_t e = 0; e < total; ++e) {
        float v[2] = {0.0f, 0.0f};
        for (int p = 0; p < n->n_parents; ++p) {
            if (scalar[p]) { v[p] = src[p][0]; continue; }
            int64_t idx = 0, rem = e;
            for (int d = 0; d < ndim; ++d) {       /* jit.cpp:65-71 */
                int64_t coord = rem / ostr[d];
                rem %= ostr[d];
                idx += coord * ls[p][d];
            }
            v[p] = src[p][idx];
        }
        out[e] = apply(n->op, v[0], v[1]);
    }
    slots[i].ptr = out; slots[i].elems = total; slots[i].owned = 1;
    return 0;
}

static int eval_sum(const ormi_b200_node* nodes, slot_t* slots, int i) {
    const ormi_b200_node* n = &nodes[i];
    const ormi_b200_node* in = &nodes[n->parents[0]];
    const slot_t* is = &slots[n->parents[0]];
    int64_t out_elems = numel(n);
    float* out = (float*)calloc((size_t)(out_elems > 0 ? out_elems : 1), sizeof(float));   /* zeros(), sum.cpp:15 */
    if (!out) { snprintf(g_err, sizeof g_err, "out of memory"); return 1; }
    const int is_max = (n->op == ORMI_OP_MAX);                   /* extension: same walk, keep the larger value */
    if (is_max) for (int64_t e = 0; e < out_elems; ++e) out[e] = -INFINITY;
    int ostr[ORMI_B200_MAX_DIMS];
    for (int d = n->ndim - 1, acc = 1; d >= 0; --d) { ostr[d] = acc; acc *= n->shape[d]; }
    for (int d = 0; d < in->ndim; ++d) {
        if (in->strides[d] == 0) {
            free(out);
            snprintf(g_err, sizeof g_err, "SUM over a stride-0 view divides by zero in the reference (sum.cpp:28)");
            return 1;
        }
    }
    for (int64_t e = 0; e < is->elems; ++e) {                    /* sum.cpp:22-48 */
        int64_t rem = e, out_flat = 0;
        int out_d = 0;
        for (int d = 0; d < in->ndim; ++d) {
            int64_t coord = rem / in->strides[d];
            rem %= in->strides[d];
            int reduced = (n->n_axes == 0);
            for (int a = 0; a < n->n_axes && !reduced; ++a) reduced = (n->axes[a] == d);
            if (!reduced) { out_flat += coord * ostr[out_d]; out_d++; }
            else if (n->keepdims) out_d++;
        }
        if (out_flat >= out_elems) {
            free(out);
            snprintf(g_err, sizeof g_err, "the reference SUM writes out of bounds here (un-broadcast of a middle dimension, adjoint.cpp:22-31)");
            return 1;
        }
        if (is_max) { if (is->ptr[e] > out[out_flat]) out[out_flat] = is->ptr[e]; }
        else out[out_flat] += is->ptr[e];
    }
    slots[i].ptr = out; slots[i].elems = out_elems; slots[i].owned = 1;
    return 0;
}

/* C[M,N] = op(A) op(B), fp32, k ascending: the definition of cblas_sgemm(alpha=1, beta=0). */
static void sgemm_def(int ta, int tb, int M, int N, int K, const float* a, int lda, const float* b, int ldb, float* c) {
    float* acc = (float*)malloc((size_t)N * sizeof(float));
    for (int i = 0; i < M; ++i) {
        for (int j = 0; j < N; ++j) acc[j] = 0.0f;
        for (int p = 0; p < K; ++p) {
            float av = ta ? a[(size_t)p * lda + i] : a[(size_t)i * lda + p];
            if (!tb) { const float* br = b + (size_t)p * ldb; for (int j = 0; j < N; ++j) acc[j] += av * br[j]; }
            else     { for (int j = 0; j < N; ++j) acc[j] += av * b[(size_t)j * ldb + p]; }
        }
        memcpy(c + (size_t)i * N, acc, (size_t)N * sizeof(float));
    }
    free(acc);
}

static int64_t batch_offset(int flat, const int* bshape, int nb, const ormi_b200_node* v) {   /* matmul.cpp:43-60 */
    int64_t off = 0;
    int tmp = flat;
    for (int i = nb - 1; i >= 0; --i) {
        int coord = tmp % bshape[i];
        tmp /= bshape[i];
        int td = i - (nb - (v->ndim - 2));
        if (td >= 0 && v->shape[td] > 1) off += (int64_t)coord * v->strides[td];
    }
    return off;
}

static int eval_matmul(const ormi_b200_node* nodes, slot_t* slots, int i) {
    const ormi_b200_node* n = &nodes[i];
    const ormi_b200_node* A = &nodes[n->parents[0]];
    const ormi_b200_node* B = &nodes[n->parents[1]];
    int M = A->shape[A->ndim - 2], K = A->shape[A->ndim - 1], N = B->shape[B->ndim - 1];
    int nb = n->ndim - 2, batch = 1;
    for (int d = 0; d < nb; ++d) batch *= n->shape[d];
    int64_t total = numel(n);
    float* out = (float*)malloc((size_t)(total > 0 ? total : 1) * sizeof(float));
    if (!out) { snprintf(g_err, sizeof g_err, "out of memory"); return 1; }
    int ta = A->strides[A->ndim - 1] != 1, tb = B->strides[B->ndim - 1] != 1;      /* matmul.cpp:37-41 */
    int lda = ta ? A->strides[A->ndim - 1] : A->strides[A->ndim - 2];
    int ldb = tb ? B->strides[B->ndim - 1] : B->strides[B->ndim - 2];
    for (int b = 0; b < batch; ++b) {
        const float* ap = slots[n->parents[0]].ptr + batch_offset(b, n->shape, nb, A);
        const float* bp = slots[n->parents[1]].ptr + batch_offset(b, n->shape, nb, B);
        sgemm_def(ta, tb, M, N, K, ap, lda, bp, ldb, out + (size_t)b * M * N);
    }
    slots[i].ptr = out; slots[i].elems = total; slots[i].owned = 1;
    return 0;
}

static double now_s(void) { struct timespec t; clock_gettime(CLOCK_MONOTONIC, &t); return t.tv_sec + 1e-9 * t.tv_nsec; }

/* Realizes out_nodes[] of a flattened graph whose realized nodes carry HOST pointers in `data`.
 * Values are copied out with the node's view strides applied. */
int oracle_port_run(const ormi_b200_node* nodes, int n, const int32_t* out_nodes, int n_out,
                    float** out_data, const int64_t* out_cap, int32_t* out_ndim, int32_t* out_shape,
                    double* seconds) {
    slot_t* slots = (slot_t*)calloc((size_t)n, sizeof(slot_t));
    char* need = (char*)calloc((size_t)n, 1);
    int rc = 0;
    for (int o = 0; o < n_out; ++o) need[out_nodes[o]] = 1;
    for (int i = n - 1; i >= 0; --i) {
        if (!need[i] || nodes[i].data) continue;
        for (int p = 0; p < nodes[i].n_parents; ++p) need[nodes[i].parents[p]] = 1;
    }
    double t0 = now_s();
    for (int i = 0; i < n && !rc; ++i) {
        if (!need[i]) continue;
        const ormi_b200_node* nd = &nodes[i];
        if (nd->data) { slots[i].ptr = (float*)nd->data; slots[i].elems = nd->data_bytes / 4; continue; }
        if (nd->op == ORMI_OP_LEAF) { snprintf(g_err, sizeof g_err, "leaf %d has no data", i); rc = 1; break; }
        if (is_view(nd->op)) { slots[i] = slots[nd->parents[0]]; slots[i].owned = 0; continue; }   /* runtime.cpp:20-23 */
        if (nd->op == ORMI_OP_SUM || nd->op == ORMI_OP_MAX) rc = eval_sum(nodes, slots, i);
        else if (nd->op == ORMI_OP_MATMUL) rc = eval_matmul(nodes, slots, i);
        else if ((nd->op >= ORMI_OP_NEG && nd->op <= ORMI_OP_POW) || nd->op == ORMI_OP_MAXIMUM || nd->op == ORMI_OP_GE) rc = eval_pointwise(nodes, slots, i);
        else { snprintf(g_err, sizeof g_err, "op %d has no CPU lowering", nd->op); rc = 1; }
    }
    if (seconds) *seconds = now_s() - t0;
    for (int o = 0; o < n_out && !rc; ++o) {
        const ormi_b200_node* nd = &nodes[out_nodes[o]];
        int64_t total = numel(nd);
        out_ndim[o] = nd->ndim;
        for (int d = 0; d < nd->ndim; ++d) out_shape[o * ORMI_B200_MAX_DIMS + d] = nd->shape[d];
        if (total > out_cap[o]) { snprintf(g_err, sizeof g_err, "output buffer too small"); rc = 1; break; }
        int idx[ORMI_B200_MAX_DIMS] = {0};
        const float* src = slots[out_nodes[o]].ptr;
        for (int64_t e = 0; e < total; ++e) {
            int64_t off = 0;
            for (int d = 0; d < nd->ndim; ++d) off += (int64_t)idx[d] * nd->strides[d];
            out_data[o][e] = src[off];
            for (int d = nd->ndim - 1; d >= 0; --d) { if (++idx[d] < nd->shape[d]) break; idx[d] = 0; }
        }
    }
    for (int i = 0; i < n; ++i) if (slots[i].owned) free(slots[i].ptr);
    free(slots); free(need);
    return rc;
}
