/*
 * cblas_sgemm for the reference's CPU backend wherever this repository compiles it: the checker under oracle/_ref
 * (test infrastructure) and the CPU half of ormi-core inside the engine library of ormi_b200/csrc/seams (ormi-core's
 * DeviceEnum::CPU path; the B200 path never calls it).  The reference links an un-pinned system OpenBLAS
 * (ormi-core/CMakeLists.txt:31-36).  This shim forwards to an OpenBLAS shared object when one can be dlopen'ed — the
 * path in ORMI_ORACLE_OPENBLAS (the Python loaders set it to the library inside the running interpreter's scipy or
 * opencv wheel), else the distribution's libopenblas — and otherwise computes the same definition
 *      C = alpha * op(A) * op(B) + beta * C        (fp32, accumulation over k in ascending order)
 * with plain loops.  oracle_cblas_backend() tells which one is active.
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <glob.h>
#include "cblas_shim/cblas.h"

typedef void (*sgemm_fn)(CBLAS_ORDER, CBLAS_TRANSPOSE, CBLAS_TRANSPOSE, int, int, int, float,
                         const float*, int, const float*, int, float, float*, int);
typedef int (*get_threads_fn)(void);

static sgemm_fn g_sgemm = 0;
static get_threads_fn g_get_threads = 0;
static int g_tried = 0;
static char g_backend[512] = "loops";

static void try_load(const char* path) {
    if (g_sgemm || !path || !*path) return;
    void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!h) return;
    sgemm_fn f = (sgemm_fn)dlsym(h, "cblas_sgemm");
    if (!f) f = (sgemm_fn)dlsym(h, "scipy_cblas_sgemm");
    if (f && f != (sgemm_fn)cblas_sgemm) {
        g_sgemm = f;
        g_get_threads = (get_threads_fn)dlsym(h, "openblas_get_num_threads");
        if (!g_get_threads) g_get_threads = (get_threads_fn)dlsym(h, "scipy_openblas_get_num_threads");
        snprintf(g_backend, sizeof g_backend, "openblas:%s", path);
    }
}

static void load_once(void) {
    if (g_tried) return;
    g_tried = 1;
    if (getenv("ORMI_ORACLE_NO_OPENBLAS")) return;
    try_load(getenv("ORMI_ORACLE_OPENBLAS"));
    const char* patterns[] = {
        "/usr/lib/x86_64-linux-gnu/libopenblas.so.0",
        "/usr/lib/x86_64-linux-gnu/openblas-pthread/libopenblas.so.0",
        "/usr/lib64/libopenblas.so.0",
        0};
    for (int i = 0; patterns[i] && !g_sgemm; ++i) {
        glob_t g;
        if (glob(patterns[i], 0, 0, &g) == 0) {
            for (size_t j = 0; j < g.gl_pathc && !g_sgemm; ++j) try_load(g.gl_pathv[j]);
        }
        globfree(&g);
    }
}

const char* oracle_cblas_backend(void) { load_once(); return g_backend; }
int oracle_cblas_threads(void) { load_once(); return g_get_threads ? g_get_threads() : 1; }

static void sgemm_loops(CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k, float alpha,
                        const float* a, int lda, const float* b, int ldb, float beta, float* c, int ldc) {
    for (int i = 0; i < m; ++i) {
        float* crow = c + (size_t)i * ldc;
        float* acc = (float*)calloc((size_t)n, sizeof(float));
        for (int p = 0; p < k; ++p) {
            float av = (ta == CblasNoTrans) ? a[(size_t)i * lda + p] : a[(size_t)p * lda + i];
            if (tb == CblasNoTrans) {
                const float* brow = b + (size_t)p * ldb;
                for (int j = 0; j < n; ++j) acc[j] += av * brow[j];
            } else {
                for (int j = 0; j < n; ++j) acc[j] += av * b[(size_t)j * ldb + p];
            }
        }
        for (int j = 0; j < n; ++j) crow[j] = alpha * acc[j] + (beta == 0.0f ? 0.0f : beta * crow[j]);
        free(acc);
    }
}

void cblas_sgemm(CBLAS_ORDER order, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k, float alpha,
                 const float* a, int lda, const float* b, int ldb, float beta, float* c, int ldc) {
    load_once();
    if (g_sgemm) { g_sgemm(order, ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc); return; }
    if (order != CblasRowMajor) { fprintf(stderr, "oracle cblas shim: only row-major is implemented\n"); abort(); }
    sgemm_loops(ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
}
