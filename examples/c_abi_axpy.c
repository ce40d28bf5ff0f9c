/* The C ABI from plain C: y = 2 * (a + b + 3) on the GPU, the expression of the reference's
 * first integration test (tests/test_backend_integration.py:13-23), submitted as a hand-built
 * CNB1 blob.  No Python, no C++: the header is C, the library is loaded at link time.
 *
 *   cc -Iinclude examples/c_abi_axpy.c -Lcharmnumeric_b200 -lcnb200 -Wl,-rpath,$PWD/charmnumeric_b200 -o c_abi_axpy
 *   ./c_abi_axpy            (needs a B200)
 *   ./c_abi_axpy --check [file]   (no GPU: builds the blob, has the library parse it, writes it to file)
 *
 * Blob grammar: see the top of charmnumeric_b200/csrc/wire.cpp. */
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "cnb200.h"

static char blob[4096];
static size_t used;

static void put_i32(int32_t v) { memcpy(blob + used, &v, 4); used += 4; }
static void put_i64(int64_t v) { memcpy(blob + used, &v, 8); used += 8; }
static void put_f64(double v) { memcpy(blob + used, &v, 8); used += 8; }

/* ast header: result_name opcode flags dtype ndims scalar shape[ndims] region(global) */
static void ast(int name, int opcode, int flags, int ndims, double scalar, int n) {
    put_i32(name); put_i32(opcode); put_i32(flags); put_i32(CN_DTYPE_F64); put_i32(ndims); put_f64(scalar);
    if (ndims == 1) put_i32(n);
    put_i32(1); /* region: whole array */
}
static void leaf_array(int name, int n) { put_i32(0); ast(name, CN_OP_NOOP, 0, 1, 0.0, n); put_i32(0); put_i32(1); }
static void leaf_scalar(double v) { put_i32(0); ast(-1, CN_OP_NOOP, 2, 0, v, 0); put_i32(0); put_i32(1); }
static void ref(int name) { put_i32(1); put_i32(name); put_i32(1); }

int main(int argc, char** argv) {
    enum { N = 32, A = 1, B = 2, T0 = 10, T1 = 11, Y = 3 };
    double a[N], b[N], y[N];
    int64_t shape[1] = {N};
    cn_context* ctx = NULL;
    int rc, i;

    /* one fusible node with three roots: t0 = a + b (temp); t1 = t0 + 3 (temp); y = 2 * t1 */
    memcpy(blob, "CNB1", 4); used = 4;
    put_i32(1);                      /* epoch */
    put_i32(1);                      /* nodes */
    put_i32(0); put_i64(1); put_i32(1); put_i32(0); put_i32(3); /* id, identifier, fusible, deps, roots */
    ast(T0, CN_OP_ADD, 1, 1, 0.0, N); put_i32(2); leaf_array(A, N); leaf_array(B, N);
    ast(T1, CN_OP_ADD, 1, 1, 0.0, N); put_i32(2); ref(T0); leaf_scalar(3.0);
    ast(Y, CN_OP_MUL, 0, 1, 0.0, N); put_i32(2); leaf_scalar(2.0); ref(T1);
    put_i32(0);                      /* no deletes */

    if (argc > 1 && strcmp(argv[1], "--check") == 0) {
        char err[256] = "";
        int nodes = 0, roots = 0;
        rc = cn_dag_check(blob, (int64_t)used, &nodes, &roots, err, (int)sizeof(err));
        printf("blob of %zu bytes: status %d (%s), %d node(s), %d root(s) %s\n", used, rc, cn_status_string(rc),
               nodes, roots, err);
        if (argc > 2) { /* also write the bytes out, for comparison with another writer */
            FILE* f = fopen(argv[2], "wb");
            if (!f || fwrite(blob, 1, used, f) != used) return 1;
            fclose(f);
        }
        return rc == CN_STATUS_OK && nodes == 1 && roots == 3 ? 0 : 1;
    }

    for (i = 0; i < N; ++i) { a[i] = 1.5; b[i] = -0.5; }
    rc = cn_context_create(0, 0, 1, &ctx);
    if (rc != CN_STATUS_OK) {
        fprintf(stderr, "no context: %s (%s)\n", cn_status_string(rc), cn_last_error(NULL));
        return 2;
    }
    if ((rc = cn_put(ctx, A, 1, shape, CN_DTYPE_F64, a)) || (rc = cn_put(ctx, B, 1, shape, CN_DTYPE_F64, b))) goto fail;

    if ((rc = cn_receive_dag(ctx, 1, (int64_t)used, blob))) goto fail;
    if ((rc = cn_get(ctx, 1, 1, Y, N, CN_DTYPE_F64, y))) goto fail;
    for (i = 0; i < N; ++i)
        if (y[i] != 8.0) { fprintf(stderr, "y[%d] = %g, expected 8\n", i, y[i]); return 1; }
    printf("y = 2 * (a + b + 3) = %g on all %d elements\n", y[0], N);
    cn_context_destroy(ctx);
    return 0;
fail:
    fprintf(stderr, "%s: %s\n", cn_status_string(rc), cn_last_error(ctx));
    cn_context_destroy(ctx);
    return 1;
}
