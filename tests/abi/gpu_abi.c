/* A C caller of the device entry points of libqk_kernels.so: GpuContext::packed_matvec and
 * the resident factorized layer, checked against plain C loops that follow the reference
 * (crates/quantibbler-kernels/src/core.rs:202-221,247-260 and
 * crates/quantibbler-server/src/engine/mod.rs:393-437).
 *
 * Exit codes: 0 = device results match; 77 = no usable device (the expected-value
 * checksums are still printed, so that a machine without a GPU can check this file's own
 * arithmetic); 1 = a check failed. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "qk_kernels.h"

static uint64_t lcg_state = 0x243F6A8885A308D3ull;
static uint32_t lcg(void) {   /* Knuth's MMIX multiplier; the test rebuilds the same stream */
    lcg_state = lcg_state * 6364136223846793005ull + 1442695040888963407ull;
    return (uint32_t)(lcg_state >> 33);
}
static double unit(void) { return (double)lcg() / 2147483648.0 * 2.0 - 1.0; }   /* [-1, 1) */

static void random_rows(uint8_t *rows, size_t n_rows, size_t n_bits) {
    size_t words = (n_bits + 7) / 8;
    for (size_t i = 0; i < n_rows; ++i)
        for (size_t j = 0; j < words; ++j) {
            uint8_t b = (uint8_t)(lcg() & 0xFF);
            size_t valid = n_bits - 8 * j;
            if (valid < 8) b &= (uint8_t)((1u << valid) - 1u);   /* pad bits zero */
            rows[i * words + j] = b;
        }
}

/* out[i] = sum_k s(i,k) * vec[k], s = +1 where the bit is set, left to right in double */
static void matvec(const uint8_t *rows, size_t n_rows, size_t n_bits, const double *vec,
                   double *out) {
    size_t words = (n_bits + 7) / 8;
    for (size_t i = 0; i < n_rows; ++i) {
        double acc = 0.0;
        for (size_t k = 0; k < n_bits; ++k) {
            int bit = (rows[i * words + k / 8] >> (k % 8)) & 1;
            acc += bit ? vec[k] : -vec[k];
        }
        out[i] = acc;
    }
}

#define ROWS 37
#define BITS 75
#define DOUT 48
#define DIN 80
#define RANK 24

int main(void) {
    static uint8_t packed[ROWS * ((BITS + 7) / 8)];
    static double vec[BITS], want_mv[ROWS], got_mv[ROWS];
    random_rows(packed, ROWS, BITS);
    for (int k = 0; k < BITS; ++k) vec[k] = unit();
    matvec(packed, ROWS, BITS, vec, want_mv);

    static uint8_t ub_rows[DOUT * ((RANK + 7) / 8)], vb_t_rows[RANK * ((DIN + 7) / 8)];
    static float s1[DOUT], s2[DIN], bias[DOUT], x[DIN], want_y[DOUT], got_y[DOUT];
    static double z[DIN], t[RANK], u[DOUT];
    random_rows(ub_rows, DOUT, RANK);
    random_rows(vb_t_rows, RANK, DIN);
    for (int i = 0; i < DOUT; ++i) s1[i] = (float)(0.001 + 0.02 * fabs(unit()));
    for (int j = 0; j < DIN; ++j) s2[j] = (float)(0.001 + 0.02 * fabs(unit()));
    for (int i = 0; i < DOUT; ++i) bias[i] = (float)(0.1 * unit());
    for (int j = 0; j < DIN; ++j) x[j] = (float)unit();
    for (int j = 0; j < DIN; ++j) z[j] = (double)(float)(s2[j] * x[j]);
    matvec(vb_t_rows, RANK, DIN, z, t);
    matvec(ub_rows, DOUT, RANK, t, u);
    for (int i = 0; i < DOUT; ++i) want_y[i] = (float)u[i] * s1[i] + bias[i];

    double sum_mv = 0.0, sum_y = 0.0, peak_y = 0.0;
    for (int i = 0; i < ROWS; ++i) sum_mv += want_mv[i] * (i + 1);
    for (int i = 0; i < DOUT; ++i) {
        sum_y += (double)want_y[i] * (i + 1);
        if (fabs(want_y[i]) > peak_y) peak_y = fabs(want_y[i]);
    }
    printf("expected matvec checksum %.17g\nexpected layer checksum %.17g\n", sum_mv, sum_y);

    qk_ctx *ctx = NULL;
    if (qk_gpu_init_at(0, &ctx) != QK_OK) {
        printf("no device: %s\n", qk_last_error());
        return 77;
    }
    int failures = 0;
    if (qk_gpu_packed_matvec(ctx, packed, sizeof packed, ROWS, BITS, vec, BITS, got_mv) != QK_OK) {
        fprintf(stderr, "packed_matvec: %s\n", qk_last_error());
        return 1;
    }
    for (int i = 0; i < ROWS; ++i)
        if (got_mv[i] != want_mv[i]) {   /* the device face sums in the same order: same bits */
            fprintf(stderr, "matvec row %d: got %.17g want %.17g\n", i, got_mv[i], want_mv[i]);
            ++failures;
        }
    /* the refusal comes from the host, before any launch (gpu.rs:123-137) */
    if (qk_gpu_packed_matvec(ctx, packed, sizeof packed, ROWS, BITS, vec, BITS - 1, got_mv) !=
            QK_ERR_VALUE ||
        strcmp(qk_last_error(), "vec must have length 75, got 74") != 0) {
        fprintf(stderr, "short vector: unexpected answer '%s'\n", qk_last_error());
        ++failures;
    }

    qk_layer *layer = NULL;
    if (qk_layer_create(ctx, ub_rows, sizeof ub_rows, vb_t_rows, sizeof vb_t_rows, DOUT, DIN, RANK,
                        s1, s2, bias, QK_F32, &layer) != QK_OK) {
        fprintf(stderr, "layer_create: %s\n", qk_last_error());
        return 1;
    }
    for (int rep = 0; rep < 2; ++rep) {
        memset(got_y, 0, sizeof got_y);
        if (qk_layer_apply_host(ctx, layer, x, DIN, got_y, DOUT) != QK_OK) {
            fprintf(stderr, "layer_apply_host: %s\n", qk_last_error());
            return 1;
        }
        for (int i = 0; i < DOUT; ++i)
            if (fabs((double)got_y[i] - (double)want_y[i]) > 1e-5 * peak_y) {
                fprintf(stderr, "layer row %d: got %.9g want %.9g\n", i, got_y[i], want_y[i]);
                ++failures;
            }
    }
    if (qk_gpu_synchronize(ctx) != QK_OK) {
        fprintf(stderr, "synchronize: %s\n", qk_last_error());
        ++failures;
    }
    qk_layer_free(layer);
    qk_gpu_free(ctx);
    if (failures) return 1;
    puts("gpu ABI ok");
    return 0;
}
