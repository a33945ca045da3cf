/* TEST INFRASTRUCTURE (oracle side) - never linked into the product library.
 *
 * Glue that lets the reference's own quantiser translation unit
 * (seedpack/ggml/ggml-quants.c, pulled in through seedpack/ggml/export.c) be compiled
 * as a stand-alone shared object, where it lies, without copying it:
 *
 *   - the handful of ggml.c symbols the quantisers call (ggml_row_size, ggml_type_size,
 *     ggml_type_name, ggml_abort).  The reference's own stubs (seedpack/ggml/stubs.c:8-24)
 *     have no entry for Q2_0, so a complete size table is supplied here instead;
 *   - a STABLE sort under the name the Makefile maps `qsort` to.  The reference's
 *     authoritative build replaces qsort by a stable insertion sort
 *     (seedpack/gpuquant.py:70-80) because IQ1_S / IQ1_M sort (value, index) pairs by
 *     value only (ggml-quants.c:4501-4505) and bf16 inputs carry many equal values.
 *     A stable merge sort gives the same permutation and keeps the 43692 x 2048-entry
 *     table construction (ggml-quants.c:3182) fast.
 */
#include <stdarg.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

struct sizes { int type, blck; size_t size; const char *name; };
static const struct sizes TYPES[] = {
    {0, 1, 4, "f32"}, {1, 1, 2, "f16"}, {2, 32, 18, "q4_0"}, {3, 32, 20, "q4_1"},
    {6, 32, 22, "q5_0"}, {7, 32, 24, "q5_1"}, {8, 32, 34, "q8_0"}, {9, 32, 36, "q8_1"},
    {10, 256, 84, "q2_K"}, {11, 256, 110, "q3_K"}, {12, 256, 144, "q4_K"}, {13, 256, 176, "q5_K"},
    {14, 256, 210, "q6_K"}, {15, 256, 292, "q8_K"}, {16, 256, 66, "iq2_xxs"}, {17, 256, 74, "iq2_xs"},
    {18, 256, 98, "iq3_xxs"}, {19, 256, 50, "iq1_s"}, {20, 32, 18, "iq4_nl"}, {21, 256, 110, "iq3_s"},
    {22, 256, 82, "iq2_s"}, {23, 256, 136, "iq4_xs"}, {29, 256, 56, "iq1_m"}, {30, 1, 2, "bf16"},
    {34, 256, 54, "tq1_0"}, {35, 256, 66, "tq2_0"}, {39, 32, 17, "mxfp4"}, {40, 64, 36, "nvfp4"},
    {41, 128, 18, "q1_0"}, {42, 64, 18, "q2_0"},
};

static const struct sizes *find(int t) {
    for (size_t i = 0; i < sizeof(TYPES) / sizeof(TYPES[0]); ++i)
        if (TYPES[i].type == t) return &TYPES[i];
    fprintf(stderr, "ref_shim: unknown ggml type %d\n", t);
    abort();
}

void ggml_abort(const char *file, int line, const char *fmt, ...) {
    va_list a;
    va_start(a, fmt);
    fprintf(stderr, "ggml abort %s:%d: ", file, line);
    vfprintf(stderr, fmt, a);
    fprintf(stderr, "\n");
    va_end(a);
    abort();
}
size_t ggml_type_size(int t) { return find(t)->size; }
size_t ggml_row_size(int t, int64_t ne) { return find(t)->size * (size_t)ne / (size_t)find(t)->blck; }
const char *ggml_type_name(int t) { return find(t)->name; }

/* stable top-down merge sort with the qsort signature */
static void msort(unsigned char *a, unsigned char *tmp, size_t n, size_t sz,
                  int (*cmp)(const void *, const void *)) {
    if (n < 2) return;
    if (n <= 8) {                     /* insertion sort: stable */
        unsigned char key[64];
        unsigned char *k = sz <= sizeof(key) ? key : (unsigned char *)malloc(sz);
        for (size_t i = 1; i < n; ++i) {
            memcpy(k, a + i * sz, sz);
            size_t j = i;
            while (j > 0 && cmp(a + (j - 1) * sz, k) > 0) { memcpy(a + j * sz, a + (j - 1) * sz, sz); --j; }
            if (j != i) memcpy(a + j * sz, k, sz);
        }
        if (k != key) free(k);
        return;
    }
    size_t h = n / 2;
    msort(a, tmp, h, sz, cmp);
    msort(a + h * sz, tmp, n - h, sz, cmp);
    size_t i = 0, j = h, o = 0;
    while (i < h && j < n) {
        if (cmp(a + j * sz, a + i * sz) < 0) { memcpy(tmp + o * sz, a + j * sz, sz); ++j; }
        else                                  { memcpy(tmp + o * sz, a + i * sz, sz); ++i; }
        ++o;
    }
    if (i < h) memcpy(tmp + o * sz, a + i * sz, (h - i) * sz);
    if (j < n) memcpy(tmp + o * sz, a + j * sz, (n - j) * sz);
    memcpy(a, tmp, n * sz);
}

void sg_ref_stable_sort(void *base, size_t n, size_t sz, int (*cmp)(const void *, const void *)) {
    if (n < 2) return;
    unsigned char *tmp = (unsigned char *)malloc(n * sz);
    msort((unsigned char *)base, tmp, n, sz, cmp);
    free(tmp);
}
