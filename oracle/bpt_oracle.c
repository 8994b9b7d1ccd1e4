/*
 * CPU restatement of the BP-Transformer hot path.  TEST INFRASTRUCTURE ONLY: the shipped
 * package never links, loads or calls this file; it exists so tests and the benchmark's
 * CPU-baseline leg have something independent of the CUDA code to compare with.
 *
 * Integer part (bit-exact contract) follows the reference's Cython builder:
 *   level table / pos      graph_builder/builder.pyx:41-62
 *   edge emission          graph_builder/builder.pyx:64-116
 *   partition_csr          graph_builder/builder.pyx:305-321
 * CSR extraction follows graph/base.py:71-86 (rows of the out-CSR are sources, rows of the
 * in-CSR are destinations, data = edge id); the order inside a row is defined here as
 * ascending edge id (stable counting sort), because the library that fixed it in the
 * reference (DGL 0.4) is not part of the reference's sources.
 *
 * Floating-point part follows the math of the reference's message-passing path
 *   score      modules/attention.py:189-200  (k[src].q[dst] + ak[e].q[dst])
 *   softmax    modules/attention.py:202-207  (edge softmax of score/sqrt(d_k) per destination)
 *   aggregate  modules/attention.py:209      (sum of v[src]*a over incoming edges)
 * which is also what the chain of graph_kernel/graphop_kernel.cu:19-202 computes op by op.
 * Gradients are the analytic derivatives of that chain.
 *
 * Build: gcc -O3 -fopenmp -shared -fPIC bpt_oracle.c -o _build/libbpt_oracle.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ level table */

/* builder.pyx:41-56: level sizes n, ceil(n/2), ... while >= 2, then a root of one node.
 * Returns the number of levels; n_nodes_arr / shift may be NULL. shift has n_lvl entries
 * used here (shift[j] = first node id of level j). */
int bpto_levels(int64_t length, uint32_t *n_nodes_arr, uint32_t *shift, int64_t *n_nodes_out) {
    int64_t n = length, total = 0;
    int lvl = 0;
    while (n >= 2) {
        if (n_nodes_arr) n_nodes_arr[lvl] = (uint32_t)n;
        if (shift) shift[lvl] = (uint32_t)total;
        total += n;
        lvl++;
        n = (n + 1) >> 1;
    }
    if (n_nodes_arr) n_nodes_arr[lvl] = 1;
    if (shift) shift[lvl] = (uint32_t)total;
    total += 1;
    lvl++;
    if (n_nodes_out) *n_nodes_out = total;
    return lvl;
}

/* builder.pyx:46-47,57-62: pos of node idx at level j is min((idx+1)*2^j - 1, length-1);
 * the root gets length-1. */
void bpto_pos(int64_t length, uint32_t *pos) {
    uint32_t nn[64], sh[64];
    int64_t total;
    int n_lvl = bpto_levels(length, nn, sh, &total);
    for (int j = 0; j < n_lvl - 1; ++j)
        for (uint32_t i = 0; i < nn[j]; ++i) {
            uint64_t p = ((uint64_t)i + 1) * ((uint64_t)1 << j) - 1;
            if (p >= (uint64_t)length) p = (uint64_t)length - 1;
            pos[sh[j] + i] = (uint32_t)p;
        }
    pos[total - 1] = (uint32_t)(length - 1);
}

/* builder.pyx:64-116.  Emits edges in the reference's order.  With src == NULL only counts.
 * Returns the number of edges. */
int64_t bpto_build(int64_t length, int triu, int step, int clip_dist,
                   uint32_t *src, uint32_t *dst, uint32_t *etype) {
    uint32_t nn[64], sh[64];
    int64_t total;
    int n_lvl = bpto_levels(length, nn, sh, &total);
    int64_t e = 0;
    const uint32_t per_lvl = 2u * (uint32_t)step + 1u;
    for (int64_t i = 0; i < length; ++i) {
        int v = (int)i;
        uint32_t shift = 0;
        int l_ptr = v - 1, r_ptr = v + 1;
        int l_ov = 0, r_ov = 0;
        for (int j = 0; j < n_lvl; ++j) {
            uint32_t base = per_lvl * (uint32_t)(j < clip_dist ? j : clip_dist);
            for (int k = 0; k < step; ++k) {
                if (!triu && (uint32_t)r_ptr < nn[j]) {
                    if (src) {
                        src[e] = r_ov ? sh[j - 1] + (((uint32_t)r_ptr << 1) + 1u) : sh[j] + (uint32_t)r_ptr;
                        dst[e] = (uint32_t)i;
                        etype[e] = base + 2u * ((uint32_t)k + 1u);
                    }
                    e++;
                    r_ov = 0;
                }
                r_ptr++;
                if (l_ptr >= 0) {
                    if (src) {
                        src[e] = l_ov ? sh[j - 1] + ((uint32_t)l_ptr << 1) : sh[j] + (uint32_t)l_ptr;
                        dst[e] = (uint32_t)i;
                        etype[e] = base + 2u * (uint32_t)k + 1u;
                    }
                    e++;
                    l_ov = 0;
                }
                l_ptr--;
            }
            if ((l_ptr & 1) == 0) l_ov = 1;
            if ((r_ptr & 1) == 1) r_ov = 1;
            r_ptr >>= 1;
            l_ptr >>= 1; /* arithmetic: -1 stays -1, -2 becomes -1 */
            if (src) {
                src[e] = (uint32_t)i;
                dst[e] = shift + (uint32_t)v;
                etype[e] = base;
            }
            e++;
            shift += nn[j];
            v >>= 1;
        }
    }
    return e;
}

/* ------------------------------------------------------------------ baseline graphs */

/* FullyConnected.build_graph, graph_builder/builder.pyx:243-267.  Returns the edge count;
 * with src == NULL only counts.  pos (length+1 entries) may be NULL. */
int64_t bpto_fully_connected(int64_t length, int triu, int64_t window,
                             uint32_t *src, uint32_t *dst, uint32_t *etype, uint32_t *pos) {
    int64_t e = 0;
    const int64_t jend = length < window + 1 ? length : window + 1;
    for (int64_t i = 0; i < length; ++i) {
        if (pos) pos[i] = (uint32_t)i;
        if (src) { src[e] = (uint32_t)i; dst[e] = (uint32_t)i; etype[e] = 0; }
        e++;
        for (int64_t j = 1; j < jend; ++j) {
            if (i >= j) {
                if (src) { src[e] = (uint32_t)(i - j); dst[e] = (uint32_t)i; etype[e] = (uint32_t)(2 * j - 1); }
                e++;
            }
            if (!triu && i + j < length) {
                if (src) { src[e] = (uint32_t)(i + j); dst[e] = (uint32_t)i; etype[e] = (uint32_t)(2 * j); }
                e++;
            }
        }
        if (src) { src[e] = (uint32_t)i; dst[e] = (uint32_t)length; etype[e] = 0; }
        e++;
    }
    if (pos) pos[length] = (uint32_t)length;
    return e;
}

/* OpenAISparse.build_graph, graph_builder/builder.pyx:171-196.  The reference's loop bounds are
 * unsigned: when c exceeds stride*j the start of range(stride*j - c, stride*j) wraps around and
 * the range is empty. */
int64_t bpto_openai_sparse(int64_t length, int64_t stride, int64_t c,
                           uint32_t *src, uint32_t *dst, uint32_t *etype, uint32_t *pos) {
    int64_t e = 0;
    for (int64_t i = 0; i < length; ++i) {
        if (pos) pos[i] = (uint32_t)i;
        for (int64_t j = (i / stride) * stride; j < i + 1; ++j) {
            if (src) { src[e] = (uint32_t)j; dst[e] = (uint32_t)i; etype[e] = 0; }
            e++;
        }
        for (int64_t j = 1; j < i / stride + 1; ++j) {
            if (stride * j < c) continue;
            for (int64_t k = stride * j - c; k < stride * j; ++k) {
                if (src) { src[e] = (uint32_t)k; dst[e] = (uint32_t)i; etype[e] = 0; }
                e++;
            }
        }
        if (src) { src[e] = (uint32_t)i; dst[e] = (uint32_t)length; etype[e] = 0; }
        e++;
    }
    if (pos) pos[length] = (uint32_t)(length - 1);
    return e;
}

/* ------------------------------------------------------------------ CSR helpers */

/* builder.pyx:305-321.  With row == NULL only counts. Returns the number of chunks. */
int64_t bpto_partition_csr(const int64_t *indptr, int64_t n_rows, int chunk,
                           int64_t *row, int64_t *indptr_out) {
    int64_t c = 0;
    for (int64_t i = 0; i < n_rows; ++i)
        for (int64_t j = indptr[i]; j < indptr[i + 1]; j += chunk) {
            if (row) { row[c] = i; indptr_out[c] = j; }
            c++;
        }
    if (row) indptr_out[c] = indptr[n_rows];
    return c;
}

/* Stable counting sort of edge ids by key (graph/base.py:72,79 with ascending-eid rows).
 * key/other have n_edges entries; out: indptr[n_rows+1], indices[n_edges] = other[eid],
 * eid[n_edges]. */
void bpto_coo_to_csr(const int64_t *key, const int64_t *other, int64_t n_edges, int64_t n_rows,
                     int64_t *indptr, int64_t *indices, int64_t *eid) {
    memset(indptr, 0, sizeof(int64_t) * (size_t)(n_rows + 1));
    for (int64_t e = 0; e < n_edges; ++e) indptr[key[e] + 1]++;
    for (int64_t i = 0; i < n_rows; ++i) indptr[i + 1] += indptr[i];
    int64_t *cur = (int64_t *)malloc(sizeof(int64_t) * (size_t)(n_rows > 0 ? n_rows : 1));
    memcpy(cur, indptr, sizeof(int64_t) * (size_t)n_rows);
    for (int64_t e = 0; e < n_edges; ++e) {
        int64_t p = cur[key[e]]++;
        indices[p] = other[e];
        eid[p] = e;
    }
    free(cur);
}

/* ------------------------------------------------------------------ attention math */

#define REAL double
#define FN(name) name##_f64
#include "bpt_oracle_attn.inc"
#undef REAL
#undef FN

#define REAL float
#define FN(name) name##_f32
#define BPTO_REAL_IS_FLOAT 1
#include "bpt_oracle_attn.inc"
#undef REAL
#undef FN

int bpto_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void bpto_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
