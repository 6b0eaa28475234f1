/*
 * grws_oracle.c -- CPU restatement of the Graph_RWS hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the CUDA library is compared against.  It is never part of the
 * product path: only the tests, the smoke check and the CPU-baseline leg of the benchmark may
 * load it.  Every function cites the reference file:line whose behaviour it restates.
 *
 * Parity pins (see tests/test_oracle_pins.py):
 *   - the BCSR layout functions are checked bit-for-bit against outputs of the reference's own
 *     csr_to_bcsr_cpu (core/wrapper/convert_wrapper.cpp:27-180) stored under tests/golden/;
 *   - philox4x32_10 is checked against the published Random123 known-answer vectors and
 *     against the cuRAND host generator;
 *   - the SpMM restatement is checked against a dense float64 product.
 * The reference ships no tests or golden vectors of its own for this path.
 *
 * Plain C99 + OpenMP.  Build: make -C oracle
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------ */
/* small helpers                                                                              */
/* ------------------------------------------------------------------------------------------ */
static int cmp_i32(const void *a, const void *b) {
    int32_t x = *(const int32_t *)a, y = *(const int32_t *)b;
    return (x > y) - (x < y);
}

/* sort + unique in place, returns number of unique values */
static int64_t sort_unique_i32(int32_t *v, int64_t n) {
    if (n <= 0) return 0;
    qsort(v, (size_t)n, sizeof(int32_t), cmp_i32);
    int64_t m = 1;
    for (int64_t i = 1; i < n; ++i)
        if (v[i] != v[m - 1]) v[m++] = v[i];
    return m;
}

static int64_t lower_bound_i32(const int32_t *v, int64_t n, int32_t key) {
    int64_t lo = 0, hi = n;
    while (lo < hi) {
        int64_t mid = (lo + hi) >> 1;
        if (v[mid] < key) lo = mid + 1; else hi = mid;
    }
    return lo;
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; a caller that wants the host's cores for a
 * timed CPU run sets the count itself. */
API void grws_oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

API int grws_oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------------------------ */
/* CSR -> BCSR  (core/wrapper/convert_wrapper.cpp:27-180)                                      */
/*   window = tile_rows consecutive rows; a window lists its sorted unique column ids          */
/*   tile_cols at a time (convert_wrapper.cpp:61-91), the last tile padded with -1 (:106);     */
/*   values are [tile][tile_rows][tile_cols] row-major, zero where there is no edge (:108),    */
/*   duplicate (row,col) entries: the last one in CSR order wins (:174).                       */
/* ------------------------------------------------------------------------------------------ */
API int64_t grws_oracle_csr_to_bcsr_count(int64_t num_rows, const int64_t *row_ptr,
                                          const int32_t *col_idx, int64_t tile_rows,
                                          int64_t tile_cols, int64_t *window_offset /*[W+1]*/) {
    int64_t W = (num_rows + tile_rows - 1) / tile_rows;
    window_offset[0] = 0;
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t w = 0; w < W; ++w) {
        int64_t r0 = w * tile_rows, r1 = r0 + tile_rows;
        if (r1 > num_rows) r1 = num_rows;
        int64_t e0 = row_ptr[r0], e1 = row_ptr[r1], n = e1 - e0;
        int64_t tiles = 0;
        if (n > 0) {
            int32_t *tmp = (int32_t *)malloc((size_t)n * sizeof(int32_t));
            memcpy(tmp, col_idx + e0, (size_t)n * sizeof(int32_t));
            int64_t u = sort_unique_i32(tmp, n);
            tiles = (u + tile_cols - 1) / tile_cols;
            free(tmp);
        }
        window_offset[w + 1] = tiles;
    }
    for (int64_t w = 0; w < W; ++w) window_offset[w + 1] += window_offset[w]; /* :96-98 */
    return window_offset[W];
}

API void grws_oracle_csr_to_bcsr_fill(int64_t num_rows, const int64_t *row_ptr,
                                      const int32_t *col_idx, const float *values,
                                      int64_t tile_rows, int64_t tile_cols,
                                      const int64_t *window_offset, int32_t *out_cols /*[T*tc]*/,
                                      float *out_vals /*[T*tr*tc]*/) {
    int64_t W = (num_rows + tile_rows - 1) / tile_rows;
    int64_t T = window_offset[W];
    for (int64_t i = 0; i < T * tile_cols; ++i) out_cols[i] = -1;               /* :106 */
    memset(out_vals, 0, (size_t)(T * tile_rows * tile_cols) * sizeof(float));    /* :108 */
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t w = 0; w < W; ++w) {
        int64_t t0 = window_offset[w], nt = window_offset[w + 1] - t0;
        if (nt == 0) continue;
        int64_t r0 = w * tile_rows, r1 = r0 + tile_rows;
        if (r1 > num_rows) r1 = num_rows;
        int64_t e0 = row_ptr[r0], e1 = row_ptr[r1], n = e1 - e0;
        int32_t *uq = (int32_t *)malloc((size_t)n * sizeof(int32_t));
        memcpy(uq, col_idx + e0, (size_t)n * sizeof(int32_t));
        int64_t u = sort_unique_i32(uq, n);
        memcpy(out_cols + t0 * tile_cols, uq, (size_t)u * sizeof(int32_t));      /* :140-143 */
        for (int64_t r = r0; r < r1; ++r) {                                      /* :150-176 */
            for (int64_t e = row_ptr[r]; e < row_ptr[r + 1]; ++e) {
                int64_t pos = lower_bound_i32(uq, u, col_idx[e]);
                int64_t tile = t0 + pos / tile_cols, ic = pos % tile_cols;
                out_vals[tile * tile_rows * tile_cols + (r - r0) * tile_cols + ic] = values[e];
            }
        }
        free(uq);
    }
}

/* ------------------------------------------------------------------------------------------ */
/* forward SpMM  C[W*16, N] = A_bcsr * B[K, N]                                                 */
/*   semantics of tcspmm_base_kernel (core/include/spmm_tc.cuh:113-193): every tile of the     */
/*   window is accumulated, a column id of -1 contributes nothing (:131-141), M = W*tile_rows  */
/*   (core/wrapper/spmm_wrapper.cu:55-63).  Accumulation here is float64 (the reference rounds */
/*   both operands to TF32 and accumulates in fp32; the parity tolerance covers that).         */
/* ------------------------------------------------------------------------------------------ */
API void grws_oracle_spmm_fwd(int64_t W, int64_t N, int64_t tile_rows, int64_t tile_cols,
                              const int64_t *window_offset, const int32_t *cols,
                              const float *vals, const float *B, int64_t ldb, float *C,
                              int64_t ldc) {
#pragma omp parallel
    {
        double *acc = (double *)malloc((size_t)(tile_rows * N) * sizeof(double));
#pragma omp for schedule(dynamic, 16)
        for (int64_t w = 0; w < W; ++w) {
            memset(acc, 0, (size_t)(tile_rows * N) * sizeof(double));
            for (int64_t t = window_offset[w]; t < window_offset[w + 1]; ++t) {
                const float *tv = vals + t * tile_rows * tile_cols;
                for (int64_t c = 0; c < tile_cols; ++c) {
                    int32_t col = cols[t * tile_cols + c];
                    if (col == -1) continue;
                    const float *brow = B + (int64_t)col * ldb;
                    for (int64_t r = 0; r < tile_rows; ++r) {
                        float a = tv[r * tile_cols + c];
                        if (a == 0.0f) continue;
                        double *ar = acc + r * N;
                        for (int64_t n = 0; n < N; ++n) ar[n] += (double)a * (double)brow[n];
                    }
                }
            }
            for (int64_t r = 0; r < tile_rows; ++r)
                for (int64_t n = 0; n < N; ++n)
                    C[(w * tile_rows + r) * ldc + n] = (float)acc[r * N + n];
        }
        free(acc);
    }
}

/* ------------------------------------------------------------------------------------------ */
/* transposed SpMM  G_in[num_cols, F] = A^T * G_out[W*16, F]                                   */
/*   semantics of spmm_bcsr_transpose_atomic_kernel (core/include/spmm_tc.cuh:238-269):        */
/*   grad_in[col] += A[r,c] * grad_out[row]; -1 columns skipped (:258), zero weights skipped   */
/*   (:264).  The reference also skips |g| < 1e-9 (:250), which changes the sum by less than   */
/*   the tolerance; this restatement adds every term, in float64, in a fixed order.    */
/* ------------------------------------------------------------------------------------------ */
API void grws_oracle_spmm_transpose(int64_t W, int64_t F, int64_t tile_rows, int64_t tile_cols,
                                    const int64_t *window_offset, const int32_t *cols,
                                    const float *vals, const float *grad_out, int64_t num_cols,
                                    float *grad_in) {
    double *acc = (double *)calloc((size_t)(num_cols * F), sizeof(double));
    /* threads own contiguous ranges of output rows (column ids of A): every thread scans all column
     * ids and adds only the entries of its own rows, so every output element is summed by one
     * thread in (window, tile, row) order: parallel over all features at once, no atomics, and the
     * same result for any thread count */
#pragma omp parallel
    {
#ifdef _OPENMP
        const int nt = omp_get_num_threads(), tid = omp_get_thread_num();
#else
        const int nt = 1, tid = 0;
#endif
        const int64_t c0 = num_cols * tid / nt, c1 = num_cols * (tid + 1) / nt;
        if (c1 > c0)
            for (int64_t w = 0; w < W; ++w)
                for (int64_t t = window_offset[w]; t < window_offset[w + 1]; ++t) {
                    const int32_t *tc = cols + t * tile_cols;
                    int any = 0;
                    for (int64_t c = 0; c < tile_cols; ++c) any |= (tc[c] >= c0 && tc[c] < c1);
                    if (!any) continue;
                    for (int64_t r = 0; r < tile_rows; ++r) {
                        const float *g = grad_out + (w * tile_rows + r) * F;
                        for (int64_t c = 0; c < tile_cols; ++c) {
                            int32_t col = tc[c];
                            if (col < c0 || col >= c1) continue;        /* -1 is in nobody's range */
                            float a = vals[t * tile_rows * tile_cols + r * tile_cols + c];
                            if (a == 0.0f) continue;
                            double *o = acc + (int64_t)col * F;
                            for (int64_t f = 0; f < F; ++f) o[f] += (double)a * (double)g[f];
                        }
                    }
                }
    }
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < num_cols * F; ++i) grad_in[i] = (float)acc[i];
    free(acc);
}

/* ------------------------------------------------------------------------------------------ */
/* reindex + prune  (core/include/reindex.cuh:33-102)                                          */
/*   window of a column = col / tile_rows with C integer division, so a -1 padding id maps to  */
/*   window 0 (:48-51); a hit becomes found*tile_rows + col % tile_rows (:73-78); a miss       */
/*   becomes column 0 and zeroes that column of the tile's values in place (:79-100).          */
/* ------------------------------------------------------------------------------------------ */
API void grws_oracle_reindex(const int32_t *in_cols, float *values, const int32_t *active_windows,
                             int64_t num_indices, int64_t num_active, int32_t tile_rows,
                             int32_t tile_cols, int32_t *out_cols) {
    for (int64_t idx = 0; idx < num_indices; ++idx) {
        int32_t g = in_cols[idx];
        int32_t target = g / tile_rows;
        int64_t left = 0, right = num_active - 1, found = -1;
        while (left <= right) {
            int64_t mid = (left + right) / 2;
            int32_t win = active_windows[mid];
            if (win == target) { found = mid; break; }
            else if (win < target) left = mid + 1;
            else right = mid - 1;
        }
        if (found != -1) {
            out_cols[idx] = (int32_t)found * tile_rows + (g % tile_rows);
        } else {
            out_cols[idx] = 0;
            int64_t blk = idx / tile_cols, cit = idx % tile_cols;
            int64_t base = blk * tile_rows * tile_cols;
            for (int32_t r = 0; r < tile_rows; ++r) values[base + r * tile_cols + cit] = 0.0f;
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* seeds -> sorted unique (window, OR-mask)  (core/wrapper/sampling_wrapper.cu:307-346)        */
/*   node -> (node / tile_rows, 1 << (node % tile_rows)); -1 seeds are dropped (:311,340-344). */
/*   returns the number of active windows.                                                     */
/* ------------------------------------------------------------------------------------------ */
API int64_t grws_oracle_windows_and_masks(const int32_t *seeds, int64_t n, int32_t tile_rows,
                                          int32_t *out_windows, int32_t *out_masks) {
    int32_t *w = (int32_t *)malloc((size_t)(n > 0 ? n : 1) * sizeof(int32_t));
    int64_t m = 0;
    for (int64_t i = 0; i < n; ++i)
        if (seeds[i] != -1) w[m++] = seeds[i] / tile_rows;
    int64_t u = sort_unique_i32(w, m);
    for (int64_t i = 0; i < u; ++i) { out_windows[i] = w[i]; out_masks[i] = 0; }
    for (int64_t i = 0; i < n; ++i) {
        if (seeds[i] == -1) continue;
        int64_t p = lower_bound_i32(w, u, seeds[i] / tile_rows);
        out_masks[p] |= (int32_t)(1u << (seeds[i] % tile_rows));
    }
    free(w);
    return u;
}

/* ------------------------------------------------------------------------------------------ */
/* Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3",   */
/* SC'11).  The reference has no random sampler (its sampler is a deterministic top-K,         */
/* core/include/sampling.cuh:65-448); the uniform sampler below is this build's own            */
/* definition and this host replay is its bit-exact specification.                             */
/* ------------------------------------------------------------------------------------------ */
#define PHILOX_M0 0xD2511F53u
#define PHILOX_M1 0xCD9E8D57u
#define PHILOX_W0 0x9E3779B9u
#define PHILOX_W1 0xBB67AE85u

API void grws_oracle_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3];
    uint32_t k0 = key[0], k1 = key[1];
    for (int r = 0; r < 10; ++r) {
        uint64_t p0 = (uint64_t)PHILOX_M0 * c0;
        uint64_t p1 = (uint64_t)PHILOX_M1 * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += PHILOX_W0; k1 += PHILOX_W1;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

/* j-th 64-bit draw of the stream keyed by (seed, node, hop): Philox counter
 * {node, hop, j >> 1, 0}, key {seed_lo, seed_hi}; draw = words (2*(j&1)+1 : 2*(j&1)). */
static uint64_t sample_draw64(uint64_t seed, uint32_t node, uint32_t hop, uint32_t j) {
    uint32_t ctr[4] = {node, hop, j >> 1, 0u};
    uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
    uint32_t o[4];
    grws_oracle_philox4x32_10(ctr, key, o);
    uint32_t lo = o[2 * (j & 1)], hi = o[2 * (j & 1) + 1];
    return ((uint64_t)hi << 32) | lo;
}

static uint64_t mulhi64(uint64_t a, uint64_t b) {
    return (uint64_t)(((unsigned __int128)a * (unsigned __int128)b) >> 64);
}

/* ------------------------------------------------------------------------------------------ */
/* one hop of uniform neighbour sampling without replacement over a CSR graph.                 */
/*   for node v with degree d and fanout f:                                                    */
/*     d <= f : all d neighbours in CSR order;                                                 */
/*     d >  f : Floyd's subset algorithm: for j = 0..f-1: t = floor(draw_j * (d-f+j+1) / 2^64);*/
/*              pick t unless an earlier pick equals t, then pick d-f+j.  Picks are emitted    */
/*              in j order.                                                                    */
/*   outputs have a fixed stride of f slots per node, unused slots are -1 / 0.                 */
/*   nodes equal to -1 produce an empty list.                                                  */
/* ------------------------------------------------------------------------------------------ */
API void grws_oracle_sample_hop(const int64_t *row_ptr, const int32_t *col_idx,
                                const float *values, const int32_t *nodes, int64_t num_nodes,
                                int32_t fanout, uint64_t seed, uint32_t hop,
                                int32_t *out_nbr /*[n*f]*/, float *out_w /*[n*f]*/,
                                int32_t *out_cnt /*[n]*/) {
#pragma omp parallel for schedule(dynamic, 256)
    for (int64_t i = 0; i < num_nodes; ++i) {
        int32_t v = nodes[i];
        int32_t *nb = out_nbr + i * fanout;
        float *ww = out_w + i * fanout;
        for (int32_t j = 0; j < fanout; ++j) { nb[j] = -1; ww[j] = 0.0f; }
        if (v < 0) { out_cnt[i] = 0; continue; }
        int64_t e0 = row_ptr[v], d = row_ptr[v + 1] - e0;
        if (d <= fanout) {
            for (int64_t j = 0; j < d; ++j) { nb[j] = col_idx[e0 + j]; ww[j] = values ? values[e0 + j] : 1.0f; }
            out_cnt[i] = (int32_t)d;
        } else {
            int64_t pick[1024];
            for (int32_t j = 0; j < fanout; ++j) {
                uint64_t bound = (uint64_t)(d - fanout + j + 1);
                int64_t t = (int64_t)mulhi64(sample_draw64(seed, (uint32_t)v, hop, (uint32_t)j), bound);
                int dup = 0;
                for (int32_t q = 0; q < j; ++q) if (pick[q] == t) { dup = 1; break; }
                pick[j] = dup ? (d - fanout + j) : t;
                nb[j] = col_idx[e0 + pick[j]];
                ww[j] = values ? values[e0 + pick[j]] : 1.0f;
            }
            out_cnt[i] = fanout;
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* dedup + reindex of one hop:                                                                 */
/*   src list = dst nodes (in the given order) followed by the ascending-sorted unique sampled */
/*   neighbours that are not dst nodes; local id of a node = its position in the src list.     */
/*   returns n_src; out_src must hold n_dst + n_dst*fanout entries; out_local [n_dst*fanout]   */
/*   gets the local id of every sampled neighbour (-1 for empty slots).                        */
/* ------------------------------------------------------------------------------------------ */
typedef struct { int32_t key, val; } kv_t;
static int cmp_kv(const void *a, const void *b) {
    int32_t x = ((const kv_t *)a)->key, y = ((const kv_t *)b)->key;
    return (x > y) - (x < y);
}

API int64_t grws_oracle_dedup_reindex(const int32_t *dst, int64_t n_dst, const int32_t *nbr,
                                      int32_t fanout, int32_t *out_src, int32_t *out_local) {
    int64_t ne = n_dst * fanout;
    kv_t *d = (kv_t *)malloc((size_t)(n_dst > 0 ? n_dst : 1) * sizeof(kv_t));
    for (int64_t i = 0; i < n_dst; ++i) { d[i].key = dst[i]; d[i].val = (int32_t)i; }
    qsort(d, (size_t)n_dst, sizeof(kv_t), cmp_kv);
    int32_t *cand = (int32_t *)malloc((size_t)(ne > 0 ? ne : 1) * sizeof(int32_t));
    int64_t nc = 0;
    for (int64_t e = 0; e < ne; ++e) {
        int32_t u = nbr[e];
        if (u < 0) continue;
        kv_t probe = {u, 0};
        if (n_dst > 0 && bsearch(&probe, d, (size_t)n_dst, sizeof(kv_t), cmp_kv)) continue;
        cand[nc++] = u;
    }
    int64_t nu = sort_unique_i32(cand, nc);
    for (int64_t i = 0; i < n_dst; ++i) out_src[i] = dst[i];
    for (int64_t i = 0; i < nu; ++i) out_src[n_dst + i] = cand[i];
    for (int64_t e = 0; e < ne; ++e) {
        int32_t u = nbr[e];
        if (u < 0) { out_local[e] = -1; continue; }
        kv_t probe = {u, 0};
        kv_t *hit = n_dst > 0 ? (kv_t *)bsearch(&probe, d, (size_t)n_dst, sizeof(kv_t), cmp_kv) : NULL;
        if (hit) {
            /* duplicates in dst: the first position wins */
            int32_t best = hit->val;
            for (kv_t *p = hit; p >= d && p->key == u; --p) if (p->val < best) best = p->val;
            for (kv_t *p = hit; p < d + n_dst && p->key == u; ++p) if (p->val < best) best = p->val;
            out_local[e] = best;
        } else {
            out_local[e] = (int32_t)(n_dst + lower_bound_i32(cand, nu, u));
        }
    }
    free(cand); free(d);
    return n_dst + nu;
}
