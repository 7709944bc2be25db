/*
 * csg_oracle.c -- CPU restatement of the reference's Chunked Greedy (csg) path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library and
 * the timed CPU baseline; nothing in the product path may call it.
 *
 * Parity status: pinned.  The reference holds no golden vectors for csg
 * (its only test, sporder/tests/smoke.c, checks permutation validity of other
 * entry points), so this restatement is pinned against outputs of the
 * reference's own CUDA library run on a B200 (tests/golden/, produced by
 * tests/golden/make_golden.py from oracle/_ref/libsporder_ref.so).
 *
 * Every function cites the reference file:line whose arithmetic it restates.
 * The reference computes on the GPU with one warp per row / per chunk; none of
 * its results depend on thread scheduling, so a sequential restatement is exact.
 * Compile without fast-math and with -ffp-contract=off.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ---- packed (weight, index) entry: sporder/src/common/weighted_index.h:15-27 ----
 * high 32 bits = IEEE bit pattern of the fp32 weight, low 32 bits = index + 1;
 * the all-zero word decodes to (index -1, weight 0). */
static inline uint64_t pack_entry(int32_t idx, float w) {
  uint32_t wb;
  memcpy(&wb, &w, 4);
  return ((uint64_t)wb << 32) | (uint32_t)(idx + 1);
}
static inline int32_t entry_index(uint64_t e) { return (int32_t)(e & 0xFFFFFFFFu) - 1; }
static inline float entry_weight(uint64_t e) {
  uint32_t wb = (uint32_t)(e >> 32);
  float w;
  memcpy(&w, &wb, 4);
  return w;
}

/* ---- parameter resolution: sporder/src/sporder.cpp:147-161 and
 * sporder/src/common/chunk_similarity_top_k.cu:111-147 ----
 * returns 0 on success, nonzero when the reference would abort. */
ORACLE_API int oracle_resolve_params(int32_t n, int32_t nnz, int32_t *k, float *ovs,
                                     int32_t *chunk, int32_t *m_used, int32_t *M) {
  if (*k <= 0) {
    int32_t a = nnz / n;
    if (a < 16) a = 16;
    if (a > 256) a = 256;
    *k = a;
  }
  if (*ovs <= 0.0f) *ovs = 4.0f;
  if (*chunk <= 0) *chunk = 1024;
  int32_t m = (int32_t)((float)(*k) * (*ovs));
  *m_used = ((m + 31) / 32) * 32; /* what the stats struct reports */
  if (*ovs < 1.0f) return 1;
  if (m > 512) return 2;
  int32_t mm = m < 1 ? 1 : m;
  *M = ((mm + 31) / 32) * 32; /* kernel instantiation chosen by the binary dispatch */
  return 0;
}

/* ---- CSR -> CSC: sporder/src/common/csr2csc.cu:62-113 ----
 * (stable sort of row-major (col,row) pairs by column => rows ascending per column) */
ORACLE_API void oracle_csr2csc_rect(int32_t n, int32_t ncols, int32_t nnz, const int32_t *ptr,
                                    const int32_t *ind, int32_t *col_ptr, int32_t *row_ind) {
  memset(col_ptr, 0, sizeof(int32_t) * ((size_t)ncols + 1));
  for (int32_t i = 0; i < nnz; ++i) col_ptr[ind[i] + 1]++;
  for (int32_t c = 0; c < ncols; ++c) col_ptr[c + 1] += col_ptr[c];
  int32_t *fill = (int32_t *)malloc(sizeof(int32_t) * ((size_t)ncols + 1));
  memcpy(fill, col_ptr, sizeof(int32_t) * ((size_t)ncols + 1));
  for (int32_t r = 0; r < n; ++r)
    for (int32_t p = ptr[r]; p < ptr[r + 1]; ++p) row_ind[fill[ind[p]]++] = r;
  free(fill);
}
ORACLE_API void oracle_csr2csc(int32_t n, int32_t nnz, const int32_t *ptr, const int32_t *ind,
                               int32_t *col_ptr, int32_t *row_ind) {
  oracle_csr2csc_rect(n, n, nnz, ptr, ind, col_ptr, row_ind);
}

/* ---- Space-Saving sketch of one row + top-k selection ----
 * container: sporder/src/common/warp_spacesaving.cuh:24-151
 * stream:    sporder/src/common/chunk_similarity_top_k.cu:39-87
 * tie rules: sporder/src/common/cuda_util.cuh:66-87
 *
 * The reference keeps M slots as CELLS = M/32 registers in each of 32 lanes.
 * Slot (lane, cell) is stored here at index lane*CELLS + cell, which is also
 * the fill order (the j-th distinct key lands in lane j/CELLS, cell j%CELLS).
 * `where` maps a chunk-local row to its slot (+1), 0 when absent: it only
 * accelerates the reference's linear key search and does not change results. */
typedef struct {
  int32_t *key;
  float *w;
  int16_t *where; /* chunk_len entries */
} sketch_t;

static void sketch_row(int32_t r, int32_t n, int32_t k, int32_t chunk, int32_t M,
                       const int32_t *ptr, const int32_t *ind, const int32_t *col_ptr,
                       const int32_t *row_ind, sketch_t *sk, uint64_t *out) {
  const int32_t CELLS = M / 32;
  const int32_t row_begin = ptr[r], row_end = ptr[r + 1];
  const int32_t row_size = row_end - row_begin;
  if (row_size == 0) return; /* chunk_similarity_top_k.cu:42-44: entries stay zero */
  const int32_t chunk_start = (r / chunk) * chunk;
  int32_t chunk_end = chunk_start + chunk;
  if (chunk_end > n || chunk_end < 0) chunk_end = n;

  int32_t filled = 0;
  for (int32_t j = 0; j < M; ++j) {
    sk->key[j] = -1;
    sk->w[j] = 0.0f;
  }
  for (int32_t p = row_begin; p < row_end; ++p) {
    const int32_t c = ind[p];
    for (int32_t q = col_ptr[c]; q < col_ptr[c + 1]; ++q) {
      const int32_t s = row_ind[q];
      if (s < chunk_start) continue;
      if (s >= chunk_end) break; /* ascending rows: nothing further emits */
      if (s == r) continue;
      /* chunk_similarity_top_k.cu:73-75: int add, int->fp32, IEEE fp32 divide */
      const float alpha = 2.0f / (float)(row_size + (ptr[s + 1] - ptr[s]));
      const int32_t loc = s - chunk_start;
      int32_t slot = sk->where[loc] - 1;
      if (slot >= 0) { /* warp_spacesaving.cuh:111-119: key present, accumulate */
        sk->w[slot] += alpha;
      } else if (filled < M) { /* :121-131: lowest lane, then lowest cell, that is empty */
        slot = filled++;
        sk->key[slot] = s;
        sk->w[slot] = alpha;
        sk->where[loc] = (int16_t)(slot + 1);
      } else { /* :133-150: evict min by (weight, cell, lane); new weight = min + alpha */
        int32_t best = 0;
        float bw = sk->w[0];
        int32_t bkey = 0; /* (cell << 5) | lane of slot 0 */
        for (int32_t j = 1; j < M; ++j) {
          const int32_t lane = j / CELLS, cell = j % CELLS;
          const int32_t tk = (cell << 5) | lane;
          const float wj = sk->w[j];
          if (wj < bw || (wj == bw && tk < bkey)) {
            bw = wj;
            bkey = tk;
            best = j;
          }
        }
        sk->where[sk->key[best] - chunk_start] = 0;
        sk->key[best] = s;
        sk->w[best] = bw + alpha;
        sk->where[loc] = (int16_t)(best + 1);
      }
    }
  }
  /* reset the direct map for the next row of this thread */
  for (int32_t j = 0; j < filled; ++j) sk->where[sk->key[j] - chunk_start] = 0;

  /* per-lane selection sort, descending weight: warp_spacesaving.cuh:71-90 */
  for (int32_t lane = 0; lane < 32; ++lane) {
    int32_t *kk = sk->key + lane * CELLS;
    float *ww = sk->w + lane * CELLS;
    for (int32_t i = 0; i < CELLS - 1; ++i) {
      int32_t best = i;
      if (kk[best] == -1) break;
      for (int32_t j = i + 1; j < CELLS; ++j) {
        if (kk[j] == -1) break;
        if (ww[j] > ww[best]) best = j;
      }
      if (best != i) {
        int32_t tk = kk[i];
        kk[i] = kk[best];
        kk[best] = tk;
        float tw = ww[i];
        ww[i] = ww[best];
        ww[best] = tw;
      }
    }
  }
  /* k rounds of arg-max over the lanes' cursors: warp_spacesaving.cuh:46-66 */
  int32_t pos[32];
  for (int32_t lane = 0; lane < 32; ++lane) pos[lane] = 0;
  for (int32_t i = 0; i < k; ++i) {
    int all_done = 1;
    for (int32_t lane = 0; lane < 32; ++lane)
      if (!(pos[lane] >= CELLS || sk->key[lane * CELLS + pos[lane]] == -1)) all_done = 0;
    if (all_done) break;
    int32_t best_lane = 0;
    float best_w = (pos[0] < CELLS) ? sk->w[pos[0]] : 0.0f;
    for (int32_t lane = 1; lane < 32; ++lane) {
      const float wl = (pos[lane] < CELLS) ? sk->w[lane * CELLS + pos[lane]] : 0.0f;
      if (wl > best_w) { /* ties keep the smaller lane (cuda_util.cuh:72-76) */
        best_w = wl;
        best_lane = lane;
      }
    }
    const int32_t j = best_lane * CELLS + pos[best_lane];
    out[i] = pack_entry(sk->key[j], sk->w[j]);
    pos[best_lane]++;
  }
}

/* ---- top-k table for all rows: chunk_similarity_top_k.cu:137-154 ----
 * table[n*k] packed entries; unused entries are zero.  col_ptr/row_ind are the
 * CSC (or the CSR itself when the caller promised symmetry: csr2csc.h:52-54). */
/* ncols > n describes a block of whole chunks cut out of a larger matrix (rows
 * renumbered from 0, columns kept): every chunk of the block sees exactly the
 * candidates it sees inside the full matrix, because candidates never leave a
 * chunk.  Used for row shards and for the bounded samples of the CPU baseline. */
ORACLE_API int oracle_csg_table_rect(int32_t n, int32_t ncols, int32_t nnz, const int32_t *ptr,
                                     const int32_t *ind, int is_symmetric, int32_t k, float ovs,
                                     int32_t chunk, uint64_t *table) {
  int32_t m_used, M;
  if (n < 1 || ncols < n) return 3;
  if (is_symmetric && ncols != n) return 3;
  if (oracle_resolve_params(n, nnz, &k, &ovs, &chunk, &m_used, &M)) return 1;
  int32_t *col_ptr = NULL, *row_ind = NULL;
  const int32_t *cp = ptr, *ri = ind;
  if (!is_symmetric) {
    col_ptr = (int32_t *)malloc(sizeof(int32_t) * ((size_t)ncols + 1));
    row_ind = (int32_t *)malloc(sizeof(int32_t) * ((size_t)(nnz > 0 ? nnz : 1)));
    oracle_csr2csc_rect(n, ncols, nnz, ptr, ind, col_ptr, row_ind);
    cp = col_ptr;
    ri = row_ind;
  }
  memset(table, 0, sizeof(uint64_t) * (size_t)n * (size_t)k);
  const int32_t span = chunk < n ? chunk : n;
#pragma omp parallel
  {
    sketch_t sk;
    sk.key = (int32_t *)malloc(sizeof(int32_t) * (size_t)M);
    sk.w = (float *)malloc(sizeof(float) * (size_t)M);
    sk.where = (int16_t *)calloc((size_t)span, sizeof(int16_t));
#pragma omp for schedule(dynamic, 16)
    for (int32_t r = 0; r < n; ++r)
      sketch_row(r, n, k, chunk, M, ptr, ind, cp, ri, &sk, table + (size_t)r * k);
    free(sk.key);
    free(sk.w);
    free(sk.where);
  }
  free(col_ptr);
  free(row_ind);
  return 0;
}

ORACLE_API int oracle_csg_table(int32_t n, int32_t nnz, const int32_t *ptr, const int32_t *ind,
                                int is_symmetric, int32_t k, float ovs, int32_t chunk,
                                uint64_t *table) {
  return oracle_csg_table_rect(n, n, nnz, ptr, ind, is_symmetric, k, ovs, chunk, table);
}

/* ---- greedy chain per chunk: sporder/src/csg/chunk_similarity_greedy.cu:14-96,
 * bitmap scan sporder/src/common/warp_visited_bitmap.cuh:99-111 ----
 * counters (may be NULL): restarts, links, sum of followed link weights. */
ORACLE_API void oracle_greedy(int32_t n, int32_t k, int32_t chunk, const uint64_t *table,
                              int32_t *order, int64_t *restarts_out, int64_t *links_out,
                              double *link_weight_out) {
  const int32_t num_chunks = (int32_t)(((int64_t)n + chunk - 1) / chunk);
  int64_t restarts = 0, links = 0;
  double link_w = 0.0;
#pragma omp parallel for schedule(dynamic, 4) reduction(+ : restarts, links, link_w)
  for (int32_t q = 0; q < num_chunks; ++q) {
    const int64_t start64 = (int64_t)q * chunk;
    const int32_t start = (int32_t)start64;
    const int32_t end = (start64 + chunk > n) ? n : (int32_t)(start64 + chunk);
    const int32_t size = end - start;
    uint8_t *visited = (uint8_t *)calloc((size_t)size, 1);
    int32_t cur = start, pos = start, scan_from = 0;
    float chunk_link_w = 0.0f; /* fp32 per chunk, then fp64 (:33,:91-93) */
    for (;;) {
      visited[cur - start] = 1;
      order[pos++] = cur;
      const uint64_t *row = table + (size_t)cur * k;
      float best_w = -1.0f;
      int32_t best_c = -1;
      for (int32_t j = 0; j < k; ++j) {
        const int32_t cand = entry_index(row[j]);
        if (cand < 0) break; /* valid entries form a prefix */
        if (cand < start || cand >= end) continue;
        if (visited[cand - start]) continue;
        const float w = entry_weight(row[j]);
        if (w > best_w || (w == best_w && cand < best_c)) {
          best_w = w;
          best_c = cand;
        }
      }
      if (best_c >= 0) {
        links += 1;
        chunk_link_w += best_w;
        cur = best_c;
        continue;
      }
      while (scan_from < size && visited[scan_from]) ++scan_from; /* smallest unvisited */
      if (scan_from >= size) break;
      cur = start + scan_from;
      restarts += 1;
    }
    link_w += (double)chunk_link_w;
    free(visited);
  }
  if (restarts_out) *restarts_out = restarts;
  if (links_out) *links_out = links;
  if (link_weight_out) *link_weight_out = link_w;
}

/* ---- table statistics: sporder/src/common/similarity_top_k.cu:120-157 ---- */
ORACLE_API void oracle_table_stats(int32_t n, int32_t k, const uint64_t *table,
                                   int64_t *total_degree, double *total_weight,
                                   int32_t *zero_rows) {
  int64_t deg = 0;
  double wsum = 0.0;
  int32_t zero = 0;
  for (int32_t r = 0; r < n; ++r) {
    int32_t d = 0;
    float rw = 0.0f;
    for (int32_t j = 0; j < k; ++j) {
      const uint64_t e = table[(size_t)r * k + j];
      if (entry_index(e) == -1) break;
      d += 1;
      rw += entry_weight(e);
    }
    deg += d;
    wsum += (double)rw;
    zero += (d == 0);
  }
  *total_degree = deg;
  *total_weight = wsum;
  *zero_rows = zero;
}

/* stats layout mirrors sporder_csg_stats_t (sporder/include/sporder.h:213-222) */
typedef struct {
  int32_t k_used;
  int32_t m_used;
  double avg_degree;
  double avg_edge_weight;
  int32_t zero_degree_rows;
  int32_t chunk_size_used;
  int32_t chain_restarts;
  double avg_followed_weight;
} oracle_csg_stats_t;

/* ---- whole pipeline: sporder.cpp:140-166 + chunk_similarity_greedy.cu:100-138 ----
 * table_out (may be NULL) receives the n*k_used table; stats may be NULL.
 * returns 0, or nonzero where the reference would abort. */
ORACLE_API int oracle_csg_rect(int32_t n, int32_t ncols, int32_t nnz, const int32_t *ptr,
                               const int32_t *ind, int is_symmetric, int32_t k, float ovs,
                               int32_t chunk, int32_t *new_order, uint64_t *table_out,
                               oracle_csg_stats_t *stats) {
  int32_t m_used, M;
  if (n < 1) return 3;
  if (oracle_resolve_params(n, nnz, &k, &ovs, &chunk, &m_used, &M)) return 1;
  uint64_t *table = table_out;
  if (!table) table = (uint64_t *)malloc(sizeof(uint64_t) * (size_t)n * (size_t)k);
  int rc = oracle_csg_table_rect(n, ncols, nnz, ptr, ind, is_symmetric, k, ovs, chunk, table);
  if (rc) {
    if (!table_out) free(table);
    return rc;
  }
  int64_t restarts = 0, links = 0;
  double link_w = 0.0;
  oracle_greedy(n, k, chunk, table, new_order, &restarts, &links, &link_w);
  if (stats) {
    int64_t deg;
    double wsum;
    int32_t zero;
    oracle_table_stats(n, k, table, &deg, &wsum, &zero);
    stats->k_used = k;
    stats->m_used = m_used;
    stats->chunk_size_used = chunk;
    stats->avg_degree = (double)deg / n; /* csg/stats_collector.cu:53-62 */
    stats->avg_edge_weight = deg > 0 ? wsum / (double)deg : 0.0;
    stats->zero_degree_rows = zero;
    stats->chain_restarts = (int32_t)restarts;
    stats->avg_followed_weight = links > 0 ? link_w / (double)links : 0.0;
  }
  if (!table_out) free(table);
  return 0;
}

ORACLE_API int oracle_csg(int32_t n, int32_t nnz, const int32_t *ptr, const int32_t *ind,
                          int is_symmetric, int32_t k, float ovs, int32_t chunk,
                          int32_t *new_order, uint64_t *table_out, oracle_csg_stats_t *stats) {
  return oracle_csg_rect(n, n, nnz, ptr, ind, is_symmetric, k, ovs, chunk, new_order, table_out,
                         stats);
}

/* ---- permutation application: sporder/src/reorder.cu:72-149 ----
 * mode 0 = rows only, 1 = symmetric (columns remapped by old2new, rows re-sorted). */
typedef struct {
  int32_t c;
  float v;
} colval_t;
static int cmp_colval(const void *a, const void *b) {
  const int32_t x = ((const colval_t *)a)->c, y = ((const colval_t *)b)->c;
  return (x > y) - (x < y);
}
ORACLE_API void oracle_reorder(int32_t n, int32_t nnz, const int32_t *ptr_old,
                               const int32_t *ind_old, const float *val_old,
                               const int32_t *new_order, int mode, int32_t *ptr_new,
                               int32_t *ind_new, float *val_new) {
  (void)nnz;
  const int with_vals = val_old != NULL && val_new != NULL;
  ptr_new[0] = 0;
  for (int32_t p = 0; p < n; ++p) {
    const int32_t src = new_order[p];
    ptr_new[p + 1] = ptr_new[p] + (ptr_old[src + 1] - ptr_old[src]);
  }
  int32_t *old2new = NULL;
  if (mode == 1) {
    old2new = (int32_t *)malloc(sizeof(int32_t) * (size_t)n);
    for (int32_t p = 0; p < n; ++p) old2new[new_order[p]] = p;
  }
#pragma omp parallel
  {
    colval_t *buf = NULL;
    size_t cap = 0;
#pragma omp for schedule(dynamic, 64)
    for (int32_t p = 0; p < n; ++p) {
      const int32_t src = new_order[p];
      const int32_t b = ptr_old[src], len = ptr_old[src + 1] - b, dst = ptr_new[p];
      if (mode == 0) {
        for (int32_t j = 0; j < len; ++j) {
          ind_new[dst + j] = ind_old[b + j];
          if (with_vals) val_new[dst + j] = val_old[b + j];
        }
        continue;
      }
      if ((size_t)len > cap) {
        cap = (size_t)len * 2;
        free(buf);
        buf = (colval_t *)malloc(sizeof(colval_t) * cap);
      }
      for (int32_t j = 0; j < len; ++j) {
        buf[j].c = old2new[ind_old[b + j]];
        buf[j].v = with_vals ? val_old[b + j] : 0.0f;
      }
      qsort(buf, (size_t)len, sizeof(colval_t), cmp_colval); /* keys are distinct */
      for (int32_t j = 0; j < len; ++j) {
        ind_new[dst + j] = buf[j].c;
        if (with_vals) val_new[dst + j] = buf[j].v;
      }
    }
    free(buf);
  }
  free(old2new);
}

/* ---- SpMM checkers (the reference has no first-party SpMM; it times third-party
 * kernels through bench/spmm/spmm_bench/base.py:48-59 and cuSPARSE through
 * sporder/src/bench_cusparse_spmm.cu:64-90).  C = A * B, B and C row-major n x w.
 * The f64 version also returns sum_j |a_ij * b_jl| for the scaled tolerance. ---- */
ORACLE_API void oracle_spmm_f64(int32_t n, int32_t w, const int32_t *ptr, const int32_t *ind,
                                const float *val, const float *B, double *C, double *Cabs) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int32_t r = 0; r < n; ++r) {
    double *c = C + (size_t)r * w;
    double *ca = Cabs ? Cabs + (size_t)r * w : NULL;
    for (int32_t l = 0; l < w; ++l) {
      c[l] = 0.0;
      if (ca) ca[l] = 0.0;
    }
    for (int32_t p = ptr[r]; p < ptr[r + 1]; ++p) {
      const double a = (double)val[p];
      const float *b = B + (size_t)ind[p] * w;
      for (int32_t l = 0; l < w; ++l) {
        const double t = a * (double)b[l];
        c[l] += t;
        if (ca) ca[l] += fabs(t);
      }
    }
  }
}

ORACLE_API void oracle_spmm_f32(int32_t n, int32_t w, const int32_t *ptr, const int32_t *ind,
                                const float *val, const float *B, float *C) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int32_t r = 0; r < n; ++r) {
    float *c = C + (size_t)r * w;
    for (int32_t l = 0; l < w; ++l) c[l] = 0.0f;
    for (int32_t p = ptr[r]; p < ptr[r + 1]; ++p) {
      const float a = val[p];
      const float *b = B + (size_t)ind[p] * w;
      for (int32_t l = 0; l < w; ++l) c[l] += a * b[l];
    }
  }
}

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
ORACLE_API void oracle_set_num_threads(int t) {
#ifdef _OPENMP
  if (t > 0) omp_set_num_threads(t);
#else
  (void)t;
#endif
}

/* Pillar count, sporder/src/count_pillars.cu:11-35,38-85: the reference keys every nonzero
 * with (row / height, column), sorts the keys and counts the distinct ones.  Restated with a
 * per-window marker array instead of a sort: a column is counted the first time a window
 * meets it.  Returns -1 on bad arguments. */
ORACLE_API int64_t oracle_count_pillars(int32_t n, int32_t ncols, const int32_t *ptr,
                                        const int32_t *ind, int32_t height) {
  if (n < 1 || ncols < 1 || height < 1) return -1;
  int32_t *last = (int32_t *)malloc(sizeof(int32_t) * (size_t)ncols);
  if (!last) return -1;
  for (int32_t c = 0; c < ncols; ++c) last[c] = -1;
  int64_t count = 0;
  for (int32_t r = 0; r < n; ++r) {
    const int32_t window = r / height;
    for (int32_t p = ptr[r]; p < ptr[r + 1]; ++p) {
      const int32_t c = ind[p];
      if (last[c] != window) {
        last[c] = window;
        ++count;
      }
    }
  }
  free(last);
  return count;
}
