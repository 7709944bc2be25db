/*
 * sporder_b200.h -- C ABI of the B200 (sm_100a) Chunked Greedy library.
 *
 * The first four entry points are the ones the reference's Python binding and C
 * callers bind for the csg path; names, argument order, argument meaning and
 * struct layouts are those of the reference header, so a program linked against
 * the reference's libsporder can load this library instead for that path.
 * Everything below them is new surface without a reference counterpart.
 *
 * Conventions (same as sporder/include/sporder.h:13-41 unless stated):
 *   - calls are synchronous: results are ready when the call returns;
 *   - d_ pointers are device memory on the context's device, h_ pointers are host
 *     memory, all other pointers are host memory;
 *   - CSR patterns are square, zero-based, column indices sorted and unique
 *     inside a row;
 *   - permutations are new2old: new row p holds old row d_new_order[p];
 *   - DIFFERENCE: the reference aborts the process on invalid arguments and CUDA
 *     errors (sporder/src/common/error_checking.h:20-29).  This library never
 *     aborts: the call returns early, outputs are unspecified, and
 *     sporder_last_error() returns the message (NULL when the last call on this
 *     thread succeeded).
 *   - `is_symmetric` is the reference's promise that the pattern equals its
 *     transpose (sporder/src/common/csr2csc.h:49-59, where the CSR arrays are then
 *     read as the CSC).  With it the library reads the column groups straight off
 *     the CSR arrays instead of sorting; results are the same as without it on a
 *     symmetric pattern.  On a pattern that is not symmetric a true promise gives a
 *     different, still valid permutation (as in the reference) and never an
 *     out-of-range access.  Row shards (sporder_csg_shard) have no such parameter.
 */
#ifndef SPORDER_B200_H
#define SPORDER_B200_H

#include <stdbool.h>
#include <stdint.h>

#define SPORDER_API __attribute__((visibility("default")))

#ifdef __cplusplus
extern "C" {
#endif

/* replaces sporder/include/sporder.h:43-52 */
typedef struct sporder_context_struct *sporder_context_t;
SPORDER_API sporder_context_t sporder_context_create(void);
SPORDER_API void sporder_context_destroy(sporder_context_t h);

/* replaces sporder/include/sporder.h:203-211 (same layout) */
typedef struct {
  double wall_ms;
  float csr2csc_ms;      /* here: the chunk-local transpose */
  float similarity_ms;   /* sketch + top-k */
  float chunk_greedy_ms; /* greedy chaining */
} sporder_csg_timing_t;

/* replaces sporder/include/sporder.h:213-222 (same layout) */
typedef struct {
  int32_t k_used;
  int32_t m_used;
  double avg_degree;
  double avg_edge_weight;
  int32_t zero_degree_rows;
  int32_t chunk_size_used;
  int32_t chain_restarts;
  double avg_followed_weight;
} sporder_csg_stats_t;

/* replaces sporder/include/sporder.h:224-228.
 * k <= 0 -> min(256, max(16, nnz / n)); oversampling <= 0 -> 4.0;
 * chunk_size <= 0 -> 1024 (sporder/src/sporder.cpp:147-155).
 * Errors (instead of the reference's abort): oversampling in (0,1),
 * int(k * oversampling) > 512, n < 1. */
SPORDER_API void sporder_chunk_similarity_greedy(
    sporder_context_t ctx, int32_t n, int32_t nnz, const int32_t *d_ptr, const int32_t *d_ind,
    bool is_symmetric, int32_t k, float oversampling, int32_t chunk_size, int32_t *d_new_order,
    sporder_csg_timing_t *timing, sporder_csg_stats_t *stats);

/* replaces sporder/include/sporder.h:128-133 (same layout) */
typedef struct {
  double wall_ms;
  float csr2csc_ms;
  float similarity_ms;
  float chunk_greedy_ms;
} sporder_cg_timing_t;

/* replaces sporder/include/sporder.h:154-167 (same layout) */
typedef struct {
  int32_t k_used;
  int32_t m_used;
  double avg_degree;
  double avg_edge_weight;
  int32_t zero_degree_rows;
  int32_t chunk_size_used;
  int32_t chain_restarts;
  double avg_followed_weight;
  double cut_weight_fraction; /* edge weight crossing chunk boundaries over total edge weight */
} sporder_cg_stats_t;

/* replaces sporder/include/sporder.h:176-182 (sporder/src/cg/chunk_greedy.cu:118-163): the
 * top-k graph of the WHOLE matrix (as sporder_similarity_graph, with the defaults
 * k <= 0 -> min(256, max(16, nnz / n)), oversampling <= 0 -> 4.0, chunk_size <= 0 -> 1024 of
 * sporder/src/sporder.cpp:118-126), then greedy chains inside chunks of chunk_size rows;
 * neighbours outside a row's chunk are skipped.  new2old permutation, as csg. */
SPORDER_API void sporder_chunk_greedy(sporder_context_t ctx, int32_t n, int32_t nnz,
                                      const int32_t *d_ptr, const int32_t *d_ind, bool is_symmetric,
                                      int32_t k, float oversampling, int32_t chunk_size,
                                      int32_t *d_new_order, sporder_cg_timing_t *timing,
                                      sporder_cg_stats_t *stats);

/* replaces sporder/include/sporder.h:312-317 (same layout) */
typedef struct {
  double wall_ms;
  float csr2csc_ms;    /* here: the transpose with the matrix as one chunk */
  float similarity_ms; /* sketch + top-k */
  float unpack_ms;
} sporder_sim_timing_t;

/* replaces sporder/include/sporder.h:322-328 (same layout) */
typedef struct {
  int32_t k_used;
  int32_t m_used;
  double avg_degree;
  double avg_edge_weight;
  int32_t zero_degree_rows;
} sporder_sim_stats_t;

/* replaces sporder/include/sporder.h:330-335 (sporder/src/similarity_graph.cu:26-107):
 * for each row up to k rows with the largest sketched Dice similarity, as
 * d_indices[r * k + j] / d_weights[r * k + j], unused entries index -1, weight 0.
 * k <= 0 -> min(32, max(16, 2 * (nnz / n))); oversampling <= 0 -> 2.0
 * (sporder/src/sporder.cpp:75-80).  The outputs must hold n * k entries for the k in
 * use; the return value is that k (the reference returns nothing), -1 on error.
 * is_symmetric: see sporder_chunk_similarity_greedy. */
SPORDER_API int32_t sporder_similarity_graph(sporder_context_t ctx, int32_t n, int32_t nnz,
                                             const int32_t *d_ptr, const int32_t *d_ind,
                                             bool is_symmetric, int32_t k, float oversampling,
                                             int32_t *d_indices, float *d_weights,
                                             sporder_sim_timing_t *timing,
                                             sporder_sim_stats_t *stats);

/* replaces sporder/include/sporder.h:276-279 (sporder/src/count_pillars.cu:38-85):
 * *count = number of distinct (row / height, column) pairs of the pattern, the
 * reordering quality metric of the reference (fewer is better).  height >= 1.
 * Rows must hold their columns in ascending order for height <= 12 (the CSR contract of
 * this library and of the reference); taller windows accept any order.  count is a host
 * pointer; the call synchronises the context's stream.  On error *count is 0 and
 * sporder_last_error() says why (the reference aborts). */
SPORDER_API void sporder_count_pillars(sporder_context_t ctx, int32_t n, int32_t nnz,
                                       const int32_t *d_ptr, const int32_t *d_ind, int32_t height,
                                       int32_t *count);

/* replaces sporder/include/sporder.h:230-233 */
typedef enum {
  SPORDER_REORDER_ROWS = 0,
  SPORDER_REORDER_SYMMETRIC = 1,
} sporder_reorder_mode_t;

/* replaces sporder/include/sporder.h:253-258 */
SPORDER_API void sporder_reorder(sporder_context_t ctx, int32_t n, int32_t nnz,
                                 const int32_t *d_ptr_old, const int32_t *d_ind_old,
                                 const float *d_val_old, const int32_t *d_new_order,
                                 sporder_reorder_mode_t mode, int32_t *d_ptr_new,
                                 int32_t *d_ind_new, float *d_val_new);

/* ---- new surface (no counterpart in the reference) ------------------------- */

/* Message of the last failed call on this thread, or NULL. */
SPORDER_API const char *sporder_last_error(void);

/* Run the context's work on `stream` (a cudaStream_t) instead of the context's
 * private stream; NULL restores the private stream.  To name the legacy default
 * stream pass cudaStreamLegacy ((cudaStream_t)0x1), not 0.  Calls stay synchronous.
 * A context serves one stream at a time: switching to another stream first waits for
 * the work the context queued on the previous one (sporder_spmm_async). */
SPORDER_API void sporder_context_set_stream(sporder_context_t ctx, void *stream);

/* Upper bound, in stream elements of 8 bytes, on the buffer that holds the materialised
 * candidate streams of the heaviest rows (rows that stream 65536 candidates or more are
 * computed fastest from such a copy).  0 = no bound beyond the built-in 2^27 elements (1 GiB).
 * Without a bound a call plans max(8 * nnz, 2^20) elements, or what the largest earlier
 * call of this context needed, never more than nnz * chunk_size.  Rows that do not fit are
 * computed by the kernel of the lighter rows; results are the same for every bound. */
SPORDER_API void sporder_context_set_stream_limit(sporder_context_t ctx, uint64_t max_elements);

/* Calls of sporder_chunk_similarity_greedy (and its variants with a table, on host buffers or
 * on a row shard) with many nonzeros run the chunk that holds the most of them ahead of the
 * rest, on a second stream of the context: that chunk's transposition first, then the
 * chains of its heaviest rows, while everything else is still being transposed.  min_nnz
 * = 0: the built-in rule (2^24 nonzeros and 64 chunks or more); > 0: every call of at least
 * min_nnz nonzeros and two chunks; < 0: never.  Results are the same either way.  No
 * reference counterpart. */
SPORDER_API void sporder_context_set_ahead_threshold(sporder_context_t ctx, int64_t min_nnz);

/* Bytes of device workspace the context currently holds (grow-only cache). */
SPORDER_API uint64_t sporder_context_workspace_bytes(sporder_context_t ctx);

/* csg that also returns the top-k table: d_table receives n * k_used packed
 * entries (high 32 bits = fp32 bits of the weight, low 32 bits = index + 1,
 * 0 = empty; the reference's internal format, sporder/src/common/weighted_index.h:15-27).
 * d_table_capacity is the number of entries d_table can hold; d_new_order may be
 * NULL to skip the greedy stage.  Returns k_used, or -1 on error. */
SPORDER_API int32_t sporder_csg_with_table(sporder_context_t ctx, int32_t n, int32_t nnz,
                                           const int32_t *d_ptr, const int32_t *d_ind,
                                           bool is_symmetric, int32_t k, float oversampling,
                                           int32_t chunk_size, int32_t *d_new_order,
                                           uint64_t *d_table, uint64_t d_table_capacity,
                                           sporder_csg_timing_t *timing,
                                           sporder_csg_stats_t *stats);

/* csg of one row shard: rows [row_base, row_base + n_rows) of a matrix with n_cols
 * columns, given as a CSR block whose d_ptr is rebased to start at 0 and whose
 * column ids are the matrix's own.  row_base must be a multiple of chunk_size so
 * that the shard holds whole chunks; then its chunks see exactly the candidates
 * they see in the full matrix and the results (d_new_order[i], table indices) are
 * the full matrix's, already offset by row_base.  k and chunk_size should be
 * passed resolved (k <= 0 would resolve from the shard's own nnz / n_rows).
 * d_new_order and d_table may be NULL.  Returns k_used, or -1 on error. */
SPORDER_API int32_t sporder_csg_shard(sporder_context_t ctx, int32_t n_rows, int32_t n_cols,
                                      int32_t row_base, int32_t nnz, const int32_t *d_ptr,
                                      const int32_t *d_ind, int32_t k, float oversampling,
                                      int32_t chunk_size, int32_t *d_new_order,
                                      uint64_t *d_table, uint64_t d_table_capacity,
                                      sporder_csg_timing_t *timing, sporder_csg_stats_t *stats);

/* csg on host buffers: copies ptr/ind to the device, reorders, copies the
 * permutation back.  Returns 0, or -1 on error. */
SPORDER_API int32_t sporder_chunk_similarity_greedy_host(
    sporder_context_t ctx, int32_t n, int32_t nnz, const int32_t *h_ptr, const int32_t *h_ind,
    bool is_symmetric, int32_t k, float oversampling, int32_t chunk_size, int32_t *h_new_order,
    sporder_csg_timing_t *timing, sporder_csg_stats_t *stats);

/* fp32 CSR SpMM: C[n x w] = A * B with B, C row-major (ld = w).  n is the number of rows
 * of A (and of C); B must hold a row for every column id in d_ind, so A may be a row block
 * of a wider matrix (the row-partitioned multi-GPU product).  The reference
 * times third-party kernels (bench/spmm/spmm_bench/base.py:48-59) and cuSPARSE
 * (sporder/src/bench_cusparse_spmm.cu:64-90) here; it has no SpMM of its own.
 * Returns 0, or -1 on error. */
SPORDER_API int32_t sporder_spmm(sporder_context_t ctx, int32_t n, int32_t nnz, int32_t w,
                                 const int32_t *d_ptr, const int32_t *d_ind, const float *d_val,
                                 const float *d_B, float *d_C);

/* Same without the final stream synchronisation (for callers that time a train
 * of launches with events on the context's stream).  Returns 0 or -1. */
SPORDER_API int32_t sporder_spmm_async(sporder_context_t ctx, int32_t n, int32_t nnz, int32_t w,
                                       const int32_t *d_ptr, const int32_t *d_ind,
                                       const float *d_val, const float *d_B, float *d_C);

/* SpMM for callers that must not trigger a device allocation (no counterpart in the
 * reference).  Same product as sporder_spmm, but it takes no context and calls no
 * cudaMalloc / cudaFree or allocating routine: the queue of long rows sits in a fixed
 * array of 512 KiB plus 256 bytes of counters inside the library image (held by every
 * GPU that loads the library until the process exits).  Meant for hosts that gave all device memory to their own
 * pool, or that ban driver allocations on their request path because those stall the
 * whole device.
 *   - limit: nnz < 65536 * 1024 (67,108,864); larger inputs are rejected with an error;
 *   - the work is queued on `stream` (a cudaStream_t; NULL = default stream) and the
 *     call returns without waiting for it;
 *   - the first call on each device looks up the array's device address; make that
 *     first call before any stream capture;
 *   - all calls share the array: calls whose kernels may overlap on one GPU race.
 * Returns 0, or -1 on error (see sporder_last_error). */
SPORDER_API int32_t sporder_spmm_static(int32_t n, int32_t nnz, int32_t w, const int32_t *d_ptr,
                                        const int32_t *d_ind, const float *d_val,
                                        const float *d_B, float *d_C, void *stream);

/* Number of kernels this library has launched in this process (all contexts). */
SPORDER_API uint64_t sporder_kernel_launches(void);

#ifdef __cplusplus
}
#endif
#endif /* SPORDER_B200_H */
