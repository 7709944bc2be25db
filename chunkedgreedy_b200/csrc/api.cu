// C ABI of the library (include/sporder_b200.h): context, parameter resolution,
// the csg pipeline driver and the thin wrappers around reorder and SpMM.
#include "../../include/sporder_b200.h"

#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace csg {

// ---- error channel ---------------------------------------------------------
namespace {
thread_local char g_err[512];
thread_local bool g_has_err = false;
std::atomic<uint64_t> g_launches{0};
}  // namespace

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  g_has_err = true;
}
bool has_error() { return g_has_err; }
void clear_error() { g_has_err = false; }
void count_launches(int k) { g_launches.fetch_add(static_cast<uint64_t>(k), std::memory_order_relaxed); }

bool ensure_workspace(Context &ctx, size_t bytes) {
  if (bytes <= ctx.ws_bytes) return true;
  CSG_CUDA(cudaStreamSynchronize(ctx.stream));
  if (ctx.ws) CSG_CUDA(cudaFree(ctx.ws));
  ctx.ws = nullptr;
  ctx.ws_bytes = 0;
  const size_t want = bytes + (bytes >> 3);  // head room so that similar sizes reuse it
  cudaError_t e = cudaMalloc(&ctx.ws, want);
  if (e != cudaSuccess) {
    cudaGetLastError();
    e = cudaMalloc(&ctx.ws, bytes);
    if (e != cudaSuccess) {
      cudaGetLastError();
      set_error("device workspace of %zu bytes: %s", bytes, cudaGetErrorString(e));
      return false;
    }
    ctx.ws_bytes = bytes;
    return true;
  }
  ctx.ws_bytes = want;
  return true;
}

// sporder/src/sporder.cpp:147-161 and the checks of
// sporder/src/common/chunk_similarity_top_k.cu:143-147
bool resolve_params(int32_t n, int32_t nnz, int32_t k, float ovs, int32_t chunk, CsgParams *out) {
  CSG_REQUIRE(n >= 1, "n must be >= 1 (got %d)", n);
  CSG_REQUIRE(nnz >= 0, "nnz must be >= 0 (got %d)", nnz);
  if (k <= 0) {
    int32_t a = nnz / n;
    if (a < 16) a = 16;
    if (a > 256) a = 256;
    k = a;
  }
  if (ovs <= 0.0f) ovs = 4.0f;
  if (chunk <= 0) chunk = 1024;
  const int32_t m = static_cast<int32_t>(static_cast<float>(k) * ovs);
  out->k = k;
  out->ovs = ovs;
  out->chunk = chunk;
  out->m_used = ((m + 31) / 32) * 32;
  CSG_REQUIRE(ovs >= 1.0f, "expect oversampling >= 1 (got %g)", static_cast<double>(ovs));
  CSG_REQUIRE(m <= 512, "expect k * oversampling <= 512 (got %d)", m);
  const int32_t mm = m < 1 ? 1 : m;
  out->M = ((mm + 31) / 32) * 32;
  return true;
}

namespace {

struct ChainStatsHost {
  unsigned long long total_degree;
  double total_weight;
  double link_weight_sum;
  int32_t zero_degree_rows;
  int32_t restarts;
  int32_t links;
  int32_t pad;
  double in_chunk_weight;
};

size_t greedy_bitmap_words(int32_t n, int32_t chunk) {
  const int32_t span = chunk < n ? chunk : n;
  const size_t words = (static_cast<size_t>(span) + 31) / 32;
  if (4 /*warps*/ * 2 * words * sizeof(uint32_t) <= 48 * 1024) return 0;
  const size_t chunks = (static_cast<size_t>(n) + chunk - 1) / chunk;
  return chunks * 2 * words;
}

constexpr uint64_t STREAM_CAP_MAX = uint64_t(1) << 27;  // 2^27 elements = 1 GiB
constexpr int32_t AHEAD_MIN_NNZ = 1 << 24;  // smaller calls do not pay for a second pipeline's launches

// Stream elements the buffer of the heaviest rows gets for this call: never more than the
// rows could stream at all (nnz * chunk span), than 1 GiB or than the caller's limit; at
// least what the largest earlier call of the context asked for, and for a first call eight
// elements per nonzero (at least 2^20: 8 MiB).
uint64_t stream_capacity(const Context &ctx, size_t nnz, size_t span) {
  uint64_t cap = static_cast<uint64_t>(nnz) * 8;
  if (cap < (uint64_t(1) << 20)) cap = uint64_t(1) << 20;
  const uint64_t seen = ctx.stream_need_seen + (ctx.stream_need_seen >> 3);
  if (cap < seen) cap = seen;
  const uint64_t most = static_cast<uint64_t>(nnz) * span;
  if (cap > most) cap = most;
  if (cap > STREAM_CAP_MAX) cap = STREAM_CAP_MAX;
  if (ctx.stream_limit && cap > ctx.stream_limit) cap = ctx.stream_limit;
  return cap < 1 ? 1 : cap;
}

// Lays out the scratch of one csg call in the context workspace.  `transpose_only` leaves
// out everything behind the chunk-local transpose (the pillar count needs no more).
// With `prio` the call runs one chunk ahead of the rest (run_csg): that part gets control
// words, work lists and tile tables of its own and a share of the stream buffer.
bool plan_scratch(Context &ctx, int32_t n, int32_t nnz, const CsgParams &p, uint64_t *user_table,
                  CsgScratch *s, int32_t greedy_chunk = 0, bool transpose_only = false,
                  CsgScratch *prio = nullptr) {
  Arena ar;
  const size_t z = static_cast<size_t>(nnz > 0 ? nnz : 1);
  const size_t o_keyA = ar.take(4 * z), o_keyB = ar.take(4 * z);
  const size_t o_payA = ar.take(4 * z), o_payB = ar.take(4 * z);
  const size_t o_cand = ar.take(8 * z), o_seg = ar.take(8 * z), o_rank = ar.take(4 * z);
  const size_t o_work = ar.take(4 * static_cast<size_t>(n));
  const size_t o_list = ar.take(4 * static_cast<size_t>(n));
  const size_t o_ctrl = ar.take(4 * CTRL_WORDS);
  // (the greedy stage may run with another chunk size than the sketch: chunk_greedy)
  size_t bw = transpose_only ? 0 : greedy_bitmap_words(n, p.chunk);
  if (greedy_chunk > 0 && greedy_bitmap_words(n, greedy_chunk) > bw) bw = greedy_bitmap_words(n, greedy_chunk);
  const size_t o_bm = ar.take(4 * (bw ? bw : 1));
  // heavy chunks hold more than 15360 nonzeros each and are cut into tiles of 4096
  const size_t chunks = (static_cast<size_t>(n) + p.chunk - 1) / p.chunk;
  size_t heavy_max = z / 15360 + 1;
  if (heavy_max > chunks) heavy_max = chunks;
  const size_t tiles_max = z / 4096 + heavy_max + 1;
  const size_t o_hc = ar.take(4 * heavy_max), o_htb = ar.take(4 * (heavy_max + 1));
  const size_t o_th = ar.take(4 * 256 * tiles_max), o_db = ar.take(4 * 256 * heavy_max);
  // streams of the heaviest rows
  const size_t span = static_cast<size_t>(p.chunk < n ? p.chunk : n);
  const size_t cap = transpose_only ? 1 : static_cast<size_t>(stream_capacity(ctx, z, span));
  const size_t hmax = cap / (size_t(1) << (SKETCH_HEAVY_BUCKET - 1)) + 1;
  const size_t o_hs = ar.take(8 * cap), o_ho = ar.take(4 * (hmax + 1));
  const size_t o_hst = ar.take(4 * hmax * 2 * (p.M / 32) * 32);
  const size_t pmax = transpose_only ? 1 : z / SKETCH_PART_COLS + hmax + 1;  // column slices of the heavy rows
  const size_t o_pb = ar.take(4 * (hmax + 2)), o_po = ar.take(4 * (pmax + 1));
  const size_t o_table = (user_table || transpose_only) ? 0 : ar.take(8 * static_cast<size_t>(n) * p.k);
  // the part that runs ahead: one chunk's worth of lists, tile tables for up to all nonzeros
  // (nothing bounds a chunk's share of them), and its share of the stream buffer - what it
  // asked for in the context's last call plus an eighth, half the buffer on a first call
  size_t cap_p = 0, hmax_p = 0, pmax_p = 0;
  size_t o_p_list = 0, o_p_ctrl = 0, o_p_hc = 0, o_p_htb = 0, o_p_th = 0, o_p_db = 0, o_p_ho = 0, o_p_hst = 0,
         o_p_pb = 0, o_p_po = 0;
  if (prio) {
    cap_p = ctx.stream_need_prio ? static_cast<size_t>(ctx.stream_need_prio + (ctx.stream_need_prio >> 3)) : cap / 2;
    if (cap_p > cap - cap / 4) cap_p = cap - cap / 4;
    if (cap_p < 1) cap_p = 1;
    hmax_p = cap_p / (size_t(1) << (SKETCH_HEAVY_BUCKET - 1)) + 1;
    if (hmax_p > span) hmax_p = span;
    pmax_p = z / SKETCH_PART_COLS + hmax_p + 1;
    o_p_list = ar.take(4 * span);
    o_p_ctrl = ar.take(4 * CTRL_WORDS);
    o_p_hc = ar.take(4 * 2);
    o_p_htb = ar.take(4 * 4);
    o_p_th = ar.take(4 * 256 * (z / 4096 + 2));
    o_p_db = ar.take(4 * 256);
    o_p_ho = ar.take(4 * (hmax_p + 1));
    o_p_hst = ar.take(4 * hmax_p * 2 * (p.M / 32) * 32);
    o_p_pb = ar.take(4 * (hmax_p + 2));
    o_p_po = ar.take(4 * (pmax_p + 1));
  }
  if (!ensure_workspace(ctx, ar.off)) return false;
  s->keyA = reinterpret_cast<uint32_t *>(ctx.ws + o_keyA);
  s->keyB = reinterpret_cast<uint32_t *>(ctx.ws + o_keyB);
  s->payA = reinterpret_cast<uint32_t *>(ctx.ws + o_payA);
  s->payB = reinterpret_cast<uint32_t *>(ctx.ws + o_payB);
  s->cand = reinterpret_cast<int2 *>(ctx.ws + o_cand);
  s->seg = reinterpret_cast<int2 *>(ctx.ws + o_seg);
  s->seg_rank = reinterpret_cast<int32_t *>(ctx.ws + o_rank);
  s->row_work = reinterpret_cast<uint32_t *>(ctx.ws + o_work);
  s->row_list = reinterpret_cast<int32_t *>(ctx.ws + o_list);
  s->ctrl = reinterpret_cast<uint32_t *>(ctx.ws + o_ctrl);
  s->table = user_table ? user_table : reinterpret_cast<uint64_t *>(ctx.ws + o_table);
  s->hstream = reinterpret_cast<int2 *>(ctx.ws + o_hs);
  s->heavy_off = reinterpret_cast<uint32_t *>(ctx.ws + o_ho);
  s->heavy_state = reinterpret_cast<int32_t *>(ctx.ws + o_hst);
  s->part_base = reinterpret_cast<uint32_t *>(ctx.ws + o_pb);
  s->part_off = reinterpret_cast<uint32_t *>(ctx.ws + o_po);
  s->stream_cap = static_cast<uint32_t>(cap);
  s->heavy_max = static_cast<uint32_t>(hmax);
  s->heavy_chunk = reinterpret_cast<int32_t *>(ctx.ws + o_hc);
  s->heavy_tile_base = reinterpret_cast<int32_t *>(ctx.ws + o_htb);
  s->tile_hist = reinterpret_cast<uint32_t *>(ctx.ws + o_th);
  s->digit_base = reinterpret_cast<uint32_t *>(ctx.ws + o_db);
  s->gbitmaps = bw ? reinterpret_cast<uint32_t *>(ctx.ws + o_bm) : nullptr;
  if (prio) {
    *prio = *s;  // the arrays indexed by nonzero, row or table entry are common to both parts
    prio->row_list = reinterpret_cast<int32_t *>(ctx.ws + o_p_list);
    prio->ctrl = reinterpret_cast<uint32_t *>(ctx.ws + o_p_ctrl);
    prio->heavy_chunk = reinterpret_cast<int32_t *>(ctx.ws + o_p_hc);
    prio->heavy_tile_base = reinterpret_cast<int32_t *>(ctx.ws + o_p_htb);
    prio->tile_hist = reinterpret_cast<uint32_t *>(ctx.ws + o_p_th);
    prio->digit_base = reinterpret_cast<uint32_t *>(ctx.ws + o_p_db);
    prio->heavy_off = reinterpret_cast<uint32_t *>(ctx.ws + o_p_ho);
    prio->heavy_state = reinterpret_cast<int32_t *>(ctx.ws + o_p_hst);
    prio->part_base = reinterpret_cast<uint32_t *>(ctx.ws + o_p_pb);
    prio->part_off = reinterpret_cast<uint32_t *>(ctx.ws + o_p_po);
    // the stream buffer is cut in two: the front for the part ahead
    prio->stream_cap = static_cast<uint32_t>(cap_p);
    prio->heavy_max = static_cast<uint32_t>(hmax_p);
    s->hstream = s->hstream + cap_p;
    s->stream_cap = static_cast<uint32_t>(cap - cap_p);
    const size_t hmax_r = (cap - cap_p) / (size_t(1) << (SKETCH_HEAVY_BUCKET - 1)) + 1;
    if (hmax_r < s->heavy_max) s->heavy_max = static_cast<uint32_t>(hmax_r);
  }
  return true;
}

// End of a call that ran the transpose (and possibly the sketch): the control words come
// back with the call's one synchronisation.  Malformed input and a refused stream slice are
// errors; the stream need of the heavy rows is remembered for the context's next call.
bool finish_call(Context &ctx, const CsgScratch &s, const CsgScratch *prio = nullptr) {
  uint32_t *h = reinterpret_cast<uint32_t *>(ctx.h_pinned);
  CSG_CUDA(cudaMemcpyAsync(h, s.ctrl, 16 * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx.stream));
  if (prio)  // (the side stream's work has been joined into ctx.stream by now)
    CSG_CUDA(cudaMemcpyAsync(h + 16, prio->ctrl, 16 * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx.stream));
  CSG_CUDA(cudaStreamSynchronize(ctx.stream));
  CSG_CUDA(cudaGetLastError());
  uint64_t need_prio = 0;
  if (prio) {  // the words of the part ahead: errors count like the others', its need is kept apart
    const uint32_t *hp = h + 16;
    need_prio = (static_cast<uint64_t>(hp[CTRL_HEAVY_NEED + 1]) << 32) | hp[CTRL_HEAVY_NEED];
    if (need_prio > STREAM_CAP_MAX) need_prio = STREAM_CAP_MAX;
    if (need_prio > ctx.stream_need_prio) ctx.stream_need_prio = need_prio;
    h[CTRL_BAD_INPUT] |= hp[CTRL_BAD_INPUT];
    h[CTRL_STREAM_OVERRUN] |= hp[CTRL_STREAM_OVERRUN];
    if (h[CTRL_CHECK] == 0 && hp[CTRL_CHECK] != 0)
      for (int i = 0; i < 3; ++i) h[CTRL_CHECK + i] = hp[CTRL_CHECK + i];
  }
  CSG_REQUIRE(h[CTRL_BAD_INPUT] == 0,
              "malformed CSR: row pointers must be non-decreasing inside [0, nnz] (results unspecified)");
  if (h[CTRL_CHECK] != 0) {  // only a build with -DSPORDER_CHECKED writes this word
    static const char *const site[] = {"?", "cand[] index of a group", "position in a stream ring",
                                       "stream offset of a heavy row", "stream key outside its chunk",
                                       "heavy-row state item", "row of the top-k table", "row list entry",
                                       "order[] position", "scatter position of a radix pass",
                                       "group position written by the transpose", "part table entry"};
    const uint32_t k = h[CTRL_CHECK] < sizeof(site) / sizeof(site[0]) ? h[CTRL_CHECK] : 0;
    const long long idx = static_cast<long long>((static_cast<uint64_t>(h[CTRL_CHECK + 2]) << 32) | h[CTRL_CHECK + 1]);
    set_error("checked build: index out of bounds (%s: %lld); results unspecified", site[k], idx);
    return false;
  }
  CSG_REQUIRE(h[CTRL_STREAM_OVERRUN] == 0,
              "internal: a heavy row's stream slice did not fit its place in the stream buffer");
  uint64_t need = ((static_cast<uint64_t>(h[CTRL_HEAVY_NEED + 1]) << 32) | h[CTRL_HEAVY_NEED]) + need_prio;
  if (need > STREAM_CAP_MAX) need = STREAM_CAP_MAX;
  if (need > ctx.stream_need_seen) ctx.stream_need_seen = need;
#ifdef CSG_ROUND_PROFILE
  if (getenv("CSG_ROUND_PROFILE")) {  // cycles per phase of the chain kernel's rounds, all warps
    unsigned long long c[12];
    if (cudaMemcpy(c, s.ctrl + CTRL_PROFILE, sizeof(c), cudaMemcpyDeviceToHost) == cudaSuccess && c[6])
      fprintf(stderr,
              "[rounds] %llu rounds, %.2f elements each; cycles per round: look-up %.0f, order %.0f, "
              "resolve %.0f, targets %.0f, limits %.0f, apply %.0f\n",
              c[6], double(c[7]) / c[6], double(c[0]) / c[6], double(c[1]) / c[6], double(c[2]) / c[6],
              double(c[3]) / c[6], double(c[4]) / c[6], double(c[5]) / c[6]);
    uint32_t heavy = 0;
    cudaMemcpy(&heavy, s.ctrl + CTRL_HEAVY_ROWS, sizeof(heavy), cudaMemcpyDeviceToHost);
    if (heavy > 4096) heavy = 4096;
    static uint32_t kcyc[4096], work[4096];
    static int32_t rows[4096];
    if (heavy && cudaMemcpy(kcyc, s.heavy_off, heavy * 4, cudaMemcpyDeviceToHost) == cudaSuccess &&
        cudaMemcpy(rows, s.row_list, heavy * 4, cudaMemcpyDeviceToHost) == cudaSuccess) {
      for (uint32_t i = 0; i < heavy; ++i)
        cudaMemcpy(&work[i], s.row_work + rows[i], 4, cudaMemcpyDeviceToHost);
      fprintf(stderr, "[rounds] %u heavy rows; slowest (row: stream elements, Mcycles, cycles/element):", heavy);
      for (int k = 0; k < 12; ++k) {
        uint32_t best = 0;
        for (uint32_t i = 1; i < heavy; ++i)
          if (kcyc[i] > kcyc[best]) best = i;
        fprintf(stderr, " [%d: %u, %.1f, %.0f]", rows[best], work[best], kcyc[best] * 1024e-6,
                work[best] ? kcyc[best] * 1024.0 / work[best] : 0.0);
        kcyc[best] = 0;
      }
      fprintf(stderr, "\n");
    }
  }
#endif
  return true;
}

// The pipeline of sporder/src/csg/chunk_similarity_greedy.cu:100-138 with the
// stages of this library: chunk-local transpose -> sketch/top-k -> greedy.
bool run_csg(Context &ctx, int32_t n, int32_t ncols, int32_t row_base, int32_t nnz,
             const int32_t *d_ptr, const int32_t *d_ind,
             int32_t k, float ovs, int32_t chunk, int32_t *d_new_order, uint64_t *d_table,
             uint64_t table_capacity, sporder_csg_timing_t *timing, sporder_csg_stats_t *stats,
             int32_t *k_used, bool symmetric = false) {
  const auto wall0 = std::chrono::steady_clock::now();
  CsgParams p;
  if (!resolve_params(n, nnz, k, ovs, chunk, &p)) return false;
  if (k_used) *k_used = p.k;
  if (stats) {
    std::memset(stats, 0, sizeof(*stats));
    stats->k_used = p.k;
    stats->m_used = p.m_used;
    stats->chunk_size_used = p.chunk;
  }
  CSG_REQUIRE(d_ptr && (d_ind || nnz == 0), "null CSR arrays");
  CSG_REQUIRE(ncols >= n && row_base >= 0 && static_cast<int64_t>(row_base) + n <= ncols,
              "row block [%d, %d + %d) does not lie inside a matrix of %d rows", row_base, row_base, n, ncols);
  CSG_REQUIRE(row_base % p.chunk == 0,
              "row_base %d is not a multiple of the chunk size %d: the block would not hold whole chunks",
              row_base, p.chunk);
  CSG_REQUIRE(!d_table || table_capacity >= static_cast<uint64_t>(n) * p.k,
              "table buffer holds %llu entries, need n * k = %llu",
              static_cast<unsigned long long>(table_capacity),
              static_cast<unsigned long long>(static_cast<uint64_t>(n) * p.k));
  CSG_CUDA(cudaSetDevice(ctx.device));
  // (a row block of a larger matrix does not hold the rows its columns name: no shortcut there)
  const bool sym_path = symmetric && row_base == 0 && n == ncols;
  // Large calls run one chunk ahead.  On power-law inputs the rows with the longest candidate
  // streams - the dependent chains that decide how long the call takes - sit in the chunk
  // with the most nonzeros, and all their chains need is that chunk's own transposition.  So
  // that chunk is transposed first, on a second stream, and its heavy rows' chains start
  // there while the context's stream transposes everything else; the two meet before the
  // greedy stage.  Results do not depend on the split (the same kernels on the same rows).
  // By default for calls of 2^24 nonzeros in 64 chunks or more, whose chunk ahead must hold 2^17
  // nonzeros: smaller calls do not pay for the second pipeline's fifteen launches.  A caller's
  // own threshold (sporder_context_set_ahead_threshold) applies to any call of two chunks.
  const int64_t chunks = (static_cast<int64_t>(n) + p.chunk - 1) / p.chunk;
  bool ahead = !sym_path && ctx.side_stream != nullptr && p.chunk <= 4096;
  int32_t ahead_chunk_nnz = 1 << 17;
  if (ctx.ahead_min_nnz == 0) {
    ahead = ahead && nnz >= AHEAD_MIN_NNZ && chunks >= 64;
  } else {
    ahead = ahead && ctx.ahead_min_nnz > 0 && nnz >= ctx.ahead_min_nnz && chunks >= 2;
    ahead_chunk_nnz = 0;
  }
  CsgScratch s, sp;
  if (!plan_scratch(ctx, n, nnz, p, d_table, &s, 0, false, ahead ? &sp : nullptr)) return false;
  cudaStream_t st = ctx.stream;
  const bool zero_table = d_table != nullptr || stats != nullptr;

  if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[0], st));
  if (!ahead) {
    if (!launch_transpose(ctx, n, ncols, nnz, p.chunk, d_ptr, d_ind, s, sym_path)) return false;
    if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[1], st));
    if (!launch_sketch(ctx, n, nnz, p, d_ptr, s, row_base, zero_table)) return false;
  } else {
    auto two_parts = [&]() -> bool {
      if (zero_table)
        CSG_CUDA(cudaMemsetAsync(s.table, 0, sizeof(uint64_t) * static_cast<size_t>(n) * p.k, st));
      if (!launch_priority_pick(ctx, n, nnz, p.chunk, d_ptr, s, sp, ahead_chunk_nnz)) return false;
      CSG_CUDA(cudaEventRecord(ctx.ev[5], st));
      CSG_CUDA(cudaStreamWaitEvent(ctx.side_stream, ctx.ev[5], 0));
      // the chunk ahead: queued first, so that the host's launches of the rest do not delay it
      if (!launch_transpose(ctx, n, ncols, nnz, p.chunk, d_ptr, d_ind, sp, false, PHASE_PRIO, s.ctrl)) return false;
      if (!launch_sketch(ctx, n, nnz, p, d_ptr, sp, row_base, false, PHASE_PRIO)) return false;
      CSG_CUDA(cudaEventRecord(ctx.ev[7], ctx.side_stream));
      if (!launch_transpose(ctx, n, ncols, nnz, p.chunk, d_ptr, d_ind, s, false, PHASE_REST, sp.ctrl)) return false;
      if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[1], st));
      CSG_CUDA(cudaStreamWaitEvent(st, ctx.ev[8], 0));
      if (!launch_sketch(ctx, n, nnz, p, d_ptr, s, row_base, false, PHASE_REST)) return false;
      CSG_CUDA(cudaStreamWaitEvent(st, ctx.ev[7], 0));
      return true;
    };
    if (!two_parts()) {
      // a launch failed with the second stream forked and not joined: nothing of this call
      // may still be running when the next one reuses the workspace
      cudaStreamSynchronize(ctx.side_stream);
      cudaStreamSynchronize(st);
      return false;
    }
  }
  if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[2], st));
  if (stats && !launch_table_stats(ctx, n, p.k, s.table, s.ctrl)) return false;
  if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[3], st));
  if (d_new_order) {
    if (!launch_greedy(ctx, n, p, s, d_new_order, stats != nullptr, row_base)) return false;
  }
  if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[4], st));
  ChainStatsHost hs;
  if (stats)
    CSG_CUDA(cudaMemcpyAsync(&hs, s.ctrl + CTRL_STATS, sizeof(hs), cudaMemcpyDeviceToHost, st));
  if (!finish_call(ctx, s, ahead ? &sp : nullptr)) return false;
  if (stats) {  // sporder/src/csg/stats_collector.cu:53-62
    stats->avg_degree = static_cast<double>(hs.total_degree) / n;
    stats->avg_edge_weight =
        hs.total_degree > 0 ? hs.total_weight / static_cast<double>(hs.total_degree) : 0.0;
    stats->zero_degree_rows = hs.zero_degree_rows;
    stats->chain_restarts = hs.restarts;
    stats->avg_followed_weight = hs.links > 0 ? hs.link_weight_sum / hs.links : 0.0;
  }
  if (timing) {
    CSG_CUDA(cudaEventElapsedTime(&timing->csr2csc_ms, ctx.ev[0], ctx.ev[1]));
    CSG_CUDA(cudaEventElapsedTime(&timing->similarity_ms, ctx.ev[1], ctx.ev[2]));
    CSG_CUDA(cudaEventElapsedTime(&timing->chunk_greedy_ms, ctx.ev[3], ctx.ev[4]));
    timing->wall_ms =
        std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - wall0).count();
  }
  return true;
}


// packed table -> separate arrays; an empty entry (0) reads as index -1, weight 0
// (sporder/src/similarity_graph.cu:13-23)
__global__ void __launch_bounds__(256) unpack_table_kernel(size_t count, const uint64_t *__restrict__ table,
                                                           int32_t *__restrict__ indices,
                                                           float *__restrict__ weights) {
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const uint64_t e = table[i];
    indices[i] = static_cast<int32_t>(static_cast<uint32_t>(e)) - 1;
    weights[i] = __uint_as_float(static_cast<uint32_t>(e >> 32));
  }
}

// The public top-k similarity graph (sporder/src/similarity_graph.cu:26-107,
// sporder/src/sporder.cpp:69-91): the same candidate stream, sketch and top-k selection as
// csg with the whole matrix as the one chunk (sporder/src/common/similarity_top_k.cu:10-51),
// other defaults (k = min(32, max(16, 2 nnz / n)), oversampling 2), results unpacked.
bool run_similarity_graph(Context &ctx, int32_t n, int32_t nnz, const int32_t *d_ptr, const int32_t *d_ind,
                          int32_t k, float ovs, int32_t *d_indices, float *d_weights,
                          sporder_sim_timing_t *timing, sporder_sim_stats_t *stats, int32_t *k_used,
                          bool symmetric = false) {
  const auto wall0 = std::chrono::steady_clock::now();
  CSG_REQUIRE(n >= 1, "n must be >= 1 (got %d)", n);
  CSG_REQUIRE(nnz >= 0, "nnz must be >= 0 (got %d)", nnz);
  if (k <= 0) {
    int32_t a = 2 * (nnz / n);
    if (a < 16) a = 16;
    if (a > 32) a = 32;
    k = a;
  }
  if (ovs <= 0.0f) ovs = 2.0f;
  CsgParams p;
  if (!resolve_params(n, nnz, k, ovs, n, &p)) return false;
  if (k_used) *k_used = p.k;
  if (stats) {
    std::memset(stats, 0, sizeof(*stats));
    stats->k_used = p.k;
    stats->m_used = p.m_used;
  }
  CSG_REQUIRE(d_ptr && (d_ind || nnz == 0), "null CSR arrays");
  CSG_REQUIRE(d_indices && d_weights, "null output arrays");
  CSG_CUDA(cudaSetDevice(ctx.device));
  CsgScratch s;
  if (!plan_scratch(ctx, n, nnz, p, nullptr, &s)) return false;
  cudaStream_t st = ctx.stream;
  if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[0], st));
  if (!launch_transpose(ctx, n, n, nnz, p.chunk, d_ptr, d_ind, s, symmetric)) return false;
  if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[1], st));
  if (!launch_sketch(ctx, n, nnz, p, d_ptr, s, 0, true)) return false;
  if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[2], st));
  if (stats && !launch_table_stats(ctx, n, p.k, s.table, s.ctrl)) return false;
  if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[3], st));
  const size_t count = static_cast<size_t>(n) * p.k;
  size_t grid = (count + 255) / 256;
  if (grid > static_cast<size_t>(ctx.num_sms) * 16) grid = static_cast<size_t>(ctx.num_sms) * 16;
  unpack_table_kernel<<<static_cast<unsigned>(grid), 256, 0, st>>>(count, s.table, d_indices, d_weights);
  CSG_CUDA(cudaGetLastError());
  count_launches(1);
  if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[4], st));
  ChainStatsHost hs;
  if (stats)
    CSG_CUDA(cudaMemcpyAsync(&hs, s.ctrl + CTRL_STATS, sizeof(hs), cudaMemcpyDeviceToHost, st));
  if (!finish_call(ctx, s)) return false;
  if (stats) {  // sporder/src/similarity_graph.cu:99-104
    stats->avg_degree = static_cast<double>(hs.total_degree) / n;
    stats->avg_edge_weight =
        hs.total_degree > 0 ? hs.total_weight / static_cast<double>(hs.total_degree) : 0.0;
    stats->zero_degree_rows = hs.zero_degree_rows;
  }
  if (timing) {
    CSG_CUDA(cudaEventElapsedTime(&timing->csr2csc_ms, ctx.ev[0], ctx.ev[1]));
    CSG_CUDA(cudaEventElapsedTime(&timing->similarity_ms, ctx.ev[1], ctx.ev[2]));
    CSG_CUDA(cudaEventElapsedTime(&timing->unpack_ms, ctx.ev[3], ctx.ev[4]));
    timing->wall_ms =
        std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - wall0).count();
  }
  return true;
}

// Chunked greedy on the global graph (sporder/src/cg/chunk_greedy.cu:118-163,
// sporder/src/sporder.cpp:112-138): the top-k graph of run_similarity_graph with the csg
// defaults (k = min(256, max(16, nnz / n)), oversampling 4), then the greedy chains inside
// chunks of chunk_size rows, candidates outside the chunk skipped.
bool run_chunk_greedy(Context &ctx, int32_t n, int32_t nnz, const int32_t *d_ptr, const int32_t *d_ind,
                      int32_t k, float ovs, int32_t chunk, int32_t *d_new_order,
                      sporder_cg_timing_t *timing, sporder_cg_stats_t *stats, bool symmetric = false) {
  const auto wall0 = std::chrono::steady_clock::now();
  CsgParams pg;  // greedy: the caller's chunk; also resolves k and oversampling
  if (!resolve_params(n, nnz, k, ovs, chunk, &pg)) return false;
  CsgParams ps = pg;  // sketch: the whole matrix is the chunk
  ps.chunk = n;
  if (stats) {
    std::memset(stats, 0, sizeof(*stats));
    stats->k_used = pg.k;
    stats->m_used = pg.m_used;
    stats->chunk_size_used = pg.chunk;
  }
  CSG_REQUIRE(d_ptr && (d_ind || nnz == 0), "null CSR arrays");
  CSG_REQUIRE(d_new_order, "null d_new_order");
  CSG_CUDA(cudaSetDevice(ctx.device));
  CsgScratch s;
  if (!plan_scratch(ctx, n, nnz, ps, nullptr, &s, pg.chunk)) return false;
  cudaStream_t st = ctx.stream;
  if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[0], st));
  if (!launch_transpose(ctx, n, n, nnz, ps.chunk, d_ptr, d_ind, s, symmetric)) return false;
  if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[1], st));
  if (!launch_sketch(ctx, n, nnz, ps, d_ptr, s, 0, stats != nullptr)) return false;
  if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[2], st));
  if (stats) {
    if (!launch_table_stats(ctx, n, pg.k, s.table, s.ctrl)) return false;
    if (!launch_in_chunk_weight(ctx, n, pg.k, pg.chunk, s.table, s.ctrl)) return false;
  }
  if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[3], st));
  if (!launch_greedy(ctx, n, pg, s, d_new_order, stats != nullptr, 0)) return false;
  if (timing) CSG_CUDA(cudaEventRecord(ctx.ev[4], st));
  ChainStatsHost hs;
  if (stats)
    CSG_CUDA(cudaMemcpyAsync(&hs, s.ctrl + CTRL_STATS, sizeof(hs), cudaMemcpyDeviceToHost, st));
  if (!finish_call(ctx, s)) return false;
  if (stats) {  // sporder/src/cg/stats_collector.cu:52-73
    stats->avg_degree = static_cast<double>(hs.total_degree) / n;
    stats->avg_edge_weight =
        hs.total_degree > 0 ? hs.total_weight / static_cast<double>(hs.total_degree) : 0.0;
    stats->zero_degree_rows = hs.zero_degree_rows;
    stats->chain_restarts = hs.restarts;
    stats->avg_followed_weight = hs.links > 0 ? hs.link_weight_sum / hs.links : 0.0;
    double cut = hs.total_weight > 0.0 ? 1.0 - hs.in_chunk_weight / hs.total_weight : 0.0;
    stats->cut_weight_fraction = cut < 0.0 ? 0.0 : (cut > 1.0 ? 1.0 : cut);
  }
  if (timing) {
    CSG_CUDA(cudaEventElapsedTime(&timing->csr2csc_ms, ctx.ev[0], ctx.ev[1]));
    CSG_CUDA(cudaEventElapsedTime(&timing->similarity_ms, ctx.ev[1], ctx.ev[2]));
    CSG_CUDA(cudaEventElapsedTime(&timing->chunk_greedy_ms, ctx.ev[3], ctx.ev[4]));
    timing->wall_ms =
        std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - wall0).count();
  }
  return true;
}

// Pillar count (sporder/src/count_pillars.cu:38-85): windows of up to 12 rows by searching
// the window's earlier rows, taller windows as the column groups of the chunk-local
// transpose with the window as the chunk.  Measured on the 65 M-nonzero R-MAT matrix the
// search costs 3 ms at height 1, 7 ms at 4 and 21 ms at 16, the transpose 26 ms at 8, 16 ms
// at 16 and 6 ms at 1024 (the reference's global key sort: 21-22 ms at every height).
constexpr int32_t PILLAR_SEARCH_ROWS = 12;

bool run_count_pillars(Context &ctx, int32_t n, int32_t nnz, const int32_t *d_ptr, const int32_t *d_ind,
                       int32_t height, int32_t *count) {
  CSG_REQUIRE(n >= 1, "n must be >= 1 (got %d)", n);
  CSG_REQUIRE(nnz >= 0, "nnz must be >= 0 (got %d)", nnz);
  CSG_REQUIRE(height >= 1, "height must be >= 1 (got %d)", height);
  CSG_REQUIRE(count, "null count");
  *count = 0;
  if (nnz == 0) return true;
  CSG_REQUIRE(d_ptr && d_ind, "null CSR arrays");
  CSG_CUDA(cudaSetDevice(ctx.device));
  unsigned long long *d_count = nullptr;
  uint32_t *d_bad = nullptr;
  if (height <= PILLAR_SEARCH_ROWS) {
    if (!ensure_workspace(ctx, 512)) return false;
    d_count = reinterpret_cast<unsigned long long *>(ctx.ws);
    d_bad = reinterpret_cast<uint32_t *>(ctx.ws + 256);
    CSG_CUDA(cudaMemsetAsync(ctx.ws, 0, 512, ctx.stream));
    if (!launch_pillars_search(ctx, n, nnz, height, d_ptr, d_ind, d_count, d_bad)) return false;
  } else {
    CsgParams p;
    if (!resolve_params(n, nnz, 1, 1.0f, height, &p)) return false;  // k = 1: smallest table the layout allows
    CsgScratch s;
    if (!plan_scratch(ctx, n, nnz, p, nullptr, &s, 0, true)) return false;
    if (!launch_transpose(ctx, n, n, nnz, p.chunk, d_ptr, d_ind, s)) return false;
    // the counter takes the place of the (now unused) sort buffer; the transpose set the flag word
    d_count = reinterpret_cast<unsigned long long *>(s.keyA);
    d_bad = s.ctrl + CTRL_BAD_INPUT;
    CSG_CUDA(cudaMemsetAsync(d_count, 0, sizeof(unsigned long long), ctx.stream));
    if (!launch_pillars_groups(ctx, nnz, s.seg_rank, d_count)) return false;
  }
  unsigned long long *h = reinterpret_cast<unsigned long long *>(ctx.h_pinned + 16);
  CSG_CUDA(cudaMemcpyAsync(h, d_count, sizeof(unsigned long long), cudaMemcpyDeviceToHost, ctx.stream));
  CSG_CUDA(cudaMemcpyAsync(ctx.h_pinned, d_bad, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx.stream));
  CSG_CUDA(cudaStreamSynchronize(ctx.stream));
  CSG_REQUIRE(ctx.h_pinned[0] == 0,
              "malformed CSR: row pointers must be non-decreasing inside [0, nnz] (results unspecified)");
  *count = static_cast<int32_t>(*h);  // at most nnz
  return true;
}

}  // namespace
}  // namespace csg

struct sporder_context_struct {
  csg::Context c;
};

extern "C" {

sporder_context_t sporder_context_create(void) {
  csg::clear_error();
  auto *h = new sporder_context_struct;
  csg::Context &c = h->c;
  auto fail = [&](cudaError_t e, const char *what) {
    csg::set_error("context: %s -> %s", what, cudaGetErrorString(e));
    delete h;
    return static_cast<sporder_context_t>(nullptr);
  };
  cudaError_t e;
  if ((e = cudaGetDevice(&c.device)) != cudaSuccess) return fail(e, "cudaGetDevice");
  if ((e = cudaStreamCreateWithFlags(&c.own_stream, cudaStreamNonBlocking)) != cudaSuccess)
    return fail(e, "cudaStreamCreate");
  c.stream = c.own_stream;
  {  // the stream of the part of a large call that runs ahead: highest priority, so that its
     // small kernels are placed before the blocks of the grids on the main stream
    int least = 0, greatest = 0;
    if ((e = cudaDeviceGetStreamPriorityRange(&least, &greatest)) != cudaSuccess) return fail(e, "stream priorities");
    if ((e = cudaStreamCreateWithPriority(&c.side_stream, cudaStreamNonBlocking, greatest)) != cudaSuccess)
      return fail(e, "cudaStreamCreateWithPriority");
  }
  cudaDeviceGetAttribute(&c.num_sms, cudaDevAttrMultiProcessorCount, c.device);
  cudaDeviceGetAttribute(&c.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, c.device);
  for (auto &ev : c.ev)
    if ((e = cudaEventCreate(&ev)) != cudaSuccess) return fail(e, "cudaEventCreate");
  if ((e = cudaMallocHost(&c.h_pinned, 64 * sizeof(int))) != cudaSuccess)
    return fail(e, "cudaMallocHost");
  return h;
}

void sporder_context_destroy(sporder_context_t h) {
  if (!h) return;
  csg::Context &c = h->c;
  cudaSetDevice(c.device);
  cudaStreamSynchronize(c.stream);
  if (c.side_stream) cudaStreamSynchronize(c.side_stream);
  if (c.ws) cudaFree(c.ws);
  if (c.stage) cudaFree(c.stage);
  for (auto &ev : c.ev)
    if (ev) cudaEventDestroy(ev);
  if (c.h_pinned) cudaFreeHost(c.h_pinned);
  if (c.own_stream) cudaStreamDestroy(c.own_stream);
  if (c.side_stream) cudaStreamDestroy(c.side_stream);
  delete h;
}

void sporder_context_set_stream(sporder_context_t h, void *stream) {
  if (!h) return;
  cudaStream_t next = stream ? static_cast<cudaStream_t>(stream) : h->c.own_stream;  // see header
  // The workspace and its control words serve one stream at a time: work still queued on the
  // previous stream (sporder_spmm_async) must be over before another stream may reuse them.
  if (next != h->c.stream) cudaStreamSynchronize(h->c.stream);
  h->c.stream = next;
}

void sporder_context_set_ahead_threshold(sporder_context_t h, int64_t min_nnz) {
  if (h) h->c.ahead_min_nnz = min_nnz;
}

void sporder_context_set_stream_limit(sporder_context_t h, uint64_t max_elements) {
  if (h) h->c.stream_limit = max_elements;
}

uint64_t sporder_context_workspace_bytes(sporder_context_t h) { return h ? h->c.ws_bytes : 0; }

const char *sporder_last_error(void) { return csg::g_has_err ? csg::g_err : nullptr; }

uint64_t sporder_kernel_launches(void) { return csg::g_launches.load(); }

void sporder_chunk_similarity_greedy(sporder_context_t ctx, int32_t n, int32_t nnz,
                                     const int32_t *d_ptr, const int32_t *d_ind, bool is_symmetric,
                                     int32_t k, float oversampling, int32_t chunk_size,
                                     int32_t *d_new_order, sporder_csg_timing_t *timing,
                                     sporder_csg_stats_t *stats) {
  csg::clear_error();
  if (!ctx) {
    csg::set_error("null context");
    return;
  }
  if (!d_new_order) {
    csg::set_error("null d_new_order");
    return;
  }
  csg::run_csg(ctx->c, n, n, 0, nnz, d_ptr, d_ind, k, oversampling, chunk_size, d_new_order, nullptr, 0,
               timing, stats, nullptr, is_symmetric);
}

int32_t sporder_csg_with_table(sporder_context_t ctx, int32_t n, int32_t nnz, const int32_t *d_ptr,
                               const int32_t *d_ind, bool is_symmetric, int32_t k,
                               float oversampling, int32_t chunk_size, int32_t *d_new_order,
                               uint64_t *d_table, uint64_t d_table_capacity,
                               sporder_csg_timing_t *timing, sporder_csg_stats_t *stats) {
  csg::clear_error();
  if (!ctx) {
    csg::set_error("null context");
    return -1;
  }
  int32_t k_used = -1;
  if (!csg::run_csg(ctx->c, n, n, 0, nnz, d_ptr, d_ind, k, oversampling, chunk_size, d_new_order, d_table,
                    d_table_capacity, timing, stats, &k_used, is_symmetric))
    return -1;
  return k_used;
}

int32_t sporder_csg_shard(sporder_context_t ctx, int32_t n_rows, int32_t n_cols, int32_t row_base,
                          int32_t nnz, const int32_t *d_ptr, const int32_t *d_ind, int32_t k,
                          float oversampling, int32_t chunk_size, int32_t *d_new_order,
                          uint64_t *d_table, uint64_t d_table_capacity,
                          sporder_csg_timing_t *timing, sporder_csg_stats_t *stats) {
  csg::clear_error();
  if (!ctx) {
    csg::set_error("null context");
    return -1;
  }
  int32_t k_used = -1;
  if (!csg::run_csg(ctx->c, n_rows, n_cols, row_base, nnz, d_ptr, d_ind, k, oversampling,
                    chunk_size, d_new_order, d_table, d_table_capacity, timing, stats, &k_used))
    return -1;
  return k_used;
}

int32_t sporder_chunk_similarity_greedy_host(sporder_context_t ctx, int32_t n, int32_t nnz,
                                             const int32_t *h_ptr, const int32_t *h_ind,
                                             bool is_symmetric, int32_t k, float oversampling,
                                             int32_t chunk_size, int32_t *h_new_order,
                                             sporder_csg_timing_t *timing,
                                             sporder_csg_stats_t *stats) {
  csg::clear_error();
  if (!ctx || !h_ptr || !h_new_order || n < 1 || nnz < 0) {
    csg::set_error("csg_host: bad arguments");
    return -1;
  }
  csg::Context &c = ctx->c;
  auto run = [&]() -> bool {
    CSG_CUDA(cudaSetDevice(c.device));
    // Device copies of the inputs and the result live in a buffer of the context that only
    // grows: a stream-ordered allocation per call went back to the driver at every
    // synchronisation and cost more than the reorder itself.
    const size_t b_ptr = (sizeof(int32_t) * (static_cast<size_t>(n) + 1) + 255) & ~size_t(255);
    const size_t b_ind = (sizeof(int32_t) * static_cast<size_t>(nnz > 0 ? nnz : 1) + 255) & ~size_t(255);
    const size_t b_ord = sizeof(int32_t) * static_cast<size_t>(n);
    if (b_ptr + b_ind + b_ord > c.stage_bytes) {
      CSG_CUDA(cudaStreamSynchronize(c.stream));
      if (c.stage) CSG_CUDA(cudaFree(c.stage));
      c.stage = nullptr;
      c.stage_bytes = 0;
      CSG_CUDA(cudaMalloc(&c.stage, b_ptr + b_ind + b_ord));
      c.stage_bytes = b_ptr + b_ind + b_ord;
    }
    int32_t *d_ptr = reinterpret_cast<int32_t *>(c.stage);
    int32_t *d_ind = reinterpret_cast<int32_t *>(c.stage + b_ptr);
    int32_t *d_order = reinterpret_cast<int32_t *>(c.stage + b_ptr + b_ind);
    CSG_CUDA(cudaMemcpyAsync(d_ptr, h_ptr, sizeof(int32_t) * (static_cast<size_t>(n) + 1),
                             cudaMemcpyHostToDevice, c.stream));
    if (nnz > 0)
      CSG_CUDA(cudaMemcpyAsync(d_ind, h_ind, sizeof(int32_t) * static_cast<size_t>(nnz),
                               cudaMemcpyHostToDevice, c.stream));
    const bool ok = csg::run_csg(c, n, n, 0, nnz, d_ptr, d_ind, k, oversampling, chunk_size, d_order,
                                 nullptr, 0, timing, stats, nullptr, is_symmetric);
    if (ok)
      CSG_CUDA(cudaMemcpyAsync(h_new_order, d_order, sizeof(int32_t) * static_cast<size_t>(n),
                               cudaMemcpyDeviceToHost, c.stream));
    CSG_CUDA(cudaStreamSynchronize(c.stream));
    return ok;
  };
  return run() ? 0 : -1;
}

void sporder_chunk_greedy(sporder_context_t ctx, int32_t n, int32_t nnz, const int32_t *d_ptr,
                          const int32_t *d_ind, bool is_symmetric, int32_t k, float oversampling,
                          int32_t chunk_size, int32_t *d_new_order, sporder_cg_timing_t *timing,
                          sporder_cg_stats_t *stats) {
  csg::clear_error();
  if (!ctx) {
    csg::set_error("null context");
    return;
  }
  csg::run_chunk_greedy(ctx->c, n, nnz, d_ptr, d_ind, k, oversampling, chunk_size, d_new_order, timing,
                        stats, is_symmetric);
}

int32_t sporder_similarity_graph(sporder_context_t ctx, int32_t n, int32_t nnz, const int32_t *d_ptr,
                                 const int32_t *d_ind, bool is_symmetric, int32_t k, float oversampling,
                                 int32_t *d_indices, float *d_weights, sporder_sim_timing_t *timing,
                                 sporder_sim_stats_t *stats) {
  csg::clear_error();
  if (!ctx) {
    csg::set_error("null context");
    return -1;
  }
  int32_t k_used = -1;
  if (!csg::run_similarity_graph(ctx->c, n, nnz, d_ptr, d_ind, k, oversampling, d_indices, d_weights,
                                 timing, stats, &k_used, is_symmetric))
    return -1;
  return k_used;
}

void sporder_count_pillars(sporder_context_t ctx, int32_t n, int32_t nnz, const int32_t *d_ptr,
                           const int32_t *d_ind, int32_t height, int32_t *count) {
  csg::clear_error();
  if (!ctx) {
    csg::set_error("null context");
    return;
  }
  csg::run_count_pillars(ctx->c, n, nnz, d_ptr, d_ind, height, count);
}

void sporder_reorder(sporder_context_t ctx, int32_t n, int32_t nnz, const int32_t *d_ptr_old,
                     const int32_t *d_ind_old, const float *d_val_old, const int32_t *d_new_order,
                     sporder_reorder_mode_t mode, int32_t *d_ptr_new, int32_t *d_ind_new,
                     float *d_val_new) {
  csg::clear_error();
  if (!ctx) {
    csg::set_error("null context");
    return;
  }
  if (mode != SPORDER_REORDER_ROWS && mode != SPORDER_REORDER_SYMMETRIC) {
    csg::set_error("invalid reorder mode");
    return;
  }
  if (n < 1 || nnz < 0 || !d_ptr_old || !d_new_order || !d_ptr_new || (nnz > 0 && (!d_ind_old || !d_ind_new))) {
    csg::set_error("reorder: bad arguments");
    return;
  }
  csg::Context &c = ctx->c;
  auto run = [&]() -> bool {
    CSG_CUDA(cudaSetDevice(c.device));
    if (!csg::launch_reorder(c, n, nnz, d_ptr_old, d_ind_old, d_val_old, d_new_order,
                             static_cast<int>(mode), d_ptr_new, d_ind_new, d_val_new))
      return false;
    CSG_CUDA(cudaStreamSynchronize(c.stream));
    CSG_CUDA(cudaGetLastError());
    return true;
  };
  run();
}

static int32_t spmm_impl(sporder_context_t ctx, int32_t n, int32_t nnz, int32_t w,
                         const int32_t *d_ptr, const int32_t *d_ind, const float *d_val,
                         const float *d_B, float *d_C, bool sync) {
  csg::clear_error();
  if (!ctx || n < 1 || nnz < 0 || !d_ptr || !d_B || !d_C || (nnz > 0 && (!d_ind || !d_val))) {
    csg::set_error("spmm: bad arguments");
    return -1;
  }
  csg::Context &c = ctx->c;
  auto run = [&]() -> bool {
    CSG_CUDA(cudaSetDevice(c.device));
    if (!csg::launch_spmm(c, n, nnz, w, d_ptr, d_ind, d_val, d_B, d_C)) return false;
    if (sync) {
      CSG_CUDA(cudaStreamSynchronize(c.stream));
      CSG_CUDA(cudaGetLastError());
    }
    return true;
  };
  return run() ? 0 : -1;
}

int32_t sporder_spmm(sporder_context_t ctx, int32_t n, int32_t nnz, int32_t w, const int32_t *d_ptr,
                     const int32_t *d_ind, const float *d_val, const float *d_B, float *d_C) {
  return spmm_impl(ctx, n, nnz, w, d_ptr, d_ind, d_val, d_B, d_C, true);
}

int32_t sporder_spmm_async(sporder_context_t ctx, int32_t n, int32_t nnz, int32_t w,
                           const int32_t *d_ptr, const int32_t *d_ind, const float *d_val,
                           const float *d_B, float *d_C) {
  return spmm_impl(ctx, n, nnz, w, d_ptr, d_ind, d_val, d_B, d_C, false);
}

}  // extern "C"
