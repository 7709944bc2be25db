// Greedy chaining inside each chunk, and the optional table statistics.
//
// Semantics restated from sporder/src/csg/chunk_similarity_greedy.cu:14-96: the
// chain starts at the chunk's first row; the next row is the unvisited in-chunk
// entry of the current row's top-k list with the largest weight (ties: smaller
// index); with none left the chain restarts at the smallest unvisited row
// (sporder/src/common/warp_visited_bitmap.cuh:99-111).  The visiting order is the
// permutation (new2old).
//
// One warp per chunk as in the reference; what changes: rows whose candidate
// stream was empty are known from the transpose (row_work == 0) and need no table
// load, the restart scan keeps a monotone cursor instead of rescanning the bitmap,
// the arg-max is two warp reductions, and the order is written 32 entries at a time.
#include "common.cuh"

namespace csg {

namespace {

constexpr int G_WARPS = 4;

struct GreedyArgs {
  int32_t n, k, chunk, num_chunks, row_base;
  const uint64_t *table;
  const uint32_t *row_work;
  int32_t *order;
  uint32_t *ctrl;      // stats block, or nullptr
  uint32_t *ctrl_all;  // the control words (checked build: where a bad index is recorded)
  uint32_t *gbitmaps;  // global bitmaps when a chunk's bitmaps do not fit shared memory
  int32_t words;       // bitmap words per chunk
};

struct ChainStats {  // lives at ctrl[CTRL_STATS ...]
  unsigned long long total_degree;
  double total_weight;
  double link_weight_sum;
  int32_t zero_degree_rows;
  int32_t restarts;
  int32_t links;
  int32_t pad;
  double in_chunk_weight;  // table weights whose candidate lies in the row's own chunk
};

// The chain of chunk q = rows [start, end), run by one warp.  STAGED: the chunk's rows of the
// table were copied to shared memory (`staged`, row-major like the table) by the block.
template <bool STAGED>
__device__ __forceinline__ void chain_chunk(const GreedyArgs &a, int32_t start, int32_t end, uint32_t *visited,
                                            const uint64_t *staged) {
  const int lane = lane_id();
  const int32_t size = end - start;
  const int32_t words = (size + 31) >> 5;
  uint32_t *nonempty = visited + a.words;
  for (int32_t w = lane; w < words; w += 32) visited[w] = 0;
  for (int32_t base = 0; base < size; base += 32) {
    const int32_t i = base + lane;
    const bool ne = (i < size) && a.row_work[start + i] != 0;
    const unsigned m = __ballot_sync(FULL, ne);
    if (lane == 0) nonempty[base >> 5] = m;
  }
  __syncwarp();

  int32_t cur = start, emitted = 0, scan = 0, mine = 0;
  int32_t restarts = 0, links = 0;
  float link_w = 0.0f;
  for (;;) {
    const int32_t loc = cur - start;
    if (lane == 0) visited[loc >> 5] |= 1u << (loc & 31);
    if (lane == (emitted & 31)) mine = cur + a.row_base;
    ++emitted;
    if ((emitted & 31) == 0 && index_ok(a.ctrl_all, CHK_ORDER, emitted, size + 1))
      a.order[start + emitted - 32 + lane] = mine;
    __syncwarp();

    int32_t best_c = -1;
    if (nonempty[loc >> 5] & (1u << (loc & 31))) {
      const uint64_t *row = STAGED ? staged + static_cast<size_t>(loc) * a.k
                                   : a.table + static_cast<size_t>(cur) * a.k;
      uint32_t best_w = 0;  // weight bits; real weights are positive
      for (int32_t j = lane; j < a.k; j += 32) {
        const uint64_t e = row[j];
        if (e == 0) break;  // valid entries form a prefix
        const int32_t cand = entry_index(e) - a.row_base;
        if (cand < start || cand >= end) continue;
        const int32_t cl = cand - start;
        if (visited[cl >> 5] & (1u << (cl & 31))) continue;
        // The next row of the chain is one of these candidates, and its list is needed as
        // soon as the arg-max below is known: ask for every candidate's list now, so that the
        // one dependent load per step finds it in L1 instead of waiting on L2.
        if (!STAGED) asm volatile("prefetch.global.L1 [%0];" ::"l"(a.table + static_cast<size_t>(cand) * a.k));
        const uint32_t wb = entry_weight_bits(e);
        if (wb > best_w || (wb == best_w && cand < best_c)) {
          best_w = wb;
          best_c = cand;
        }
      }
      const uint32_t g = __reduce_max_sync(FULL, best_w);
      if (g != 0u) {
        const uint32_t c = (best_w == g) ? static_cast<uint32_t>(best_c) : 0xFFFFFFFFu;
        best_c = static_cast<int32_t>(__reduce_min_sync(FULL, c));
        links += 1;
        link_w += __uint_as_float(g);
      } else {
        best_c = -1;
      }
    }
    if (best_c >= 0) {
      cur = best_c;
      continue;
    }
    // Restart at the smallest unvisited row; `scan` only moves forward.  A row without a
    // list (no bit in `nonempty`) would be emitted, find no neighbour and restart again, one
    // dependent step each - and on many inputs most rows are like that.  They change nothing
    // for the rows behind them, so all unvisited rows without a list in front of the first
    // unvisited row WITH a list are emitted here at once, in index order, as the chain
    // would have emitted them one by one (each of them counts as one restart).
    int32_t nxt = -1;
    for (int32_t base = scan; base < words; base += 32) {
      const int32_t w = base + lane;
      uint32_t fr = 0, ne = 0;
      if (w < words) {
        fr = ~visited[w];
        if (w == words - 1 && (size & 31)) fr &= (1u << (size & 31)) - 1u;
        ne = nonempty[w];
      }
      const uint32_t listed = fr & ne, bare = fr & ~ne;
      const unsigned mb = __ballot_sync(FULL, listed != 0);
      const int lb = mb ? __ffs(mb) - 1 : 32;  // lane of the first word that holds a row with a list
      const uint32_t fb = __shfl_sync(FULL, listed, lb & 31);
      const int bitb = mb ? __ffs(fb) - 1 : 0;
      uint32_t take = lane < lb ? bare : (lane == lb ? bare & ((1u << bitb) - 1u) : 0u);
      if (__any_sync(FULL, take != 0)) {
        const int32_t cnt = __popc(take);
        int32_t incl = cnt;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const int32_t t = __shfl_up_sync(FULL, incl, off);
          if (lane >= off) incl += t;
        }
        const int32_t total = __shfl_sync(FULL, incl, 31);
        // entries still waiting in registers go out first, then the run, in place
        if (lane < (emitted & 31)) a.order[start + (emitted & ~31) + lane] = mine;
        int32_t at = start + emitted + incl - cnt;
        if (w < words) visited[w] |= take;
        while (take) {
          const int b = __ffs(take) - 1;
          take &= take - 1;
          if (index_ok(a.ctrl_all, CHK_ORDER, at - start, size)) a.order[at] = start + (w << 5) + b + a.row_base;
          ++at;
        }
        emitted += total;
        restarts += total;
        __syncwarp();
        // the block of 32 that is being filled now: its first entries are already in memory
        if (lane < (emitted & 31)) mine = a.order[start + (emitted & ~31) + lane];
      }
      if (mb) {
        scan = base + lb;
        nxt = (scan << 5) + bitb;
        break;
      }
    }
    if (nxt < 0) break;
    cur = start + nxt;
    restarts += 1;
  }
  if ((emitted & 31) != 0 && lane < (emitted & 31)) a.order[start + (emitted & ~31) + lane] = mine;

  if (a.ctrl && lane == 0) {
    ChainStats *st = reinterpret_cast<ChainStats *>(a.ctrl + CTRL_STATS);
    atomicAdd(&st->restarts, restarts);
    atomicAdd(&st->links, links);
    atomicAdd(&st->link_weight_sum, static_cast<double>(link_w));
  }
}

__global__ void __launch_bounds__(G_WARPS * 32) greedy_kernel(GreedyArgs a) {
  extern __shared__ uint32_t g_smem[];
  const int warp = threadIdx.x >> 5;
  const int32_t q = blockIdx.x * G_WARPS + warp;
  if (q >= a.num_chunks) return;
  const int64_t start64 = static_cast<int64_t>(q) * a.chunk;
  const int32_t start = static_cast<int32_t>(start64);
  const int32_t end = (start64 + a.chunk > a.n) ? a.n : static_cast<int32_t>(start64 + a.chunk);
  // two bitmaps per chunk: visited, and "row has a non-empty top-k list"
  uint32_t *visited = a.gbitmaps ? a.gbitmaps + static_cast<size_t>(q) * 2 * a.words
                                 : g_smem + static_cast<size_t>(warp) * 2 * a.words;
  chain_chunk<false>(a, start, end, visited, nullptr);
}

// With no more chunks than SMs there are too few chains to hide one another's latency, and a
// step is one dependent read of a table row: a block per chunk copies the chunk's rows of the
// table into shared memory first (1024 rows x 16 entries = 128 KB), and one warp runs the
// chain on that copy.
constexpr int GS_THREADS = 256;
__global__ void __launch_bounds__(GS_THREADS, 1) greedy_staged_kernel(GreedyArgs a) {
  extern __shared__ __align__(16) uint32_t g_smem[];
  const int32_t q = blockIdx.x;
  const int64_t start64 = static_cast<int64_t>(q) * a.chunk;
  const int32_t start = static_cast<int32_t>(start64);
  const int32_t end = (start64 + a.chunk > a.n) ? a.n : static_cast<int32_t>(start64 + a.chunk);
  uint32_t *visited = g_smem;
  uint64_t *staged = reinterpret_cast<uint64_t *>(g_smem + ((2 * a.words + 3) & ~3));
  const size_t entries = static_cast<size_t>(end - start) * a.k;
  const uint64_t *src = a.table + static_cast<size_t>(start) * a.k;
  for (size_t i = threadIdx.x; i < entries; i += GS_THREADS) staged[i] = src[i];
  __syncthreads();
  if (threadIdx.x < 32) chain_chunk<true>(a, start, end, visited, staged);
}

// sporder/src/common/similarity_top_k.cu:120-157
__global__ void table_stats_kernel(int32_t n, int32_t k, const uint64_t *__restrict__ table,
                                   uint32_t *ctrl) {
  unsigned long long deg = 0;
  double wsum = 0.0;
  int32_t zero = 0;
  for (int32_t r = blockIdx.x * blockDim.x + threadIdx.x; r < n; r += gridDim.x * blockDim.x) {
    const uint64_t *row = table + static_cast<size_t>(r) * k;
    int32_t d = 0;
    float rw = 0.0f;
    for (int32_t j = 0; j < k; ++j) {
      const uint64_t e = row[j];
      if (entry_index(e) == -1) break;
      d += 1;
      rw += __uint_as_float(entry_weight_bits(e));
    }
    deg += d;
    wsum += rw;
    zero += (d == 0);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    deg += __shfl_down_sync(FULL, deg, off);
    wsum += __shfl_down_sync(FULL, wsum, off);
    zero += __shfl_down_sync(FULL, zero, off);
  }
  if (lane_id() == 0) {
    ChainStats *st = reinterpret_cast<ChainStats *>(ctrl + CTRL_STATS);
    if (deg) {
      atomicAdd(&st->total_degree, deg);
      atomicAdd(&st->total_weight, wsum);
    }
    if (zero) atomicAdd(&st->zero_degree_rows, zero);
  }
}

// Weight of the table entries that stay inside their row's chunk, for the fraction of the
// graph a chunked ordering cuts (sporder/src/cg/chunk_greedy.cu:66-68,111-112;
// cg/stats_collector.cu:66-72).  Summed in fp64.
__global__ void __launch_bounds__(256) in_chunk_weight_kernel(int32_t n, int32_t k, int32_t chunk,
                                                              const uint64_t *__restrict__ table,
                                                              uint32_t *ctrl) {
  double mine = 0.0;
  for (int32_t r = blockIdx.x * blockDim.x + threadIdx.x; r < n; r += gridDim.x * blockDim.x) {
    const int64_t start = static_cast<int64_t>(r / chunk) * chunk;
    const int64_t end = start + chunk < n ? start + chunk : n;
    const uint64_t *row = table + static_cast<size_t>(r) * k;
    for (int32_t j = 0; j < k; ++j) {
      const uint64_t e = row[j];
      if (e == 0) break;
      const int32_t cand = entry_index(e);
      if (cand >= start && cand < end) mine += static_cast<double>(__uint_as_float(entry_weight_bits(e)));
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mine += __shfl_down_sync(FULL, mine, off);
  if ((threadIdx.x & 31) == 0 && mine != 0.0)
    atomicAdd(&reinterpret_cast<ChainStats *>(ctrl + CTRL_STATS)->in_chunk_weight, mine);
}

}  // namespace

bool launch_in_chunk_weight(Context &ctx, int32_t n, int32_t k, int32_t chunk, const uint64_t *table,
                            uint32_t *ctrl) {
  int grid = (n + 255) / 256;
  if (grid > ctx.num_sms * 8) grid = ctx.num_sms * 8;
  in_chunk_weight_kernel<<<grid, 256, 0, ctx.stream>>>(n, k, chunk, table, ctrl);
  CSG_CUDA(cudaGetLastError());
  count_launches(1);
  return true;
}

bool launch_greedy(Context &ctx, int32_t n, const CsgParams &p, CsgScratch &s,
                   int32_t *d_new_order, bool with_stats, int32_t row_base) {
  GreedyArgs a;
  a.n = n;
  a.k = p.k;
  a.chunk = p.chunk;
  a.row_base = row_base;
  a.num_chunks = static_cast<int32_t>((static_cast<int64_t>(n) + p.chunk - 1) / p.chunk);
  a.table = s.table;
  a.row_work = s.row_work;
  a.order = d_new_order;
  a.ctrl = with_stats ? s.ctrl : nullptr;
  a.ctrl_all = s.ctrl;
  const int32_t span = p.chunk < n ? p.chunk : n;
  a.words = (span + 31) / 32;
  size_t smem = static_cast<size_t>(G_WARPS) * 2 * a.words * sizeof(uint32_t);
  a.gbitmaps = nullptr;
  if (smem > 48 * 1024) {  // very large chunks: bitmaps in global memory
    CSG_REQUIRE(s.gbitmaps != nullptr, "greedy: no global bitmap space was reserved");
    a.gbitmaps = s.gbitmaps;
    smem = 0;
  }
  // few chunks: one block per chunk with the chunk's table rows in shared memory, if they fit
  const size_t staged_bytes = static_cast<size_t>((2 * a.words + 3) & ~3) * sizeof(uint32_t) +
                              static_cast<size_t>(span) * p.k * sizeof(uint64_t);
  if (a.num_chunks <= ctx.num_sms && staged_bytes + 1024 <= static_cast<size_t>(ctx.smem_optin)) {
    CSG_CUDA(cudaFuncSetAttribute(greedy_staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(staged_bytes)));
    greedy_staged_kernel<<<a.num_chunks, GS_THREADS, staged_bytes, ctx.stream>>>(a);
    CSG_CUDA(cudaGetLastError());
    count_launches(1);
    return true;
  }
  const int grid = (a.num_chunks + G_WARPS - 1) / G_WARPS;
  greedy_kernel<<<grid, G_WARPS * 32, smem, ctx.stream>>>(a);
  CSG_CUDA(cudaGetLastError());
  count_launches(1);
  return true;
}

bool launch_table_stats(Context &ctx, int32_t n, int32_t k, const uint64_t *table, uint32_t *ctrl) {
  int grid = (n + 255) / 256;
  if (grid > ctx.num_sms * 8) grid = ctx.num_sms * 8;
  table_stats_kernel<<<grid, 256, 0, ctx.stream>>>(n, k, table, ctrl);
  CSG_CUDA(cudaGetLastError());
  count_launches(1);
  return true;
}

}  // namespace csg
