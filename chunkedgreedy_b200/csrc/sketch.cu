// Per-row Space-Saving sketch over the in-chunk candidate stream, then top-k.
//
// Semantics restated from the reference, bit for bit:
//   stream order  sporder/src/common/chunk_similarity_top_k.cu:52-84
//                 (columns of the row ascending; rows of a column ascending;
//                 only rows of the row's own chunk, never the row itself)
//   Dice term     :73-75  alpha = 2.0f / float(|r| + |s|), IEEE fp32 divide
//   container     sporder/src/common/warp_spacesaving.cuh:31-44,109-150
//                 (hit: w += alpha; else first empty slot in (lane, cell) order;
//                 else evict the slot with the least (weight, cell, lane) and
//                 give it weight min + alpha)
//   top-k         :46-66,71-90 (per-lane selection sort by weight, then k rounds
//                 of arg-max over the lanes' cursors, ties to the smaller lane)
//
// What differs is the machinery.  The candidate stream comes from the chunk-local
// transpose (coalesced, no out-of-chunk entries), rows are taken from a work list
// ordered heaviest first (the stream of one row is inherently sequential, so the
// longest rows must start first), and a sketch step costs one vote plus, on a miss
// with a full sketch, two warp reductions (redux.sync) instead of ten shuffles.
#include "common.cuh"

namespace csg {

namespace {

constexpr int S_THREADS = 128;

struct SketchArgs {
  int32_t n, nnz, k, row_base;
  const int32_t *ptr;
  const int2 *seg;
  const int2 *cand;
  const int32_t *row_list;
  uint32_t *ctrl;
  uint64_t *table;
};

// The sketch of one row: CELLS slots per lane.  Slot (lane, cell) is the
// (lane*CELLS + cell)-th to be filled.
template <int CELLS>
struct Sketch {
  int32_t key[CELLS];
  float w[CELLS];
  int32_t filled;  // warp-uniform

  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int c = 0; c < CELLS; ++c) {
      key[c] = -1;
      w[c] = 0.0f;
    }
    filled = 0;
  }

  // one stream element, all lanes hold the same (s, a)
  __device__ __forceinline__ void add(int32_t s, float a) {
    bool hit = false;
#pragma unroll
    for (int c = 0; c < CELLS; ++c) {
      if (key[c] == s) {
        w[c] += a;
        hit = true;
      }
    }
    if (__any_sync(FULL, hit)) return;
    const int lane = lane_id();
    if (filled < 32 * CELLS) {
      const int owner = filled / CELLS, cell = filled % CELLS;
      if (lane == owner) {
#pragma unroll
        for (int c = 0; c < CELLS; ++c) {
          if (c == cell) {
            key[c] = s;
            w[c] = a;
          }
        }
      }
      ++filled;
      return;
    }
    // full: evict the least (weight, cell, lane).  Weights are positive, so their
    // bit patterns order like the values.
    uint32_t lw = __float_as_uint(w[0]);
    int lc = 0;
#pragma unroll
    for (int c = 1; c < CELLS; ++c) {
      const uint32_t wc = __float_as_uint(w[c]);
      if (wc < lw) {
        lw = wc;
        lc = c;
      }
    }
    const uint32_t gmin = __reduce_min_sync(FULL, lw);
    const uint32_t tie = (lw == gmin) ? static_cast<uint32_t>((lc << 5) | lane) : 0xFFFFFFFFu;
    const uint32_t win = __reduce_min_sync(FULL, tie);
    if (lane == static_cast<int>(win & 31u)) {
#pragma unroll
      for (int c = 0; c < CELLS; ++c) {
        if (c == lc) {
          key[c] = s;
          w[c] = w[c] + a;
        }
      }
    }
  }

  __device__ __forceinline__ void local_sort_descending() {
    // the reference's selection sort, including where it stops
#pragma unroll
    for (int i = 0; i < CELLS - 1; ++i) {
      if (key[i] == -1) break;
      int best = i;
      float best_w = w[i];
#pragma unroll
      for (int j = i + 1; j < CELLS; ++j) {
        if (key[j] == -1) break;
        if (w[j] > best_w) {
          best = j;
          best_w = w[j];
        }
      }
      if (best != i) {
        // dynamic register index: resolved with selects after unrolling
        int32_t bk = key[i];
        float bw = w[i];
#pragma unroll
        for (int j = i + 1; j < CELLS; ++j) {
          if (j == best) {
            const int32_t tk = key[j];
            const float tw = w[j];
            key[j] = bk;
            w[j] = bw;
            bk = tk;
            bw = tw;
          }
        }
        key[i] = bk;
        w[i] = bw;
      }
    }
  }

  // writes the valid prefix of the row's k entries (the table is pre-zeroed)
  __device__ __forceinline__ void select_top_k(int32_t k, uint64_t *out, int32_t row_base) {
    local_sort_descending();
    const int lane = lane_id();
    int pos = 0;
    uint64_t mine = 0;
    int i = 0;
    for (; i < k; ++i) {
      float wc = 0.0f;
      int32_t kc = -1;
#pragma unroll
      for (int c = 0; c < CELLS; ++c) {
        if (c == pos) {
          wc = w[c];
          kc = key[c];
        }
      }
      const uint32_t wb = __float_as_uint(wc);
      const uint32_t g = __reduce_max_sync(FULL, wb);
      if (g == 0u) break;  // every lane is past its last filled slot
      const int wl = __ffs(__ballot_sync(FULL, wb == g)) - 1;
      const int32_t ek = __shfl_sync(FULL, kc, wl);
      if (lane == (i & 31)) mine = pack_entry(ek + row_base, __uint_as_float(g));
      if (lane == wl) ++pos;
      if ((i & 31) == 31) {
        out[(i - 31) + lane] = mine;
        mine = 0;
      }
    }
    if ((i & 31) != 0 && lane < (i & 31)) out[(i & ~31) + lane] = mine;
  }
};

template <int CELLS>
__global__ void __launch_bounds__(S_THREADS) sketch_kernel(SketchArgs a) {
  const int lane = lane_id();
  const uint32_t listed = a.ctrl[CTRL_ROWS_LISTED];
  Sketch<CELLS> sk;
  for (;;) {
    uint32_t item = 0;
    if (lane == 0) item = atomicAdd(&a.ctrl[CTRL_ROW_TICKET], 1u);
    item = __shfl_sync(FULL, item, 0);
    if (item >= listed) break;
    const int32_t r = a.row_list[item];
    const int32_t rb = a.ptr[r], re = a.ptr[r + 1];
    const int32_t rs = re - rb;
    if (rb < 0 || rs < 0 || re > a.nnz) {  // malformed row pointers: flag and skip
      if (lane == 0) atomicExch(&a.ctrl[CTRL_BAD_INPUT], 1u);
      continue;
    }
    sk.clear();
    for (int32_t pb = rb; pb < re; pb += 32) {
      const int32_t p = pb + lane;
      int2 sg = make_int2(0, 0);
      if (p < re) sg = a.seg[p];
      unsigned act = __ballot_sync(FULL, sg.y >= 2);
      while (act) {
        const int j = __ffs(act) - 1;
        act &= act - 1;
        const int32_t st = __shfl_sync(FULL, sg.x, j);
        const int32_t len = __shfl_sync(FULL, sg.y, j);
        for (int32_t base = 0; base < len; base += 32) {
          const int32_t i = base + lane;
          int32_t s = -1;
          float al = 0.0f;
          if (i < len) {
            const int2 c = a.cand[st + i];
            if (c.x != r) {
              s = c.x;
              al = 2.0f / static_cast<float>(rs + c.y);
            }
          }
          unsigned todo = __ballot_sync(FULL, s >= 0);
          while (todo) {
            const int t = __ffs(todo) - 1;
            todo &= todo - 1;
            sk.add(__shfl_sync(FULL, s, t), __shfl_sync(FULL, al, t));
          }
        }
      }
    }
    sk.select_top_k(a.k, a.table + static_cast<size_t>(r) * a.k, a.row_base);
  }
}

template <int CELLS>
bool launch_one(Context &ctx, const SketchArgs &a) {
  int per_sm = 0;
  CSG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sketch_kernel<CELLS>, S_THREADS, 0));
  if (per_sm < 1) per_sm = 1;
  sketch_kernel<CELLS><<<ctx.num_sms * per_sm, S_THREADS, 0, ctx.stream>>>(a);
  CSG_CUDA(cudaGetLastError());
  count_launches(1);
  return true;
}

}  // namespace

bool launch_sketch(Context &ctx, int32_t n, int32_t nnz, const CsgParams &p, const int32_t *d_ptr,
                   CsgScratch &s, int32_t row_base) {
  SketchArgs a;
  a.n = n;
  a.nnz = nnz;
  a.k = p.k;
  a.row_base = row_base;
  a.ptr = d_ptr;
  a.seg = s.seg;
  a.cand = s.cand;
  a.row_list = s.row_list;
  a.ctrl = s.ctrl;
  a.table = s.table;
  // rows without candidates are never visited: their entries must read as empty
  CSG_CUDA(cudaMemsetAsync(s.table, 0, sizeof(uint64_t) * static_cast<size_t>(n) * p.k, ctx.stream));
  switch (p.M / 32) {
#define CSG_CASE(C) \
  case C:           \
    return launch_one<C>(ctx, a);
    CSG_CASE(1) CSG_CASE(2) CSG_CASE(3) CSG_CASE(4) CSG_CASE(5) CSG_CASE(6) CSG_CASE(7) CSG_CASE(8)
    CSG_CASE(9) CSG_CASE(10) CSG_CASE(11) CSG_CASE(12) CSG_CASE(13) CSG_CASE(14) CSG_CASE(15)
    CSG_CASE(16)
#undef CSG_CASE
    default:
      set_error("sketch capacity %d is not a multiple of 32 in [32, 512]", p.M);
      return false;
  }
}

}  // namespace csg
