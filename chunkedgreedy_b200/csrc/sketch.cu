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
// What differs is the machinery.  One warp consumes one row's stream, as in the
// reference, but
//  * rows come from a work list ordered heaviest first: the stream of one row is an
//    order-dependent chain, so the longest rows must start first;
//  * stream elements are PRODUCED in batches into shared memory - lane-parallel over the
//    column groups of the chunk-local transpose, coalesced for long groups, Dice terms
//    computed here - and CONSUMED from there in a tight loop, so group bookkeeping,
//    address arithmetic, the divide and DRAM latency stay out of the dependent chain;
//  * a step on a full sketch costs three redux.sync (the cheapest warp collective on
//    this part): one hit test and two for the eviction victim of the NEXT miss, which
//    is computed ahead of time from each lane's cached two smallest weights (see
//    Sketch::add_full);
//  * the rows with the longest streams set the run time of the whole call, and a warp
//    that shares its scheduler with seven others takes 1.6x longer per step.  Those rows
//    (65536 stream elements or more) take a path of their own: their streams are written
//    out to memory by the whole grid (heavy_expand_kernel, one warp per 128 columns),
//    then a chain kernel runs one warp per row and one warp per scheduler - one block per
//    SM, kept alone there by its shared-memory request - doing nothing but consuming.  The
//    kernel of all other rows follows as a programmatic dependent launch: it starts as
//    soon as the chain kernel's blocks are running and fills the SMs that kernel leaves or
//    frees;
//  * for sketches of up to 128 slots the chain kernel does not step through the stream one
//    element at a time: it resolves the longest prefix of the next 32 elements whose
//    outcome can be read off the sketch as it stands, all lanes at once (see "the chains
//    in rounds" below) - 16 elements per round on the longest R-MAT rows, at under half
//    the cost of 16 sequential steps.  Larger sketches keep the element-wise chain
//    (heavy_consume_kernel);
//  * a large call runs in two parts (see run_csg): the chunk with the most nonzeros on a
//    stream of its own, ahead of the rest.  Both parts go through launch_cells with their own
//    lists and control words; their chain kernels have eight warps per block, and only the
//    critical rows - those long enough to decide when the call ends - keep a scheduler to
//    themselves.
#include "common.cuh"

namespace csg {

namespace {

constexpr int S_WARPS = 4;
constexpr int S_THREADS = 32 * S_WARPS;
constexpr int S_RING = 256;    // stream elements per batch, light rows
constexpr int H_PART = SKETCH_PART_COLS;  // columns of a heavy row expanded by one warp: small enough
                                         // that a slice of hub columns (up to chunk-1 candidates
                                         // each) does not become the last warp to finish
constexpr int S_LONG = 48;     // groups with at least this many pending entries are copied by the whole warp

struct SketchArgs {
  int32_t n, nnz, k, row_base, chunk;
  const int32_t *ptr;
  const int2 *seg;
  const int32_t *seg_rank;
  const int2 *cand;
  const int32_t *row_list;
  const uint32_t *row_work;
  uint32_t *ctrl;
  uint64_t *table;
  // materialised streams of the heavy rows
  int2 *hstream;
  uint32_t *heavy_off;
  int32_t *heavy_state;
  uint32_t stream_cap, heavy_max;
  uint32_t *part_base;  // first part of each heavy row, plus the total
  uint32_t *part_off;   // per part: entries it produces, then its offset in hstream
};

// The sketch of one row: CELLS slots per lane, all in registers.  Slot (lane, cell) is
// the (lane*CELLS + cell)-th to be filled; its number is lane*CELLS + cell.
template <int CELLS>
struct Sketch {
  int32_t key[CELLS];
  float w[CELLS];
  int32_t filled;      // warp-uniform
  // valid while the sketch is full:
  uint32_t gmin;       // weight bits of the slot the next miss evicts (same in all lanes)
  int32_t gown;        // its lane
  int32_t gcell;       // its cell
  uint32_t l1w, l2w;   // this lane's smallest and second smallest weight (bits) ...
  int32_t l1c, l2c;    // ... and their cells, ordered by (weight, cell)
  int32_t lane;        // read once through volatile asm: a re-read of the special
                       // register inside the dependent chain costs ~25 cycles each time

  __device__ __forceinline__ void bind_lane() {
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(lane));
  }

  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int c = 0; c < CELLS; ++c) {
      key[c] = -1;
      w[c] = 0.0f;
    }
    filled = 0;
    gmin = 0;
    gown = gcell = 0;
    l1w = l2w = 0;
    l1c = l2c = 0;
  }

  // Weights are positive, so their bit patterns order like the values.  Strict
  // comparisons keep the smaller cell first among equal weights.
  __device__ __forceinline__ void lane_top2() {
    l1w = __float_as_uint(w[0]);
    l1c = 0;
    l2w = 0xFFFFFFFFu;
    l2c = CELLS;  // "none": loses every tie
#pragma unroll
    for (int c = 1; c < CELLS; ++c) {
      const uint32_t x = __float_as_uint(w[c]);
      const bool first = x < l1w, second = x < l2w;
      l2w = first ? l1w : (second ? x : l2w);
      l2c = first ? l1c : (second ? c : l2c);
      l1w = first ? x : l1w;
      l1c = first ? c : l1c;
    }
  }

  // Victim of the next eviction given every lane's smallest (weight, cell): the least
  // (weight, cell, lane).  Two dependent redux.sync.
  __device__ __forceinline__ void find_victim(uint32_t lw, int32_t lc, uint32_t &vmin, int32_t &vown,
                                              int32_t &vcell) const {
    vmin = __reduce_min_sync(FULL, lw);
    const uint32_t t = (lw == vmin) ? static_cast<uint32_t>((lc << 5) | lane) : 0xFFFFFFFFu;
    const uint32_t win = __reduce_min_sync(FULL, t);
    vown = static_cast<int32_t>(win & 31u);
    vcell = static_cast<int32_t>(win >> 5);
  }

  __device__ __forceinline__ void refresh_victim() {
    lane_top2();
    find_victim(l1w, l1c, gmin, gown, gcell);
  }

  // slot (lane, cell) holding key s, or -1.  Warp-uniform result.
  __device__ __forceinline__ int32_t find_slot(int32_t s) const {
    int hit_cell = -1;
#pragma unroll
    for (int c = 0; c < CELLS; ++c) hit_cell = (key[c] == s) ? c : hit_cell;
    const uint32_t hs = __reduce_min_sync(
        FULL, hit_cell >= 0 ? static_cast<uint32_t>(lane * CELLS + hit_cell) : 0xFFFFFFFFu);
    return static_cast<int32_t>(hs);
  }

  __device__ __forceinline__ void add_weight(int32_t slot, float a) {
    const int hl = slot / CELLS, hc = slot % CELLS;
    const bool me = lane == hl;
#pragma unroll
    for (int c = 0; c < CELLS; ++c) w[c] = (me & (c == hc)) ? w[c] + a : w[c];
  }

  __device__ __forceinline__ void put(int32_t slot, int32_t s, float wv) {
    const int ol = slot / CELLS, oc = slot % CELLS;
    const bool me = lane == ol;
#pragma unroll
    for (int c = 0; c < CELLS; ++c) {
      const bool p = me & (c == oc);
      w[c] = p ? wv : w[c];
      key[c] = p ? s : key[c];
    }
  }

  // one stream element while the sketch still has empty slots
  __device__ __forceinline__ void add_filling(int32_t s, float a) {
    const int32_t slot = find_slot(s);
    if (slot >= 0) {
      add_weight(slot, a);
      return;
    }
    put(filled, s, a);
    ++filled;
    if (filled == 32 * CELLS) refresh_victim();
  }

  // One stream element with the sketch full.  Only the victim's lane can change its
  // smallest weight on a miss, and its new smallest is either the re-inserted slot or
  // its cached second smallest: the speculative victim search therefore starts after one
  // add, one compare and one select, and the bookkeeping of the lane's own top-2 runs
  // beside the reductions instead of in front of them.  Written with selects only: a
  // lane-divergent branch here costs more than the rest of the step.
  __device__ __forceinline__ void add_full(int32_t s, float a) {
    const bool own = lane == gown;
    const float wnew = __uint_as_float(gmin) + a;
    const uint32_t nb = __float_as_uint(wnew);
    const int32_t slot = find_slot(s);
    // speculation: this element misses and replaces the cached victim
    const bool new_first = (nb < l2w) | ((nb == l2w) & (gcell < l2c));
    const uint32_t sw = own ? (new_first ? nb : l2w) : l1w;
    const int32_t sc = own ? (new_first ? gcell : l2c) : l1c;
    uint32_t smin;
    int32_t sown, scell;
    find_victim(sw, sc, smin, sown, scell);
    if (slot < 0) {  // miss (warp-uniform): commit
      const int32_t gslot = gown * CELLS + gcell;
      put(gslot, s, wnew);
      if (CELLS <= 2) {  // the lane's pair, reordered
        l2w = own ? (new_first ? l2w : nb) : l2w;
        l2c = own ? (new_first ? l2c : gcell) : l2c;
        l1w = sw;
        l1c = sc;
      } else {
        lane_top2();
      }
      gmin = smin;
      gown = sown;
      gcell = scell;
    } else {  // hit: the speculation is void
      add_weight(slot, a);
      lane_top2();
      if (slot / CELLS == gown) find_victim(l1w, l1c, gmin, gown, gcell);
    }
  }

  // this lane's smallest (weight, cell): all the victim search of the table steps needs
  __device__ __forceinline__ void lane_min() {
    l1w = __float_as_uint(w[0]);
    l1c = 0;
#pragma unroll
    for (int c = 1; c < CELLS; ++c) {
      const uint32_t x = __float_as_uint(w[c]);
      const bool first = x < l1w;
      l1w = first ? x : l1w;
      l1c = first ? c : l1c;
    }
  }

  // ---- steps with a key -> slot table --------------------------------------------------
  // One byte per row of the chunk in shared memory (0 = not in the sketch, else slot + 1)
  // answers "is the key there, and where" with one broadcast load instead of CELLS compares
  // and a warp reduction, and the victim is only looked for when an element misses (two
  // reductions per miss, none per hit).  Fewer instructions per element than add_full, which
  // is what counts where many warps share a scheduler; add_full's speculation buys latency,
  // which counts where a warp has a scheduler to itself.
  __device__ __forceinline__ void add_filling_tab(int32_t s, float a, uint8_t *tab, int32_t cbase) {
    const int q = tab[s - cbase];
    if (q) {  // (same address in all lanes: the branch is uniform)
      add_weight(q - 1, a);
      return;
    }
    put(filled, s, a);
    if (lane == 0) tab[s - cbase] = static_cast<uint8_t>(filled + 1);
    ++filled;
    if (filled == 32 * CELLS) lane_min();
    __syncwarp();
  }

  __device__ __forceinline__ void add_full_tab(int32_t s, float a, uint8_t *tab, int32_t cbase) {
    const int q = tab[s - cbase];
    if (q) {  // hit
      add_weight(q - 1, a);
      lane_min();
      return;
    }
    find_victim(l1w, l1c, gmin, gown, gcell);
    const float wnew = __uint_as_float(gmin) + a;
    const int32_t gslot = gown * CELLS + gcell;
    if (lane == gown) {
      int32_t old_key = key[0];
#pragma unroll
      for (int c = 1; c < CELLS; ++c) old_key = (c == gcell) ? key[c] : old_key;
      tab[old_key - cbase] = 0;
      tab[s - cbase] = static_cast<uint8_t>(gslot + 1);
    }
    put(gslot, s, wnew);
    lane_min();
    __syncwarp();
  }

  // the table is empty again for the next row
  __device__ __forceinline__ void clear_tab(uint8_t *tab, int32_t cbase) const {
#pragma unroll
    for (int c = 0; c < CELLS; ++c)
      if (key[c] >= 0) tab[key[c] - cbase] = 0;
    __syncwarp();
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

  // writes the row's k entries: the valid prefix, then zeros
  __device__ __forceinline__ void select_top_k(int32_t k, uint64_t *out, int32_t row_base) {
    local_sort_descending();
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
    for (int j = i + lane; j < k; j += 32) out[j] = 0;  // the stages behind stop at the first empty entry
  }
};

// Producer side of one row: walks the row's column groups 32 at a time (one per lane)
// and writes the stream, in order and without the row itself, into the warp's ring.
template <int RING>
struct Producer {
  const SketchArgs &a;
  int32_t r, rb, re, rs;
  int32_t pb;         // CSR position of lane 0's column in the current window
  int32_t gst, glen;  // this lane's group: first entry, length (0 when it has no candidates)
  int32_t grank;      // index of row r inside the group
  int32_t done;       // stream entries of this lane's group already produced
  int2 nsg;           // next window, requested one window ahead
  int32_t nrank;

  __device__ __forceinline__ Producer(const SketchArgs &args) : a(args) {}

  // cand[idx], idx from a group descriptor the transpose wrote (checked build: tested)
  __device__ __forceinline__ int2 cand_at(int32_t idx) const {
    return index_ok(a.ctrl, CHK_CAND, idx, a.nnz) ? a.cand[idx] : make_int2(r, 1);
  }

  __device__ __forceinline__ void load_next(int32_t p) {
    nsg = make_int2(0, 0);
    nrank = 0;
    if (p < re) {
      nsg = a.seg[p];
      nrank = a.seg_rank[p];
    }
  }
  __device__ __forceinline__ void take_window() {
    gst = nsg.x;
    glen = nsg.y >= 2 ? nsg.y : 0;
    grank = nrank;
    done = 0;
  }
  // columns [row_begin, row_end) of row `row` (CSR positions), which has row_size entries
  __device__ __forceinline__ void begin(int32_t row, int32_t row_begin, int32_t row_end,
                                        int32_t row_size) {
    r = row;
    rb = row_begin;
    re = row_end;
    rs = row_size;
    pb = rb;
    load_next(pb + lane_id());
    take_window();
    load_next(pb + 32 + lane_id());
  }

  // entry q of this lane's group with the row itself skipped -> (row, alpha)
  __device__ __forceinline__ void emit(int32_t q, int32_t *ring_s, float *ring_a, int32_t at) const {
    const int2 e = cand_at(gst + q + (q >= grank ? 1 : 0));
    ring_s[at] = e.x;
    ring_a[at] = 2.0f / static_cast<float>(rs + e.y);
  }

  // Fills the ring with up to RING elements; returns how many.  0 = stream finished.
  __device__ __forceinline__ int produce(int32_t *ring_s, float *ring_a) {
    const int lane = lane_id();
    int fill = 0;
    for (;;) {
      const int32_t rem = glen > 0 ? glen - 1 - done : 0;
      const unsigned pending = __ballot_sync(FULL, rem > 0);
      if (pending == 0u) {  // window exhausted: next 32 columns
        pb += 32;
        if (pb >= re) break;
        take_window();
        load_next(pb + 32 + lane);
        continue;
      }
      if (fill >= RING) break;
      const unsigned longs = __ballot_sync(FULL, rem >= S_LONG);
      const int first = __ffs(pending) - 1;
      if ((longs >> first) & 1u) {
        // the next group in stream order is a long one: whole warp, coalesced
        const int32_t g_st = __shfl_sync(FULL, gst, first);
        const int32_t g_rank = __shfl_sync(FULL, grank, first);
        const int32_t g_done = __shfl_sync(FULL, done, first);
        const int32_t g_rem = __shfl_sync(FULL, rem, first);
        const int32_t take = g_rem < RING - fill ? g_rem : RING - fill;
        for (int32_t i0 = 0; i0 < take; i0 += 128) {
          int2 e[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int32_t q = g_done + i0 + u * 32 + lane;
            if (i0 + u * 32 + lane < take) e[u] = cand_at(g_st + q + (q >= g_rank ? 1 : 0));
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int32_t i = i0 + u * 32 + lane;
            if (i < take && index_ok(a.ctrl, CHK_RING, fill + i, RING)) {
              ring_s[fill + i] = e[u].x;
              ring_a[fill + i] = 2.0f / static_cast<float>(rs + e[u].y);
            }
          }
        }
        if (lane == first) done += take;
        fill += take;
        continue;
      }
      // leading run of short groups, from `first` up to (not including) the first long
      // group: lane-parallel, ring positions from a prefix sum
      const unsigned later_longs = longs & ~((1u << first) - 1u);
      const int stop = later_longs ? __ffs(later_longs) - 1 : 32;
      const int32_t mine = (lane >= first && lane < stop) ? rem : 0;
      int32_t incl = mine;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int32_t t = __shfl_up_sync(FULL, incl, off);
        if (lane >= off) incl += t;
      }
      const int32_t space = RING - fill;
      const int32_t before = incl - mine;
      int32_t take = space - before;
      take = take < 0 ? 0 : (take > mine ? mine : take);
      {
        // eight independent loads in flight per lane: the copy is latency bound otherwise
        const int32_t at0 = fill + before;
        int32_t i = 0;
        for (; i + 8 <= take; i += 8) {
          int2 e[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int32_t q = done + i + u;
            e[u] = cand_at(gst + q + (q >= grank ? 1 : 0));
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (index_ok(a.ctrl, CHK_RING, at0 + i + u, RING)) {
              ring_s[at0 + i + u] = e[u].x;
              ring_a[at0 + i + u] = 2.0f / static_cast<float>(rs + e[u].y);
            }
          }
        }
        int2 e[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int32_t q = done + i + u;
          if (i + u < take) e[u] = cand_at(gst + q + (q >= grank ? 1 : 0));
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (i + u < take && index_ok(a.ctrl, CHK_RING, at0 + i + u, RING)) {
            ring_s[at0 + i + u] = e[u].x;
            ring_a[at0 + i + u] = 2.0f / static_cast<float>(rs + e[u].y);
          }
        }
      }
      done += take;
      const int32_t total = __shfl_sync(FULL, incl, 31);
      fill += total < space ? total : space;
    }
    __syncwarp();
    return fill;
  }
};

// Feeds `cnt` staged stream elements to the sketch.
template <int CELLS>
__device__ __forceinline__ void consume(Sketch<CELLS> &sk, const int32_t *bs, const float *ba,
                                        int cnt) {
  int t = 0;
  for (; t < cnt && sk.filled < 32 * CELLS; ++t) sk.add_filling(bs[t], ba[t]);
  if (t < cnt) {  // full sketch: the dependent chain, next element requested one step ahead
    int32_t ns = bs[t];
    float na = ba[t];
#pragma unroll 1
    for (; t < cnt; ++t) {
      const int32_t cs = ns;
      const float cf = na;
      const int nt = t + 1 < cnt ? t + 1 : t;
      ns = bs[nt];
      na = ba[nt];
      sk.add_full(cs, cf);
    }
  }
}

// The same with the key -> slot table (see Sketch::add_full_tab).
// A stream key as an index into a table over the chunk's rows: in the checked build a key
// outside the chunk is recorded and replaced by the chunk's first row.
__device__ __forceinline__ int32_t key_in_chunk(uint32_t *ctrl, int32_t s, int32_t cbase, int32_t span) {
  return index_ok(ctrl, CHK_KEY, static_cast<long long>(s) - cbase, span) ? s : cbase;
}

template <int CELLS>
__device__ __forceinline__ void consume_tab(Sketch<CELLS> &sk, uint8_t *tab, int32_t cbase, const int32_t *bs,
                                            const float *ba, int cnt, uint32_t *ctrl, int32_t span) {
  int t = 0;
  for (; t < cnt && sk.filled < 32 * CELLS; ++t) sk.add_filling_tab(key_in_chunk(ctrl, bs[t], cbase, span), ba[t], tab, cbase);
#pragma unroll 1
  for (; t < cnt; ++t) sk.add_full_tab(key_in_chunk(ctrl, bs[t], cbase, span), ba[t], tab, cbase);
}

__device__ __forceinline__ bool row_bounds_ok(const SketchArgs &a, int32_t rb, int32_t re) {
  if (rb < 0 || re < rb || re > a.nnz) {  // malformed row pointers: flag and skip
    if (lane_id() == 0) atomicExch(&a.ctrl[CTRL_BAD_INPUT], 1u);
    return false;
  }
  return true;
}

// All rows below the heavy threshold: one warp per row, producing and consuming in turn.
// TAB: with a key -> slot table per warp (tab_bytes each, dynamic shared memory); without it
// for chunks whose tables would not fit and for sketches of more than 224 slots (the table
// holds slot numbers in a byte).
template <int CELLS, bool TAB>
__global__ void __launch_bounds__(S_THREADS) sketch_kernel(SketchArgs a, int after_primary, int tab_bytes) {
  extern __shared__ __align__(16) unsigned char light_dyn[];
  __shared__ int32_t ring_s[S_WARPS][S_RING];
  __shared__ float ring_a[S_WARPS][S_RING];
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  const uint32_t listed = a.ctrl[CTRL_ROWS_LISTED];
  int32_t *bs = ring_s[warp];
  float *ba = ring_a[warp];
  uint8_t *tab = light_dyn + static_cast<size_t>(warp) * tab_bytes;
  if (TAB) {
    for (int i = lane * 16; i < tab_bytes; i += 32 * 16) *reinterpret_cast<uint4 *>(tab + i) = make_uint4(0, 0, 0, 0);
    __syncwarp();
  }
  Sketch<CELLS> sk;
  sk.bind_lane();
  Producer<S_RING> prod(a);
  for (;;) {
    uint32_t item = 0;
    if (lane == 0) item = atomicAdd(&a.ctrl[CTRL_ROW_TICKET], 1u);  // starts after the heavy rows
    item = __shfl_sync(FULL, item, 0);
    if (item >= listed) break;
    const int32_t r = a.row_list[item];
    if (!index_ok(a.ctrl, CHK_LIST, r, a.n)) continue;
    const int32_t rb = a.ptr[r], re = a.ptr[r + 1];
    if (!row_bounds_ok(a, rb, re)) continue;
    const int32_t cbase = (r / a.chunk) * a.chunk;
    sk.clear();
    prod.begin(r, rb, re, re - rb);
    for (;;) {
      const int cnt = prod.produce(bs, ba);
      if (cnt == 0) break;
      if (TAB)
        consume_tab<CELLS>(sk, tab, cbase, bs, ba, cnt, a.ctrl, tab_bytes);
      else
        consume<CELLS>(sk, bs, ba, cnt);
      __syncwarp();
    }
    if (TAB) sk.clear_tab(tab, cbase);
    sk.select_top_k(a.k, a.table + static_cast<size_t>(r) * a.k, a.row_base);
  }
  // Launched as the programmatic dependent of the heavy-chain kernel, this kernel starts
  // while that one is still running; it must not be seen as finished before it.
  if (after_primary) asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---- heavy rows through materialised streams ------------------------------------------
// offsets of the heavy rows' streams in hstream; trims the heavy set to what fits
__global__ void __launch_bounds__(1024) heavy_offsets_kernel(SketchArgs a) {
  __shared__ unsigned long long sm[32];
  __shared__ unsigned long long carry_s;
  __shared__ uint32_t count_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t H = a.ctrl[CTRL_HEAVY_ROWS];
  if (H > a.heavy_max) H = a.heavy_max;
  if (threadIdx.x == 0) {
    carry_s = 0;
    count_s = H;
  }
  __syncthreads();
  for (uint32_t base = 0; base < H; base += 1024) {
    const uint32_t i = base + threadIdx.x;
    uint32_t v = 0, np = 0;
    if (i < H) {
      const int32_t r = a.row_list[i];
      v = a.row_work[r];
      np = static_cast<uint32_t>((a.ptr[r + 1] - a.ptr[r] + H_PART - 1) / H_PART);
    }
    // parts first (same scan, second value packed in the high half of 64 bits)
    unsigned long long pk = (static_cast<unsigned long long>(np) << 43) | v;  // sums: < 2^21 parts, < 2^43 entries
    unsigned long long incl = pk;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned long long t = __shfl_up_sync(FULL, incl, off);
      if (lane >= off) incl += t;
    }
    if (lane == 31) sm[warp] = incl;
    __syncthreads();
    unsigned long long wbase = 0, tot = 0;
    for (int w = 0; w < 32; ++w) {
      const unsigned long long t = sm[w];
      if (w < warp) wbase += t;
      tot += t;
    }
    const unsigned long long carry = carry_s;
    const unsigned long long excl = carry + wbase + incl - pk;
    if (i < H) {
      const unsigned long long e_off = excl & ((1ull << 43) - 1);
      a.heavy_off[i] = static_cast<uint32_t>(e_off > 0xFFFFFFFFull ? 0xFFFFFFFFull : e_off);
      a.part_base[i] = static_cast<uint32_t>(excl >> 43);
      // first row that does not fit the stream buffer, or whose slices would overflow the
      // 21 bits the scan has for their count: it and the rows behind it stay with the light rows
      if (e_off + v > a.stream_cap || (excl >> 43) + np >= (1ull << 21)) atomicMin(&count_s, i);
    }
    __syncthreads();
    if (threadIdx.x == 0) carry_s = carry + tot;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const uint32_t Hc = count_s;
    // parts of the rows that stay heavy: part_base[Hc] closes the table
    if (Hc == H)
      a.part_base[H] = static_cast<uint32_t>(carry_s >> 43);
    // (when trimmed, part_base[Hc] already holds the first dropped row's base)
    a.ctrl[CTRL_HEAVY_PARTS] = Hc == H ? static_cast<uint32_t>(carry_s >> 43) : a.part_base[Hc];
    a.ctrl[CTRL_HEAVY_ROWS] = count_s;
    a.ctrl[CTRL_ROW_TICKET] = count_s;  // the other rows' tickets start behind the heavy ones
    a.ctrl[CTRL_HEAVY_TICKET] = 0;
    a.ctrl[CTRL_HEAVY_TICKET + 1] = 0;
  }
}

// part -> (heavy row, column range).  Uniform over the warp.
struct PartRef {
  uint32_t item;
  int32_t r, pb, pe, row_size;
};
__device__ __forceinline__ PartRef part_ref(const SketchArgs &a, uint32_t part, uint32_t heavy) {
  uint32_t lo = 0, hi = heavy;  // part_base[lo] <= part < part_base[hi]
  while (hi - lo > 1) {
    const uint32_t mid = (lo + hi) >> 1;
    if (a.part_base[mid] <= part)
      lo = mid;
    else
      hi = mid;
  }
  PartRef p;
  p.item = lo;
  p.r = a.row_list[lo];
  const int32_t rb = a.ptr[p.r], re = a.ptr[p.r + 1];
  p.row_size = re - rb;
  p.pb = rb + static_cast<int32_t>(part - a.part_base[lo]) * H_PART;
  p.pe = p.pb + H_PART < re ? p.pb + H_PART : re;
  if (rb < 0 || re < rb || re > a.nnz) {  // malformed row pointers: nothing to do
    atomicExch(&a.ctrl[CTRL_BAD_INPUT], 1u);
    p.pe = p.pb;
  }
  return p;
}

// stream entries every part (H_PART columns of a heavy row) will produce
__global__ void __launch_bounds__(256) heavy_part_count_kernel(SketchArgs a) {
  const int lane = lane_id();
  const uint32_t heavy = a.ctrl[CTRL_HEAVY_ROWS], parts = a.ctrl[CTRL_HEAVY_PARTS];
  const uint32_t warps = (gridDim.x * blockDim.x) >> 5;
  for (uint32_t part = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; part < parts; part += warps) {
    const PartRef p = part_ref(a, part, heavy);
    uint32_t cnt = 0;
    for (int32_t q = p.pb + lane; q < p.pe; q += 32) {
      const int32_t len = a.seg[q].y;
      cnt += len >= 2 ? static_cast<uint32_t>(len - 1) : 0u;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) cnt += __shfl_down_sync(FULL, cnt, off);
    if (lane == 0) a.part_off[part] = cnt;
  }
}

// counts -> offsets (exclusive scan in place, one block)
__global__ void __launch_bounds__(1024) heavy_part_scan_kernel(SketchArgs a) {
  __shared__ uint32_t sm[32];
  __shared__ uint32_t carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t parts = a.ctrl[CTRL_HEAVY_PARTS];
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (uint32_t base = 0; base < parts; base += 1024) {
    const uint32_t i = base + threadIdx.x;
    const uint32_t v = i < parts ? a.part_off[i] : 0u;
    uint32_t incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t t = __shfl_up_sync(FULL, incl, off);
      if (lane >= off) incl += t;
    }
    if (lane == 31) sm[warp] = incl;
    __syncthreads();
    uint32_t wbase = 0, tot = 0;
    for (int w = 0; w < 32; ++w) {
      const uint32_t t = sm[w];
      if (w < warp) wbase += t;
      tot += t;
    }
    const uint32_t carry = carry_s;
    if (i < parts) a.part_off[i] = carry + wbase + incl - v;
    __syncthreads();
    if (threadIdx.x == 0) carry_s = carry + tot;
    __syncthreads();
  }
}

// one warp per part: its slice of the row's stream, written out in order
__global__ void __launch_bounds__(S_THREADS) heavy_expand_kernel(SketchArgs a) {
  __shared__ int32_t ring_s[S_WARPS][S_RING];
  __shared__ float ring_a[S_WARPS][S_RING];
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  const uint32_t heavy = a.ctrl[CTRL_HEAVY_ROWS], parts = a.ctrl[CTRL_HEAVY_PARTS];
  int32_t *bs = ring_s[warp];
  float *ba = ring_a[warp];
  Producer<S_RING> prod(a);
  for (;;) {
    uint32_t part = 0;
    if (lane == 0) part = atomicAdd(&a.ctrl[CTRL_HEAVY_TICKET], 1u);
    part = __shfl_sync(FULL, part, 0);
    if (part >= parts) break;
    const PartRef p = part_ref(a, part, heavy);
    if (p.pe <= p.pb) continue;
    if (!index_ok(a.ctrl, CHK_LIST, p.r, a.n)) continue;
    uint32_t at = a.part_off[part];
    int2 *out = a.hstream + at;
    prod.begin(p.r, p.pb, p.pe, p.row_size);
    for (;;) {
      const int cnt = prod.produce(bs, ba);
      if (cnt == 0) break;
      // The offsets were laid out from the rows' work counters; a slice that would pass the
      // end of the buffer all the same (counters and groups out of step) is refused, not written.
      if (cnt > static_cast<int>(a.stream_cap) || at > a.stream_cap - static_cast<uint32_t>(cnt)) {
        if (lane == 0) atomicExch(&a.ctrl[CTRL_STREAM_OVERRUN], 1u);
        break;
      }
      for (int i = lane; i < cnt; i += 32) out[i] = make_int2(bs[i], __float_as_int(ba[i]));
      out += cnt;
      at += static_cast<uint32_t>(cnt);
      __syncwarp();
    }
  }
}

// The dependent chains: one warp per heavy row, one warp per scheduler (one block per SM,
// kept alone there by its shared-memory request), reading the stream back in batches.
// The finished sketch goes to memory; the top-k selection is a kernel of its own, because
// with it in the same function the compiler schedules this loop 1.5x slower.
template <int CELLS>
__global__ void __launch_bounds__(S_THREADS, 1) heavy_consume_kernel(SketchArgs a) {
  extern __shared__ __align__(16) unsigned char heavy_pad[];  // only there to fill the SM
  __shared__ int32_t ring_s[S_WARPS][S_RING];
  __shared__ float ring_a[S_WARPS][S_RING];
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  if (heavy_pad[0] == 255 && a.n < 0) return;  // keeps the padding referenced
  // every block of this grid is resident now (one per SM): let the kernel of the other
  // rows, launched behind this one in the same stream, start on whatever is left
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t heavy = a.ctrl[CTRL_HEAVY_ROWS];
  int32_t *bs = ring_s[warp];
  float *ba = ring_a[warp];
  Sketch<CELLS> sk;
  sk.bind_lane();
  for (;;) {
    uint32_t item = 0;
    if (lane == 0) item = atomicAdd(&a.ctrl[CTRL_HEAVY_TICKET + 1], 1u);
    item = __shfl_sync(FULL, item, 0);
    if (item >= heavy) break;
    const int32_t r = a.row_list[item];
    const uint32_t total = a.row_work[r];
    const int2 *in = a.hstream + a.heavy_off[item];
    sk.clear();
    for (uint32_t base = 0; base < total; base += S_RING) {
      const int cnt = static_cast<int>(total - base < S_RING ? total - base : S_RING);
      for (int i = lane; i < cnt; i += 32) {
        const int2 e = in[base + i];
        bs[i] = e.x;
        ba[i] = __int_as_float(e.y);
      }
      __syncwarp();
      consume<CELLS>(sk, bs, ba, cnt);
      __syncwarp();
    }
    int32_t *st = a.heavy_state + static_cast<size_t>(item) * (2 * CELLS * 32);
#pragma unroll
    for (int c = 0; c < CELLS; ++c) {
      st[(2 * c) * 32 + lane] = sk.key[c];
      st[(2 * c + 1) * 32 + lane] = __float_as_int(sk.w[c]);
    }
  }
}

// ---- the chains in rounds ---------------------------------------------------------------
// A full sketch behaves like a queue ordered by (weight, slot code): a miss takes the
// least entry and puts it back heavier, so within a short stretch of the stream the i-th
// miss takes the i-th entry of the order as it stood at the start of the stretch.  A round
// looks at the next 32 stream elements, one per lane, and resolves the longest prefix for
// which that holds, all lanes at once.  With the sketch state S0 at the start of the round,
// m(L) misses among the first L elements and E_0 < E_1 < ... the entries of S0 in order,
// the prefix of length L is resolved exactly as the sequential container would when
//   (1) no two of its misses carry the same key (the second would be a hit on the first),
//   (2) no hit of the prefix lands on one of E_0 .. E_{m(L)-1} (taken before or after the
//       hit, the sequential outcome would differ from the one read off S0), and
//   (3) every entry put back, E_i with weight w(E_i) + alpha, stays above E_{m(L)-1}, so it
//       is not taken again inside the prefix.
// All three only get harder as L grows, so every lane computes the longest prefix its own
// element allows and one redux.sync takes the minimum; L >= 1 always.  Then miss number i
// rewrites slot E_i, hits add their alpha (hits on one key all add the same alpha, so
// their order is immaterial), and the next round starts L elements further on.  While the
// sketch still has empty slots only (1) applies and miss number i fills the next i-th slot.
// On the longest R-MAT rows a round resolves 16 elements on average in about 1000 cycles,
// where 16 sequential steps take 2200.  State lives in shared memory: weights and keys by
// slot code, a key -> slot table over the chunk's rows, and the per-round order.
// Diagnostic builds (python -m chunkedgreedy_b200.build --profile-rounds[=2]), printed by the
// host when CSG_ROUND_PROFILE is set in the environment: -DCSG_ROUND_PROFILE=1 records the
// run time of every heavy row (two clock reads per row), =2 also the cycles per phase of the
// longest row's whole-window rounds (which slows those rounds down).
#if defined(CSG_ROUND_PROFILE) && CSG_ROUND_PROFILE >= 2
#define PROF_DECL unsigned long long prof_t0 = clock64(), prof_t1
#define PROF_MARK(i)                                \
  do {                                              \
    prof_t1 = clock64();                            \
    prof[i] += prof_t1 - prof_t0;                   \
    prof_t0 = prof_t1;                              \
  } while (0)
#define PROF_ADD(i, v) prof[i] += (v)
#else
#define PROF_DECL
#define PROF_MARK(i)
#define PROF_ADD(i, v)
#endif

constexpr int H_RING = 1024;    // stream elements staged per batch
constexpr int ROUND_CELLS = 4;  // largest sketch (cells per lane) resolved in rounds
// Whole-window rounds and the table steps of the light rows are used for sketches of 64 slots
// (two cells per lane: k = 16 at the default oversampling, the benchmark's configuration).
// With 128 slots both measured slower on the R-MAT GCN configuration (sketch stage 55.5 ms
// without either, 62.4 with the whole-window rounds, 65.3 with the table steps, 72.0 with
// both): the ranking of a round grows with the square of the sketch, and a step's work per
// lane with its cells.  With 32 slots a window of 32 can take every entry.
constexpr int WINDOW_CELLS = 2;
constexpr int TRIAL_ROUNDS = 8;     // rounds of each kind a row times before it settles on one ...
constexpr int COMMIT_ROUNDS = 160;  // ... for this many rounds
constexpr int ROUND_RING_BYTES = S_WARPS * 2 * H_RING * 8;

template <int CELLS>
struct RoundState {
  static constexpr int M = 32 * CELLS;
  __align__(16) uint32_t w[M];   // weight bits by slot code (cell * 32 + lane)
  __align__(16) int32_t key[M];
  __align__(16) uint32_t sw[M];  // S0 in ascending (weight, code) order: weights ...
  int32_t si[M];                 // ... and slot codes
  int32_t rank[M];               // position of each slot in that order
  int32_t sk[M];                 // ... and keys
  int32_t miss_pos[32];          // lane of the i-th miss of the window
  uint32_t fence_sink;           // see phase_fence
#ifdef SPORDER_CHECKED
  uint32_t *ctrl;                // checked build: where a key outside its chunk is recorded ...
  int32_t span;                  // ... and the rows the key tables cover
#endif
};

// The key of a stream element as the rounds use it: in the checked build a key outside the
// chunk's table is recorded and replaced by the chunk's first row.
template <int CELLS, bool TAB>
__device__ __forceinline__ int32_t round_key(const RoundState<CELLS> &st, int32_t s, int32_t cbase) {
#ifdef SPORDER_CHECKED
  if (TAB) return key_in_chunk(st.ctrl, s, cbase, st.span);
#endif
  (void)st;
  (void)cbase;
  return s;
}

// Slot that holds key s, or -1.  With TAB from the key -> slot table of the chunk (one byte
// per row); without it - chunks whose tables would not fit shared memory - by comparing s
// with every slot's key (keys are unique in a sketch, empty slots hold -1).
template <int CELLS, bool TAB>
__device__ __forceinline__ int slot_of(const RoundState<CELLS> &st, const uint8_t *tab, int32_t cbase,
                                       int32_t s) {
  if (TAB) return static_cast<int>(tab[s - cbase]) - 1;
  int q = -1;
#pragma unroll
  for (int i4 = 0; i4 < 8 * CELLS; ++i4) {
    const int4 kk = reinterpret_cast<const int4 *>(st.key)[i4];
    q = kk.x == s ? 4 * i4 : q;
    q = kk.y == s ? 4 * i4 + 1 : q;
    q = kk.z == s ? 4 * i4 + 2 : q;
    q = kk.w == s ? 4 * i4 + 3 : q;
  }
  return q;
}

// Keeps the phases of a round apart in the instruction schedule.  Left alone, ptxas
// interleaves the window look-up, the count and the limit look-ups, and the round takes
// 1220 cycles; with a read of %clock between them (which it does not move code across, as
// long as the value is used) it takes 995.  The values go to a word nobody reads.
__device__ __forceinline__ void phase_fence(uint32_t &sink) {
  uint32_t t;
  asm volatile("mov.u32 %0, %%clock;" : "=r"(t));
  sink ^= t;
}

// One round on a full sketch; returns the number of stream elements resolved (>= 1).
template <int CELLS, bool TAB>
__device__ __forceinline__ int round_full(RoundState<CELLS> &st, uint8_t *tab, int32_t cbase,
                                          const int2 *ring, int p, int cnt, int lane,
                                          uint32_t &sink) {
  constexpr int M = 32 * CELLS;
  const uint32_t below = (1u << lane) - 1u;
  phase_fence(sink);
  const bool valid = p + lane < cnt;
  const int2 elem = valid ? ring[p + lane] : make_int2(0, 0);
  const int32_t s = round_key<CELLS, TAB>(st, elem.x, cbase);
  const float al = __int_as_float(elem.y);
  uint32_t mine[CELLS];
  int32_t mykey[CELLS];
#pragma unroll
  for (int c = 0; c < CELLS; ++c) {
    mine[c] = st.w[c * 32 + lane];
    mykey[c] = st.key[c * 32 + lane];
  }
  const int q = valid ? slot_of<CELLS, TAB>(st, tab, cbase, s) : 0;
  const bool miss = valid && q < 0;
  const bool hit = valid && q >= 0;
  // lanes carrying the same key: a second miss of a key ends the prefix (1); hits of one
  // key are added by the first of them
  const unsigned same = __match_any_sync(FULL, valid ? s : -1 - lane);
  const uint32_t wq = st.w[hit ? q : 0];
  const uint32_t missing = __ballot_sync(FULL, miss);
  const int mtot = __popc(missing);
  const int mrank = __popc(missing & below);
  phase_fence(sink);
  // Position of this lane's slots in the (weight, code) order of S0: the number of entries
  // (x, i) below (mine, code).  Weight bit patterns are below 2^31, so x < y is the sign of
  // x - y, and "below" is x < mine + 1 for a smaller code i, x < mine for a larger one.
  // Four chains per slot: one long chain would run at add latency.
  int pos[CELLS];
  {
    int32_t acc[CELLS][4];
#pragma unroll
    for (int c = 0; c < CELLS; ++c) acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0;
    uint4 v[M / 4];
#pragma unroll
    for (int i4 = 0; i4 < M / 4; ++i4) v[i4] = reinterpret_cast<const uint4 *>(st.w)[i4];
#pragma unroll
    for (int i4 = 0; i4 < M / 4; ++i4) {
      const uint32_t x[4] = {v[i4].x, v[i4].y, v[i4].z, v[i4].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = i4 * 4 + e, ci = i >> 5, li = i & 31;
        const uint32_t lower = (below >> li) & 1u;  // code li of this cell is below this lane's
#pragma unroll
        for (int c = 0; c < CELLS; ++c) {
          uint32_t d = x[e] - mine[c];
          if (ci < c) d -= 1u;
          else if (ci == c) d -= lower;
          acc[c][e] += static_cast<int32_t>(d) >> 31;
        }
      }
    }
#pragma unroll
    for (int c = 0; c < CELLS; ++c) pos[c] = -((acc[c][0] + acc[c][1]) + (acc[c][2] + acc[c][3]));
  }
#pragma unroll
  for (int c = 0; c < CELLS; ++c) {
    st.sw[pos[c]] = mine[c];
    st.si[pos[c]] = c * 32 + lane;
    st.sk[pos[c]] = mykey[c];
    st.rank[c * 32 + lane] = pos[c];
  }
  phase_fence(sink);
  if (miss) st.miss_pos[mrank] = lane;
  __syncwarp();
  phase_fence(sink);
  // every lane reads what either kind of element needs, then selects
  const int rho = st.rank[hit ? q : 0];
  const int tgt = st.si[mrank];
  const uint32_t base = st.sw[mrank];
  const int32_t old_key = st.sk[mrank];
  const uint32_t top = st.sw[mtot > 0 ? mtot - 1 : 0];
  const int at_hit = st.miss_pos[rho & 31];
  const int at_next = st.miss_pos[(mrank + 1) & 31];
  const uint32_t nb = __float_as_uint(__uint_as_float(base) + al);
  int lim = valid ? 32 : lane;
  if (hit) {  // (2): this hit and the miss that takes its slot cannot share a prefix
    const int at = rho < mtot ? at_hit : 32;
    lim = at > lane ? at : lane;
  }
  if (miss) {
    // (3): above the heaviest entry any miss of this window can take, the weight put back
    // is safe.  Otherwise (rare) the prefix ends before the next miss, or before this one
    // if the sum did not even grow.
    if (nb <= top) lim = nb > base ? (mrank + 1 < mtot ? at_next : 32) : lane;
    if (same & below) lim = lane;  // (1)
  }
  phase_fence(sink);
  int L = static_cast<int>(__reduce_min_sync(FULL, static_cast<uint32_t>(lim)));
  L = L < 1 ? 1 : L;  // one element alone is always resolved exactly
  const bool applies = lane < L;
  const unsigned mates = same & (L >= 32 ? FULL : (1u << L) - 1u);
  const int times = __popc(mates);
  float wv = __uint_as_float(wq) + al;
  if (times > 1) wv += al;
  if (times > 2)
    for (int t = 2; t < times; ++t) wv += al;
  if (applies && miss) {
    if (TAB) tab[old_key - cbase] = 0;
    st.key[tgt] = s;
    st.w[tgt] = nb;
    if (TAB) tab[s - cbase] = static_cast<uint8_t>(tgt + 1);
  }
  if (applies && hit && (mates & below) == 0u) st.w[q] = __float_as_uint(wv);  // first hit of its key
  __syncwarp();
  return L;
}

// One round on a full sketch of 64 slots or more that resolves the WHOLE window.  The three
// conditions of round_full end a prefix at the first element whose outcome cannot be read off
// the order of S0 directly.  Almost all of those are hits on an entry that the misses of the
// window are about to take, and their outcome still follows from S0 by a little bookkeeping:
//   * the misses take the entries of S0 in order, but skip an entry that a hit has made
//     heavier before they reached it (put back one Dice term heavier, an entry lands behind
//     everything a window of 32 can take: checked below, not assumed);
//   * an element whose key S0 holds in an entry that was taken before the element's turn is
//     a miss, not a hit, and takes the next entry like any other miss;
//   * a second element with the key of an earlier one is a hit on the entry the first one
//     left, whichever kind the first one was.
// Only the first element of each key ("leader") with its entry among the 32 lightest can go
// either way: with P misses before element j and b skipped entries below its entry's rank r,
// the entry is gone iff P + b > r.  Bounds on P + b settle most of them without looking at
// the others (see "slack" below); a window where one stays undecided walks them in stream
// order (a handful per window, state in two 32-bit masks, every lane computing the same).
// The miss with i misses before it
// then takes the (i+1)-th entry that no hit holds back.  The read-off is exact as long as
// nothing put back or made heavier is light enough to be taken again inside the window; an
// element whose new weight does not clear the heaviest entry taken ends the prefix before the
// next miss behind it (before itself, if its weight did not grow at all).  On the heaviest
// R-MAT rows that happens in one window of 32,000 (the row's own Dice terms dominate) to one
// in ten (rows whose terms vary more), and a round resolves 32.0 resp. 29.3 elements where
// round_full resolves 16.4 on the former; it costs about 1.8 times a round_full, which is why
// rounds_row times both kinds on every row and keeps the one that resolves more per cycle.
#ifdef CSG_WINDOW_FENCES
#define WINDOW_FENCE(s) phase_fence(s)
#else
#define WINDOW_FENCE(s)
#endif
template <int CELLS, bool TAB>
__device__ __forceinline__ int round_window(RoundState<CELLS> &st, uint8_t *tab, uint32_t *mates,
                                            int32_t cbase, const int2 *ring, int p, int cnt, int lane,
                                            uint32_t &sink, unsigned long long *prof) {
  constexpr int M = 32 * CELLS;
  static_assert(CELLS >= 2, "a window of 32 needs more than 32 slots");
  const uint32_t below = (1u << lane) - 1u;
  PROF_DECL;
  WINDOW_FENCE(sink);
  const bool valid = p + lane < cnt;
  const int2 elem = valid ? ring[p + lane] : make_int2(0, 0);
  const int32_t s = round_key<CELLS, TAB>(st, elem.x, cbase);
  const float al = __int_as_float(elem.y);
  // Lanes that carry the same key: every lane sets its bit in a word of shared memory under
  // its key and reads the word back (cleared again at the end of the round).  match.any, the
  // instruction made for this, takes some 380 cycles here; it serves chunks too large for
  // the table.
  if (mates != nullptr && valid) atomicOr(&mates[s - cbase], 1u << lane);
  uint32_t mine[CELLS];
  int32_t mykey[CELLS];
#pragma unroll
  for (int c = 0; c < CELLS; ++c) {
    mine[c] = st.w[c * 32 + lane];
    mykey[c] = st.key[c * 32 + lane];
  }
  const int q = valid ? slot_of<CELLS, TAB>(st, tab, cbase, s) : -1;
  const bool present = valid && q >= 0;  // S0 holds the key
  const uint32_t wq = st.w[present ? q : 0];
  WINDOW_FENCE(sink);
  PROF_MARK(0);
  // position of this lane's slots in the (weight, code) order of S0 (see round_full)
  int pos[CELLS];
  {
    int32_t acc[CELLS][4];
#pragma unroll
    for (int c = 0; c < CELLS; ++c) acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0;
    uint4 v[M / 4];
#pragma unroll
    for (int i4 = 0; i4 < M / 4; ++i4) v[i4] = reinterpret_cast<const uint4 *>(st.w)[i4];
#pragma unroll
    for (int i4 = 0; i4 < M / 4; ++i4) {
      const uint32_t x[4] = {v[i4].x, v[i4].y, v[i4].z, v[i4].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = i4 * 4 + e, ci = i >> 5, li = i & 31;
        const uint32_t lower = (below >> li) & 1u;
#pragma unroll
        for (int c = 0; c < CELLS; ++c) {
          uint32_t d = x[e] - mine[c];
          if (ci < c) d -= 1u;
          else if (ci == c) d -= lower;
          acc[c][e] += static_cast<int32_t>(d) >> 31;
        }
      }
    }
#pragma unroll
    for (int c = 0; c < CELLS; ++c) pos[c] = -((acc[c][0] + acc[c][1]) + (acc[c][2] + acc[c][3]));
  }
#pragma unroll
  for (int c = 0; c < CELLS; ++c) st.rank[c * 32 + lane] = pos[c];
  __syncwarp();
  WINDOW_FENCE(sink);
  PROF_MARK(1);
  const int rho = present ? st.rank[q] : M;
  unsigned same;
  if (mates != nullptr)
    same = valid ? mates[s - cbase] : 0u;
  else
    same = __match_any_sync(FULL, valid ? s : -1 - lane);
  const bool leader = valid && (same & below) == 0u;  // first element of its key in the window
  // Which leaders miss: those S0 does not hold, and those whose entry is gone by their turn.
  // An open element (leader, entry among the 32 lightest) with `before` certain misses and
  // `nth` open elements in front of it: at least `before`, at most `before + nth` entries
  // below its own are taken or skipped by its turn, so rank < before means gone and
  // rank >= before + nth means still there, whatever the open elements in front did.  Most
  // windows have only such elements; the others are walked in stream order.
  const uint32_t absent = __ballot_sync(FULL, leader && !present);
  const bool open = leader && present && rho < 32;
  uint32_t open_set = __ballot_sync(FULL, open);
  const int slack = rho - __popc(absent & below);
  const bool sure_gone = open && slack < 0;
  const bool sure_held = open && slack >= __popc(open_set & below);
  uint32_t flipped = __ballot_sync(FULL, sure_gone);  // lanes whose entry was taken before their turn
  uint32_t held = __reduce_or_sync(FULL, sure_held ? 1u << (rho & 31) : 0u);  // ranks a hit holds back
  if (__any_sync(FULL, open && !sure_gone && !sure_held)) {
    flipped = 0u;
    held = 0u;
    while (open_set) {
      const int j = __ffs(open_set) - 1;
      open_set &= open_set - 1u;
      const int r = __shfl_sync(FULL, rho, j);
      const int before = __popc((absent | flipped) & ((1u << j) - 1u));
      const int skipped = __popc(held & ((1u << r) - 1u));
      if (before + skipped > r)
        flipped |= 1u << j;
      else
        held |= 1u << r;
    }
  }
  PROF_MARK(2);
  const uint32_t missing = absent | flipped;
  const int mtot = __popc(missing);
  const bool miss = (missing >> lane) & 1u;
  // The i-th miss takes the i-th entry of the order that no hit holds back: the owners of those
  // entries write them out in that numbering (rank minus the held ranks below it).
#pragma unroll
  for (int c = 0; c < CELLS; ++c) {
    const int r = pos[c];
    if (r < 32 && ((held >> r) & 1u) == 0u) {
      const int at = r - __popc(held & ((1u << r) - 1u));
      st.sw[at] = mine[c];
      st.si[at] = c * 32 + lane;
      st.sk[at] = mykey[c];
      st.miss_pos[at] = r;
    }
  }
  __syncwarp();
  WINDOW_FENCE(sink);
  PROF_MARK(3);
  const int mine_i = miss ? __popc(missing & below) : 0;
  const int last_i = mtot > 0 ? mtot - 1 : 0;
  const int tgt = st.si[mine_i];
  const uint32_t base = st.sw[mine_i];
  const int32_t old_key = st.sk[mine_i];
  const uint32_t top = st.sw[last_i];
  const int t_last = mtot > 0 ? st.miss_pos[last_i] : -1;  // rank of the heaviest entry taken
  const uint32_t behind = missing & ~(below | (1u << lane));
  const int next_miss = behind ? __ffs(behind) - 1 : 32;
  const uint32_t nb = __float_as_uint(__uint_as_float(base) + al);
  const uint32_t hv = __float_as_uint(__uint_as_float(wq) + al);
  int lim = valid ? 32 : lane;
  if (mtot > 0) {
    if (miss && nb <= top) lim = nb > base ? next_miss : lane;
    if (leader && present && !miss && rho <= t_last && hv <= top) lim = hv > wq ? next_miss : lane;
  }
  WINDOW_FENCE(sink);
  int L = static_cast<int>(__reduce_min_sync(FULL, static_cast<uint32_t>(lim)));
  L = L < 1 ? 1 : L;  // one element alone is always resolved exactly
  PROF_MARK(4);
  const bool applies = lane < L && leader;
  const int times = __popc(same & (L >= 32 ? FULL : (1u << L) - 1u));
  float wv = miss ? __uint_as_float(nb) : __uint_as_float(hv);
  for (int k = 1; k < times; ++k) wv += al;  // later elements of the key, in stream order
  if (TAB && applies && miss) tab[old_key - cbase] = 0;
  if (mates != nullptr && valid) mates[s - cbase] = 0u;
  // (a key taken by one miss may be put back by a later one, which then is a flipped lane:
  // clear first, then set)
  if (flipped) __syncwarp();
  if (applies && miss) {
    st.key[tgt] = s;
    st.w[tgt] = __float_as_uint(wv);
    if (TAB) tab[s - cbase] = static_cast<uint8_t>(tgt + 1);
  }
  if (applies && !miss) st.w[q] = __float_as_uint(wv);
  __syncwarp();
  PROF_MARK(5);
  PROF_ADD(6, 1);
  PROF_ADD(7, L);
  return L;
}

// One round while the sketch has empty slots; `filled` is updated.
template <int CELLS, bool TAB>
__device__ __forceinline__ int round_fill(RoundState<CELLS> &st, uint8_t *tab, int32_t cbase,
                                          const int2 *ring, int p, int cnt, int lane,
                                          int &filled) {
  constexpr int M = 32 * CELLS;
  const uint32_t below = (1u << lane) - 1u;
  const bool valid = p + lane < cnt;
  const int2 elem = valid ? ring[p + lane] : make_int2(0, 0);
  const int32_t s = round_key<CELLS, TAB>(st, elem.x, cbase);
  const float al = __int_as_float(elem.y);
  const int q = valid ? slot_of<CELLS, TAB>(st, tab, cbase, s) : 0;
  const bool miss = valid && q < 0;
  const bool hit = valid && q >= 0;
  const uint32_t missing = __ballot_sync(FULL, miss);
  const int mrank = __popc(missing & below);
  const unsigned same = __match_any_sync(FULL, valid ? s : -1 - lane);
  int lim = valid ? 32 : lane;
  if (miss && ((same & below) || mrank >= M - filled)) lim = lane;
  const int L = static_cast<int>(__reduce_min_sync(FULL, static_cast<uint32_t>(lim)));
  const unsigned prefix = L >= 32 ? FULL : (1u << L) - 1u;
  if (lane < L) {
    if (miss) {
      const int j = filled + mrank;  // j-th slot to be filled: lane j / CELLS, cell j % CELLS
      const int code = (j % CELLS) * 32 + j / CELLS;
      st.key[code] = s;
      st.w[code] = __float_as_uint(al);
      if (TAB) tab[s - cbase] = static_cast<uint8_t>(code + 1);
    } else if (hit && ((same & prefix) & below) == 0u) {
      float wv = __uint_as_float(st.w[q]);
      for (int t = __popc(same & prefix); t > 0; --t) wv += al;
      st.w[q] = __float_as_uint(wv);
    }
  }
  filled += __popc(missing & prefix);
  __syncwarp();
  return L;
}

// Same contract as heavy_consume_kernel (one warp per heavy row, one block per SM, final
// sketch to heavy_state), resolving the stream in rounds.  The dynamic shared memory that
// keeps the block alone on its SM holds the key -> slot tables, `tab_bytes` per warp.
// copies `cnt` stream elements into a ring buffer without passing through registers
__device__ __forceinline__ void stage_batch(int2 *ring, const int2 *in, int cnt, int lane) {
  for (int i = lane; i < cnt; i += 32) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(ring + i));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(in + i) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// The whole-window rounds as a function of their own (like rounds_row below: compiled into one
// body with the strict rounds, each kind loses speed to the other's registers and schedule).
// Whole-window rounds on [p, cnt) of a batch, at most `left` of them.
template <int CELLS, bool TAB>
__device__ __noinline__ int window_rounds(RoundState<CELLS> &st, uint8_t *tab, uint32_t *mates,
                                          int32_t cbase, const int2 *ring, int p, int cnt, int &left,
                                          unsigned long long *prof) {
  const int lane = lane_id();
  uint32_t sink = 0;
  while (p < cnt && left > 0) {
    p += round_window<CELLS, TAB>(st, tab, mates, cbase, ring, p, cnt, lane, sink, prof);
    --left;
  }
  if (lane == 0) st.fence_sink = sink;
  return p;
}

// One heavy row, start to finish: stream batches in, rounds, final sketch out.  Not
// inlined: compiled as part of the kernel's ticket loop the same rounds take 1280 cycles
// instead of 1000.
template <int CELLS, bool TAB>
__device__ __noinline__ void rounds_row(const int2 *in, uint32_t total, int32_t cbase,
                                        RoundState<CELLS> &st, uint8_t *tab, uint32_t *mates, int2 *ring0,
                                        int2 *ring1, int32_t *out, unsigned long long *prof_out) {
  constexpr int M = 32 * CELLS;
  const int lane = lane_id();
  unsigned long long prof[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
  (void)prof;
  (void)prof_out;
#pragma unroll
  for (int c = 0; c < CELLS; ++c) {
    st.key[c * 32 + lane] = -1;
    st.w[c * 32 + lane] = 0u;
  }
  int filled = 0, buf = 0;
  // (see the loop below) kind of round in use, rounds left in the stretch, the trial being
  // booked (0 window, 1 strict, -1 none), and what the trials resolved in how many cycles
#ifdef CSG_STRICT_ONLY
  int mode = 1, left = 1 << 30, trial = -1;
#else
  int mode = 0, left = TRIAL_ROUNDS, trial = 0;

#endif
  long long got[2] = {0, 0}, took[2] = {0, 0};
  int streak = 0, last_mode = -1;
  uint32_t sink = 0;
  __syncwarp();
  stage_batch(ring0, in, static_cast<int>(total < H_RING ? total : H_RING), lane);
  for (uint32_t base = 0; base < total; base += H_RING) {
    const int cnt = static_cast<int>(total - base < H_RING ? total - base : H_RING);
    const uint32_t next = base + H_RING;
    if (next < total)
      stage_batch(buf ? ring0 : ring1, in + next, static_cast<int>(total - next < H_RING ? total - next : H_RING), lane);
    else
      asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // all but the newest group: this batch is in
    __syncwarp();
    const int2 *ring = buf ? ring1 : ring0;
    int p = 0;
    while (p < cnt && filled < M) p += round_fill<CELLS, TAB>(st, tab, cbase, ring, p, cnt, lane, filled);
    if constexpr (CELLS == WINDOW_CELLS) {
      // Which kind of round is faster depends on the row: a whole-window round costs more and
      // pays where it resolves (nearly) the whole window - rows whose own length dominates their
      // Dice terms.  Where the terms vary widely, entries put back light are taken again at
      // once, either kind ends after a few elements and the cheaper one wins; and how often a
      // strict round is cut short depends on the sketch size.  So the row measures: a few
      // rounds of each kind against the clock, then a long stretch of the kind that resolved
      // more elements per cycle, and again.
      while (p < cnt) {
        const int before = p;
        const long long t0 = clock64();
        if (mode == 0) {
          p = window_rounds<CELLS, TAB>(st, tab, mates, cbase, ring, p, cnt, left, prof);
        } else {  // (in line: as a function of its own this kind runs a tenth slower)
          while (p < cnt && left > 0) {
            p += round_full<CELLS, TAB>(st, tab, cbase, ring, p, cnt, lane, sink);
            --left;
          }
        }
        if (trial >= 0) {  // a trial stretch: book it
          got[trial] += p - before;
          took[trial] += clock64() - t0;
        }
        if (left == 0) {
          if (trial == 0) {  // window tried: now the strict kind
            trial = 1;
            mode = 1;
            left = TRIAL_ROUNDS;
          } else {
            if (trial == 1)  // both tried: elements per cycle, compared without dividing
              mode = got[0] * took[1] >= got[1] * took[0] ? 0 : 1;
            if (trial == 1) {
              // the stretch grows while the same kind keeps winning (up to 16 times as long)
              streak = mode == last_mode ? (streak < 4 ? streak + 1 : 4) : 0;
              last_mode = mode;
              trial = -1;
              left = COMMIT_ROUNDS << streak;
            } else {  // a committed stretch is over: measure again
              trial = 0;
              mode = 0;
              left = TRIAL_ROUNDS;
              got[0] = got[1] = 0;
              took[0] = took[1] = 0;
            }
          }
        }
      }
    } else {  // other sketch sizes: strict rounds (see WINDOW_CELLS)
      while (p < cnt) p += round_full<CELLS, TAB>(st, tab, cbase, ring, p, cnt, lane, sink);
    }
    buf ^= 1;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int c = 0; c < CELLS; ++c) {
    const int32_t kk = st.key[c * 32 + lane];
    out[(2 * c) * 32 + lane] = kk;
    out[(2 * c + 1) * 32 + lane] = static_cast<int32_t>(st.w[c * 32 + lane]);
    if (TAB && kk >= 0) tab[kk - cbase] = 0;  // the table is empty again for the next row
  }
  if (lane == 0) st.fence_sink = sink;
#ifdef CSG_ROUND_PROFILE
  if (lane == 0 && prof_out != nullptr)
    for (int i = 0; i < 12; ++i) atomicAdd(prof_out + i, prof[i]);
#endif
  __syncwarp();
}

// WARPS per block: four (a scheduler each) for the chains that decide how long the call
// takes; eight, two to a scheduler, for the chains of the rest of a call that runs one chunk
// ahead - they have time to spare and then hold half as many SMs.
template <int CELLS, int WARPS>
__global__ void __launch_bounds__(32 * WARPS, 1) heavy_rounds_kernel(SketchArgs a, int tab_bytes, int mates_words) {
  // dynamic shared memory: two stream buffers per warp (the next batch lands while this
  // one is consumed), then the key tables
  extern __shared__ __align__(16) unsigned char heavy_dyn[];
  constexpr int RING_BYTES = WARPS * 2 * H_RING * 8;
  int2(*rings)[2][H_RING] = reinterpret_cast<int2(*)[2][H_RING]>(heavy_dyn);
  __shared__ RoundState<CELLS> state[WARPS];
  const int lane = lane_id(), warp = threadIdx.x >> 5;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t heavy = a.ctrl[CTRL_HEAVY_ROWS];
  uint8_t *tab = heavy_dyn + RING_BYTES + static_cast<size_t>(warp) * tab_bytes;
  // (behind the four key tables: a word per row of the chunk and warp for round_window's
  // duplicate detection, when it fits)
  uint32_t *mates = mates_words > 0
                        ? reinterpret_cast<uint32_t *>(heavy_dyn + RING_BYTES + static_cast<size_t>(WARPS) * tab_bytes) +
                              static_cast<size_t>(warp) * mates_words
                        : nullptr;
  for (int i = lane; i < mates_words; i += 32) mates[i] = 0u;

#ifdef SPORDER_CHECKED
  if (lane == 0) {
    state[warp].ctrl = a.ctrl;
    state[warp].span = tab_bytes;
  }
  __syncwarp();
#endif
  for (int i = lane * 16; i < tab_bytes; i += 32 * 16) *reinterpret_cast<uint4 *>(tab + i) = make_uint4(0, 0, 0, 0);
  // Blocks of eight warps (a call that runs one chunk ahead): the first blocks take the critical
  // rows at the head of the list with four of their warps (the other four leave at once, so
  // those chains have a scheduler each); the blocks behind them take the other rows eight at a
  // time, in list order, so that the rows fill as few SMs as they can and blocks without rows
  // leave at once.  Blocks of four warps draw tickets.
  auto run_row = [&](uint32_t item) {
    const int32_t r = a.row_list[item];
    // checked build: the row, its place in the state array and its stream's extent
    if (!index_ok(a.ctrl, CHK_LIST, r, a.n) || !index_ok(a.ctrl, CHK_STATE, item, a.heavy_max) ||
        !index_ok(a.ctrl, CHK_STREAM, static_cast<long long>(a.heavy_off[item]) + a.row_work[r],
                  static_cast<long long>(a.stream_cap) + 1))
      return;
    int32_t *out = a.heavy_state + static_cast<size_t>(item) * (2 * CELLS * 32);
#ifdef CSG_ROUND_PROFILE
    const unsigned long long row_t0 = clock64();
    const uint32_t row_off = a.heavy_off[item];
#endif
    if (tab_bytes > 0)
      rounds_row<CELLS, true>(a.hstream + a.heavy_off[item], a.row_work[r], (r / a.chunk) * a.chunk,
                              state[warp], tab, mates, rings[warp][0], rings[warp][1], out,
                              item == 0 ? reinterpret_cast<unsigned long long *>(a.ctrl + CTRL_PROFILE)
                                        : nullptr);  // (profile build: the longest row only)
    else  // chunk too large for key tables in shared memory
      rounds_row<CELLS, false>(a.hstream + a.heavy_off[item], a.row_work[r], 0, state[warp], nullptr,
                               nullptr, rings[warp][0], rings[warp][1], out,
                               reinterpret_cast<unsigned long long *>(a.ctrl + CTRL_PROFILE));
#ifdef CSG_ROUND_PROFILE
    // the row's stream offset is no longer needed: its place takes the row's run time (in
    // units of 1024 cycles), for the host to list the slowest rows
    (void)row_off;
    if (lane == 0) a.heavy_off[item] = static_cast<uint32_t>((clock64() - row_t0) >> 10);
#endif
  };
  if constexpr (WARPS == S_WARPS) {
    for (;;) {
      uint32_t item = 0;
      if (lane == 0) item = atomicAdd(&a.ctrl[CTRL_HEAVY_TICKET + 1], 1u);
      item = __shfl_sync(FULL, item, 0);
      if (item >= heavy) break;
      run_row(item);
    }
  } else {
    uint32_t crit = a.ctrl[CTRL_CRITICAL_ROWS];
    crit = crit < heavy ? crit : heavy;
    uint32_t sparse_blocks = (crit + S_WARPS - 1) / S_WARPS;
    if (sparse_blocks >= gridDim.x) {  // no block left for other rows: all rows alike
      sparse_blocks = gridDim.x;
      crit = heavy;
    }
    uint32_t item, stride, last = heavy;
    if (blockIdx.x < sparse_blocks) {
      if (warp >= S_WARPS) return;
      item = blockIdx.x * S_WARPS + warp;
      stride = sparse_blocks * S_WARPS;
      last = crit;
    } else {
      item = crit + (blockIdx.x - sparse_blocks) * WARPS + warp;
      stride = (gridDim.x - sparse_blocks) * WARPS;
    }
    for (; item < last; item += stride) run_row(item);
  }
}

template <int CELLS>
__global__ void __launch_bounds__(S_THREADS) heavy_topk_kernel(SketchArgs a) {
  const int lane = lane_id();
  const uint32_t heavy = a.ctrl[CTRL_HEAVY_ROWS];
  const uint32_t warps = (gridDim.x * blockDim.x) >> 5;
  Sketch<CELLS> sk;
  sk.bind_lane();
  for (uint32_t item = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; item < heavy; item += warps) {
    const int32_t *st = a.heavy_state + static_cast<size_t>(item) * (2 * CELLS * 32);
    sk.clear();
#pragma unroll
    for (int c = 0; c < CELLS; ++c) {
      sk.key[c] = st[(2 * c) * 32 + lane];
      sk.w[c] = __int_as_float(st[(2 * c + 1) * 32 + lane]);
    }
    const int32_t r = a.row_list[item];
    sk.select_top_k(a.k, a.table + static_cast<size_t>(r) * a.k, a.row_base);
  }
}

template <int CELLS>
bool launch_cells(Context &ctx, const SketchArgs &a, int phase) {
  // A call that runs one chunk ahead has two of these sequences in flight: the chunk ahead on
  // the side stream with a quarter of the SMs for its chains, the rest on the context's stream
  // with the other three quarters (a chain block takes a whole SM, and the kernel of the other
  // rows starts only when every chain block has one).
  cudaStream_t st = phase == PHASE_PRIO ? ctx.side_stream : ctx.stream;
  const int chain_blocks = phase == PHASE_PRIO   ? prio_chain_blocks(ctx.num_sms)
                           : phase == PHASE_REST ? ctx.num_sms - prio_chain_blocks(ctx.num_sms)
                                                 : ctx.num_sms;
  heavy_offsets_kernel<<<1, 1024, 0, st>>>(a);
  CSG_CUDA(cudaGetLastError());
  heavy_part_count_kernel<<<ctx.num_sms * 4, 256, 0, st>>>(a);
  CSG_CUDA(cudaGetLastError());
  heavy_part_scan_kernel<<<1, 1024, 0, st>>>(a);
  CSG_CUDA(cudaGetLastError());
  heavy_expand_kernel<<<ctx.num_sms * 8, S_THREADS, 0, st>>>(a);
  CSG_CUDA(cudaGetLastError());
  // (the rest of the call starts its own chains only behind this point: by then the chains
  // ahead, next in their stream, hold their SMs, and the kernel of the other rows cannot
  // settle on them first)
  if (phase == PHASE_PRIO) CSG_CUDA(cudaEventRecord(ctx.ev[8], st));
  // The chain kernel asks for all the shared memory of an SM, so that it runs one block
  // per SM.  Sketches of up to ROUND_CELLS cells per lane are resolved in rounds, with key
  // tables for a block's four warps (one byte per row of a chunk each) when they fit in there.
  bool in_rounds = false;
  if constexpr (CELLS <= ROUND_CELLS) {
    auto launch_rounds = [&](auto kernel, int warps, int blocks, bool must_fit, bool *launched) -> bool {
      cudaFuncAttributes fa;
      CSG_CUDA(cudaFuncGetAttributes(&fa, kernel));
      const int pad = ctx.smem_optin - 1024 - static_cast<int>(fa.sharedSizeBytes);
      const int64_t ring_bytes = static_cast<int64_t>(warps) * 2 * H_RING * 8;
      int64_t tab_bytes = (static_cast<int64_t>(a.chunk) + 15) / 16 * 16;
      if (ring_bytes + tab_bytes * warps > pad) tab_bytes = 0;  // slots found by comparing keys
      // round_window's duplicate detector: four bytes per row of the chunk and warp, if they fit too
      int64_t mates_words = tab_bytes;
      if (tab_bytes == 0 || ring_bytes + 5 * tab_bytes * warps > pad) mates_words = 0;
      *launched = false;
      if (must_fit && (mates_words == 0 || pad < ring_bytes)) return true;  // (the caller falls back)
      CSG_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pad));
      kernel<<<blocks, 32 * warps, pad, st>>>(a, static_cast<int>(tab_bytes), static_cast<int>(mates_words));
      CSG_CUDA(cudaGetLastError());
      *launched = true;
      return true;
    };
    if (phase != PHASE_ALL && CELLS == WINDOW_CELLS) {
      // eight chains to an SM, if all their tables fit, critical rows apart (see the kernel)
      if (!launch_rounds(heavy_rounds_kernel<CELLS, 2 * S_WARPS>, 2 * S_WARPS, chain_blocks, true, &in_rounds))
        return false;
    }
    if (!in_rounds &&
        !launch_rounds(heavy_rounds_kernel<CELLS, S_WARPS>, S_WARPS, chain_blocks, false, &in_rounds))
      return false;
  }
  if (!in_rounds) {
    const int pad = ctx.smem_optin - 1024 - 2 * S_WARPS * S_RING * 4;
    CSG_CUDA(cudaFuncSetAttribute(heavy_consume_kernel<CELLS>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, pad));
    heavy_consume_kernel<CELLS><<<chain_blocks, S_THREADS, pad, st>>>(a);
    CSG_CUDA(cudaGetLastError());
  }
  // The other rows run beside the heavy chains: their kernel follows in the same stream
  // as a programmatic dependent launch, so its blocks are placed only after every block
  // of the chain kernel is running (and has its SM to itself), and it fills the SMs that
  // stay or fall free.  It waits for the chain kernel before it ends (see sketch_kernel).
  // key -> slot tables for its warps when a chunk's table is small enough that the blocks of an
  // SM still fit (16 KB per block) and slot numbers fit a byte
  int light_tab = 0;
  if constexpr (CELLS == WINDOW_CELLS) {
    const int64_t want = (static_cast<int64_t>(a.chunk < a.n ? a.chunk : a.n) + 15) / 16 * 16;
    if (want <= 4096) light_tab = static_cast<int>(want);
  }
  auto launch_light = [&](auto kernel, int tab_bytes) -> bool {
    const int dyn = tab_bytes * S_WARPS;
    int per_sm = 0;
    CSG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, S_THREADS, dyn));
    if (per_sm < 1) per_sm = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctx.num_sms * per_sm);
    cfg.blockDim = dim3(S_THREADS);
    cfg.dynamicSmemBytes = dyn;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // The chunk ahead has listed only its heavy rows: its kernel of the other rows has work
    // only if some of them did not fit the stream buffer.  It runs behind the chains in plain
    // stream order, where its idle blocks would otherwise sit on the SMs until the chains end.
    cfg.numAttrs = phase == PHASE_PRIO ? 0 : 1;
    CSG_CUDA(cudaLaunchKernelEx(&cfg, kernel, a, phase == PHASE_PRIO ? 0 : 1, tab_bytes));
    return true;
  };
  if constexpr (CELLS == WINDOW_CELLS) {
    if (light_tab > 0) {
      if (!launch_light(sketch_kernel<CELLS, true>, light_tab)) return false;
    } else if (!launch_light(sketch_kernel<CELLS, false>, 0)) {
      return false;
    }
  } else if (!launch_light(sketch_kernel<CELLS, false>, 0)) {
    return false;
  }
  heavy_topk_kernel<CELLS><<<ctx.num_sms, S_THREADS, 0, st>>>(a);
  CSG_CUDA(cudaGetLastError());
  count_launches(7);
  return true;
}

}  // namespace

bool launch_sketch(Context &ctx, int32_t n, int32_t nnz, const CsgParams &p, const int32_t *d_ptr,
                   CsgScratch &s, int32_t row_base, bool zero_table, int phase) {
  SketchArgs a;
  a.n = n;
  a.nnz = nnz;
  a.k = p.k;
  a.row_base = row_base;
  a.chunk = p.chunk;
  a.ptr = d_ptr;
  a.seg = s.seg;
  a.seg_rank = s.seg_rank;
  a.cand = s.cand;
  a.row_list = s.row_list;
  a.row_work = s.row_work;
  a.hstream = s.hstream;
  a.heavy_off = s.heavy_off;
  a.heavy_state = s.heavy_state;
  a.stream_cap = s.stream_cap;
  a.heavy_max = s.heavy_max;
  a.part_base = s.part_base;
  a.part_off = s.part_off;
  a.ctrl = s.ctrl;
  a.table = s.table;
  // Rows without candidates are never visited.  The greedy stage knows them from their work
  // count and never reads their entries; whoever reads the whole table (its export, the
  // statistics) needs them to read as empty.
  if (zero_table)
    CSG_CUDA(cudaMemsetAsync(s.table, 0, sizeof(uint64_t) * static_cast<size_t>(n) * p.k, ctx.stream));
  switch (p.M / 32) {
#define CSG_CASE(C) \
  case C:           \
    return launch_cells<C>(ctx, a, phase);
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
