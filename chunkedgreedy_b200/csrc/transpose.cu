// Chunk-local transpose.
//
// The reference builds a full CSC with a device-wide radix sort
// (sporder/src/common/csr2csc.cu:38-115) and then, per row, scans whole column
// lists to pick out the rows of the row's own chunk
// (sporder/src/common/chunk_similarity_top_k.cu:52-84).  Candidates never leave
// the chunk, so this library transposes every chunk on its own: the chunk's
// (column, position) pairs are sorted by column with a stable LSD radix sort,
// column groups are found, and the kernels emit
//   cand[]  : the chunk's rows grouped by column, rows ascending inside a group,
//             each with its row length (what the Dice term needs);
//   seg[p]  : for nonzero p (CSR order) the group of its column: (first, length),
//             and seg_rank[p], the place of p's own row inside that group;
//   row_work: per row, how many candidates its stream will hold.
// Chunks of up to T_LS nonzeros are handled start to finish by one thread block in
// shared memory (one read of the CSR slice, no intermediate traffic).  Heavier
// chunks - on power-law inputs a handful of chunks hold millions of nonzeros, and
// the rows with the longest streams live in exactly those - are cut into tiles and
// sorted by the whole grid: per pass a tile histogram, a per-chunk scan and a
// stable tile scatter, then a group search per element.
// A caller-promised symmetric pattern needs no sort at all: column c's rows inside a chunk
// are the entries of ROW c that fall into the chunk's row range, already ascending, so the
// CSR arrays themselves serve as cand[] (with the row lengths looked up) and a group is a
// sub-range of row c found by binary search (symmetric_groups_kernel).  The reference takes
// the same promise and reads the aliased CSR arrays as the CSC
// (sporder/src/common/csr2csc.h:52-54); like there, a false promise gives a different
// (still valid) permutation, never an out-of-range access.
#include "common.cuh"

namespace csg {

namespace {

constexpr int T_THREADS = 512;
constexpr int T_WARPS = T_THREADS / 32;
constexpr int T_IPT = 8;
constexpr int T_TILE = T_THREADS * T_IPT;  // 4096
constexpr int T_LS = 15360;                // largest chunk (nonzeros) sorted in shared memory
constexpr int T_RP = 2048;                 // largest chunk (rows) with row tables in shared memory

struct TransposeArgs {
  int32_t n, nnz, chunk, num_chunks, passes;
  const int32_t *ptr, *ind;
  uint32_t *keyA, *keyB, *payA, *payB;
  int2 *cand, *seg;
  int32_t *seg_rank;
  uint32_t *row_work;
  uint32_t *ctrl;
  // heavy chunks (more than T_LS nonzeros)
  int32_t *heavy_chunk;      // chunk ids, in arrival order
  int32_t *heavy_tile_base;  // first tile of each heavy chunk, plus the total
  uint32_t *tile_hist;       // [tile][256] digit counts, then offsets
  uint32_t *digit_base;      // [heavy chunk][256]
  // a call that runs one chunk ahead: the control words that name the chunk, and whether this
  // pass leaves that chunk out (nullptr / false otherwise)
  const uint32_t *ctrl_main;
  bool skip_prio;
};

struct ChunkSpan {
  int32_t cs, rows, b, L;
};

__device__ __forceinline__ ChunkSpan chunk_span(const TransposeArgs &a, int32_t q) {
  ChunkSpan c;
  const int64_t cs64 = static_cast<int64_t>(q) * a.chunk;
  c.cs = static_cast<int32_t>(cs64);
  const int32_t ce = (cs64 + a.chunk > a.n) ? a.n : static_cast<int32_t>(cs64 + a.chunk);
  c.rows = ce - c.cs;
  c.b = a.ptr[c.cs];
  c.L = a.ptr[ce] - c.b;
  if (c.b < 0 || c.L < 0 || c.L > a.nnz - c.b) {  // malformed row pointers: flag and skip
    atomicExch(&a.ctrl[CTRL_BAD_INPUT], 1u);
    c.L = 0;
  }
  return c;
}

struct Shared {
  uint32_t wc[T_WARPS * 256];
  uint32_t hist[256];
  uint32_t binbase[256];
  int32_t warp_last[T_WARPS];
  int32_t carry;
  int32_t ticket;
  int32_t sptr[T_RP + 1];
  uint32_t row_work[T_RP];
  uint32_t skey[2][T_LS];
  uint16_t spay[2][T_LS];
};

// One stable counting pass on an 8-bit digit.  FIRST reads the keys from the CSR
// column array and uses the position as payload.
template <typename PayT, bool FIRST>
__device__ void radix_pass(const uint32_t *kin, const PayT *pin, uint32_t *kout, PayT *pout,
                           int L, int shift, Shared &sh, uint32_t *ctrl) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < 256) sh.hist[tid] = 0;
  __syncthreads();
  for (int i = tid; i < L; i += T_THREADS) atomicAdd(&sh.hist[(kin[i] >> shift) & 255u], 1u);
  __syncthreads();
  if (warp == 0) {  // exclusive scan of 256 bins, 8 per lane
    uint32_t v[8], s = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[j] = sh.hist[lane * 8 + j];
      s += v[j];
    }
    uint32_t incl = s;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      uint32_t t = __shfl_up_sync(FULL, incl, off);
      if (lane >= off) incl += t;
    }
    uint32_t run = incl - s;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      sh.binbase[lane * 8 + j] = run;
      run += v[j];
    }
  }
  __syncthreads();

  for (int tb = 0; tb < L; tb += T_TILE) {
    for (int j = tid; j < T_WARPS * 256; j += T_THREADS) sh.wc[j] = 0;
    __syncthreads();
    uint32_t key[T_IPT], rk[T_IPT];
    PayT pay[T_IPT];
    const int wbase = tb + warp * (32 * T_IPT);
#pragma unroll
    for (int i = 0; i < T_IPT; ++i) {
      const int idx = wbase + i * 32 + lane;
      const bool valid = idx < L;
      key[i] = valid ? kin[idx] : 0u;
      if (FIRST)
        pay[i] = static_cast<PayT>(idx);
      else
        pay[i] = valid ? pin[idx] : PayT(0);
      const uint32_t d = valid ? ((key[i] >> shift) & 255u) : 256u;
      const unsigned peers = match_digit(d);
      const int leader = __ffs(peers) - 1;
      uint32_t pre = 0;
      if (lane == leader && valid) {
        pre = sh.wc[warp * 256 + d];
        sh.wc[warp * 256 + d] = pre + __popc(peers);
      }
      pre = __shfl_sync(FULL, pre, leader);
      rk[i] = pre + __popc(peers & ((1u << lane) - 1u));
      __syncwarp();
    }
    __syncthreads();
    if (tid < 256) {  // per digit: running offsets over the warps, carried over tiles
      uint32_t run = sh.binbase[tid];
#pragma unroll
      for (int w = 0; w < T_WARPS; ++w) {
        const uint32_t t = sh.wc[w * 256 + tid];
        sh.wc[w * 256 + tid] = run;
        run += t;
      }
      sh.binbase[tid] = run;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < T_IPT; ++i) {
      const int idx = wbase + i * 32 + lane;
      if (idx < L) {
        const uint32_t d = (key[i] >> shift) & 255u;
        const uint32_t dst = sh.wc[warp * 256 + d] + rk[i];
        if (index_ok(ctrl, CHK_SORT, dst, L)) {
          kout[dst] = key[i];
          pout[dst] = pay[i];
        }
      }
    }
    __syncthreads();
  }
}

// Row that owns CSR position x: largest row with ptr[row] <= x, searched in
// [row_lo, row_hi] over either the shared copy of the chunk's row pointers or the
// global array.
__device__ __forceinline__ int32_t row_of(const int32_t *p, int32_t lo, int32_t hi, int32_t x) {
  // invariant: p[lo] <= x < p[hi]
  while (hi - lo > 1) {
    const int32_t mid = lo + ((hi - lo) >> 1);
    if (p[mid] <= x)
      lo = mid;
    else
      hi = mid;
  }
  return lo;
}

// After the sort: K = sorted columns, P = positions (chunk-local).  S / LN are the
// free ping-pong buffers, reused for the group start of every element and the
// group length stored at the group's first element.
template <typename PayT>
__device__ void emit_groups(const uint32_t *K, const PayT *P, uint32_t *S, PayT *LN, int L,
                            int32_t b, int32_t cs, int32_t rows, bool rows_in_smem,
                            const TransposeArgs &a, Shared &sh) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) sh.carry = 0;
  __syncthreads();
  for (int tb = 0; tb < L; tb += T_TILE) {
    const int wbase = tb + warp * (32 * T_IPT);
    int32_t last = -1;
    int32_t st[T_IPT];
    uint32_t key[T_IPT];
#pragma unroll
    for (int i = 0; i < T_IPT; ++i) {
      const int idx = wbase + i * 32 + lane;
      const bool valid = idx < L;
      key[i] = valid ? K[idx] : 0u;
      const uint32_t prev = (valid && idx > 0) ? K[idx - 1] : 0u;
      const bool head = valid && (idx == 0 || key[i] != prev);
      const unsigned hm = __ballot_sync(FULL, head);
      const unsigned le = hm & (FULL >> (31 - lane));
      st[i] = le ? (wbase + i * 32 + (31 - __clz(le))) : last;
      if (hm) last = wbase + i * 32 + (31 - __clz(hm));
    }
    if (lane == 0) sh.warp_last[warp] = last;
    __syncthreads();
    int32_t carry = sh.carry;
    for (int w = 0; w < warp; ++w) {
      const int32_t t = sh.warp_last[w];
      if (t >= 0) carry = t;
    }
#pragma unroll
    for (int i = 0; i < T_IPT; ++i) {
      const int idx = wbase + i * 32 + lane;
      if (idx < L) {
        const int32_t s = st[i] >= 0 ? st[i] : carry;
        S[idx] = static_cast<uint32_t>(s);
        const bool tail = (idx == L - 1) || (K[idx + 1] != key[i]);
        if (tail) LN[s] = static_cast<PayT>(idx + 1 - s);
      }
    }
    __syncthreads();
    if (tid == 0) {
      int32_t c = sh.carry;
      for (int w = 0; w < T_WARPS; ++w)
        if (sh.warp_last[w] >= 0) c = sh.warp_last[w];
      sh.carry = c;
    }
    __syncthreads();
  }
  for (int i = tid; i < L; i += T_THREADS) {
    const int32_t p = static_cast<int32_t>(P[i]);
    const int32_t st = static_cast<int32_t>(S[i]);
    if (!index_ok(a.ctrl, CHK_GROUP, p, L) || !index_ok(a.ctrl, CHK_GROUP, st, L)) continue;
    const int32_t len = static_cast<int32_t>(LN[st]);
    int32_t row;
    if (rows_in_smem)
      row = cs + row_of(sh.sptr, 0, rows, b + p);
    else
      row = row_of(a.ptr, cs, cs + rows, b + p);
    const int32_t rl = rows_in_smem ? (sh.sptr[row - cs + 1] - sh.sptr[row - cs])
                                    : (a.ptr[row + 1] - a.ptr[row]);
    a.cand[b + i] = make_int2(row, rl);
    a.seg[b + p] = make_int2(b + st, len);
    a.seg_rank[b + p] = i - st;
    if (len >= 2) {
      // (a row's count can pass 32 bits when the chunk is the whole matrix: it sticks at the
      // ceiling, which the sketch stage reads as "does not fit the stream buffer")
      if (rows_in_smem)
        saturating_add(&sh.row_work[row - cs], static_cast<uint32_t>(len - 1));
      else
        saturating_add(&a.row_work[row], static_cast<uint32_t>(len - 1));
    }
  }
}

__global__ void __launch_bounds__(T_THREADS, 1) transpose_kernel(TransposeArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Shared &sh = *reinterpret_cast<Shared *>(smem_raw);
  const int tid = threadIdx.x;
  for (;;) {
    __syncthreads();
    if (tid == 0) sh.ticket = static_cast<int32_t>(atomicAdd(&a.ctrl[CTRL_CHUNK_TICKET], 1u));
    __syncthreads();
    const int32_t q = sh.ticket;
    if (q >= a.num_chunks) break;
    const ChunkSpan c = chunk_span(a, q);
    const int32_t cs = c.cs, rows = c.rows, b = c.b;
    const int L = c.L;
    if (L > T_LS || L == 0) continue;  // heavy chunks go through the tiled kernels
    const bool rows_in_smem = rows <= T_RP;
    if (rows_in_smem) {
      for (int i = tid; i <= rows; i += T_THREADS) sh.sptr[i] = a.ptr[cs + i];
      for (int i = tid; i < rows; i += T_THREADS) sh.row_work[i] = 0;
    }
    __syncthreads();
    const uint32_t *kin0 = reinterpret_cast<const uint32_t *>(a.ind + b);
    const int P = a.passes;
    radix_pass<uint16_t, true>(kin0, nullptr, sh.skey[0], sh.spay[0], L, 0, sh, a.ctrl);
    for (int ps = 1; ps < P; ++ps)
      radix_pass<uint16_t, false>(sh.skey[(ps - 1) & 1], sh.spay[(ps - 1) & 1], sh.skey[ps & 1],
                                  sh.spay[ps & 1], L, 8 * ps, sh, a.ctrl);
    const int f = (P - 1) & 1;
    emit_groups<uint16_t>(sh.skey[f], sh.spay[f], sh.skey[f ^ 1], sh.spay[f ^ 1], L, b, cs, rows,
                          rows_in_smem, a, sh);
    __syncthreads();
    if (rows_in_smem)
      for (int i = tid; i < rows; i += T_THREADS) a.row_work[cs + i] = sh.row_work[i];
  }
}

// ---- heavy chunks: tiled, whole-grid sort ----------------------------------------

__global__ void classify_chunks_kernel(TransposeArgs a) {
  for (int32_t q = blockIdx.x * blockDim.x + threadIdx.x; q < a.num_chunks;
       q += gridDim.x * blockDim.x) {
    const ChunkSpan c = chunk_span(a, q);
    if (a.skip_prio && static_cast<uint32_t>(q) == a.ctrl_main[CTRL_PRIO]) continue;
    if (c.L > T_LS) a.heavy_chunk[atomicAdd(&a.ctrl[CTRL_HEAVY_COUNT], 1u)] = q;
  }
}

// The chunk that runs ahead of the rest: the one with the most nonzeros, if it is a heavy
// chunk of at least min_nnz nonzeros (a row that streams 65,536 candidates or more needs a
// chunk about that big).  It becomes the only entry of `ap`'s list of heavy chunks.
__global__ void __launch_bounds__(1024) pick_priority_kernel(TransposeArgs a, TransposeArgs ap, int32_t min_nnz) {
  __shared__ unsigned long long best[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long mine = 0;  // (nonzeros << 32) | ~chunk: the first of equally heavy chunks wins
  for (int32_t q = threadIdx.x; q < a.num_chunks; q += blockDim.x) {
    const ChunkSpan c = chunk_span(a, q);
    const unsigned long long v = (static_cast<unsigned long long>(c.L) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(q));
    mine = v > mine ? v : mine;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const unsigned long long t = __shfl_down_sync(FULL, mine, off);
    mine = t > mine ? t : mine;
  }
  if (lane == 0) best[warp] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 32; ++w) mine = best[w] > mine ? best[w] : mine;
    const int32_t L = static_cast<int32_t>(mine >> 32);
    const uint32_t q = 0xFFFFFFFFu - static_cast<uint32_t>(mine);
    const bool on = L > T_LS && L >= min_nnz;
    a.ctrl[CTRL_PRIO] = on ? q : PRIO_NONE;
    ap.ctrl[CTRL_PRIO] = on ? q : PRIO_NONE;
    ap.ctrl[CTRL_HEAVY_COUNT] = on ? 1u : 0u;
    ap.heavy_chunk[0] = on ? static_cast<int32_t>(q) : 0;
  }
}

// Work list of the chunk ahead: its rows that stream 65,536 candidates or more (the other
// rows of the chunk go with everybody else's), longest stream first, so that the eight rows a
// block of the chain kernel takes are of a length and the block is done when they are.  The
// critical rows - at least half as long as the longest, the ones that can decide when the call
// ends; their chains keep a scheduler to themselves - are then the head of the list.  One block;
// a chunk has at most PRIO_MAX_CHUNK rows.
constexpr int PRIO_MAX_CHUNK = 4096;
__global__ void __launch_bounds__(1024) priority_rows_kernel(TransposeArgs ap, int32_t *row_list) {
  __shared__ int32_t s_row[PRIO_MAX_CHUNK];
  __shared__ uint32_t s_work[PRIO_MAX_CHUNK];
  __shared__ uint32_t count, critical;
  __shared__ unsigned long long need;
  if (threadIdx.x == 0) {
    count = 0;
    need = 0;
    critical = 0;
  }
  __syncthreads();
  const uint32_t prio = ap.ctrl[CTRL_PRIO];
  uint32_t longest = 0;
  if (prio != PRIO_NONE && ap.chunk <= PRIO_MAX_CHUNK) {
    const int64_t start = static_cast<int64_t>(prio) * ap.chunk;
    const int64_t end = start + ap.chunk < ap.n ? start + ap.chunk : ap.n;
    for (int64_t r = start + threadIdx.x; r < end; r += blockDim.x) {
      const uint32_t t = ap.row_work[r];
      if (t >= (1u << (SKETCH_HEAVY_BUCKET - 1))) {
        const uint32_t at = atomicAdd(&count, 1u);
        s_row[at] = static_cast<int32_t>(r);
        s_work[at] = t;
        atomicAdd(&need, static_cast<unsigned long long>(t));
      }
    }
    __syncthreads();
    const uint32_t H = count;
    // place of every row in the order (longer stream first, then smaller row id)
    for (uint32_t i = threadIdx.x; i < H; i += blockDim.x) {
      const uint32_t w = s_work[i];
      const int32_t r = s_row[i];
      uint32_t before = 0;
      for (uint32_t j = 0; j < H; ++j) {
        const uint32_t wj = s_work[j];
        before += (wj > w || (wj == w && s_row[j] < r)) ? 1u : 0u;
      }
      row_list[before] = r;
      if (before == 0) longest = w;
    }
    // (the thread that placed the first row knows the longest stream)
    const uint32_t top = __reduce_max_sync(FULL, longest);
    if ((threadIdx.x & 31) == 0 && top) atomicMax(&critical, top);  // borrowed as a maximum for a moment
    __syncthreads();
    longest = critical;
    __syncthreads();
    if (threadIdx.x == 0) critical = 0;
    __syncthreads();
    const uint32_t bar = longest - longest / 2;
    uint32_t mine = 0;
    for (uint32_t i = threadIdx.x; i < H; i += blockDim.x) mine += s_work[i] >= bar ? 1u : 0u;
    mine = __reduce_add_sync(FULL, mine);
    if ((threadIdx.x & 31) == 0 && mine) atomicAdd(&critical, mine);
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    ap.ctrl[CTRL_ROWS_LISTED] = count;
    ap.ctrl[CTRL_HEAVY_ROWS] = count;
    ap.ctrl[CTRL_CRITICAL_ROWS] = critical;
    ap.ctrl[CTRL_CRITICAL_TICKET] = 0;
    ap.ctrl[CTRL_LONGEST] = longest;
    ap.ctrl[CTRL_ROW_TICKET] = count;
    ap.ctrl[CTRL_HEAVY_TICKET] = 0;
    ap.ctrl[CTRL_HEAVY_TICKET + 1] = 0;
    *reinterpret_cast<unsigned long long *>(ap.ctrl + CTRL_HEAVY_NEED) = need;
  }
}

// exclusive scan of the heavy chunks' tile counts (one block)
__global__ void __launch_bounds__(1024) heavy_tiles_kernel(TransposeArgs a) {
  __shared__ int32_t sm[32];
  __shared__ int32_t carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int32_t H = static_cast<int32_t>(a.ctrl[CTRL_HEAVY_COUNT]);
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int32_t base = 0; base < H; base += 1024) {
    const int32_t i = base + threadIdx.x;
    int32_t v = 0;
    if (i < H) v = (chunk_span(a, a.heavy_chunk[i]).L + T_TILE - 1) / T_TILE;
    int32_t incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int32_t t = __shfl_up_sync(FULL, incl, off);
      if (lane >= off) incl += t;
    }
    if (lane == 31) sm[warp] = incl;
    __syncthreads();
    int32_t wbase = 0, tot = 0;
    for (int w = 0; w < 32; ++w) {
      const int32_t t = sm[w];
      if (w < warp) wbase += t;
      tot += t;
    }
    const int32_t carry = carry_s;
    if (i < H) a.heavy_tile_base[i] = carry + wbase + incl - v;
    __syncthreads();
    if (threadIdx.x == 0) carry_s = carry + tot;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    a.heavy_tile_base[H] = carry_s;
    a.ctrl[CTRL_HEAVY_TILES] = static_cast<uint32_t>(carry_s);
  }
}

struct TileRef {
  int32_t h, b, L, off, cnt, cs, rows;
};

// tile t -> its heavy chunk and range (uniform over the block)
__device__ __forceinline__ TileRef tile_ref(const TransposeArgs &a, int32_t t, int32_t H) {
  int32_t lo = 0, hi = H;  // heavy_tile_base[lo] <= t < heavy_tile_base[hi]
  while (hi - lo > 1) {
    const int32_t mid = (lo + hi) >> 1;
    if (a.heavy_tile_base[mid] <= t)
      lo = mid;
    else
      hi = mid;
  }
  const ChunkSpan c = chunk_span(a, a.heavy_chunk[lo]);
  TileRef r;
  r.h = lo;
  r.b = c.b;
  r.L = c.L;
  r.cs = c.cs;
  r.rows = c.rows;
  r.off = (t - a.heavy_tile_base[lo]) * T_TILE;
  r.cnt = c.L - r.off < T_TILE ? c.L - r.off : T_TILE;
  return r;
}

__device__ __forceinline__ const uint32_t *pass_src_keys(const TransposeArgs &a, int ps, int32_t b) {
  if (ps == 0) return reinterpret_cast<const uint32_t *>(a.ind + b);
  return ((ps - 1) & 1 ? a.keyB : a.keyA) + b;
}

__global__ void __launch_bounds__(T_THREADS) heavy_hist_kernel(TransposeArgs a, int ps) {
  __shared__ uint32_t hist[256];
  const int32_t TT = static_cast<int32_t>(a.ctrl[CTRL_HEAVY_TILES]);
  const int32_t H = static_cast<int32_t>(a.ctrl[CTRL_HEAVY_COUNT]);
  const int shift = 8 * ps;
  for (int32_t t = blockIdx.x; t < TT; t += gridDim.x) {
    const TileRef r = tile_ref(a, t, H);
    const uint32_t *kin = pass_src_keys(a, ps, r.b) + r.off;
    if (threadIdx.x < 256) hist[threadIdx.x] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < r.cnt; i += T_THREADS) atomicAdd(&hist[(kin[i] >> shift) & 255u], 1u);
    __syncthreads();
    if (threadIdx.x < 256) a.tile_hist[static_cast<size_t>(t) * 256 + threadIdx.x] = hist[threadIdx.x];
    __syncthreads();
  }
}

// per heavy chunk: counts -> offsets of every (tile, digit) inside the digit's run,
// and the start of every digit's run
__global__ void __launch_bounds__(256) heavy_scan_kernel(TransposeArgs a) {
  __shared__ uint32_t sm[8];
  const int32_t H = static_cast<int32_t>(a.ctrl[CTRL_HEAVY_COUNT]);
  const int d = threadIdx.x, lane = d & 31, warp = d >> 5;
  for (int32_t h = blockIdx.x; h < H; h += gridDim.x) {
    const int32_t t0 = a.heavy_tile_base[h], t1 = a.heavy_tile_base[h + 1];
    // a chunk of millions of nonzeros has hundreds of tiles: sixteen loads in flight per
    // thread, or the walk costs one memory latency per tile
    uint32_t run = 0;
    for (int32_t tb = t0; tb < t1; tb += 16) {
      uint32_t v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u)
        v[u] = tb + u < t1 ? a.tile_hist[static_cast<size_t>(tb + u) * 256 + d] : 0u;
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        if (tb + u < t1) a.tile_hist[static_cast<size_t>(tb + u) * 256 + d] = run;
        run += v[u];
      }
    }
    uint32_t incl = run;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t t = __shfl_up_sync(FULL, incl, off);
      if (lane >= off) incl += t;
    }
    __syncthreads();
    if (lane == 31) sm[warp] = incl;
    __syncthreads();
    uint32_t wbase = 0;
    for (int w = 0; w < warp; ++w) wbase += sm[w];
    a.digit_base[static_cast<size_t>(h) * 256 + d] = wbase + incl - run;
  }
}

__global__ void __launch_bounds__(T_THREADS) heavy_scatter_kernel(TransposeArgs a, int ps) {
  __shared__ uint32_t wc[T_WARPS * 256];
  const int32_t TT = static_cast<int32_t>(a.ctrl[CTRL_HEAVY_TILES]);
  const int32_t H = static_cast<int32_t>(a.ctrl[CTRL_HEAVY_COUNT]);
  const int shift = 8 * ps;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int32_t t = blockIdx.x; t < TT; t += gridDim.x) {
    const TileRef r = tile_ref(a, t, H);
    const uint32_t *kin = pass_src_keys(a, ps, r.b) + r.off;
    const uint32_t *pin = ps == 0 ? nullptr : ((ps - 1) & 1 ? a.payB : a.payA) + r.b + r.off;
    uint32_t *kout = (ps & 1 ? a.keyB : a.keyA) + r.b;
    uint32_t *pout = (ps & 1 ? a.payB : a.payA) + r.b;
    for (int j = tid; j < T_WARPS * 256; j += T_THREADS) wc[j] = 0;
    __syncthreads();
    uint32_t key[T_IPT], rk[T_IPT], pay[T_IPT];
    const int wbase = warp * (32 * T_IPT);
#pragma unroll
    for (int i = 0; i < T_IPT; ++i) {
      const int idx = wbase + i * 32 + lane;
      const bool valid = idx < r.cnt;
      key[i] = valid ? kin[idx] : 0u;
      pay[i] = ps == 0 ? static_cast<uint32_t>(r.off + idx) : (valid ? pin[idx] : 0u);
      const uint32_t d = valid ? ((key[i] >> shift) & 255u) : 256u;
      const unsigned peers = match_digit(d);
      const int leader = __ffs(peers) - 1;
      uint32_t pre = 0;
      if (lane == leader && valid) {
        pre = wc[warp * 256 + d];
        wc[warp * 256 + d] = pre + __popc(peers);
      }
      pre = __shfl_sync(FULL, pre, leader);
      rk[i] = pre + __popc(peers & ((1u << lane) - 1u));
      __syncwarp();
    }
    __syncthreads();
    if (tid < 256) {
      uint32_t run = a.digit_base[static_cast<size_t>(r.h) * 256 + tid] +
                     a.tile_hist[static_cast<size_t>(t) * 256 + tid];
#pragma unroll
      for (int w = 0; w < T_WARPS; ++w) {
        const uint32_t v = wc[w * 256 + tid];
        wc[w * 256 + tid] = run;
        run += v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < T_IPT; ++i) {
      const int idx = wbase + i * 32 + lane;
      if (idx < r.cnt) {
        const uint32_t d = (key[i] >> shift) & 255u;
        const uint32_t dst = wc[warp * 256 + d] + rk[i];
        if (index_ok(a.ctrl, CHK_SORT, dst, r.L)) {
          kout[dst] = key[i];
          pout[dst] = pay[i];
        }
      }
    }
    __syncthreads();
  }
}

// Group of every sorted element by two bounded binary searches: a column group
// has at most one entry per row of the chunk, so its ends lie within `rows`
// positions of the element.  For chunks of up to E_ROWS rows the searches run on
// shared-memory copies - the tile's keys with a halo of rows-1 on either side and the
// chunk's row pointers - and the rows' work counters are summed in shared memory first:
// on global memory the kernel was bound by the latency of some thirty dependent loads per
// element and by atomics of a whole tile landing on the same few hub rows.
constexpr int E_ROWS = 1024;
__global__ void __launch_bounds__(T_THREADS) heavy_emit_kernel(TransposeArgs a) {
  __shared__ uint32_t skey[T_TILE + 2 * (E_ROWS - 1)];
  __shared__ int32_t sptr[E_ROWS + 1];
  __shared__ uint32_t swork[E_ROWS];
  const int32_t TT = static_cast<int32_t>(a.ctrl[CTRL_HEAVY_TILES]);
  const int32_t H = static_cast<int32_t>(a.ctrl[CTRL_HEAVY_COUNT]);
  const int f = (a.passes - 1) & 1;
  for (int32_t t = blockIdx.x; t < TT; t += gridDim.x) {
    const TileRef r = tile_ref(a, t, H);
    const uint32_t *K = (f ? a.keyB : a.keyA) + r.b;
    const uint32_t *P = (f ? a.payB : a.payA) + r.b;
    const bool staged = r.rows <= E_ROWS;
    int32_t w0 = 0;  // first sorted position held in skey
    if (staged) {
      w0 = r.off - (r.rows - 1) < 0 ? 0 : r.off - (r.rows - 1);
      const int32_t w1 = r.off + r.cnt + (r.rows - 1) < r.L ? r.off + r.cnt + (r.rows - 1) : r.L;
      for (int32_t j = threadIdx.x; j < w1 - w0; j += T_THREADS) skey[j] = K[w0 + j];
      for (int32_t j = threadIdx.x; j <= r.rows; j += T_THREADS) sptr[j] = a.ptr[r.cs + j];
      for (int32_t j = threadIdx.x; j < r.rows; j += T_THREADS) swork[j] = 0u;
      __syncthreads();
    }
    for (int li = threadIdx.x; li < r.cnt; li += T_THREADS) {
      const int32_t i = r.off + li;
      const uint32_t key = staged ? skey[i - w0] : K[i];
      int32_t lo = i - (r.rows - 1) < 0 ? 0 : i - (r.rows - 1), hi = i;  // first index with K >= key
      while (lo < hi) {
        const int32_t mid = (lo + hi) >> 1;
        if ((staged ? skey[mid - w0] : K[mid]) < key)
          lo = mid + 1;
        else
          hi = mid;
      }
      const int32_t st = lo;
      lo = i + 1;
      hi = i + r.rows < r.L ? i + r.rows : r.L;  // first index with K > key
      while (lo < hi) {
        const int32_t mid = (lo + hi) >> 1;
        if ((staged ? skey[mid - w0] : K[mid]) <= key)
          lo = mid + 1;
        else
          hi = mid;
      }
      const int32_t len = lo - st;
      const int32_t p = static_cast<int32_t>(P[i]);
      if (!index_ok(a.ctrl, CHK_GROUP, p, r.L)) continue;
      int32_t row, rl;
      if (staged) {
        const int32_t lr = row_of(sptr, 0, r.rows, r.b + p);
        row = r.cs + lr;
        rl = sptr[lr + 1] - sptr[lr];
        if (len >= 2) saturating_add(&swork[lr], static_cast<uint32_t>(len - 1));
      } else {
        row = row_of(a.ptr, r.cs, r.cs + r.rows, r.b + p);
        rl = a.ptr[row + 1] - a.ptr[row];
        if (len >= 2) saturating_add(&a.row_work[row], static_cast<uint32_t>(len - 1));
      }
      a.cand[r.b + i] = make_int2(row, rl);
      a.seg[r.b + p] = make_int2(r.b + st, len);
      a.seg_rank[r.b + p] = i - st;
    }
    if (staged) {
      __syncthreads();
      for (int32_t j = threadIdx.x; j < r.rows; j += T_THREADS)
        if (swork[j]) saturating_add(&a.row_work[r.cs + j], swork[j]);
      __syncthreads();
    }
  }
}

// ---- symmetric pattern: groups read off the CSR arrays --------------------------------
// One thread per nonzero p = (r, c): cand[p] = (c, length of row c) - cand is the column
// array with lengths attached - and the group of column c in r's chunk is the part of row c
// inside [chunk start, chunk end), found with three binary searches over row c that run in
// step (the two ends and r's own place).  Blocks take tiles of Y_TILE positions; the rows a
// tile touches are found once per tile and their pointers staged in shared memory.
constexpr int Y_THREADS = 256;
constexpr int Y_TILE = 2048;
constexpr int Y_ROWS = 2048;  // rows of a tile with pointers in shared memory (more: searched in global memory)

__global__ void __launch_bounds__(Y_THREADS) symmetric_groups_kernel(TransposeArgs a) {
  __shared__ int32_t sptr[Y_ROWS + 1];
  __shared__ int32_t span[2];
  const int tid = threadIdx.x, lane = tid & 31;
  const int32_t tiles = (a.nnz + Y_TILE - 1) / Y_TILE;
  if (a.ptr[0] != 0 || a.ptr[a.n] != a.nnz) {  // the row search below relies on both ends
    if (tid == 0) atomicExch(&a.ctrl[CTRL_BAD_INPUT], 1u);
    return;
  }
  for (int32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int32_t p_first = tile * Y_TILE;
    const int32_t p_end = a.nnz - p_first < Y_TILE ? a.nnz : p_first + Y_TILE;
    __syncthreads();
    if (tid < 2) span[tid] = row_of(a.ptr, 0, a.n, tid ? p_end - 1 : p_first);
    __syncthreads();
    const int32_t r_first = span[0], r_last = span[1] < span[0] ? span[0] : span[1];
    const int32_t nrows = r_last - r_first + 1;
    const bool staged = nrows <= Y_ROWS;
    if (staged)
      for (int32_t i = tid; i <= nrows; i += Y_THREADS) sptr[i] = a.ptr[r_first + i];
    __syncthreads();
    for (int32_t p0 = p_first; p0 < p_end; p0 += Y_THREADS) {
      const int32_t p = p0 + tid;
      int32_t r = -1;
      uint32_t add = 0;
      if (p < p_end) {
        r = staged ? r_first + row_of(sptr, 0, nrows, p) : row_of(a.ptr, r_first, r_last + 1, p);
        const int32_t rb = a.ptr[r], re = a.ptr[r + 1];
        const int32_t c = a.ind[p];
        int32_t pc = 0, pe = 0;
        bool ok = p >= rb && p < re && c >= 0 && c < a.n;  // (row pointers that are not ascending fail here)
        if (ok) {
          pc = a.ptr[c];
          pe = a.ptr[c + 1];
          ok = pc >= 0 && pe >= pc && pe <= a.nnz;
        }
        if (!ok) {
          atomicExch(&a.ctrl[CTRL_BAD_INPUT], 1u);
          a.cand[p] = make_int2(r, 1);
          a.seg[p] = make_int2(p, 0);
          a.seg_rank[p] = 0;
        } else {
          a.cand[p] = make_int2(c, pe - pc);
          const int64_t q0 = static_cast<int64_t>(r / a.chunk) * a.chunk;
          const int64_t q1 = q0 + a.chunk;
          // first entries of row c not below the chunk start, the chunk end and r
          int32_t lo_a = pc, hi_a = pe, lo_b = pc, hi_b = pe, lo_r = pc, hi_r = pe;
          while (lo_a < hi_a || lo_b < hi_b || lo_r < hi_r) {
            const int32_t ma = (lo_a + hi_a) >> 1, mb = (lo_b + hi_b) >> 1, mr = (lo_r + hi_r) >> 1;
            const int32_t va = lo_a < hi_a ? a.ind[ma] : 0;
            const int32_t vb = lo_b < hi_b ? a.ind[mb] : 0;
            const int32_t vr = lo_r < hi_r ? a.ind[mr] : 0;
            if (lo_a < hi_a) {
              if (va < q0) lo_a = ma + 1; else hi_a = ma;
            }
            if (lo_b < hi_b) {
              if (vb < q1) lo_b = mb + 1; else hi_b = mb;
            }
            if (lo_r < hi_r) {
              if (vr < r) lo_r = mr + 1; else hi_r = mr;
            }
          }
          // (rows that are not sorted can cross the three results: keep them ordered)
          const int32_t first = lo_a;
          const int32_t last = lo_b < first ? first : lo_b;
          int32_t at = lo_r < first ? first : lo_r;
          at = at > last ? last : at;
          const int32_t len = last - first;
          a.seg[p] = make_int2(first, len);
          a.seg_rank[p] = at - first;
          if (len >= 2) add = static_cast<uint32_t>(len - 1);
        }
      }
      // the candidates each row will see: one atomic per warp where the warp sits in one row
      const int32_t r_lead = __shfl_sync(FULL, r, 0);
      if (__all_sync(FULL, r == r_lead || r < 0) && r_lead >= 0 && __all_sync(FULL, add < (1u << 26))) {
        const uint32_t sum = __reduce_add_sync(FULL, add);
        if (lane == 0 && sum) saturating_add(&a.row_work[r_lead], sum);
      } else if (add) {
        saturating_add(&a.row_work[r], add);
      }
    }
  }
}

// rows per power-of-two bucket of row_work
// rows of the chunk that runs ahead which that part of the call takes itself
__device__ __forceinline__ bool taken_ahead(uint32_t prio, int32_t chunk, int32_t r, uint32_t work) {
  return prio != PRIO_NONE && work >= (1u << (SKETCH_HEAVY_BUCKET - 1)) &&
         static_cast<uint32_t>(r / chunk) == prio;
}

__global__ void __launch_bounds__(256) bucket_count_kernel(int32_t n, const uint32_t *row_work,
                                                           uint32_t *ctrl, int32_t chunk, bool skip_prio) {
  __shared__ uint32_t bucket[33];
  __shared__ unsigned long long need;
  if (threadIdx.x < 33) bucket[threadIdx.x] = 0;
  if (threadIdx.x == 0) need = 0;
  __syncthreads();
  const uint32_t prio = skip_prio ? ctrl[CTRL_PRIO] : PRIO_NONE;
  for (int32_t r = blockIdx.x * blockDim.x + threadIdx.x; r < n; r += gridDim.x * blockDim.x) {
    uint32_t t = __ldcg(row_work + r);
    if (taken_ahead(prio, chunk, r, t)) t = 0;
    if (t) atomicAdd(&bucket[32 - __clz(t)], 1u);
    // stream elements of the rows heavy enough for a materialised stream: what the stream
    // buffer would have to hold for all of them (the host sizes the next call's buffer by it)
    if (t >= (1u << (SKETCH_HEAVY_BUCKET - 1))) atomicAdd(&need, static_cast<unsigned long long>(t));
  }
  __syncthreads();
  if (threadIdx.x < 33 && bucket[threadIdx.x])
    atomicAdd(&ctrl[CTRL_BUCKET_COUNT + threadIdx.x], bucket[threadIdx.x]);
  if (threadIdx.x == 0 && need)
    atomicAdd(reinterpret_cast<unsigned long long *>(ctrl + CTRL_HEAVY_NEED), need);
}

// Heaviest bucket first: rows with 2^(b-1) <= work < 2^b sit in bucket b.
// ctrl_ahead: the control words of the chunk that runs ahead, when the call has one.  The rows
// of this list that are within a factor of four of the longest stream of the whole call (their
// bucket is the top one or the one below) count as critical like the long rows of the chunk
// ahead: their chains keep a scheduler to themselves (see heavy_rounds_kernel).
__global__ void bucket_scan_kernel(uint32_t *ctrl, const uint32_t *ctrl_ahead) {
  if (threadIdx.x == 0) {
    uint32_t run = 0;
    int top = 0;
    for (int b = 32; b >= 1; --b) {
      ctrl[CTRL_BUCKET_BASE + b] = run;
      run += ctrl[CTRL_BUCKET_COUNT + b];
      ctrl[CTRL_BUCKET_FILL + b] = 0;
      if (top == 0 && ctrl[CTRL_BUCKET_COUNT + b]) top = b;
    }
    if (ctrl_ahead) {
      const uint32_t longest = ctrl_ahead[CTRL_LONGEST];
      const int top_ahead = longest ? 32 - __clz(longest) : 0;
      top = top_ahead > top ? top_ahead : top;
      int from = top - 1 > SKETCH_HEAVY_BUCKET ? top - 1 : SKETCH_HEAVY_BUCKET;
      ctrl[CTRL_CRITICAL_ROWS] = from <= 32 ? ctrl[CTRL_BUCKET_BASE + from - 1] : 0u;  // rows of buckets >= from
      ctrl[CTRL_CRITICAL_TICKET] = 0;
    }
    ctrl[CTRL_ROWS_LISTED] = run;
    // rows with at least 2^(SKETCH_HEAVY_BUCKET-1) stream elements head the list; the
    // heavy sketch kernel takes them, the other kernel's tickets start behind them
    const uint32_t heavy = ctrl[CTRL_BUCKET_BASE + SKETCH_HEAVY_BUCKET - 1];
    ctrl[CTRL_HEAVY_ROWS] = heavy;
    ctrl[CTRL_HEAVY_TICKET] = 0;
    ctrl[CTRL_ROW_TICKET] = heavy;
  }
}

__global__ void row_list_kernel(int32_t n, const uint32_t *__restrict__ row_work, uint32_t *ctrl,
                                int32_t *__restrict__ row_list, int32_t chunk, bool skip_prio) {
  const int lane = threadIdx.x & 31;
  const int32_t total = gridDim.x * blockDim.x;
  const uint32_t prio = skip_prio ? ctrl[CTRL_PRIO] : PRIO_NONE;
  for (int32_t base = blockIdx.x * blockDim.x; base < n; base += total) {
    const int32_t r = base + threadIdx.x;
    uint32_t t = r < n ? row_work[r] : 0u;
    if (r < n && taken_ahead(prio, chunk, r, t)) t = 0;
    const uint32_t bkt = t ? (32 - __clz(t)) : 0u;
    const unsigned peers = __match_any_sync(FULL, bkt);
    if (bkt) {
      const int leader = __ffs(peers) - 1;
      uint32_t pre = 0;
      if (lane == leader) pre = atomicAdd(&ctrl[CTRL_BUCKET_FILL + bkt], __popc(peers));
      pre = __shfl_sync(peers, pre, leader);
      row_list[ctrl[CTRL_BUCKET_BASE + bkt] + pre + __popc(peers & ((1u << lane) - 1u))] = r;
    }
  }
}

}  // namespace

namespace {
TransposeArgs transpose_args(int32_t n, int32_t ncols, int32_t nnz, int32_t chunk, const int32_t *d_ptr,
                             const int32_t *d_ind, const CsgScratch &s) {
  TransposeArgs a;
  a.n = n;
  a.nnz = nnz;
  a.chunk = chunk;
  a.num_chunks = static_cast<int32_t>((static_cast<int64_t>(n) + chunk - 1) / chunk);
  int bits = 1;
  while (bits < 32 && (static_cast<int64_t>(1) << bits) < ncols) ++bits;  // column ids < ncols
  a.passes = (bits + 7) / 8;
  a.ptr = d_ptr;
  a.ind = d_ind;
  a.keyA = s.keyA;
  a.keyB = s.keyB;
  a.payA = s.payA;
  a.payB = s.payB;
  a.cand = s.cand;
  a.seg = s.seg;
  a.seg_rank = s.seg_rank;
  a.row_work = s.row_work;
  a.ctrl = s.ctrl;
  a.heavy_chunk = s.heavy_chunk;
  a.heavy_tile_base = s.heavy_tile_base;
  a.tile_hist = s.tile_hist;
  a.digit_base = s.digit_base;
  a.ctrl_main = nullptr;
  a.skip_prio = false;
  return a;
}
}  // namespace

bool launch_priority_pick(Context &ctx, int32_t n, int32_t nnz, int32_t chunk, const int32_t *d_ptr,
                          CsgScratch &s, CsgScratch &prio, int32_t min_chunk_nnz) {
  const TransposeArgs a = transpose_args(n, n, nnz, chunk, d_ptr, nullptr, s);
  const TransposeArgs ap = transpose_args(n, n, nnz, chunk, d_ptr, nullptr, prio);
  cudaStream_t st = ctx.stream;
  CSG_CUDA(cudaMemsetAsync(s.ctrl, 0, sizeof(uint32_t) * CTRL_WORDS, st));
  CSG_CUDA(cudaMemsetAsync(prio.ctrl, 0, sizeof(uint32_t) * CTRL_WORDS, st));
  CSG_CUDA(cudaMemsetAsync(s.row_work, 0, sizeof(uint32_t) * static_cast<size_t>(n), st));
  pick_priority_kernel<<<1, 1024, 0, st>>>(a, ap, min_chunk_nnz);
  CSG_CUDA(cudaGetLastError());
  count_launches(1);
  return true;
}

// phase PHASE_ALL: the whole transposition on the context's stream.  PHASE_PRIO (on the side
// stream, `s` = the scratch of the part that runs ahead): the one chunk launch_priority_pick
// named, then that chunk's list of heavy rows; ctx.ev[6] marks the end of its transposition.
// PHASE_REST (context's stream): every other chunk, then - once ev[6] has passed, because the
// lists read the work counters of all rows - the lists of everything the part ahead left.
bool launch_transpose(Context &ctx, int32_t n, int32_t ncols, int32_t nnz, int32_t chunk, const int32_t *d_ptr,
                      const int32_t *d_ind, CsgScratch &s, bool symmetric, int phase, uint32_t *ctrl_other) {
  // ctrl_other: the control words of the other part of a call that runs one chunk ahead
  TransposeArgs a = transpose_args(n, ncols, nnz, chunk, d_ptr, d_ind, s);
  a.ctrl_main = phase == PHASE_PRIO && ctrl_other ? ctrl_other : s.ctrl;
  const uint32_t *ctrl_ahead = phase == PHASE_REST ? ctrl_other : nullptr;
  a.skip_prio = phase == PHASE_REST;
  const size_t smem = sizeof(Shared);
  CSG_CUDA(cudaFuncSetAttribute(transpose_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(smem)));
  cudaStream_t st = phase == PHASE_PRIO ? ctx.side_stream : ctx.stream;
  if (phase == PHASE_ALL) {
    CSG_CUDA(cudaMemsetAsync(s.ctrl, 0, sizeof(uint32_t) * CTRL_WORDS, st));
    CSG_CUDA(cudaMemsetAsync(s.row_work, 0, sizeof(uint32_t) * static_cast<size_t>(n), st));
  }
  int lgrid = (n + 255) / 256;
  if (lgrid > ctx.num_sms * 8) lgrid = ctx.num_sms * 8;
  if (phase == PHASE_ALL && symmetric && n == ncols && nnz > 0) {
    // the caller's promise: the pattern is its own transpose
    int ygrid = (nnz + Y_TILE - 1) / Y_TILE;
    if (ygrid > ctx.num_sms * 8) ygrid = ctx.num_sms * 8;
    symmetric_groups_kernel<<<ygrid, Y_THREADS, 0, st>>>(a);
    CSG_CUDA(cudaGetLastError());
    bucket_count_kernel<<<lgrid, 256, 0, st>>>(n, s.row_work, s.ctrl, chunk, false);
    CSG_CUDA(cudaGetLastError());
    bucket_scan_kernel<<<1, 32, 0, st>>>(s.ctrl, nullptr);
    CSG_CUDA(cudaGetLastError());
    row_list_kernel<<<lgrid, 256, 0, st>>>(n, s.row_work, s.ctrl, s.row_list, chunk, false);
    CSG_CUDA(cudaGetLastError());
    count_launches(4);
    return true;
  }
  if (phase != PHASE_PRIO) {  // (the part ahead got its one heavy chunk from launch_priority_pick)
    int cgrid = (a.num_chunks + 255) / 256;
    if (cgrid > ctx.num_sms * 4) cgrid = ctx.num_sms * 4;
    classify_chunks_kernel<<<cgrid, 256, 0, st>>>(a);
    CSG_CUDA(cudaGetLastError());
  }
  heavy_tiles_kernel<<<1, 1024, 0, st>>>(a);
  CSG_CUDA(cudaGetLastError());
  // heavy chunks first: the rows with the longest streams live in them
  const int hgrid = ctx.num_sms * 2;
  int sgrid = a.num_chunks < ctx.num_sms ? a.num_chunks : ctx.num_sms;
  if (phase == PHASE_PRIO) sgrid = 1;
  for (int ps = 0; ps < a.passes; ++ps) {
    heavy_hist_kernel<<<hgrid, T_THREADS, 0, st>>>(a, ps);
    CSG_CUDA(cudaGetLastError());
    heavy_scan_kernel<<<sgrid, 256, 0, st>>>(a);
    CSG_CUDA(cudaGetLastError());
    heavy_scatter_kernel<<<hgrid, T_THREADS, 0, st>>>(a, ps);
    CSG_CUDA(cudaGetLastError());
  }
  heavy_emit_kernel<<<hgrid * 2, T_THREADS, 0, st>>>(a);
  CSG_CUDA(cudaGetLastError());
  if (phase == PHASE_PRIO) {
    priority_rows_kernel<<<1, 1024, 0, st>>>(a, s.row_list);
    CSG_CUDA(cudaGetLastError());
    CSG_CUDA(cudaEventRecord(ctx.ev[6], st));  // the rest may read this chunk's work counters and its longest stream
    count_launches(3 + 3 * a.passes);
    return true;
  }
  const int grid = a.num_chunks < ctx.num_sms ? a.num_chunks : ctx.num_sms;
  transpose_kernel<<<grid, T_THREADS, smem, st>>>(a);
  CSG_CUDA(cudaGetLastError());
  if (phase == PHASE_REST) CSG_CUDA(cudaStreamWaitEvent(st, ctx.ev[6], 0));
  bucket_count_kernel<<<lgrid, 256, 0, st>>>(n, s.row_work, s.ctrl, chunk, phase == PHASE_REST);
  CSG_CUDA(cudaGetLastError());
  bucket_scan_kernel<<<1, 32, 0, st>>>(s.ctrl, phase == PHASE_REST ? ctrl_ahead : nullptr);
  CSG_CUDA(cudaGetLastError());
  row_list_kernel<<<lgrid, 256, 0, st>>>(n, s.row_work, s.ctrl, s.row_list, chunk, phase == PHASE_REST);
  CSG_CUDA(cudaGetLastError());
  count_launches(7 + 3 * a.passes);
  return true;
}

}  // namespace csg
