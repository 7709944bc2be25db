// Apply a permutation to a CSR matrix: rows only, or rows and columns
// (P A P^T) with every output row re-sorted.
//
// Semantics of sporder/src/reorder.cu:72-149: new row p is old row
// new_order[p]; in symmetric mode column c becomes old2new[c] and the row is
// sorted by its new column ids, values moving with their columns; ptr_new is
// the inclusive scan of the gathered row lengths with ptr_new[0] = 0.
//
// The reference gathers into scratch and runs a device-wide segmented sort.  Here
// a row is gathered, remapped and sorted by as much hardware as it needs:
//   * rows of up to 32 entries (the bulk) in registers: a warp reads the descriptors of 32
//     consecutive new rows with coalesced loads, then sorts four rows of up to 8 entries,
//     two of up to 16 or one of up to 32 at a time in segments of the warp (bitonic
//     network over shuffles);
//   * rows of up to 256 entries by one warp each, two, four or eight entries per lane in
//     registers (strides of 32 and more are exchanges between a lane's own registers);
//   * rows of up to 4096 entries by one thread block: every warp sorts runs of 256 in
//     registers, the runs are merged in shared memory by rank (an entry's place in the
//     merged run is its own index plus the number of smaller entries in the partner run,
//     found by binary search - keys are distinct), the last merge writes the output;
//   * longer rows - on power-law inputs single rows hold 10^5 entries - as tiles of 4096
//     sorted the same way into a scratch copy by as many blocks as there are tiles, then one
//     pass that places every entry at the sum of its ranks in all tiles of its row.
// A permutation that keeps every row and column inside its block of 1024 (every csg order
// with the default chunk size does) needs less: the old row is sorted by column, so the new
// row is already sorted block by block and only the entries of one block have to be ordered
// among themselves.  ptr_new_kernel notices such a permutation, and rows of more than 32
// entries then go through apply_runs_kernel: slices of 2048 entries, remapped into shared
// memory with a halo, every entry placed at the start of its block's run plus the number of
// smaller entries in the run (rows of up to 256 entries: the same by one warp per row).
// No row is gathered by a single warp any more (that alone cost 6 ms on a row of 98 k
// entries), and no sort runs on global memory (the in-place network cost another 17 ms).
#include "common.cuh"

namespace csg {

namespace {

constexpr int R_THREADS = 256;
constexpr int R_SCAN_IPT = 8;
constexpr int R_SCAN_TILE = R_THREADS * R_SCAN_IPT;  // rows per scan block
constexpr int LOCAL_BITS = 10;                       // blocks of 1024 rows / columns: the default csg chunk
constexpr int R_WARP = 256;                          // longest row sorted by one warp in registers
constexpr int R_MED = 4096;                          // longest row (and tile of a longer row) sorted in shared memory

__device__ __forceinline__ int32_t block_exclusive_scan(int32_t v, int32_t *total, int32_t *sm) {
  // sm: R_THREADS/32 ints of shared memory
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t incl = v;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int32_t t = __shfl_up_sync(FULL, incl, off);
    if (lane >= off) incl += t;
  }
  __syncthreads();
  if (lane == 31) sm[warp] = incl;
  __syncthreads();
  int32_t base = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < R_THREADS / 32; ++w) {
    const int32_t t = sm[w];
    if (w < warp) base += t;
    tot += t;
  }
  *total = tot;
  return base + incl - v;
}

__global__ void __launch_bounds__(R_THREADS) len_block_sums_kernel(
    int32_t n, const int32_t *__restrict__ ptr_old, const int32_t *__restrict__ new_order,
    int32_t *__restrict__ block_sums) {
  __shared__ int32_t sm[R_THREADS / 32];
  const int32_t base = blockIdx.x * R_SCAN_TILE;
  int32_t s = 0;
#pragma unroll
  for (int i = 0; i < R_SCAN_IPT; ++i) {
    const int32_t p = base + i * R_THREADS + threadIdx.x;
    if (p < n) {
      const int32_t src = new_order[p];
      s += ptr_old[src + 1] - ptr_old[src];
    }
  }
  int32_t tot;
  block_exclusive_scan(s, &tot, sm);
  if (threadIdx.x == 0) block_sums[blockIdx.x] = tot;
}

__global__ void __launch_bounds__(1024) scan_block_sums_kernel(int32_t nb, int32_t *block_sums) {
  // exclusive scan in place, one block, any nb
  __shared__ int32_t sm[32];
  __shared__ int32_t carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int32_t base = 0; base < nb; base += 1024) {
    const int32_t i = base + threadIdx.x;
    const int32_t v = i < nb ? block_sums[i] : 0;
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
    if (i < nb) block_sums[i] = carry + wbase + incl - v;
    __syncthreads();
    if (threadIdx.x == 0) carry_s = carry + tot;
    __syncthreads();
  }
}

__global__ void __launch_bounds__(R_THREADS) ptr_new_kernel(
    int32_t n, const int32_t *__restrict__ ptr_old, const int32_t *__restrict__ new_order,
    const int32_t *__restrict__ block_sums, int32_t *__restrict__ ptr_new,
    int32_t *__restrict__ old2new, uint32_t *__restrict__ leaves_block) {
  __shared__ int32_t sm[R_THREADS / 32];
  __shared__ int moved;
  if (threadIdx.x == 0) moved = 0;
  __syncthreads();
  // thread t owns R_SCAN_IPT consecutive rows so that one block scan suffices
  const int32_t first = blockIdx.x * R_SCAN_TILE + threadIdx.x * R_SCAN_IPT;
  int32_t len[R_SCAN_IPT], s = 0;
#pragma unroll
  for (int i = 0; i < R_SCAN_IPT; ++i) {
    const int32_t p = first + i;
    len[i] = 0;
    if (p < n) {
      const int32_t src = new_order[p];
      len[i] = ptr_old[src + 1] - ptr_old[src];
      if (old2new) old2new[src] = p;
      if ((src >> LOCAL_BITS) != (p >> LOCAL_BITS)) moved = 1;  // leaves its block of 1024
    }
    s += len[i];
  }
  __syncthreads();
  if (threadIdx.x == 0 && moved) atomicExch(leaves_block, 1u);
  int32_t tot;
  int32_t run = block_sums[blockIdx.x] + block_exclusive_scan(s, &tot, sm);
  if (blockIdx.x == 0 && threadIdx.x == 0) ptr_new[0] = 0;
#pragma unroll
  for (int i = 0; i < R_SCAN_IPT; ++i) {
    const int32_t p = first + i;
    run += len[i];
    if (p < n) ptr_new[p + 1] = run;
  }
}

struct ApplyArgs {
  int32_t n;
  const int32_t *ptr_old, *ind_old;
  const float *val_old;      // nullptr: pattern only
  const int32_t *new_order;
  const int32_t *old2new;    // nullptr: rows only (no remap, no sort)
  const int32_t *ptr_new;
  int32_t *ind_new;
  float *val_new;
  int32_t *queue_warp, *queue_block;  // new rows of 33..R_WARP entries / of up to R_MED
  int2 *queue_long;                   // longer rows: (new row, number of its first tile)
  int2 *queue_runs;                   // block-local permutation, rows past R_WARP: (new row, slice)
  uint32_t *counters;                 // [0] warp rows, [1] block rows, [2..3] packed (long rows, tiles),
                                      // [4] set when the permutation leaves blocks of 1024,
                                      // [6] slices in queue_runs
  int32_t *tmp_key;                   // scratch copy of the long rows' sorted tiles, indexed like ind_new
  float *tmp_val;
};
constexpr int CNT_WARP = 0, CNT_BLOCK = 1, CNT_LONG = 2, CNT_MOVED = 4, CNT_RUNS = 6;
constexpr int RUN_SLICE = 2048;                      // entries of a row one block orders at a time
constexpr int RUN_HALO = (1 << LOCAL_BITS) - 1;      // a run holds at most 1024 entries

// Rows of up to W entries, 32 / W of them at a time: each row in a segment of W lanes.
// `mask` names the lanes whose row (src, len, dst) belongs to this size class.
template <int W>
__device__ __forceinline__ void apply_class(const ApplyArgs &a, unsigned mask, int32_t src, int32_t len,
                                            int32_t dst, int lane) {
  constexpr int PER_PASS = 32 / W;
  const int sub = lane / W, j = lane % W;
  while (mask) {
    const unsigned bit = __fns(mask, 0, sub + 1);  // the (sub+1)-th row of the class, if any
    const bool have = bit < 32u;
    const int from = have ? static_cast<int>(bit) : 0;
    const int32_t s = __shfl_sync(FULL, src, from);
    const int32_t l = __shfl_sync(FULL, len, from);
    const int32_t d = __shfl_sync(FULL, dst, from);
#pragma unroll
    for (int r = 0; r < PER_PASS; ++r) mask &= mask - 1u;  // (0 & anything stays 0)
    const bool mine = have && j < l;
    int32_t key = 0x7FFFFFFF;
    float v = 0.0f;
    if (mine) {
      const int32_t c = a.ind_old[s + j];
      key = a.old2new ? a.old2new[c] : c;
      if (a.val_new) v = a.val_old[s + j];
    }
    if (a.old2new) {
#pragma unroll
      for (int k = 2; k <= W; k <<= 1) {
#pragma unroll
        for (int x = k >> 1; x > 0; x >>= 1) {
          const int32_t ok = __shfl_xor_sync(FULL, key, x);
          const float ov = __shfl_xor_sync(FULL, v, x);
          const bool up = (j & k) == 0;
          const bool lower = (j & x) == 0;
          const bool take = (up == lower) ? (ok < key) : (ok > key);
          if (take) {
            key = ok;
            v = ov;
          }
        }
      }
    }
    if (mine) {
      a.ind_new[d + j] = key;
      if (a.val_new) a.val_new[d + j] = v;
    }
  }
}

// One warp per 32 consecutive new rows: descriptors with coalesced loads, rows of up to 32
// entries finished here, longer rows queued for the kernels behind.
__global__ void __launch_bounds__(R_THREADS) apply_short_kernel(ApplyArgs a) {
  const int lane = threadIdx.x & 31;
  const int32_t warps = (gridDim.x * blockDim.x) >> 5;
  const int32_t batches = (a.n + 31) / 32;
  for (int32_t batch = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; batch < batches; batch += warps) {
    const int32_t p = batch * 32 + lane;
    int32_t src = 0, len = 0, dst = 0;
    if (p < a.n) {
      const int32_t src_row = a.new_order[p];
      src = a.ptr_old[src_row];
      len = a.ptr_old[src_row + 1] - src;
      dst = a.ptr_new[p];
    }
    if (len > R_WARP && a.old2new && a.counters[CNT_MOVED] == 0u) {  // block-local permutation
      const uint32_t slices = static_cast<uint32_t>((len + RUN_SLICE - 1) / RUN_SLICE);
      const uint32_t first = atomicAdd(&a.counters[CNT_RUNS], slices);
      for (uint32_t t = 0; t < slices; ++t) a.queue_runs[first + t] = make_int2(p, static_cast<int32_t>(t));
    } else if (len > 32) {
      if (len <= R_WARP) {
        a.queue_warp[atomicAdd(&a.counters[CNT_WARP], 1u)] = p;
      } else if (len <= R_MED) {
        a.queue_block[atomicAdd(&a.counters[CNT_BLOCK], 1u)] = p;
      } else {
        const unsigned long long tiles = static_cast<unsigned long long>((len + R_MED - 1) / R_MED);
        const unsigned long long old = atomicAdd(
            reinterpret_cast<unsigned long long *>(a.counters + CNT_LONG), (1ull << 32) | tiles);
        a.queue_long[old >> 32] = make_int2(p, static_cast<int32_t>(old & 0xFFFFFFFFu));
      }
    }
    apply_class<8>(a, __ballot_sync(FULL, len > 0 && len <= 8), src, len, dst, lane);
    apply_class<16>(a, __ballot_sync(FULL, len > 8 && len <= 16), src, len, dst, lane);
    apply_class<32>(a, __ballot_sync(FULL, len > 16 && len <= 32), src, len, dst, lane);
  }
}

// Bitonic network over the 32 * EPL entries of a warp, ascending.  Entry e sits in register
// e / 32 of lane e % 32: partners at a distance below 32 are reached by shuffles, partners
// further away are the lane's own registers.  The stages are a loop, not unrolled code: fully
// unrolled, the three instances of the network were so much code that the warps of a block,
// each at another stage, spent most of their time waiting for instructions to be fetched.
template <int EPL, int DR>
__device__ __forceinline__ void local_exchange(int32_t (&key)[EPL], float (&val)[EPL], int k) {
#pragma unroll
  for (int r = 0; r < EPL; ++r) {
    if ((r & DR) == 0 && r + DR < EPL) {
      const bool up = ((r * 32) & k) == 0;  // k >= 64 here: the bit lies in r
      const bool swap = up ? (key[r + DR] < key[r]) : (key[r + DR] > key[r]);
      const int32_t k0 = key[r], k1 = key[r + DR];
      const float v0 = val[r], v1 = val[r + DR];
      key[r] = swap ? k1 : k0;
      key[r + DR] = swap ? k0 : k1;
      val[r] = swap ? v1 : v0;
      val[r + DR] = swap ? v0 : v1;
    }
  }
}

template <int EPL>
__device__ __forceinline__ void warp_sort(int32_t (&key)[EPL], float (&val)[EPL], int lane) {
#pragma unroll 1
  for (int k = 2; k <= 32 * EPL; k <<= 1) {
#pragma unroll 1
    for (int x = k >> 1; x > 0; x >>= 1) {
      if (x >= 32) {
        if (x == 128) local_exchange<EPL, 4>(key, val, k);
        if (x == 64) local_exchange<EPL, 2>(key, val, k);
        if (x == 32) local_exchange<EPL, 1>(key, val, k);
      } else {
        const bool lower = (lane & x) == 0;
#pragma unroll
        for (int r = 0; r < EPL; ++r) {
          const int e = r * 32 + lane;
          const int32_t ok = __shfl_xor_sync(FULL, key[r], x);
          const float ov = __shfl_xor_sync(FULL, val[r], x);
          const bool up = (e & k) == 0;
          const bool take = (up == lower) ? (ok < key[r]) : (ok > key[r]);
          key[r] = take ? ok : key[r];
          val[r] = take ? ov : val[r];
        }
      }
    }
  }
}

// One row of up to 32 * EPL entries, gathered, remapped, sorted and written by one warp.
template <int EPL>
__device__ __forceinline__ void warp_row(const ApplyArgs &a, int32_t src, int32_t L, int32_t dst, int lane) {
  int32_t key[EPL];
  float val[EPL];
#pragma unroll
  for (int r = 0; r < EPL; ++r) {
    const int32_t i = r * 32 + lane;
    key[r] = 0x7FFFFFFF;
    val[r] = 0.0f;
    if (i < L) {
      key[r] = a.old2new[a.ind_old[src + i]];
      if (a.val_new) val[r] = a.val_old[src + i];
    }
  }
  warp_sort<EPL>(key, val, lane);
#pragma unroll
  for (int r = 0; r < EPL; ++r) {
    const int32_t i = r * 32 + lane;
    if (i < L) {
      a.ind_new[dst + i] = key[r];
      if (a.val_new) a.val_new[dst + i] = val[r];
    }
  }
}

// One warp per queued row of 33..R_WARP entries.
// Block-local permutation, rows of more than R_WARP entries: one block per slice of RUN_SLICE
// entries.  The old row is sorted by column and the permutation keeps every column in its
// block of 1024, so the remapped row is a sequence of runs, one per block, in the right
// order; an entry's place is the start of its run plus the number of smaller entries in the
// run.  The slice is staged with a halo of 1023 entries on either side: no run is longer
// than 1024.
__global__ void __launch_bounds__(R_THREADS) apply_runs_kernel(ApplyArgs a) {
  __shared__ int32_t skey[RUN_SLICE + 2 * RUN_HALO];
  if (!a.old2new || a.counters[CNT_MOVED] != 0u) return;
  const int32_t total = static_cast<int32_t>(a.counters[CNT_RUNS]);
  for (int32_t id = blockIdx.x; id < total; id += gridDim.x) {
    const int2 q = a.queue_runs[id];  // (new row, slice)
    const int32_t src_row = a.new_order[q.x];
    const int32_t src = a.ptr_old[src_row], L = a.ptr_old[src_row + 1] - src;
    const int32_t dst = a.ptr_new[q.x];
    const int32_t s0 = q.y * RUN_SLICE;
    const int32_t s1 = s0 + RUN_SLICE < L ? s0 + RUN_SLICE : L;
    const int32_t w0 = s0 - RUN_HALO < 0 ? 0 : s0 - RUN_HALO;
    const int32_t w1 = s1 + RUN_HALO < L ? s1 + RUN_HALO : L;
    __syncthreads();
    for (int32_t j = w0 + threadIdx.x; j < w1; j += R_THREADS) skey[j - w0] = a.old2new[a.ind_old[src + j]];
    __syncthreads();
    for (int32_t i = s0 + threadIdx.x; i < s1; i += R_THREADS) {
      const int32_t x = skey[i - w0];
      const int32_t blk = x >> LOCAL_BITS;
      int32_t below = 0;
      int32_t j = i - 1;
      for (; j >= w0 && (skey[j - w0] >> LOCAL_BITS) == blk; --j) below += skey[j - w0] < x ? 1 : 0;
      const int32_t run_start = j + 1;
      for (j = i + 1; j < w1 && (skey[j - w0] >> LOCAL_BITS) == blk; ++j) below += skey[j - w0] < x ? 1 : 0;
      a.ind_new[dst + run_start + below] = x;
      if (a.val_new) a.val_new[dst + run_start + below] = a.val_old[src + i];
    }
  }
}

// The same for a row of up to R_WARP entries, by one warp: the whole row is staged.
__device__ __forceinline__ void warp_row_runs(const ApplyArgs &a, int32_t *skey, int32_t src, int32_t L,
                                              int32_t dst, int lane) {
  __syncwarp();
  for (int32_t j = lane; j < L; j += 32) skey[j] = a.old2new[a.ind_old[src + j]];
  __syncwarp();
  for (int32_t i = lane; i < L; i += 32) {
    const int32_t x = skey[i];
    const int32_t blk = x >> LOCAL_BITS;
    int32_t below = 0;
    int32_t j = i - 1;
    for (; j >= 0 && (skey[j] >> LOCAL_BITS) == blk; --j) below += skey[j] < x ? 1 : 0;
    const int32_t run_start = j + 1;
    for (j = i + 1; j < L && (skey[j] >> LOCAL_BITS) == blk; ++j) below += skey[j] < x ? 1 : 0;
    a.ind_new[dst + run_start + below] = x;
    if (a.val_new) a.val_new[dst + run_start + below] = a.val_old[src + i];
  }
}

__global__ void __launch_bounds__(R_THREADS) apply_warp_kernel(ApplyArgs a) {
  __shared__ int32_t staged[R_THREADS / 32][R_WARP];
  const int lane = threadIdx.x & 31;
  const bool local = a.old2new && a.counters[CNT_MOVED] == 0u;  // block-local permutation
  const uint32_t count = a.counters[CNT_WARP];
  const uint32_t warps = (gridDim.x * blockDim.x) >> 5;
  for (uint32_t item = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; item < count; item += warps) {
    const int32_t p = a.queue_warp[item];
    const int32_t src_row = a.new_order[p];
    const int32_t src = a.ptr_old[src_row], L = a.ptr_old[src_row + 1] - src;
    const int32_t dst = a.ptr_new[p];
    if (!a.old2new) {  // rows only: a copy
      for (int32_t i = lane; i < L; i += 32) {
        a.ind_new[dst + i] = a.ind_old[src + i];
        if (a.val_new) a.val_new[dst + i] = a.val_old[src + i];
      }
    } else if (local) {
      warp_row_runs(a, staged[threadIdx.x >> 5], src, L, dst, lane);
    } else if (L <= 64) {
      warp_row<2>(a, src, L, dst, lane);
    } else if (L <= 128) {
      warp_row<4>(a, src, L, dst, lane);
    } else {
      warp_row<8>(a, src, L, dst, lane);
    }
  }
}

// ---- up to R_MED entries by one block ---------------------------------------------------
// Shared memory: two copies of (keys, values).  Sorts the L <= R_MED entries that
// fetch(i) delivers (remapped key and value of entry i) and hands entry number q of the
// sorted order to put(q, key, value).  Runs of 256 are sorted in registers by the warps;
// merges by rank: an entry moves to its own index in its run plus the number of smaller
// entries in the partner run.
struct BlockSortShared {
  int32_t key[2][R_MED];
  float val[2][R_MED];
};

// number of entries of run[0..len) below x (keys are distinct)
__device__ __forceinline__ int32_t rank_in_run(const int32_t *run, int32_t len, int32_t x) {
  int32_t lo = 0, hi = len;
  while (lo < hi) {
    const int32_t mid = (lo + hi) >> 1;
    if (run[mid] < x)
      lo = mid + 1;
    else
      hi = mid;
  }
  return lo;
}

template <typename Fetch, typename Put>
__device__ void block_sort(BlockSortShared &sh, int32_t L, bool with_val, Fetch fetch, Put put) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int WARPS = R_THREADS / 32;
  __syncthreads();  // the buffers may still be read by the previous use
  for (int32_t base = warp * R_WARP; base < L; base += WARPS * R_WARP) {
    int32_t key[8];
    float val[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int32_t i = base + r * 32 + lane;
      key[r] = 0x7FFFFFFF;
      val[r] = 0.0f;
      if (i < L) fetch(i, key[r], val[r]);
    }
    warp_sort<8>(key, val, lane);
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int32_t i = base + r * 32 + lane;
      if (i < L) {  // the padding sorts behind every entry: the run's entries come first
        sh.key[0][i] = key[r];
        if (with_val) sh.val[0][i] = val[r];
      }
    }
  }
  __syncthreads();
  int cur = 0;
  for (int32_t run = R_WARP; run < L || run == R_WARP; run <<= 1) {
    const bool last = (run << 1) >= L;  // the merge that leaves one run: it delivers the result
    for (int32_t i = threadIdx.x; i < L; i += R_THREADS) {
      const int32_t q = i / run, o = i - q * run;
      const int32_t partner = (q ^ 1) * run;
      int32_t plen = L - partner;
      plen = plen < 0 ? 0 : (plen > run ? run : plen);
      const int32_t x = sh.key[cur][i];
      const int32_t at = (q >> 1) * (run << 1) + o + rank_in_run(sh.key[cur] + partner, plen, x);
      const float v = with_val ? sh.val[cur][i] : 0.0f;
      if (last) {
        put(at, x, v);
      } else {
        sh.key[cur ^ 1][at] = x;
        if (with_val) sh.val[cur ^ 1][at] = v;
      }
    }
    __syncthreads();
    if (last) break;
    cur ^= 1;
  }
}

// One block per queued row of R_WARP + 1 .. R_MED entries.
__global__ void __launch_bounds__(R_THREADS) apply_block_kernel(ApplyArgs a) {
  extern __shared__ __align__(16) unsigned char apply_smem[];
  BlockSortShared &sh = *reinterpret_cast<BlockSortShared *>(apply_smem);
  const uint32_t count = a.counters[CNT_BLOCK];
  for (uint32_t item = blockIdx.x; item < count; item += gridDim.x) {
    const int32_t p = a.queue_block[item];
    const int32_t src_row = a.new_order[p];
    const int32_t src = a.ptr_old[src_row], L = a.ptr_old[src_row + 1] - src;
    const int32_t dst = a.ptr_new[p];
    if (!a.old2new) {  // rows only: a copy
      for (int32_t i = threadIdx.x; i < L; i += R_THREADS) {
        a.ind_new[dst + i] = a.ind_old[src + i];
        if (a.val_new) a.val_new[dst + i] = a.val_old[src + i];
      }
      continue;
    }
    block_sort(
        sh, L, a.val_new != nullptr,
        [&](int32_t i, int32_t &k, float &v) {
          k = a.old2new[a.ind_old[src + i]];
          if (a.val_new) v = a.val_old[src + i];
        },
        [&](int32_t q, int32_t k, float v) {
          a.ind_new[dst + q] = k;
          if (a.val_new) a.val_new[dst + q] = v;
        });
  }
}

// ---- rows longer than R_MED ----------------------------------------------------------------
struct LongTile {
  int32_t src, L, dst, tile, tiles;
};
// tile number -> its row (binary search on the queue entries' first tile numbers, ascending
// by construction) and its place in the row
__device__ __forceinline__ LongTile long_tile(const ApplyArgs &a, int32_t id, int32_t queued) {
  int32_t lo = 0, hi = queued;  // queue_long[lo].y <= id < queue_long[hi].y
  while (hi - lo > 1) {
    const int32_t mid = (lo + hi) >> 1;
    if (a.queue_long[mid].y <= id)
      lo = mid;
    else
      hi = mid;
  }
  const int2 q = a.queue_long[lo];
  const int32_t src_row = a.new_order[q.x];
  LongTile t;
  t.src = a.ptr_old[src_row];
  t.L = a.ptr_old[src_row + 1] - t.src;
  t.dst = a.ptr_new[q.x];
  t.tile = id - q.y;
  t.tiles = (t.L + R_MED - 1) / R_MED;
  return t;
}

// One block per tile of R_MED entries of a long row: remapped and sorted into the scratch copy
// (rows only: copied straight to the output).
__global__ void __launch_bounds__(R_THREADS) apply_tiles_kernel(ApplyArgs a) {
  extern __shared__ __align__(16) unsigned char apply_smem[];
  BlockSortShared &sh = *reinterpret_cast<BlockSortShared *>(apply_smem);
  const int32_t queued = static_cast<int32_t>(a.counters[CNT_LONG + 1]);
  const int32_t total = static_cast<int32_t>(a.counters[CNT_LONG]);
  for (int32_t id = blockIdx.x; id < total; id += gridDim.x) {
    const LongTile t = long_tile(a, id, queued);
    const int32_t off = t.tile * R_MED;
    const int32_t len = t.L - off < R_MED ? t.L - off : R_MED;
    if (!a.old2new) {
      for (int32_t i = threadIdx.x; i < len; i += R_THREADS) {
        a.ind_new[t.dst + off + i] = a.ind_old[t.src + off + i];
        if (a.val_new) a.val_new[t.dst + off + i] = a.val_old[t.src + off + i];
      }
      continue;
    }
    block_sort(
        sh, len, a.val_new != nullptr,
        [&](int32_t i, int32_t &k, float &v) {
          k = a.old2new[a.ind_old[t.src + off + i]];
          if (a.val_new) v = a.val_old[t.src + off + i];
        },
        [&](int32_t q, int32_t k, float v) {
          a.tmp_key[t.dst + off + q] = k;
          if (a.val_new) a.tmp_val[t.dst + off + q] = v;
        });
  }
}

// One block per tile again: every entry goes to the sum of its ranks in all tiles of its row
// (its own index in its own tile).
__global__ void __launch_bounds__(R_THREADS) apply_merge_kernel(ApplyArgs a) {
  if (!a.old2new) return;
  const int32_t queued = static_cast<int32_t>(a.counters[CNT_LONG + 1]);
  const int32_t total = static_cast<int32_t>(a.counters[CNT_LONG]);
  for (int32_t id = blockIdx.x; id < total; id += gridDim.x) {
    const LongTile t = long_tile(a, id, queued);
    const int32_t off = t.tile * R_MED;
    const int32_t len = t.L - off < R_MED ? t.L - off : R_MED;
    const int32_t *row = a.tmp_key + t.dst;
    for (int32_t i = threadIdx.x; i < len; i += R_THREADS) {
      const int32_t x = row[off + i];
      int32_t at = i;
      for (int32_t other = 0; other < t.tiles; ++other) {
        if (other == t.tile) continue;
        const int32_t oo = other * R_MED;
        at += rank_in_run(row + oo, t.L - oo < R_MED ? t.L - oo : R_MED, x);
      }
      a.ind_new[t.dst + at] = x;
      if (a.val_new) a.val_new[t.dst + at] = a.tmp_val[t.dst + off + i];
    }
  }
}

}  // namespace

size_t reorder_workspace_bytes(int32_t n, int32_t nnz, int mode) {
  Arena ar;
  const int32_t nb = (n + R_SCAN_TILE - 1) / R_SCAN_TILE;
  ar.take(sizeof(int32_t) * (static_cast<size_t>(nb) + 1));
  ar.take(256);                                         // queue counters
  ar.take(sizeof(int32_t) * (static_cast<size_t>(nnz) / 32 + 1));      // rows of 33..R_WARP entries
  ar.take(sizeof(int32_t) * (static_cast<size_t>(nnz) / R_WARP + 1));  // rows of up to R_MED
  ar.take(sizeof(int2) * (static_cast<size_t>(nnz) / R_MED + 1));      // longer rows
  ar.take(sizeof(int2) * (static_cast<size_t>(nnz) / R_WARP + 1));     // slices of a block-local permutation
  if (mode == 1) {
    ar.take(sizeof(int32_t) * static_cast<size_t>(n));  // old2new
    ar.take(sizeof(int32_t) * static_cast<size_t>(nnz > 0 ? nnz : 1));  // sorted tiles: keys
    ar.take(sizeof(float) * static_cast<size_t>(nnz > 0 ? nnz : 1));    // ... and values
  }
  return ar.off;
}

bool launch_reorder(Context &ctx, int32_t n, int32_t nnz, const int32_t *d_ptr_old,
                    const int32_t *d_ind_old, const float *d_val_old, const int32_t *d_new_order,
                    int mode, int32_t *d_ptr_new, int32_t *d_ind_new, float *d_val_new) {
  const bool symmetric = mode == 1;
  const bool with_vals = d_val_old != nullptr && d_val_new != nullptr;
  if (!ensure_workspace(ctx, reorder_workspace_bytes(n, nnz, mode))) return false;
  Arena ar;
  const int32_t nb = (n + R_SCAN_TILE - 1) / R_SCAN_TILE;
  int32_t *block_sums = reinterpret_cast<int32_t *>(ctx.ws + ar.take(sizeof(int32_t) * (static_cast<size_t>(nb) + 1)));
  ApplyArgs a;
  a.n = n;
  a.ptr_old = d_ptr_old;
  a.ind_old = d_ind_old;
  a.val_old = with_vals ? d_val_old : nullptr;
  a.new_order = d_new_order;
  a.ptr_new = d_ptr_new;
  a.ind_new = d_ind_new;
  a.val_new = with_vals ? d_val_new : nullptr;
  a.counters = reinterpret_cast<uint32_t *>(ctx.ws + ar.take(256));
  a.queue_warp = reinterpret_cast<int32_t *>(ctx.ws + ar.take(sizeof(int32_t) * (static_cast<size_t>(nnz) / 32 + 1)));
  a.queue_block = reinterpret_cast<int32_t *>(ctx.ws + ar.take(sizeof(int32_t) * (static_cast<size_t>(nnz) / R_WARP + 1)));
  a.queue_long = reinterpret_cast<int2 *>(ctx.ws + ar.take(sizeof(int2) * (static_cast<size_t>(nnz) / R_MED + 1)));
  a.queue_runs = reinterpret_cast<int2 *>(ctx.ws + ar.take(sizeof(int2) * (static_cast<size_t>(nnz) / R_WARP + 1)));
  a.old2new = nullptr;
  a.tmp_key = nullptr;
  a.tmp_val = nullptr;
  int32_t *old2new = nullptr;
  if (symmetric) {
    old2new = reinterpret_cast<int32_t *>(ctx.ws + ar.take(sizeof(int32_t) * static_cast<size_t>(n)));
    a.old2new = old2new;
    a.tmp_key = reinterpret_cast<int32_t *>(ctx.ws + ar.take(sizeof(int32_t) * static_cast<size_t>(nnz > 0 ? nnz : 1)));
    a.tmp_val = reinterpret_cast<float *>(ctx.ws + ar.take(sizeof(float) * static_cast<size_t>(nnz > 0 ? nnz : 1)));
  }
  const int sort_smem = static_cast<int>(sizeof(BlockSortShared));
  CSG_CUDA(cudaFuncSetAttribute(apply_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sort_smem));
  CSG_CUDA(cudaFuncSetAttribute(apply_tiles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sort_smem));
  CSG_CUDA(cudaMemsetAsync(a.counters, 0, 8 * sizeof(uint32_t), ctx.stream));
  len_block_sums_kernel<<<nb, R_THREADS, 0, ctx.stream>>>(n, d_ptr_old, d_new_order, block_sums);
  CSG_CUDA(cudaGetLastError());
  scan_block_sums_kernel<<<1, 1024, 0, ctx.stream>>>(nb, block_sums);
  CSG_CUDA(cudaGetLastError());
  ptr_new_kernel<<<nb, R_THREADS, 0, ctx.stream>>>(n, d_ptr_old, d_new_order, block_sums, d_ptr_new,
                                                   old2new, a.counters + CNT_MOVED);
  CSG_CUDA(cudaGetLastError());
  int64_t want = ((static_cast<int64_t>(n) + 31) / 32 * 32 + R_THREADS - 1) / R_THREADS;
  int grid = static_cast<int>(want < ctx.num_sms * 8 ? want : ctx.num_sms * 8);
  if (grid < 1) grid = 1;
  apply_short_kernel<<<grid, R_THREADS, 0, ctx.stream>>>(a);
  CSG_CUDA(cudaGetLastError());
  apply_runs_kernel<<<ctx.num_sms * 8, R_THREADS, 0, ctx.stream>>>(a);
  CSG_CUDA(cudaGetLastError());
  apply_warp_kernel<<<ctx.num_sms * 6, R_THREADS, 0, ctx.stream>>>(a);
  CSG_CUDA(cudaGetLastError());
  apply_block_kernel<<<ctx.num_sms * 3, R_THREADS, sort_smem, ctx.stream>>>(a);
  CSG_CUDA(cudaGetLastError());
  apply_tiles_kernel<<<ctx.num_sms * 3, R_THREADS, sort_smem, ctx.stream>>>(a);
  CSG_CUDA(cudaGetLastError());
  apply_merge_kernel<<<ctx.num_sms * 4, R_THREADS, 0, ctx.stream>>>(a);
  CSG_CUDA(cudaGetLastError());
  count_launches(9);
  return true;
}

}  // namespace csg
