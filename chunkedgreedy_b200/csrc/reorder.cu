// Apply a permutation to a CSR matrix: rows only, or rows and columns
// (P A P^T) with every output row re-sorted.
//
// Semantics of sporder/src/reorder.cu:72-149: new row p is old row
// new_order[p]; in symmetric mode column c becomes old2new[c] and the row is
// sorted by its new column ids, values moving with their columns; ptr_new is
// the inclusive scan of the gathered row lengths with ptr_new[0] = 0.
//
// The reference gathers into scratch and runs a device-wide segmented sort.  Here
// a row is gathered, remapped and sorted where it sits: rows of up to 32 entries
// (the bulk) in the registers of one warp, rows that fit shared memory by one
// thread block, longer rows by one thread block in place in global memory.  The
// sorting network has only ascending comparators, so a row needs no padding.
#include "common.cuh"

namespace csg {

namespace {

constexpr int R_THREADS = 256;
constexpr int R_SCAN_IPT = 8;
constexpr int R_SCAN_TILE = R_THREADS * R_SCAN_IPT;  // rows per scan block
constexpr int R_MED = 2048;                          // longest row sorted in shared memory

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
    int32_t *__restrict__ old2new) {
  __shared__ int32_t sm[R_THREADS / 32];
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
    }
    s += len[i];
  }
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

// All-ascending bitonic network over arr[0..L): comparators whose upper end is
// >= L touch only virtual +inf entries and are skipped.  Keys are distinct.
template <int NTHREADS>
__device__ void block_sort_asc(int32_t *keys, float *vals, int32_t L) {
  int32_t P = 1;
  while (P < L) P <<= 1;
  for (int32_t k = 2; k <= P; k <<= 1) {
    // flip step: i pairs with the mirror position inside its k-block
    for (int32_t t = threadIdx.x; t < (P >> 1); t += NTHREADS) {
      const int32_t half = k >> 1;
      const int32_t blk = t / half, off = t % half;
      const int32_t i = blk * k + off, l = blk * k + (k - 1 - off);
      if (l < L) {
        const int32_t a = keys[i], b = keys[l];
        if (b < a) {
          keys[i] = b;
          keys[l] = a;
          if (vals) {
            const float va = vals[i];
            vals[i] = vals[l];
            vals[l] = va;
          }
        }
      }
    }
    __syncthreads();
    for (int32_t j = k >> 2; j > 0; j >>= 1) {
      for (int32_t t = threadIdx.x; t < (P >> 1); t += NTHREADS) {
        const int32_t i = ((t / j) * (j << 1)) + (t % j), l = i + j;
        if (l < L) {
          const int32_t a = keys[i], b = keys[l];
          if (b < a) {
            keys[i] = b;
            keys[l] = a;
            if (vals) {
              const float va = vals[i];
              vals[i] = vals[l];
              vals[l] = va;
            }
          }
        }
      }
      __syncthreads();
    }
  }
}

// One warp per new row.  Rows of <= 32 entries are finished here; longer rows are
// gathered (and remapped) unsorted and queued for the block kernels.
__global__ void __launch_bounds__(R_THREADS) gather_rows_kernel(
    int32_t n, const int32_t *__restrict__ ptr_old, const int32_t *__restrict__ ind_old,
    const float *__restrict__ val_old, const int32_t *__restrict__ new_order,
    const int32_t *__restrict__ old2new, const int32_t *__restrict__ ptr_new,
    int32_t *__restrict__ ind_new, float *__restrict__ val_new, int32_t *__restrict__ queue,
    uint32_t *__restrict__ queue_count) {
  const int lane = threadIdx.x & 31;
  const int32_t warps = (gridDim.x * blockDim.x) >> 5;
  for (int32_t p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; p < n; p += warps) {
    const int32_t src_row = new_order[p];
    const int32_t src = ptr_old[src_row], len = ptr_old[src_row + 1] - src;
    const int32_t dst = ptr_new[p];
    if (old2new && len <= 32) {
      int32_t key = 0x7FFFFFFF;
      float v = 0.0f;
      if (lane < len) {
        key = old2new[ind_old[src + lane]];
        if (val_new) v = val_old[src + lane];
      }
      if (len > 1) {
#pragma unroll
        for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
          for (int j = k >> 1; j > 0; j >>= 1) {
            const int32_t ok = __shfl_xor_sync(FULL, key, j);
            const float ov = __shfl_xor_sync(FULL, v, j);
            const bool up = (lane & k) == 0;
            const bool lower = (lane & j) == 0;
            const bool take = (up == lower) ? (ok < key) : (ok > key);
            if (take) {
              key = ok;
              v = ov;
            }
          }
        }
      }
      if (lane < len) {
        ind_new[dst + lane] = key;
        if (val_new) val_new[dst + lane] = v;
      }
      continue;
    }
    for (int32_t i = lane; i < len; i += 32) {
      const int32_t c = ind_old[src + i];
      ind_new[dst + i] = old2new ? old2new[c] : c;
      if (val_new) val_new[dst + i] = val_old[src + i];
    }
    if (old2new && lane == 0) queue[atomicAdd(queue_count, 1u)] = p;
  }
}

__global__ void __launch_bounds__(R_THREADS) sort_long_rows_kernel(
    const int32_t *__restrict__ ptr_new, int32_t *ind_new, float *val_new,
    const int32_t *__restrict__ queue, const uint32_t *__restrict__ queue_count) {
  __shared__ int32_t skey[R_MED];
  __shared__ float sval[R_MED];
  const uint32_t count = *queue_count;
  for (uint32_t item = blockIdx.x; item < count; item += gridDim.x) {
    const int32_t p = queue[item];
    const int32_t b = ptr_new[p], L = ptr_new[p + 1] - b;
    __syncthreads();
    if (L <= R_MED) {
      for (int32_t i = threadIdx.x; i < L; i += R_THREADS) {
        skey[i] = ind_new[b + i];
        if (val_new) sval[i] = val_new[b + i];
      }
      __syncthreads();
      block_sort_asc<R_THREADS>(skey, val_new ? sval : nullptr, L);
      for (int32_t i = threadIdx.x; i < L; i += R_THREADS) {
        ind_new[b + i] = skey[i];
        if (val_new) val_new[b + i] = sval[i];
      }
    } else {
      block_sort_asc<R_THREADS>(ind_new + b, val_new ? val_new + b : nullptr, L);
    }
  }
}

}  // namespace

size_t reorder_workspace_bytes(int32_t n, int32_t nnz, int mode) {
  (void)nnz;
  Arena ar;
  const int32_t nb = (n + R_SCAN_TILE - 1) / R_SCAN_TILE;
  ar.take(sizeof(int32_t) * (static_cast<size_t>(nb) + 1));
  if (mode == 1) {
    ar.take(sizeof(int32_t) * static_cast<size_t>(n));  // old2new
    ar.take(sizeof(int32_t) * static_cast<size_t>(n));  // queue of rows longer than a warp
    ar.take(256);                                       // queue counter
  }
  return ar.off;
}

bool launch_reorder(Context &ctx, int32_t n, int32_t nnz, const int32_t *d_ptr_old,
                    const int32_t *d_ind_old, const float *d_val_old, const int32_t *d_new_order,
                    int mode, int32_t *d_ptr_new, int32_t *d_ind_new, float *d_val_new) {
  (void)nnz;
  const bool symmetric = mode == 1;
  const bool with_vals = d_val_old != nullptr && d_val_new != nullptr;
  if (!ensure_workspace(ctx, reorder_workspace_bytes(n, nnz, mode))) return false;
  Arena ar;
  const int32_t nb = (n + R_SCAN_TILE - 1) / R_SCAN_TILE;
  int32_t *block_sums = reinterpret_cast<int32_t *>(ctx.ws + ar.take(sizeof(int32_t) * (static_cast<size_t>(nb) + 1)));
  int32_t *old2new = nullptr, *queue = nullptr;
  uint32_t *queue_count = nullptr;
  if (symmetric) {
    old2new = reinterpret_cast<int32_t *>(ctx.ws + ar.take(sizeof(int32_t) * static_cast<size_t>(n)));
    queue = reinterpret_cast<int32_t *>(ctx.ws + ar.take(sizeof(int32_t) * static_cast<size_t>(n)));
    queue_count = reinterpret_cast<uint32_t *>(ctx.ws + ar.take(256));
    CSG_CUDA(cudaMemsetAsync(queue_count, 0, sizeof(uint32_t), ctx.stream));
  }
  len_block_sums_kernel<<<nb, R_THREADS, 0, ctx.stream>>>(n, d_ptr_old, d_new_order, block_sums);
  CSG_CUDA(cudaGetLastError());
  scan_block_sums_kernel<<<1, 1024, 0, ctx.stream>>>(nb, block_sums);
  CSG_CUDA(cudaGetLastError());
  ptr_new_kernel<<<nb, R_THREADS, 0, ctx.stream>>>(n, d_ptr_old, d_new_order, block_sums, d_ptr_new,
                                                   old2new);
  CSG_CUDA(cudaGetLastError());
  int64_t want = (static_cast<int64_t>(n) * 32 + R_THREADS - 1) / R_THREADS;
  int grid = static_cast<int>(want < ctx.num_sms * 16 ? want : ctx.num_sms * 16);
  if (grid < 1) grid = 1;
  gather_rows_kernel<<<grid, R_THREADS, 0, ctx.stream>>>(
      n, d_ptr_old, d_ind_old, with_vals ? d_val_old : nullptr, d_new_order, old2new, d_ptr_new,
      d_ind_new, with_vals ? d_val_new : nullptr, queue, queue_count);
  CSG_CUDA(cudaGetLastError());
  if (symmetric) {
    sort_long_rows_kernel<<<ctx.num_sms * 4, R_THREADS, 0, ctx.stream>>>(
        d_ptr_new, d_ind_new, with_vals ? d_val_new : nullptr, queue, queue_count);
    CSG_CUDA(cudaGetLastError());
  }
  count_launches(symmetric ? 5 : 4);
  return true;
}

}  // namespace csg
