// Pillar count: the number of distinct (row window, column) pairs of a CSR pattern,
// window = row / height - the reordering quality metric of the reference
// (sporder/src/count_pillars.cu:38-85, which builds a 64-bit key per nonzero, radix-sorts
// all of them and counts the key changes).
//
// Here no global sort is made.  For short windows: the rows of a window are consecutive, so
// a nonzero (r, c) is the first of its pillar exactly when c occurs in none of the rows
// between the window's first row and r; with sorted rows that is at most height-1 short
// binary searches per nonzero, over data the neighbouring lanes have just touched.  One
// warp per row, lanes over its nonzeros.  Taller windows go through the chunk-local
// transpose of the csg path with the window as the chunk: the pillars are its column
// groups (the driver in api.cu picks the path).
#include "common.cuh"

namespace csg {

namespace {

constexpr unsigned FULL = 0xFFFFFFFFu;

__global__ void __launch_bounds__(256) pillars_search_kernel(int32_t n, int32_t nnz, int32_t height,
                                                             const int32_t *__restrict__ ptr,
                                                             const int32_t *__restrict__ ind,
                                                             unsigned long long *count, uint32_t *bad) {
  const int lane = threadIdx.x & 31;
  const int32_t warps = (gridDim.x * blockDim.x) >> 5;
  unsigned long long mine = 0;
  for (int32_t r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < n; r += warps) {
    const int32_t rb = ptr[r], re = ptr[r + 1];
    if (rb < 0 || re < rb || re > nnz) {  // malformed row pointers: flag and skip
      if (lane == 0) atomicExch(bad, 1u);
      continue;
    }
    const int32_t first = (r / height) * height;
    for (int32_t p = rb + lane; p < re; p += 32) {
      const int32_t c = ind[p];
      bool seen = p > rb && ind[p - 1] == c;  // a column repeated inside the row counts once
      for (int32_t q = first; q < r && !seen; ++q) {
        int32_t lo = ptr[q], hi = ptr[q + 1];  // first position of row q with a column >= c
        if (lo < 0 || hi < lo || hi > nnz) break;  // flagged by the warp that owns row q
        const int32_t end = hi;
        while (lo < hi) {
          const int32_t mid = lo + ((hi - lo) >> 1);
          if (ind[mid] < c)
            lo = mid + 1;
          else
            hi = mid;
        }
        seen = lo < end && ind[lo] == c;
      }
      mine += seen ? 0u : 1u;
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mine += __shfl_down_sync(FULL, mine, off);
  if (lane == 0 && mine) atomicAdd(count, mine);
}

// column groups of the chunk-local transpose = nonzeros that come first in their group
__global__ void __launch_bounds__(256) pillars_groups_kernel(int32_t nnz, const int32_t *__restrict__ seg_rank,
                                                             unsigned long long *count) {
  const int lane = threadIdx.x & 31;
  unsigned long long mine = 0;
  for (int32_t p = blockIdx.x * blockDim.x + threadIdx.x; p < nnz; p += gridDim.x * blockDim.x)
    mine += seg_rank[p] == 0 ? 1u : 0u;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mine += __shfl_down_sync(FULL, mine, off);
  if (lane == 0 && mine) atomicAdd(count, mine);
}

}  // namespace

bool launch_pillars_search(Context &ctx, int32_t n, int32_t nnz, int32_t height, const int32_t *d_ptr,
                           const int32_t *d_ind, unsigned long long *d_count, uint32_t *d_bad) {
  int grid = (n + 7) / 8;
  if (grid > ctx.num_sms * 16) grid = ctx.num_sms * 16;
  pillars_search_kernel<<<grid, 256, 0, ctx.stream>>>(n, nnz, height, d_ptr, d_ind, d_count, d_bad);
  CSG_CUDA(cudaGetLastError());
  count_launches(1);
  return true;
}

bool launch_pillars_groups(Context &ctx, int32_t nnz, const int32_t *seg_rank, unsigned long long *d_count) {
  int grid = (nnz + 255) / 256;
  if (grid > ctx.num_sms * 16) grid = ctx.num_sms * 16;
  pillars_groups_kernel<<<grid, 256, 0, ctx.stream>>>(nnz, seg_rank, d_count);
  CSG_CUDA(cudaGetLastError());
  count_launches(1);
  return true;
}

}  // namespace csg
