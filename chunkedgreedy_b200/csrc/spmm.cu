// fp32 CSR SpMM, C[n x w] = A[n x n] * B[n x w], B and C row-major.
//
// The reference has no first-party SpMM: it times third-party tensor-core kernels
// through bench/spmm/spmm_bench/base.py:48-59 and cuSPARSE through
// sporder/src/bench_cusparse_spmm.cu:64-90.  This kernel is the fp32 CUDA-core
// SpMM the reordered matrix is fed to: the work is the gather of one B row per
// nonzero (4*w bytes), so the kernel is a bandwidth kernel and its job is to keep
// many row gathers in flight.
//
// Row tiling: a group of G = w/VEC lanes (VEC = 4 floats where w allows) owns one
// row piece and walks its nonzeros; every lane of the group loads its VEC columns
// of B[col] (one coalesced segment per group) and accumulates in registers.  A
// warp therefore handles 32/G row pieces at once.  Rows longer than SPLIT are cut
// into pieces that are added with atomics (C is zeroed first for those rows), so a
// hub row never serialises on one warp.
#include <mutex>

#include "../../include/sporder_b200.h"
#include "common.cuh"

namespace csg {

namespace {

constexpr int M_THREADS = 256;
constexpr int SPLIT = 1024;  // longest row piece one lane group walks

template <int VEC>
__device__ __forceinline__ void load_b(const float *p, float (&out)[VEC]) {
  if (VEC == 4) {
    const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
    out[0] = t.x;
    out[1] = t.y;
    out[2] = t.z;
    out[3] = t.w;
  } else if (VEC == 2) {
    const float2 t = __ldg(reinterpret_cast<const float2 *>(p));
    out[0] = t.x;
    out[1] = t.y;
  } else {
    out[0] = __ldg(p);
  }
}

struct SpmmArgs {
  int32_t n, w;
  const int32_t *ptr, *ind;
  const float *val;
  const float *B;
  float *C;
  int32_t *long_rows;     // rows longer than SPLIT, appended by the first launch
  uint32_t *long_count;
};

// One row piece [pb, pe) of `row` for the lane group: G lanes, VEC columns each,
// one column panel of G*VEC at a time when w is wider.
template <int G, int VEC>
__device__ __forceinline__ void row_piece(const SpmmArgs &a, int32_t row, int32_t pb, int32_t pe,
                                          int gl, bool accumulate) {
  const int panels = a.w / (G * VEC);
  for (int panel = 0; panel < panels; ++panel) {
    const int32_t col0 = panel * G * VEC + gl * VEC;
    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = 0.0f;
    int32_t p = pb;
    // four gathers in flight per lane
    for (; p + 4 <= pe; p += 4) {
      int32_t c[4];
      float x[4];
      float b[4][VEC];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        c[u] = __ldg(a.ind + p + u);
        x[u] = __ldg(a.val + p + u);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) load_b<VEC>(a.B + static_cast<size_t>(c[u]) * a.w + col0, b[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] = fmaf(x[u], b[u][v], acc[v]);
    }
    for (; p < pe; ++p) {
      const int32_t c = __ldg(a.ind + p);
      const float x = __ldg(a.val + p);
      float b[VEC];
      load_b<VEC>(a.B + static_cast<size_t>(c) * a.w + col0, b);
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[v] = fmaf(x, b[v], acc[v]);
    }
    float *out = a.C + static_cast<size_t>(row) * a.w + col0;
    if (accumulate) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) atomicAdd(out + v, acc[v]);
    } else if (VEC == 4) {
      *reinterpret_cast<float4 *>(out) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    } else if (VEC == 2) {
      *reinterpret_cast<float2 *>(out) = make_float2(acc[0], acc[1]);
    } else {
      out[0] = acc[0];
    }
  }
}

// First launch: one lane group per row.  Rows longer than SPLIT are zeroed and
// queued instead of computed.
template <int G, int VEC>
__global__ void __launch_bounds__(M_THREADS) spmm_rows_kernel(SpmmArgs a) {
  constexpr int PER_WARP = 32 / G;
  const int lane = threadIdx.x & 31;
  const int sub = lane / G, gl = lane % G;
  const int32_t warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int32_t warps = (gridDim.x * blockDim.x) >> 5;
  for (int32_t base = warp_global * PER_WARP; base < a.n; base += warps * PER_WARP) {
    const int32_t row = base + sub;
    if (row >= a.n) continue;
    const int32_t pb = a.ptr[row], pe = a.ptr[row + 1];
    if (pe - pb > SPLIT) {
      for (int32_t j = gl; j < a.w; j += G) a.C[static_cast<size_t>(row) * a.w + j] = 0.0f;
      if (gl == 0) a.long_rows[atomicAdd(a.long_count, 1u)] = row;
      continue;
    }
    row_piece<G, VEC>(a, row, pb, pe, gl, false);
  }
}

// Second launch: the queued long rows, SPLIT nonzeros per lane group, added with
// atomics.  Every group walks the (short) queue and takes the pieces that fall to it.
template <int G, int VEC>
__global__ void __launch_bounds__(M_THREADS) spmm_long_kernel(SpmmArgs a) {
  constexpr int PER_WARP = 32 / G;
  const int lane = threadIdx.x & 31;
  const int sub = lane / G, gl = lane % G;
  const int32_t group = ((blockIdx.x * blockDim.x + threadIdx.x) >> 5) * PER_WARP + sub;
  const int32_t groups = ((gridDim.x * blockDim.x) >> 5) * PER_WARP;
  const uint32_t count = *a.long_count;
  int32_t turn = 0;  // running piece number over the whole queue
  for (uint32_t li = 0; li < count; ++li) {
    const int32_t row = a.long_rows[li];
    const int32_t b = a.ptr[row], e = a.ptr[row + 1];
    const int32_t pieces = (e - b + SPLIT - 1) / SPLIT;
    // first piece of this row that falls to this group
    int32_t first = (group - turn) % groups;
    if (first < 0) first += groups;
    for (int32_t pc = first; pc < pieces; pc += groups) {
      const int32_t pb = b + pc * SPLIT;
      const int32_t pe = (pb + SPLIT < e) ? pb + SPLIT : e;
      row_piece<G, VEC>(a, row, pb, pe, gl, true);
    }
    turn = (turn + pieces) % groups;
  }
}

template <int G, int VEC>
bool launch_variant(Context &ctx, const SpmmArgs &a) {
  const int per_warp = 32 / G;
  int64_t warps = (static_cast<int64_t>(a.n) + per_warp - 1) / per_warp;
  int64_t blocks = (warps * 32 + M_THREADS - 1) / M_THREADS;
  const int64_t cap = static_cast<int64_t>(ctx.num_sms) * 32;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  spmm_rows_kernel<G, VEC><<<static_cast<int>(blocks), M_THREADS, 0, ctx.stream>>>(a);
  CSG_CUDA(cudaGetLastError());
  spmm_long_kernel<G, VEC><<<ctx.num_sms * 4, M_THREADS, 0, ctx.stream>>>(a);
  CSG_CUDA(cudaGetLastError());
  count_launches(2);
  return true;
}

}  // namespace

bool launch_spmm(Context &ctx, int32_t n, int32_t nnz, int32_t w, const int32_t *d_ptr,
                 const int32_t *d_ind, const float *d_val, const float *d_B, float *d_C) {
  CSG_REQUIRE(w >= 1, "spmm: dense width must be >= 1");
  SpmmArgs a;
  a.n = n;
  a.w = w;
  a.ptr = d_ptr;
  a.ind = d_ind;
  a.val = d_val;
  a.B = d_B;
  a.C = d_C;
  // queue of rows longer than SPLIT (at most nnz / SPLIT of them)
  Arena ar;
  const size_t o_cnt = ar.take(256);
  const size_t o_rows = ar.take(sizeof(int32_t) * (static_cast<size_t>(nnz) / SPLIT + 1));
  if (!ensure_workspace(ctx, ar.off)) return false;
  a.long_count = reinterpret_cast<uint32_t *>(ctx.ws + o_cnt);
  a.long_rows = reinterpret_cast<int32_t *>(ctx.ws + o_rows);
  CSG_CUDA(cudaMemsetAsync(a.long_count, 0, sizeof(uint32_t), ctx.stream));

  const bool al16 = (reinterpret_cast<uintptr_t>(d_B) % 16 == 0) && (reinterpret_cast<uintptr_t>(d_C) % 16 == 0);
  if (w % 128 == 0 && al16) return launch_variant<32, 4>(ctx, a);
  if (w % 64 == 0 && al16) return launch_variant<16, 4>(ctx, a);
  if (w % 32 == 0 && al16) return launch_variant<8, 4>(ctx, a);
  if (w % 16 == 0 && al16) return launch_variant<4, 4>(ctx, a);
  if (w % 32 == 0) return launch_variant<32, 1>(ctx, a);
  if (w % 8 == 0) return launch_variant<8, 1>(ctx, a);
  if (w % 4 == 0) return launch_variant<4, 1>(ctx, a);
  if (w % 2 == 0) return launch_variant<2, 1>(ctx, a);
  return launch_variant<1, 1>(ctx, a);
}

}  // namespace csg

// ---------------------------------------------------------------------------------
// SpMM without any allocation.
//
// Some hosts of this library must not see a cudaMalloc from it: applications that
// have handed all device memory to an allocator of their own (a tensor framework's
// caching pool run with a fixed memory share, a database buffer pool), where a
// driver allocation inside a library call can fail outright or push the process
// over its budget; and request paths that ban driver allocations because
// cudaMalloc / cudaFree stall every stream of the device.  For them the queue of
// long rows -- the only scratch the SpMM kernels need -- lives in a fixed array
// that is part of the loaded library image, so every GPU that loads the library
// holds these 256 KiB until the process exits.
//
// The array is shared by every call in the process and keeps what the last call
// left in it; the call clears the one counter that must start at zero.  Two calls
// whose kernels can overlap on the same GPU (different streams) would race on it.
namespace csg {
namespace {

constexpr int STATIC_MAX_LONG_ROWS = 65536;  // queue capacity
constexpr int STATIC_QUEUE_OFFSET = 64;      // words; the counter owns the first 256 bytes
static __device__ __align__(256) uint32_t g_spmm_static_scratch[STATIC_QUEUE_OFFSET +
                                                                STATIC_MAX_LONG_ROWS];

// In host code the symbol above is only a stand-in, not a device address: the real
// address is asked for once per device, with that device current.
constexpr int MAX_DEVICES = 64;
std::mutex g_static_mutex;
uint32_t *g_static_addr[MAX_DEVICES] = {};

bool static_scratch_address(int device, uint32_t **out) {
  std::lock_guard<std::mutex> lock(g_static_mutex);
  CSG_REQUIRE(device >= 0 && device < MAX_DEVICES, "spmm_static: device %d out of range", device);
  if (!g_static_addr[device]) {
    void *p = nullptr;
    CSG_CUDA(cudaGetSymbolAddress(&p, g_spmm_static_scratch));
    g_static_addr[device] = static_cast<uint32_t *>(p);
  }
  *out = g_static_addr[device];
  return true;
}

bool run_spmm_static(int32_t n, int32_t nnz, int32_t w, const int32_t *d_ptr, const int32_t *d_ind,
                     const float *d_val, const float *d_B, float *d_C, cudaStream_t stream) {
  CSG_REQUIRE(n >= 1 && nnz >= 0 && w >= 1, "spmm_static: bad sizes n=%d nnz=%d w=%d", n, nnz, w);
  CSG_REQUIRE(d_ptr && d_B && d_C && (nnz == 0 || (d_ind && d_val)), "spmm_static: null array");
  // at most nnz / SPLIT rows can be longer than SPLIT; all of them must fit the queue
  CSG_REQUIRE(static_cast<int64_t>(nnz) / SPLIT + 1 <= STATIC_MAX_LONG_ROWS,
              "spmm_static: nnz = %d exceeds the fixed scratch (at most %lld nonzeros); use sporder_spmm",
              nnz, static_cast<long long>(STATIC_MAX_LONG_ROWS - 1) * SPLIT + SPLIT - 1);
  Context tmp;  // stack object only: stream and SM count for the launch geometry
  CSG_CUDA(cudaGetDevice(&tmp.device));
  CSG_CUDA(cudaDeviceGetAttribute(&tmp.num_sms, cudaDevAttrMultiProcessorCount, tmp.device));
  tmp.stream = stream;
  uint32_t *scratch = nullptr;
  if (!static_scratch_address(tmp.device, &scratch)) return false;
  SpmmArgs a;
  a.n = n;
  a.w = w;
  a.ptr = d_ptr;
  a.ind = d_ind;
  a.val = d_val;
  a.B = d_B;
  a.C = d_C;
  a.long_count = scratch;
  a.long_rows = reinterpret_cast<int32_t *>(scratch + STATIC_QUEUE_OFFSET);
  CSG_CUDA(cudaMemsetAsync(a.long_count, 0, sizeof(uint32_t), stream));  // last call's count
  const bool al16 = (reinterpret_cast<uintptr_t>(d_B) % 16 == 0) &&
                    (reinterpret_cast<uintptr_t>(d_C) % 16 == 0);
  if (w % 128 == 0 && al16) return launch_variant<32, 4>(tmp, a);
  if (w % 64 == 0 && al16) return launch_variant<16, 4>(tmp, a);
  if (w % 32 == 0 && al16) return launch_variant<8, 4>(tmp, a);
  if (w % 16 == 0 && al16) return launch_variant<4, 4>(tmp, a);
  if (w % 32 == 0) return launch_variant<32, 1>(tmp, a);
  if (w % 8 == 0) return launch_variant<8, 1>(tmp, a);
  if (w % 4 == 0) return launch_variant<4, 1>(tmp, a);
  if (w % 2 == 0) return launch_variant<2, 1>(tmp, a);
  return launch_variant<1, 1>(tmp, a);
}

}  // namespace
}  // namespace csg

extern "C" int32_t sporder_spmm_static(int32_t n, int32_t nnz, int32_t w, const int32_t *d_ptr,
                                       const int32_t *d_ind, const float *d_val, const float *d_B,
                                       float *d_C, void *stream) {
  csg::clear_error();
  return csg::run_spmm_static(n, nnz, w, d_ptr, d_ind, d_val, d_B, d_C,
                              static_cast<cudaStream_t>(stream))
             ? 0
             : -1;
}
