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
// row piece and walks its nonzeros four at a time; every lane of the group loads its
// VEC columns of B[col] (one coalesced segment per group) and accumulates in
// registers.  A warp therefore handles 32/G rows at once, and each group fetches its
// next row from a ticket counter the moment it is done, so uneven row lengths do not
// idle lanes.  Rows longer than SPLIT are cut into pieces that all groups share and
// that are added with atomics (C is zeroed first for those rows), so a hub row never
// serialises on one warp.
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
  // scratch: [0] row ticket, [2..3] packed (long rows, pieces) counter, then the queue
  uint32_t *ctrl;
  int2 *long_rows;  // (row, first piece number), in piece order
};

constexpr int CTRL_TICKET = 0;
constexpr int CTRL_PACKED = 2;  // 64-bit: high word = long rows queued, low word = pieces so far
constexpr int CTRL_SCRATCH_WORDS = 64;

// FMA of up to four nonzeros [p, p + cnt) of one row into acc, loads issued together.
template <int G, int VEC>
__device__ __forceinline__ void fma4(const SpmmArgs &a, int32_t p, int cnt, int32_t col0,
                                     float (&acc)[VEC]) {
  int32_t c[4];
  float x[4];
  float b[4][VEC];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const bool on = u < cnt;
    c[u] = on ? __ldg(a.ind + p + u) : 0;
    x[u] = on ? __ldg(a.val + p + u) : 0.0f;
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    if (u < cnt) {
      load_b<VEC>(a.B + static_cast<size_t>(c[u]) * a.w + col0, b[u]);
    } else {
#pragma unroll
      for (int v = 0; v < VEC; ++v) b[u][v] = 0.0f;
    }
  }
#pragma unroll
  for (int u = 0; u < 4; ++u)
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = fmaf(x[u], b[u][v], acc[v]);
}

template <int VEC>
__device__ __forceinline__ void store_c(float *out, const float (&acc)[VEC], bool accumulate) {
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

// First launch.  Every lane group is persistent: it takes the next row from a ticket
// counter as soon as its current row is finished, so the groups of a warp never wait
// for the one with the longest row.  Rows longer than SPLIT are zeroed and queued for
// the second launch.  (w == G * VEC here; wider matrices take the panel kernel.)
template <int G, int VEC>
__global__ void __launch_bounds__(M_THREADS) spmm_rows_kernel(SpmmArgs a) {
  const int lane = threadIdx.x & 31;
  const int gl = lane % G;
  const unsigned gmask = (G == 32) ? FULL : (((1u << G) - 1u) << (lane - gl));
  const int32_t col0 = gl * VEC;
  int32_t row = -1, p = 0, pe = 0;
  bool done = false;
  float acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = 0.0f;
  for (;;) {
    if (p >= pe && !done) {
      if (row >= 0) store_c<VEC>(a.C + static_cast<size_t>(row) * a.w + col0, acc, false);
      int32_t r = 0;
      if (gl == 0) r = static_cast<int32_t>(atomicAdd(&a.ctrl[CTRL_TICKET], 1u));
      r = __shfl_sync(gmask, r, lane - gl);
      row = -1;
      if (r >= a.n) {
        done = true;
      } else {
        const int32_t b = a.ptr[r], e = a.ptr[r + 1];
        if (e - b > SPLIT) {
          for (int32_t j = gl * VEC; j < a.w; j += G * VEC)
#pragma unroll
            for (int v = 0; v < VEC; ++v) a.C[static_cast<size_t>(r) * a.w + j + v] = 0.0f;
          if (gl == 0) {
            const unsigned long long pieces = static_cast<unsigned long long>((e - b + SPLIT - 1) / SPLIT);
            const unsigned long long old = atomicAdd(
                reinterpret_cast<unsigned long long *>(a.ctrl + CTRL_PACKED), (1ull << 32) | pieces);
            a.long_rows[old >> 32] = make_int2(r, static_cast<int32_t>(old & 0xFFFFFFFFu));
          }
        } else {
          row = r;
          p = b;
          pe = e;
#pragma unroll
          for (int v = 0; v < VEC; ++v) acc[v] = 0.0f;
        }
      }
    }
    if (__all_sync(FULL, done)) break;
    const int cnt = pe - p < 4 ? pe - p : 4;
    if (cnt > 0) fma4<G, VEC>(a, p, cnt, col0, acc);
    p += cnt;
  }
}

// Matrices wider than one panel of G*VEC columns: one lane group per row and panel loop.
template <int G, int VEC>
__global__ void __launch_bounds__(M_THREADS) spmm_panel_kernel(SpmmArgs a) {
  constexpr int PER_WARP = 32 / G;
  const int lane = threadIdx.x & 31;
  const int sub = lane / G, gl = lane % G;
  const int32_t warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int32_t warps = (gridDim.x * blockDim.x) >> 5;
  const int panels = a.w / (G * VEC);
  for (int32_t base = warp_global * PER_WARP; base < a.n; base += warps * PER_WARP) {
    const int32_t row = base + sub;
    if (row >= a.n) continue;
    const int32_t pb = a.ptr[row], pe = a.ptr[row + 1];
    if (pe - pb > SPLIT) {
      for (int32_t j = gl; j < a.w; j += G) a.C[static_cast<size_t>(row) * a.w + j] = 0.0f;
      if (gl == 0) {
        const unsigned long long pieces = static_cast<unsigned long long>((pe - pb + SPLIT - 1) / SPLIT);
        const unsigned long long old = atomicAdd(
            reinterpret_cast<unsigned long long *>(a.ctrl + CTRL_PACKED), (1ull << 32) | pieces);
        a.long_rows[old >> 32] = make_int2(row, static_cast<int32_t>(old & 0xFFFFFFFFu));
      }
      continue;
    }
    for (int panel = 0; panel < panels; ++panel) {
      const int32_t col0 = panel * G * VEC + gl * VEC;
      float acc[VEC];
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[v] = 0.0f;
      for (int32_t p = pb; p < pe; p += 4) fma4<G, VEC>(a, p, pe - p < 4 ? pe - p : 4, col0, acc);
      store_c<VEC>(a.C + static_cast<size_t>(row) * a.w + col0, acc, false);
    }
  }
}

// Second launch: the pieces (SPLIT nonzeros each) of the queued long rows, spread over
// all lane groups; piece number -> queue entry by binary search on the entries' first
// piece numbers (ascending by construction).  Partial rows are added with atomics.
template <int G, int VEC>
__global__ void __launch_bounds__(M_THREADS) spmm_long_kernel(SpmmArgs a) {
  constexpr int PER_WARP = 32 / G;
  const int lane = threadIdx.x & 31;
  const int sub = lane / G, gl = lane % G;
  const int32_t group = ((blockIdx.x * blockDim.x + threadIdx.x) >> 5) * PER_WARP + sub;
  const int32_t groups = ((gridDim.x * blockDim.x) >> 5) * PER_WARP;
  const int32_t queued = static_cast<int32_t>(a.ctrl[CTRL_PACKED + 1]);
  const int32_t total = static_cast<int32_t>(a.ctrl[CTRL_PACKED]);
  const int panels = a.w / (G * VEC);
  for (int32_t id = group; id < total; id += groups) {
    int32_t lo = 0, hi = queued;  // long_rows[lo].y <= id < long_rows[hi].y
    while (hi - lo > 1) {
      const int32_t mid = (lo + hi) >> 1;
      if (a.long_rows[mid].y <= id)
        lo = mid;
      else
        hi = mid;
    }
    const int2 q = a.long_rows[lo];
    const int32_t b = a.ptr[q.x], e = a.ptr[q.x + 1];
    const int32_t pb = b + (id - q.y) * SPLIT;
    const int32_t pe = pb + SPLIT < e ? pb + SPLIT : e;
    for (int panel = 0; panel < panels; ++panel) {
      const int32_t col0 = panel * G * VEC + gl * VEC;
      float acc[VEC];
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[v] = 0.0f;
      for (int32_t p = pb; p < pe; p += 4) fma4<G, VEC>(a, p, pe - p < 4 ? pe - p : 4, col0, acc);
      store_c<VEC>(a.C + static_cast<size_t>(q.x) * a.w + col0, acc, true);
    }
  }
}

template <int G, int VEC>
bool launch_variant(Context &ctx, const SpmmArgs &a) {
  const int per_warp = 32 / G;
  if (a.w == G * VEC) {  // one panel: persistent groups, a few waves worth of them
    spmm_rows_kernel<G, VEC><<<ctx.num_sms * 8, M_THREADS, 0, ctx.stream>>>(a);
  } else {
    int64_t warps = (static_cast<int64_t>(a.n) + per_warp - 1) / per_warp;
    int64_t blocks = (warps * 32 + M_THREADS - 1) / M_THREADS;
    const int64_t cap = static_cast<int64_t>(ctx.num_sms) * 32;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    spmm_panel_kernel<G, VEC><<<static_cast<int>(blocks), M_THREADS, 0, ctx.stream>>>(a);
  }
  CSG_CUDA(cudaGetLastError());
  spmm_long_kernel<G, VEC><<<ctx.num_sms * 8, M_THREADS, 0, ctx.stream>>>(a);
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
  // scratch: counters and the queue of rows longer than SPLIT (at most nnz / SPLIT of them)
  Arena ar;
  const size_t o_ctrl = ar.take(sizeof(uint32_t) * CTRL_SCRATCH_WORDS);
  const size_t o_rows = ar.take(sizeof(int2) * (static_cast<size_t>(nnz) / SPLIT + 1));
  if (!ensure_workspace(ctx, ar.off)) return false;
  a.ctrl = reinterpret_cast<uint32_t *>(ctx.ws + o_ctrl);
  a.long_rows = reinterpret_cast<int2 *>(ctx.ws + o_rows);
  CSG_CUDA(cudaMemsetAsync(a.ctrl, 0, sizeof(uint32_t) * CTRL_SCRATCH_WORDS, ctx.stream));

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
// holds these 512 KiB until the process exits.
//
// The array is shared by every call in the process and keeps what the last call
// left in it; the call clears the counters that must start at zero.  Two calls
// whose kernels can overlap on the same GPU (different streams) would race on it.
namespace csg {
namespace {

constexpr int STATIC_MAX_LONG_ROWS = 65536;  // queue capacity (entries of 8 bytes)
constexpr int STATIC_QUEUE_OFFSET = CTRL_SCRATCH_WORDS;  // words; counters own the first 256 bytes
static __device__ __align__(256) uint32_t g_spmm_static_scratch[STATIC_QUEUE_OFFSET +
                                                                2 * STATIC_MAX_LONG_ROWS];

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
  a.ctrl = scratch;
  a.long_rows = reinterpret_cast<int2 *>(scratch + STATIC_QUEUE_OFFSET);
  // the counters keep the previous call's values: clear them (the queue is overwritten)
  CSG_CUDA(cudaMemsetAsync(a.ctrl, 0, sizeof(uint32_t) * CTRL_SCRATCH_WORDS, stream));
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
