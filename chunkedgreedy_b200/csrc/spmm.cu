// fp32 CSR SpMM, C[n x w] = A[n x n] * B[n x w], B and C row-major.
//
// The reference has no first-party SpMM: it times third-party tensor-core kernels
// through bench/spmm/spmm_bench/base.py:48-59 and cuSPARSE through
// sporder/src/bench_cusparse_spmm.cu:64-90.  This kernel is the fp32 CUDA-core
// SpMM the reordered matrix is fed to: the work is the gather of one B row per
// nonzero (4*w bytes), so the kernel is a bandwidth kernel and its job is to keep
// many row gathers in flight.
//
// Row tiling: a group of G lanes owns one row and walks its nonzeros up to eight at a
// time; every lane of the group loads its VEC columns of B[col] (one coalesced segment per
// group), for PAN panels of G*VEC columns at once, and accumulates in registers.  A warp
// therefore handles 32/G rows at once.  Rows are handed out in two levels.  The rows are cut
// into units of equal cost, where a row costs ROW_COST plus its nonzeros: unit u holds the
// rows r with ROW_COST * r + ptr[r] in [u * T, (u + 1) * T), found by searching the row
// pointers, so a stretch of hub rows and a stretch of empty rows make equally many units.  A
// warp draws a unit from one global counter (one atomic per unit), stages the unit's row
// pointers in shared memory with one coalesced read, and its groups take the rows of the
// unit one by one as they finish, so uneven row lengths idle no lanes and no counter is
// hammered once per row.  (Batches of a fixed number of rows left the SMs idle 60 % of the
// kernel on a power-law matrix: one warp drew 128 hub rows.)  Rows longer than SPLIT are cut
// into pieces that all groups share and that are added with atomics (C is zeroed first for
// those rows), so a hub row never serialises on one warp.  The matrix is read once and marked as streaming data (evict
// first), so that it does not push rows of B out of the L2 cache.
#include <mutex>

#include "../../include/sporder_b200.h"
#include "common.cuh"

namespace csg {

namespace {

constexpr int M_THREADS = 256;
constexpr int M_WARPS = M_THREADS / 32;
constexpr int M_BLOCKS_PER_SM = 3;
constexpr int SPLIT = 1024;      // longest row one lane group walks alone
constexpr int LONG_PIECE = 256;  // nonzeros per piece of a longer row
constexpr int ROW_COST = 4;      // cost of a row beside its nonzeros, in nonzeros
constexpr int UNIT_MAX = 2048;   // largest unit cost; a unit holds at most UNIT_MAX / ROW_COST rows
constexpr int BATCH_MAX = UNIT_MAX / ROW_COST;

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

// base + c * wbytes as one 32 x 32 -> 64 bit multiply-add (written as a 64-bit product of
// converted operands the compiler builds it from four multiplies and two shifts, which on
// short rows was a third of all instructions executed)
__device__ __forceinline__ const float *b_row(const char *base, int32_t c, int32_t wbytes) {
  long long out;
  asm("mad.wide.s32 %0, %1, %2, %3;" : "=l"(out) : "r"(c), "r"(wbytes), "l"(reinterpret_cast<long long>(base)));
  return reinterpret_cast<const float *>(out);
}

struct SpmmArgs {
  int32_t n, w, nnz, unit;  // unit: cost per unit of rows (T)
  const int32_t *ptr, *ind;
  const float *val;
  const float *B;
  float *C;
  // scratch: [0] row ticket, [2..3] packed (long rows, pieces) counter, then the queue
  uint32_t *ctrl;
  int2 *long_rows;  // (row, first piece number), in piece order
};

// First row r in [0, n] with ROW_COST * r + ptr[r] >= target, n + 1 when there is none.  Two
// searches at once: lanes 0-15 look for target_lo, lanes 16-31 for target_hi, sixteen probes
// per step, so a search costs log16(n) dependent loads instead of log2(n).
__device__ __forceinline__ void unit_bounds(const SpmmArgs &a, long long target_lo, long long target_hi,
                                            int32_t *first, int32_t *last) {
  const int lane = threadIdx.x & 31, i = lane & 15;
  const long long target = lane < 16 ? target_lo : target_hi;
  long long lo = 0, hi = static_cast<long long>(a.n) + 1;  // the answer lies in [lo, hi]
  while (__any_sync(FULL, lo < hi)) {
    const long long len = hi - lo;
    const long long step = (len + 15) / 16;
    long long idx = lo + (i + 1) * step - 1;
    if (idx > hi - 1) idx = hi - 1;
    bool pred = false;
    if (lo < hi) pred = ROW_COST * idx + __ldg(a.ptr + idx) >= target;
    const unsigned votes = (__ballot_sync(FULL, pred) >> (lane & 16)) & 0xFFFFu;
    if (lo < hi) {
      if (votes) {
        const int f = __ffs(votes) - 1;
        long long top = lo + (f + 1) * step - 1;
        if (top > hi - 1) top = hi - 1;
        lo = lo + f * step;
        hi = top;
      } else {
        lo = hi;
      }
    }
  }
  *first = static_cast<int32_t>(__shfl_sync(FULL, lo, 0));
  *last = static_cast<int32_t>(__shfl_sync(FULL, lo, 16));
}

constexpr int CTRL_TICKET = 0;
constexpr int CTRL_PACKED = 2;  // 64-bit: high word = long rows queued, low word = pieces so far
constexpr int CTRL_SCRATCH_WORDS = 64;

// gathers in flight per group and step: eight rows of B, four where a lane already
// fetches two panels of each
template <int PAN>
struct Step {
  static constexpr int U = PAN >= 2 ? 4 : 8;
};

// FMA of up to U nonzeros [p, p + cnt) of one row into acc, for the panels
// pn0 .. pn0 + PAN - 1, all loads of a kind issued together.
template <int G, int VEC, int PAN, int U = Step<PAN>::U>
__device__ __forceinline__ void fma_step(const SpmmArgs &a, int32_t p, int cnt, int32_t col0,
                                         float (&acc)[PAN][VEC]) {
  int32_t c[U];
  float x[U];
  float b[U][PAN][VEC];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const bool on = u < cnt;
    c[u] = on ? __ldcs(a.ind + p + u) : 0;
    x[u] = on ? __ldcs(a.val + p + u) : 0.0f;
  }
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (u < cnt) {
      const float *src = b_row(reinterpret_cast<const char *>(a.B + col0), c[u], a.w * 4);
#pragma unroll
      for (int pn = 0; pn < PAN; ++pn) load_b<VEC>(src + pn * G * VEC, b[u][pn]);
    } else {
#pragma unroll
      for (int pn = 0; pn < PAN; ++pn)
#pragma unroll
        for (int v = 0; v < VEC; ++v) b[u][pn][v] = 0.0f;
    }
  }
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int pn = 0; pn < PAN; ++pn)
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[pn][v] = fmaf(x[u], b[u][pn][v], acc[pn][v]);
}

template <int VEC>
__device__ __forceinline__ void store_c(float *out, const float (&acc)[VEC], bool accumulate) {
  if (accumulate) {
#pragma unroll
    for (int v = 0; v < VEC; ++v) atomicAdd(out + v, acc[v]);
  } else if (VEC == 4) {
    __stcs(reinterpret_cast<float4 *>(out), make_float4(acc[0], acc[1], acc[2], acc[3]));
  } else if (VEC == 2) {
    __stcs(reinterpret_cast<float2 *>(out), make_float2(acc[0], acc[1]));
  } else {
    __stcs(out, acc[0]);
  }
}

// ---- units of short rows ---------------------------------------------------------------
// A unit whose rows all have at most SHORT_MAX nonzeros (every unit of a mesh or a road
// network) needs none of the machinery of spmm_rows_kernel's walk: the warp copies the
// (column, value) pairs of as many rows as fit S_PAIRS into shared memory with coalesced
// loads, its lane groups take those rows in turn, and a row is worked off in pieces of exactly
// as many nonzeros as it has left - no predicates, no padding, one shared-memory read per
// nonzero.  On the 9-point stencil the general walk executes some 470 instructions per four
// rows (opcode counts of a profiler run: a third of them integer multiply-adds for
// addresses, predicates and moves), and the kernel there is bound by instruction issue.
constexpr int SHORT_MAX = 16;
constexpr int S_PAIRS = 448;  // pairs staged per warp

// true when every row of the staged unit is well-formed and has at most SHORT_MAX nonzeros
__device__ __forceinline__ bool unit_is_short(const int32_t *wp, int32_t bcount, int32_t nnz, int lane) {
  int32_t worst = 0;
  for (int k = lane; k < bcount; k += 32) {
    const int32_t b = wp[k], e = wp[k + 1];
    int32_t len = e - b;
    if (b < 0 || e < b || e > nnz) len = SHORT_MAX + 1;  // malformed: the general path deals with it
    worst = len > worst ? len : worst;
  }
  return __reduce_max_sync(FULL, worst) <= SHORT_MAX;
}

// N nonzeros of a row, pairs at sp[0 .. N): gather and FMA
template <int G, int VEC, int PAN, int N>
__device__ __forceinline__ void short_slots(const int2 *sp, const char *bcol, int32_t wbytes,
                                            float (&acc)[PAN][VEC]) {
  int2 pr[N];
  float b[N][PAN][VEC];
#pragma unroll
  for (int j = 0; j < N; ++j) pr[j] = sp[j];
#pragma unroll
  for (int j = 0; j < N; ++j) {
    const float *src = b_row(bcol, pr[j].x, wbytes);
#pragma unroll
    for (int pn = 0; pn < PAN; ++pn) load_b<VEC>(src + pn * G * VEC, b[j][pn]);
  }
#pragma unroll
  for (int j = 0; j < N; ++j) {
    const float x = __int_as_float(pr[j].y);
#pragma unroll
    for (int pn = 0; pn < PAN; ++pn)
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[pn][v] = fmaf(x, b[j][pn][v], acc[pn][v]);
  }
}

// all rows [bfirst, bfirst + bcount) of a short unit; wp holds their row pointers, sp is the
// warp's pair buffer
template <int G, int VEC, int PAN>
__device__ __forceinline__ void short_rows(const SpmmArgs &a, const int32_t *wp, int2 *sp, int32_t bfirst,
                                           int32_t bcount, int lane) {
  constexpr int PER_WARP = 32 / G;
  constexpr int UC = Step<PAN>::U;
  const int sub = lane / G, gl = lane % G;
  const int panels = a.w / (G * VEC);
  const int32_t wbytes = a.w * 4;
  int32_t r0 = 0;
  while (r0 < bcount) {
    // rows [r0, r1): as many as the pair buffer holds (at least S_PAIRS / SHORT_MAX of them)
    const int32_t p0 = wp[r0];
    int32_t lo = r0 + 1, hi = bcount;
    while (lo < hi) {
      const int32_t mid = (lo + hi + 1) >> 1;
      if (wp[mid] - p0 <= S_PAIRS)
        lo = mid;
      else
        hi = mid - 1;
    }
    const int32_t r1 = lo, cnt = wp[r1] - p0;
    __syncwarp();  // the rows before are done with the buffer
    for (int32_t k = lane; k < cnt; k += 32)
      sp[k] = make_int2(__ldcs(a.ind + p0 + k), __float_as_int(__ldcs(a.val + p0 + k)));
    __syncwarp();
    for (int32_t idx = r0 + sub; idx < r1; idx += PER_WARP) {
      const int32_t b = wp[idx] - p0, e = wp[idx + 1] - p0;
      float *out = a.C + static_cast<size_t>(bfirst + idx) * a.w + gl * VEC;
      for (int pn0 = 0; pn0 < panels; pn0 += PAN) {
        float acc[PAN][VEC];
#pragma unroll
        for (int pn = 0; pn < PAN; ++pn)
#pragma unroll
          for (int v = 0; v < VEC; ++v) acc[pn][v] = 0.0f;
        const char *bcol = reinterpret_cast<const char *>(a.B + pn0 * (G * VEC) + gl * VEC);
        // pieces of UC nonzeros while more than CAP are left, then all the rest in one piece:
        // every gather of a piece is issued before its first FMA, so a row of nine costs one
        // trip to memory, not two
        constexpr int CAP = UC + 1;
        int32_t q = b;
        for (; e - q > CAP; q += UC) short_slots<G, VEC, PAN, UC>(sp + q, bcol, wbytes, acc);
        switch (e - q) {
#define CSG_REST(N)                                              \
  case N:                                                        \
    if constexpr (N <= CAP) short_slots<G, VEC, PAN, N>(sp + q, bcol, wbytes, acc); \
    break;
          CSG_REST(1) CSG_REST(2) CSG_REST(3) CSG_REST(4) CSG_REST(5) CSG_REST(6) CSG_REST(7) CSG_REST(8)
          CSG_REST(9) CSG_REST(10)
#undef CSG_REST
          default:
            break;
        }
#pragma unroll
        for (int pn = 0; pn < PAN; ++pn) store_c<VEC>(out + (pn0 + pn) * (G * VEC), acc[pn], false);
      }
    }
    r0 = r1;
  }
}

// First launch: all rows of up to SPLIT nonzeros.  Every lane group is persistent: it takes
// the next row of its warp's unit as soon as its current row is finished, so the groups of
// a warp never wait for the one with the longest row.  Rows longer than SPLIT are zeroed and
// queued for the second launch.  A row is walked once per PAN panels (w = panels * G * VEC).
template <int G, int VEC, int PAN>
__global__ void __launch_bounds__(M_THREADS, M_BLOCKS_PER_SM) spmm_rows_kernel(SpmmArgs a) {
  constexpr int U = Step<PAN>::U;
  __shared__ int32_t sptr[M_WARPS][BATCH_MAX + 1];
  __shared__ int2 spair[M_WARPS][S_PAIRS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gl = lane % G;
  const unsigned below_group = (1u << (lane - gl)) - 1u;  // lanes of the groups in front of mine
  int32_t *wp = sptr[warp];
  const int panels = a.w / (G * VEC);
  // warp-uniform: the rows in hand [bfirst, bfirst + bcount) and how many of them are given out
  int32_t bfirst = 0, bcount = 0, bnext = 0;
  bool exhausted = false;
  bool short_unit = false;  // the unit in hand goes to short_rows once every group is idle
  // group-uniform: the row in hand (-1: none), its extent, the walk's position and panel
  int32_t row = -1, pb = 0, p = 0, pe = 0, pn0 = 0;
  float acc[PAN][VEC];
#pragma unroll
  for (int pn = 0; pn < PAN; ++pn)
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[pn][v] = 0.0f;
  for (;;) {
    if (row >= 0 && p >= pe) {  // end of a walk: store, then the next panels or a new row
      float *out = a.C + static_cast<size_t>(row) * a.w + pn0 * (G * VEC) + gl * VEC;
#pragma unroll
      for (int pn = 0; pn < PAN; ++pn) {
        store_c<VEC>(out + pn * G * VEC, acc[pn], false);
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[pn][v] = 0.0f;
      }
      pn0 += PAN;
      if (pn0 < panels)
        p = pb;
      else
        row = -1;
    }
    const unsigned want = __ballot_sync(FULL, row < 0 && gl == 0);  // groups without a row
    if (want) {
      if (bnext >= bcount && !exhausted) {  // the warp draws its next unit of rows
        uint32_t t = 0;
        if (lane == 0) t = atomicAdd(&a.ctrl[CTRL_TICKET], 1u);
        t = __shfl_sync(FULL, t, 0);
        bnext = 0;
        bcount = 0;
        const long long total = static_cast<long long>(ROW_COST) * a.n + a.nnz;
        if (static_cast<long long>(t) * a.unit > total) {
          exhausted = true;
        } else {
          int32_t first, last;
          unit_bounds(a, static_cast<long long>(t) * a.unit, (static_cast<long long>(t) + 1) * a.unit,
                      &first, &last);
          if (last > a.n) last = a.n;
          if (first < last) {
            bfirst = first;
            bcount = last - first;  // at most unit / ROW_COST <= BATCH_MAX rows
            if (bcount > BATCH_MAX) bcount = BATCH_MAX;  // (only with row pointers that decrease)
            __syncwarp();
            for (int k = lane; k <= bcount; k += 32) wp[k] = __ldg(a.ptr + bfirst + k);
            __syncwarp();
            short_unit = unit_is_short(wp, bcount, a.nnz, lane);
          }
        }
      }
      bool hold = false;  // a short unit in hand: no row of it is handed out one by one
      {
        if (short_unit) {
          hold = true;
          // (groups still walking a row of the unit before finish it first)
          if (__ballot_sync(FULL, row >= 0) == 0u) {
            short_rows<G, VEC, PAN>(a, wp, spair[warp], bfirst, bcount, lane);
            bnext = bcount;
            short_unit = false;
            // (no group holds a row here: saying so frees the walk's registers for short_rows)
            row = -1;
            pb = p = pe = pn0 = 0;
#pragma unroll
            for (int pn = 0; pn < PAN; ++pn)
#pragma unroll
              for (int v = 0; v < VEC; ++v) acc[pn][v] = 0.0f;
          }
        }
      }
      if (!hold && row < 0) {
        const int idx = bnext + __popc(want & below_group);
        if (idx < bcount) {
          int32_t b = wp[idx], e = wp[idx + 1];
          if (b < 0 || e < b || e > a.nnz) e = b = 0;  // malformed row pointers: an empty row
          const int32_t r = bfirst + idx;
          if (e - b > SPLIT) {
            for (int32_t j = gl * VEC; j < a.w; j += G * VEC)
#pragma unroll
              for (int v = 0; v < VEC; ++v) a.C[static_cast<size_t>(r) * a.w + j + v] = 0.0f;
            if (gl == 0) {
              const unsigned long long pieces =
                  static_cast<unsigned long long>((e - b + LONG_PIECE - 1) / LONG_PIECE);
              const unsigned long long old = atomicAdd(
                  reinterpret_cast<unsigned long long *>(a.ctrl + CTRL_PACKED), (1ull << 32) | pieces);
              a.long_rows[old >> 32] = make_int2(r, static_cast<int32_t>(old & 0xFFFFFFFFu));
            }
          } else {
            row = r;
            pb = p = b;
            pe = e;
            pn0 = 0;
          }
        }
      }
      if (!hold) {
        const int given = bnext + __popc(want);
        bnext = given < bcount ? given : bcount;
      }
      if (exhausted && __ballot_sync(FULL, row >= 0) == 0u) break;
    }
    if (row >= 0 && p < pe) {
      const int cnt = pe - p < U ? pe - p : U;
      fma_step<G, VEC, PAN>(a, p, cnt, pn0 * (G * VEC) + gl * VEC, acc);
      p += cnt;
      // a short tail (a row of nine nonzeros is a full step and one more) goes along in the
      // same turn of the loop: the turn, with its hand-out of rows, costs more than the tail
      if (pe - p > 0 && pe - p <= U / 2) {
        fma_step<G, VEC, PAN, U / 2>(a, p, pe - p, pn0 * (G * VEC) + gl * VEC, acc);
        p = pe;
      }
    }
  }
}

// Second launch: the pieces (LONG_PIECE nonzeros each) of the queued long rows, spread over
// all lane groups; piece number -> queue entry by binary search on the entries' first
// piece numbers (ascending by construction).  Partial rows are added with atomics.
template <int G, int VEC, int PAN>
__global__ void __launch_bounds__(M_THREADS, M_BLOCKS_PER_SM) spmm_long_kernel(SpmmArgs a) {
  constexpr int PER_WARP = 32 / G;
  constexpr int U = Step<PAN>::U;
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
    const int32_t pb = b + (id - q.y) * LONG_PIECE;
    const int32_t pe = pb + LONG_PIECE < e ? pb + LONG_PIECE : e;
    for (int pn0 = 0; pn0 < panels; pn0 += PAN) {
      const int32_t col0 = pn0 * (G * VEC) + gl * VEC;
      float acc[PAN][VEC];
#pragma unroll
      for (int pn = 0; pn < PAN; ++pn)
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[pn][v] = 0.0f;
      for (int32_t p = pb; p < pe; p += U) fma_step<G, VEC, PAN>(a, p, pe - p < U ? pe - p : U, col0, acc);
#pragma unroll
      for (int pn = 0; pn < PAN; ++pn)
        store_c<VEC>(a.C + static_cast<size_t>(q.x) * a.w + col0 + pn * G * VEC, acc[pn], true);
    }
  }
}

template <int G, int VEC, int PAN>
bool launch_variant(Context &ctx, SpmmArgs a) {
  // cost per unit: enough units that every warp of the grid draws several of them
  const int grid = ctx.num_sms * M_BLOCKS_PER_SM;
  const long long total = static_cast<long long>(ROW_COST) * a.n + a.nnz;
  long long unit = total / (static_cast<long long>(grid) * M_WARPS * 8);
  if (unit < 128) unit = 128;
  if (unit > UNIT_MAX) unit = UNIT_MAX;
  a.unit = static_cast<int32_t>(unit);
  spmm_rows_kernel<G, VEC, PAN><<<grid, M_THREADS, 0, ctx.stream>>>(a);
  CSG_CUDA(cudaGetLastError());
  spmm_long_kernel<G, VEC, PAN><<<grid, M_THREADS, 0, ctx.stream>>>(a);
  CSG_CUDA(cudaGetLastError());
  count_launches(2);
  return true;
}

// Lane groups by dense width: float4 columns per lane where the width and the alignment of
// B and C allow, single floats otherwise; two panels per walk when the panel count is even.
bool dispatch_spmm(Context &ctx, const SpmmArgs &a) {
  const int w = a.w;
  const bool al16 = (reinterpret_cast<uintptr_t>(a.B) % 16 == 0) && (reinterpret_cast<uintptr_t>(a.C) % 16 == 0);
  if (w % 256 == 0 && al16) return launch_variant<32, 4, 2>(ctx, a);
  if (w % 128 == 0 && al16) return launch_variant<32, 4, 1>(ctx, a);
  if (w % 64 == 0 && al16) return launch_variant<16, 4, 1>(ctx, a);
  if (w % 32 == 0 && al16) return launch_variant<8, 4, 1>(ctx, a);
  if (w % 16 == 0 && al16) return launch_variant<4, 4, 1>(ctx, a);
  if (w % 32 == 0) return launch_variant<32, 1, 1>(ctx, a);
  if (w % 8 == 0) return launch_variant<8, 1, 1>(ctx, a);
  if (w % 4 == 0) return launch_variant<4, 1, 1>(ctx, a);
  if (w % 2 == 0) return launch_variant<2, 1, 1>(ctx, a);
  return launch_variant<1, 1, 1>(ctx, a);
}

}  // namespace

bool launch_spmm(Context &ctx, int32_t n, int32_t nnz, int32_t w, const int32_t *d_ptr,
                 const int32_t *d_ind, const float *d_val, const float *d_B, float *d_C) {
  CSG_REQUIRE(w >= 1, "spmm: dense width must be >= 1");
  SpmmArgs a;
  a.n = n;
  a.w = w;
  a.nnz = nnz;
  a.unit = UNIT_MAX;
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
  return dispatch_spmm(ctx, a);
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
  a.nnz = nnz;
  a.unit = UNIT_MAX;
  a.ptr = d_ptr;
  a.ind = d_ind;
  a.val = d_val;
  a.B = d_B;
  a.C = d_C;
  a.ctrl = scratch;
  a.long_rows = reinterpret_cast<int2 *>(scratch + STATIC_QUEUE_OFFSET);
  // the counters keep the previous call's values: clear them (the queue is overwritten)
  CSG_CUDA(cudaMemsetAsync(a.ctrl, 0, sizeof(uint32_t) * CTRL_SCRATCH_WORDS, stream));
  return dispatch_spmm(tmp, a);
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
