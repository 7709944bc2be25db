// Shared declarations of the B200 csg library: context, error channel,
// workspace arena and the launch functions of each stage.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

namespace csg {

// ---- error channel -------------------------------------------------------
// The reference aborts the process on invalid arguments and CUDA errors
// (sporder/src/common/error_checking.h:20-29).  On a shared GPU pool this
// library records the message per thread and returns instead.
void set_error(const char *fmt, ...);
bool has_error();
void clear_error();
void count_launches(int k);  // feeds sporder_kernel_launches()

#define CSG_CUDA(call)                                                                  \
  do {                                                                                  \
    cudaError_t e__ = (call);                                                           \
    if (e__ != cudaSuccess) {                                                           \
      ::csg::set_error("%s:%d: %s -> %s", __FILE__, __LINE__, #call,                    \
                       cudaGetErrorString(e__));                                        \
      return false;                                                                     \
    }                                                                                   \
  } while (0)

#define CSG_REQUIRE(cond, ...)                                                          \
  do {                                                                                  \
    if (!(cond)) {                                                                      \
      ::csg::set_error(__VA_ARGS__);                                                    \
      return false;                                                                     \
    }                                                                                   \
  } while (0)

// ---- context ---------------------------------------------------------------
// Counterpart of sporder::context (sporder/src/common/context.h:67-197): one
// stream, the device it was created on, and a grow-only device workspace so a
// warm call allocates nothing.
struct Context {
  int device = 0;
  cudaStream_t stream = nullptr;  // stream every launch of this context uses
  cudaStream_t own_stream = nullptr;
  int num_sms = 0;
  int smem_optin = 0;  // max dynamic shared memory per block (opt-in)
  char *ws = nullptr;  // device workspace
  size_t ws_bytes = 0;
  cudaEvent_t ev[10] = {};  // [0..4] stage times; [5..8] fork, joins and order of a call that runs one chunk ahead
  int *h_pinned = nullptr;  // small pinned host buffer for counters (64 ints)
  char *stage = nullptr;    // device copies of host inputs (host-buffer entry point), kept between calls
  size_t stage_bytes = 0;
  // Buffer for the materialised candidate streams of the heaviest rows (sketch.cu), in stream
  // elements of 8 bytes.  A call starts from a size in proportion to its input; every call
  // reports what all its heavy rows together would have needed, and the next call of the
  // context plans that much (rows that do not fit are still computed, by the slower kernel of
  // the light rows, so results never depend on the size).
  uint64_t stream_need_seen = 0;   // largest need any call of this context reported
  uint64_t stream_need_prio = 0;   // ... and the share of it that the rows running ahead asked for
  // Second stream (higher priority) for the part of a large call that runs ahead of the rest:
  // the transposition and the chains of the chunk that holds the most nonzeros (see run_csg).
  cudaStream_t side_stream = nullptr;
  // nonzeros from which a call runs one chunk ahead: 0 = the built-in threshold, negative =
  // never, positive = the caller's threshold (sporder_context_set_ahead_threshold)
  int64_t ahead_min_nnz = 0;
  uint64_t stream_limit = 0;       // caller's upper bound (sporder_context_set_stream_limit), 0 = none
};

bool ensure_workspace(Context &ctx, size_t bytes);

// Bump allocator over the context workspace (256-byte aligned blocks).
struct Arena {
  size_t off = 0;
  size_t take(size_t bytes) {
    size_t o = off;
    off += (bytes + 255) & ~size_t(255);
    return o;
  }
};

// ---- resolved csg parameters (sporder/src/sporder.cpp:147-161) ---------------
struct CsgParams {
  int32_t k;
  float ovs;
  int32_t chunk;
  int32_t m_used;  // value the stats struct reports
  int32_t M;       // sketch capacity actually used (multiple of 32, <= 512)
};
bool resolve_params(int32_t n, int32_t nnz, int32_t k, float ovs, int32_t chunk, CsgParams *out);

// ---- device scratch of one csg call -------------------------------------------
struct CsgScratch {
  // chunk-local transpose (see transpose.cu)
  uint32_t *keyA, *keyB, *payA, *payB;  // ping-pong buffers of the global sort path
  int2 *cand;                           // (row, row length) grouped by (chunk, column), rows ascending
  int2 *seg;                            // per nonzero: (first index into cand, group length)
  int32_t *seg_rank;                    // per nonzero: index of its own row inside that group
  uint32_t *row_work;                   // candidates each row will see
  // work list of rows with candidates, heaviest bucket first
  int32_t *row_list;
  uint32_t *ctrl;  // [0]=chunk ticket [1]=row ticket [2]=rows listed [3..] see CTRL_* below
  uint64_t *table;  // n*k packed top-k entries
  uint32_t *gbitmaps;  // greedy bitmaps when they do not fit shared memory, else nullptr
  // materialised candidate streams of the heaviest rows (see sketch.cu)
  int2 *hstream;
  uint32_t *heavy_off;
  int32_t *heavy_state;
  uint32_t stream_cap, heavy_max;
  uint32_t *part_base, *part_off;
  // tiled sort of heavy chunks (see transpose.cu)
  int32_t *heavy_chunk, *heavy_tile_base;
  uint32_t *tile_hist, *digit_base;
};
enum {
  CTRL_CHUNK_TICKET = 0,
  CTRL_ROW_TICKET = 1,
  CTRL_ROWS_LISTED = 2,
  CTRL_BAD_INPUT = 3,      // set by a kernel that met row pointers outside [0, nnz]
  CTRL_HEAVY_COUNT = 4,    // chunks sorted by the tiled path
  CTRL_HEAVY_TILES = 5,    // their tiles
  CTRL_HEAVY_ROWS = 6,     // rows at the head of row_list that the heavy sketch kernel takes
  CTRL_HEAVY_TICKET = 7,   // and the word after it: a second ticket
  CTRL_HEAVY_PARTS = 9,    // column slices of the heavy rows
  CTRL_HEAVY_NEED = 10,    // and the word after it: stream elements of all rows of heavy weight (64-bit)
  CTRL_STREAM_OVERRUN = 12,  // set by heavy_expand_kernel when a slice would pass the stream buffer
  CTRL_CHECK = 13,         // checked build: site of the first index out of bounds, then the index (64-bit)
  CTRL_BUCKET_COUNT = 16,  // 33 entries
  CTRL_PRIO = 50,          // chunk whose heavy rows run ahead of the rest (PRIO_NONE: no such chunk)
  CTRL_CRITICAL_ROWS = 51,  // rows at the head of the chunk ahead's list whose chains keep a scheduler each
  CTRL_CRITICAL_TICKET = 52,
  CTRL_LONGEST = 53,       // longest candidate stream of the chunk ahead
  CTRL_BUCKET_BASE = 56,   // 33 entries
  CTRL_BUCKET_FILL = 96,   // 33 entries
  CTRL_STATS = 136,        // see greedy.cu (8-byte aligned)
  CTRL_PROFILE = 168,      // 16 64-bit counters, written only by a build with -DCSG_ROUND_PROFILE
  CTRL_WORDS = 200
};

constexpr uint32_t PRIO_NONE = 0xFFFFFFFFu;
// phases of a call that runs one chunk ahead: everything (no such split), the chunk ahead, the rest
enum CallPhase { PHASE_ALL = 0, PHASE_PRIO = 1, PHASE_REST = 2 };
// SMs the chains of the chunk ahead may hold (the other chains get the remaining ones)
inline int prio_chain_blocks(int num_sms) { return num_sms / 4 > 0 ? num_sms / 4 : 1; }

constexpr int SKETCH_PART_COLS = 128;   // columns of a heavy row whose stream one warp writes out
constexpr int SKETCH_HEAVY_BUCKET = 17;  // rows streaming >= 65536 candidates are "heavy"

// stage launchers; all enqueue on ctx.stream and return false after set_error()
bool launch_transpose(Context &ctx, int32_t n, int32_t ncols, int32_t nnz, int32_t chunk, const int32_t *d_ptr,
                      const int32_t *d_ind, CsgScratch &s, bool symmetric = false, int phase = PHASE_ALL,
                      uint32_t *ctrl_other = nullptr);
// start of a call that runs one chunk ahead: clears the counters of both parts and names the chunk
bool launch_priority_pick(Context &ctx, int32_t n, int32_t nnz, int32_t chunk, const int32_t *d_ptr,
                          CsgScratch &s, CsgScratch &prio, int32_t min_chunk_nnz);
bool launch_sketch(Context &ctx, int32_t n, int32_t nnz, const CsgParams &p, const int32_t *d_ptr,
                   CsgScratch &s, int32_t row_base, bool zero_table, int phase = PHASE_ALL);
bool launch_greedy(Context &ctx, int32_t n, const CsgParams &p, CsgScratch &s,
                   int32_t *d_new_order, bool with_stats, int32_t row_base);
bool launch_pillars_search(Context &ctx, int32_t n, int32_t nnz, int32_t height, const int32_t *d_ptr,
                           const int32_t *d_ind, unsigned long long *d_count, uint32_t *d_bad);
bool launch_pillars_groups(Context &ctx, int32_t nnz, const int32_t *seg_rank, unsigned long long *d_count);
bool launch_in_chunk_weight(Context &ctx, int32_t n, int32_t k, int32_t chunk, const uint64_t *table,
                            uint32_t *ctrl);
bool launch_table_stats(Context &ctx, int32_t n, int32_t k, const uint64_t *table, uint32_t *ctrl);

bool launch_reorder(Context &ctx, int32_t n, int32_t nnz, const int32_t *d_ptr_old,
                    const int32_t *d_ind_old, const float *d_val_old, const int32_t *d_new_order,
                    int mode, int32_t *d_ptr_new, int32_t *d_ind_new, float *d_val_new);
size_t reorder_workspace_bytes(int32_t n, int32_t nnz, int mode);

bool launch_spmm(Context &ctx, int32_t n, int32_t nnz, int32_t w, const int32_t *d_ptr,
                 const int32_t *d_ind, const float *d_val, const float *d_B, float *d_C);

// ---- small device helpers -------------------------------------------------------
#ifdef __CUDACC__
constexpr unsigned FULL = 0xFFFFFFFFu;
__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// ---- checked build ----------------------------------------------------------------------
// Compiled with -DSPORDER_CHECKED (python -m chunkedgreedy_b200.build --checked) every index
// that a kernel derives from data another kernel wrote - positions in the transposed chunk,
// stream offsets, table slots, list entries - is tested before use; the first one out of
// bounds is recorded (site, index) and the access is skipped, so the kernel runs on with
// harmless values and the host reports the site instead of the GPU faulting.  This stands in
// for compute-sanitizer on machines where that tool may not be run.  In the normal build the
// test is a constant `true` and costs nothing.
enum CheckSite : uint32_t {
  CHK_CAND = 1,      // cand[] index from a group descriptor
  CHK_RING = 2,      // position in a warp's stream ring
  CHK_STREAM = 3,    // hstream[] offset of a heavy row
  CHK_KEY = 4,       // stream key outside its chunk (key -> slot table)
  CHK_STATE = 5,     // heavy_state[] / heavy_off[] item
  CHK_TABLE = 6,     // row of the top-k table
  CHK_LIST = 7,      // row_list[] entry
  CHK_ORDER = 8,     // order[] position in the greedy stage
  CHK_SORT = 9,      // scatter position of a radix pass
  CHK_GROUP = 10,    // group start / position written by the transpose
  CHK_PART = 11,     // part_off[] / part_base[] entry
};
#ifdef SPORDER_CHECKED
__device__ __forceinline__ bool index_ok(uint32_t *ctrl, uint32_t site, long long idx, long long bound) {
  if (idx >= 0 && idx < bound) return true;
  if (atomicCAS(&ctrl[CTRL_CHECK], 0u, site) == 0u) {
    ctrl[CTRL_CHECK + 1] = static_cast<uint32_t>(static_cast<unsigned long long>(idx));
    ctrl[CTRL_CHECK + 2] = static_cast<uint32_t>(static_cast<unsigned long long>(idx) >> 32);
  }
  return false;
}
#else
__device__ __forceinline__ bool index_ok(uint32_t *, uint32_t, long long, long long) { return true; }
#endif

// counter += v, sticking at 0xFFFFFFFF instead of wrapping.  Whoever sees the sum wrap puts
// the ceiling back; the last operation on a counter that ever wrapped is such a repair, so
// once all adders are done the counter reads 0xFFFFFFFF ("more than fits").
__device__ __forceinline__ void saturating_add(uint32_t *counter, uint32_t v) {
  const uint32_t old = atomicAdd(counter, v);
  if (old + v < old) atomicMax(counter, 0xFFFFFFFFu);
}

// Lanes of the warp whose 8-bit digit equals this lane's (d in [0, 255]; lanes that pass
// d = 256 take no part and get their own bit).  Eight ballots and eight selects: match.any, the
// instruction made for this, measures some 380 cycles per call on this part with a lone warp,
// this sequence about 80.
__device__ __forceinline__ unsigned match_digit(uint32_t d) {
  unsigned peers = __ballot_sync(FULL, d < 256u);
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    const unsigned has = __ballot_sync(FULL, (d >> b) & 1u);
    peers &= ((d >> b) & 1u) ? has : ~has;
  }
  return d < 256u ? peers : 1u << (threadIdx.x & 31);
}

// packed entry of the top-k table; wire format of the reference
// (sporder/src/common/weighted_index.h:15-27): high word = fp32 bits of the
// weight, low word = index + 1, all-zero = empty.
__device__ __forceinline__ uint64_t pack_entry(int32_t idx, float w) {
  return (static_cast<uint64_t>(__float_as_uint(w)) << 32) | static_cast<uint32_t>(idx + 1);
}
__device__ __forceinline__ int32_t entry_index(uint64_t e) {
  return static_cast<int32_t>(static_cast<uint32_t>(e)) - 1;
}
__device__ __forceinline__ uint32_t entry_weight_bits(uint64_t e) {
  return static_cast<uint32_t>(e >> 32);
}
#endif

}  // namespace csg
