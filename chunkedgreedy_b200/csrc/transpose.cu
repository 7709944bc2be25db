// Chunk-local transpose.
//
// The reference builds a full CSC with a device-wide radix sort
// (sporder/src/common/csr2csc.cu:38-115) and then, per row, scans whole column
// lists to pick out the rows of the row's own chunk
// (sporder/src/common/chunk_similarity_top_k.cu:52-84).  Candidates never leave
// the chunk, so this library transposes every chunk on its own: one thread block
// sorts the chunk's (column, position) pairs by column (stable LSD radix sort, in
// shared memory when the chunk fits, in global ping-pong buffers otherwise),
// finds the column groups and emits
//   cand[]  : the chunk's rows grouped by column, rows ascending inside a group,
//             each with its row length (what the Dice term needs);
//   seg[p]  : for nonzero p (CSR order) the group of its column: (first, length);
//   row_work: per row, how many candidates its stream will hold.
// A caller-promised symmetric pattern needs no separate path: the transpose of a
// symmetric pattern restricted to the chunk is what the reference reads from the
// aliased CSR arrays (sporder/src/common/csr2csc.h:52-54).
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
  uint32_t *row_work;
  uint32_t *ctrl;
};

struct Shared {
  uint32_t wc[T_WARPS * 256];
  uint32_t hist[256];
  uint32_t binbase[256];
  int32_t warp_last[T_WARPS];
  int32_t carry;
  int32_t ticket;
  uint32_t bucket[33];
  int32_t sptr[T_RP + 1];
  uint32_t row_work[T_RP];
  uint32_t skey[2][T_LS];
  uint16_t spay[2][T_LS];
};

// One stable counting pass on an 8-bit digit.  FIRST reads the keys from the CSR
// column array and uses the position as payload.
template <typename PayT, bool FIRST>
__device__ void radix_pass(const uint32_t *kin, const PayT *pin, uint32_t *kout, PayT *pout,
                           int L, int shift, Shared &sh) {
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
      const unsigned peers = __match_any_sync(FULL, d);
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
        kout[dst] = key[i];
        pout[dst] = pay[i];
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
    if (len >= 2) {
      if (rows_in_smem)
        atomicAdd(&sh.row_work[row - cs], static_cast<uint32_t>(len - 1));
      else
        atomicAdd(&a.row_work[row], static_cast<uint32_t>(len - 1));
    }
  }
}

__global__ void __launch_bounds__(T_THREADS, 1) transpose_kernel(TransposeArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Shared &sh = *reinterpret_cast<Shared *>(smem_raw);
  const int tid = threadIdx.x;
  if (tid < 33) sh.bucket[tid] = 0;
  for (;;) {
    __syncthreads();
    if (tid == 0) sh.ticket = static_cast<int32_t>(atomicAdd(&a.ctrl[CTRL_CHUNK_TICKET], 1u));
    __syncthreads();
    const int32_t q = sh.ticket;
    if (q >= a.num_chunks) break;
    const int64_t cs64 = static_cast<int64_t>(q) * a.chunk;
    const int32_t cs = static_cast<int32_t>(cs64);
    const int32_t ce = (cs64 + a.chunk > a.n) ? a.n : static_cast<int32_t>(cs64 + a.chunk);
    const int32_t rows = ce - cs;
    const int32_t b = a.ptr[cs];
    int L = a.ptr[ce] - b;
    if (b < 0 || L < 0 || L > a.nnz - b) {  // malformed row pointers: flag and skip
      if (tid == 0) atomicExch(&a.ctrl[CTRL_BAD_INPUT], 1u);
      L = 0;
    }
    const bool rows_in_smem = rows <= T_RP;
    if (rows_in_smem) {
      for (int i = tid; i <= rows; i += T_THREADS) sh.sptr[i] = a.ptr[cs + i];
      for (int i = tid; i < rows; i += T_THREADS) sh.row_work[i] = 0;
    }
    __syncthreads();
    if (L > 0) {
      const uint32_t *kin0 = reinterpret_cast<const uint32_t *>(a.ind + b);
      const int P = a.passes;
      if (L <= T_LS) {
        radix_pass<uint16_t, true>(kin0, nullptr, sh.skey[0], sh.spay[0], L, 0, sh);
        for (int ps = 1; ps < P; ++ps)
          radix_pass<uint16_t, false>(sh.skey[(ps - 1) & 1], sh.spay[(ps - 1) & 1], sh.skey[ps & 1],
                                      sh.spay[ps & 1], L, 8 * ps, sh);
        const int f = (P - 1) & 1;
        emit_groups<uint16_t>(sh.skey[f], sh.spay[f], sh.skey[f ^ 1], sh.spay[f ^ 1], L, b, cs, rows,
                              rows_in_smem, a, sh);
      } else {
        uint32_t *kb[2] = {a.keyA + b, a.keyB + b};
        uint32_t *pb[2] = {a.payA + b, a.payB + b};
        radix_pass<uint32_t, true>(kin0, nullptr, kb[0], pb[0], L, 0, sh);
        for (int ps = 1; ps < P; ++ps)
          radix_pass<uint32_t, false>(kb[(ps - 1) & 1], pb[(ps - 1) & 1], kb[ps & 1], pb[ps & 1], L,
                                      8 * ps, sh);
        const int f = (P - 1) & 1;
        emit_groups<uint32_t>(kb[f], pb[f], kb[f ^ 1], pb[f ^ 1], L, b, cs, rows, rows_in_smem, a,
                              sh);
      }
    }
    __syncthreads();
    if (rows_in_smem) {
      for (int i = tid; i < rows; i += T_THREADS) {
        const uint32_t t = sh.row_work[i];
        a.row_work[cs + i] = t;
        if (t) atomicAdd(&sh.bucket[32 - __clz(t)], 1u);
      }
    } else {
      for (int i = tid; i < rows; i += T_THREADS) {
        const uint32_t t = __ldcg(&a.row_work[cs + i]);  // accumulated with global atomics
        if (t) atomicAdd(&sh.bucket[32 - __clz(t)], 1u);
      }
    }
  }
  __syncthreads();
  if (tid < 33 && sh.bucket[tid]) atomicAdd(&a.ctrl[CTRL_BUCKET_COUNT + tid], sh.bucket[tid]);
}

// Heaviest bucket first: rows with 2^(b-1) <= work < 2^b sit in bucket b.
__global__ void bucket_scan_kernel(uint32_t *ctrl) {
  if (threadIdx.x == 0) {
    uint32_t run = 0;
    for (int b = 32; b >= 1; --b) {
      ctrl[CTRL_BUCKET_BASE + b] = run;
      run += ctrl[CTRL_BUCKET_COUNT + b];
      ctrl[CTRL_BUCKET_FILL + b] = 0;
    }
    ctrl[CTRL_ROWS_LISTED] = run;
  }
}

__global__ void row_list_kernel(int32_t n, const uint32_t *__restrict__ row_work, uint32_t *ctrl,
                                int32_t *__restrict__ row_list) {
  const int lane = threadIdx.x & 31;
  const int32_t total = gridDim.x * blockDim.x;
  for (int32_t base = blockIdx.x * blockDim.x; base < n; base += total) {
    const int32_t r = base + threadIdx.x;
    const uint32_t t = r < n ? row_work[r] : 0u;
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

bool launch_transpose(Context &ctx, int32_t n, int32_t ncols, int32_t nnz, int32_t chunk, const int32_t *d_ptr,
                      const int32_t *d_ind, CsgScratch &s) {
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
  a.row_work = s.row_work;
  a.ctrl = s.ctrl;
  const size_t smem = sizeof(Shared);
  CSG_CUDA(cudaFuncSetAttribute(transpose_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(smem)));
  CSG_CUDA(cudaMemsetAsync(s.ctrl, 0, sizeof(uint32_t) * CTRL_WORDS, ctx.stream));
  CSG_CUDA(cudaMemsetAsync(s.row_work, 0, sizeof(uint32_t) * static_cast<size_t>(n), ctx.stream));
  const int grid = a.num_chunks < ctx.num_sms ? a.num_chunks : ctx.num_sms;
  transpose_kernel<<<grid, T_THREADS, smem, ctx.stream>>>(a);
  CSG_CUDA(cudaGetLastError());
  bucket_scan_kernel<<<1, 32, 0, ctx.stream>>>(s.ctrl);
  CSG_CUDA(cudaGetLastError());
  int lgrid = (n + 255) / 256;
  if (lgrid > ctx.num_sms * 8) lgrid = ctx.num_sms * 8;
  row_list_kernel<<<lgrid, 256, 0, ctx.stream>>>(n, s.row_work, s.ctrl, s.row_list);
  CSG_CUDA(cudaGetLastError());
  count_launches(3);
  return true;
}

}  // namespace csg
