// Test-infrastructure shim linked INTO the reference build (oracle/_ref/): it
// exposes the reference's internal csg top-k table, which the reference's public
// C ABI never returns.  It only calls reference functions through the reference's
// own internal headers (sporder/src/common/csr2csc.h:49-70,
// sporder/src/common/chunk_similarity_top_k.h:18-23); it holds no algorithm.
// Never linked into the product library.
#include "common/chunk_similarity_top_k.h"
#include "common/context.h"
#include "common/csr2csc.h"
#include "common/weighted_index.h"
#include <cstdint>

extern "C" __attribute__((visibility("default"))) void
refshim_csg_table(int32_t n, int32_t nnz, const int32_t *d_ptr, const int32_t *d_ind,
                  bool is_symmetric, int32_t k, float oversampling, int32_t chunk_size,
                  uint64_t *d_table /* n*k packed entries, device */) {
  sporder::context ctx;
  sporder::resolved_csc csc = sporder::resolve_csc(ctx, n, nnz, d_ptr, d_ind, is_symmetric);
  sporder::multi_chunk_similarity_top_k(
      ctx, n, k, chunk_size, oversampling, d_ptr, d_ind, csc.d_ptr, csc.d_ind,
      reinterpret_cast<sporder::weighted_index *>(d_table));
  sporder::release_csc(ctx, csc);
  ctx.wait();
}
