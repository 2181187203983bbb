// Shapes, the workspace layout and the split-KV schedule shared by the decode, schedule and combine kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mla {

constexpr int CKV = 512;          // latent channels (packed E2M1, 256 bytes per token)
constexpr int KPE = 64;           // rope channels (E4M3)
constexpr int TOKEN_BYTES = 352;  // 256 + 32 + 64
constexpr int TILE = 128;         // tokens per tile = rows of one tcgen05 MMA
constexpr int HALF = 64;          // tokens per staging slot

// One unit of work of a decode CTA: `ntiles` consecutive 128-token tiles of request `b`, head group `hg`, starting
// at token `tok0`; tokens at or beyond `tok_end` are masked. Its partial result goes to slot `cta + w`.
struct Seg {
  int b, hg, tok0, ntiles, tok_end, w, cta, pad;
};
static_assert(sizeof(Seg) == 32, "Seg is read as two 16-byte words");

// Workspace (device memory owned by the caller):
//   header     16 x int32   [0] error status (sticky), [1] total tiles, [2] tiles per CTA
//   cta_range  n_cta x int2 items [first, last) that intersect the CTA's tile range
//   item_range W x int2     CTAs [first, last] that hold a piece of item w (last < first: the item is empty)
//   segs       (n_cta + W) x Seg, indexed by slot = cta + w
//   lse_part   (n_cta + W) x heads_per_cta floats, log2 units
//   o_part     (n_cta + W) x heads_per_cta x 512 floats, each normalised by its own sum
struct WsLayout {
  size_t header, cta_range, item_range, segs, lse_part, o_part, total;
};
__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
__host__ __device__ inline WsLayout ws_layout(int n_cta, long long W, int heads_per_cta) {
  WsLayout l;
  const size_t slots = size_t(n_cta) + size_t(W);
  size_t off = 0;
  l.header = off, off = align_up(off + 64, 256);
  l.cta_range = off, off = align_up(off + size_t(n_cta) * 8, 256);
  l.item_range = off, off = align_up(off + size_t(W) * 8, 256);
  l.segs = off, off = align_up(off + slots * sizeof(Seg), 256);
  l.lse_part = off, off = align_up(off + slots * heads_per_cta * 4, 256);
  l.o_part = off, off = align_up(off + slots * heads_per_cta * CKV * 4, 256);
  l.total = off;
  return l;
}

// Item numbering: w = (b * splits + z) * head_groups + hg, so that the head groups of one (request, split) are
// neighbours in the flattened tile order and re-read the same KV range close together in time.
struct Problem {
  int batch, heads, heads_per_cta, head_groups, splits, chunk, n_cta;
  __host__ __device__ long long items() const { return (long long)batch * splits * head_groups; }
};

// 128-token tiles of (request, split) pair bz = b * splits + z: the split covers tokens [z * chunk, (z + 1) * chunk) of the request.
__device__ __forceinline__ int sched_tiles(const int* kv_lens, const Problem& pb, int bz) {
  const int b = bz / pb.splits, z = bz % pb.splits;
  long long n = (long long)kv_lens[b] - (long long)z * pb.chunk;
  n = n < 0 ? 0 : (n > pb.chunk ? pb.chunk : n);
  return int((n + TILE - 1) / TILE);
}

enum Status : int {
  kOk = 0,
  kWaitTimeout = 1,   // a bounded wait inside the decode kernel gave up
  kBadSchedule = 2,   // schedule kernel: batch * splits exceeds its scan capacity
  kBadPage = 3,       // a page id of a request's live range lies outside [0, num_pages): its rows were not loaded
  kPeerTimeout = 4,   // cross-GPU merge: another GPU's record was not announced within the wait limit
};

}  // namespace mla
