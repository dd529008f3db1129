// Strided byte movers: one kernel serves the stale-KV scatter, PipeFusion patch
// copies (local or into a peer's mapped buffer) and parameter-slice migration.
//
// A "piece" is a 3-level box  [n_outer][rows][row_bytes]  with independent
// source and destination pitches. Up to kMaxPieces pieces travel in kernel
// parameter space, so a launch needs neither a device-side table nor a copy.
// Each piece picks the widest vector (16/8/4/2/1 bytes) its addresses, pitches
// and row length allow; CTAs of blockIdx.y stride over the piece's vectors.
// These kernels are HBM- (or NVLink-) bound: 16-byte accesses, consecutive
// threads on consecutive addresses, 4 loads in flight per thread.
#include <cuda_runtime.h>
#include <string.h>

#include "host_common.h"

namespace hdit {
namespace {

constexpr int kMaxPieces = 40;
constexpr int kCopyThreads = 256;

struct Piece {
  const char* src;
  char* dst;
  long long n_outer, src_outer_pitch, dst_outer_pitch;
  long long rows, src_pitch, dst_pitch;
  long long row_bytes;
  int vec;  // bytes per access
  int pad;
};

struct PieceTable {
  Piece p[kMaxPieces];
  int n;
};

__device__ __forceinline__ void row_offsets(const Piece& pc, unsigned long long row, long long& so, long long& dof) {
  if (pc.n_outer == 1) {
    so = static_cast<long long>(row) * pc.src_pitch;
    dof = static_cast<long long>(row) * pc.dst_pitch;
  } else {
    // the host checked that n_outer * rows fits 32 bits
    const unsigned o = static_cast<unsigned>(row) / static_cast<unsigned>(pc.rows);
    const unsigned r = static_cast<unsigned>(row) - o * static_cast<unsigned>(pc.rows);
    so = o * pc.src_outer_pitch + r * pc.src_pitch;
    dof = o * pc.dst_outer_pitch + r * pc.dst_pitch;
  }
}

// Thread `tid` of `nthreads` copies vectors tid, tid + nthreads, ... of the piece. The (row, column)
// position advances by a fixed (rows, columns) step with carry, so the loop has no division.
template <typename V>
__device__ __forceinline__ void copy_piece(const Piece& pc, long long tid, long long nthreads) {
  const unsigned long long vpr = static_cast<unsigned long long>(pc.row_bytes) / sizeof(V);
  const unsigned long long nrows = static_cast<unsigned long long>(pc.n_outer) * pc.rows;
  unsigned long long row = static_cast<unsigned long long>(tid) / vpr;
  unsigned long long col = static_cast<unsigned long long>(tid) - row * vpr;
  const unsigned long long step_row = static_cast<unsigned long long>(nthreads) / vpr;
  const unsigned long long step_col = static_cast<unsigned long long>(nthreads) - step_row * vpr;
  constexpr int kUnroll = 4;
  while (row < nrows) {
    V v[kUnroll];
    long long doff[kUnroll];
    bool live[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      live[u] = row < nrows;
      if (live[u]) {
        long long so;
        row_offsets(pc, row, so, doff[u]);
        doff[u] += col * sizeof(V);
        v[u] = *reinterpret_cast<const V*>(pc.src + so + col * sizeof(V));
      }
      row += step_row;
      col += step_col;
      if (col >= vpr) {
        col -= vpr;
        ++row;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (live[u]) *reinterpret_cast<V*>(pc.dst + doff[u]) = v[u];
  }
}

__global__ void __launch_bounds__(kCopyThreads) copy_pieces_kernel(const __grid_constant__ PieceTable tab) {
  const Piece& pc = tab.p[blockIdx.x];
  const long long tid = static_cast<long long>(blockIdx.y) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.y) * blockDim.x;
  switch (pc.vec) {
    case 16: copy_piece<uint4>(pc, tid, nthreads); break;
    case 8: copy_piece<uint2>(pc, tid, nthreads); break;
    case 4: copy_piece<uint32_t>(pc, tid, nthreads); break;
    case 2: copy_piece<uint16_t>(pc, tid, nthreads); break;
    default: copy_piece<uint8_t>(pc, tid, nthreads); break;
  }
}

int pick_vec(const hdit_copy_piece& d) {
  const uintptr_t bits = reinterpret_cast<uintptr_t>(d.src) | reinterpret_cast<uintptr_t>(d.dst) |
                         static_cast<uintptr_t>(d.row_bytes) |
                         (d.rows > 1 ? static_cast<uintptr_t>(d.src_pitch | d.dst_pitch) : 0) |
                         (d.n_outer > 1 ? static_cast<uintptr_t>(d.src_outer_pitch | d.dst_outer_pitch) : 0);
  if ((bits & 15) == 0) return 16;
  if ((bits & 7) == 0) return 8;
  if ((bits & 3) == 0) return 4;
  if ((bits & 1) == 0) return 2;
  return 1;
}

}  // namespace
}  // namespace hdit

extern "C" int hdit_copy_pieces(const hdit_copy_piece* pieces, int64_t n, void* stream) {
  using namespace hdit;
  if (n < 0 || (n > 0 && pieces == nullptr)) return set_error(HDIT_ERR_BAD_ARG, "bad piece list");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int64_t i = 0;
  while (i < n) {
    PieceTable tab;
    tab.n = 0;
    long long max_bytes = 0;
    for (; i < n && tab.n < kMaxPieces; ++i) {
      const hdit_copy_piece& d = pieces[i];
      if (d.n_outer < 0 || d.rows < 0 || d.row_bytes < 0) return set_error(HDIT_ERR_BAD_ARG, "negative piece extent");
      const long long bytes = static_cast<long long>(d.n_outer) * d.rows * d.row_bytes;
      if (bytes == 0) continue;
      if (d.n_outer > 1 && static_cast<long long>(d.n_outer) * d.rows > 0xffffffffLL)
        return set_error(HDIT_ERR_TOO_LARGE, "piece %lld: n_outer * rows exceeds 2^32", (long long)i);
      if (d.src == nullptr || d.dst == nullptr) return set_error(HDIT_ERR_BAD_ARG, "null pointer in piece %lld", (long long)i);
      Piece& pc = tab.p[tab.n++];
      pc.src = static_cast<const char*>(d.src);
      pc.dst = static_cast<char*>(d.dst);
      pc.n_outer = d.n_outer;
      pc.src_outer_pitch = d.src_outer_pitch;
      pc.dst_outer_pitch = d.dst_outer_pitch;
      pc.rows = d.rows;
      pc.src_pitch = d.src_pitch;
      pc.dst_pitch = d.dst_pitch;
      pc.row_bytes = d.row_bytes;
      pc.vec = pick_vec(d);
      pc.pad = 0;
      if (bytes > max_bytes) max_bytes = bytes;
    }
    if (tab.n == 0) continue;
    // Enough CTAs per piece to cover the largest one at 4 x 16 B per thread, capped so the
    // whole grid stays near a few waves of the 148 SMs.
    long long per_cta = static_cast<long long>(kCopyThreads) * 64;
    long long gy = (max_bytes + per_cta - 1) / per_cta;
    const long long cap = (148LL * 16 + tab.n - 1) / tab.n;
    if (gy > cap) gy = cap;
    if (gy < 1) gy = 1;
    dim3 grid(static_cast<unsigned>(tab.n), static_cast<unsigned>(gy));
    copy_pieces_kernel<<<grid, kCopyThreads, 0, st>>>(tab);
    HDIT_CUDA_OK(cudaGetLastError());
  }
  return HDIT_OK;
}

extern "C" int hdit_kv_scatter(void* kv_cache, const void* new_k, const void* new_v, int64_t batch, int64_t cache_tokens,
                               int64_t token_start, int64_t n_tokens, int64_t row_bytes, int64_t new_token_pitch,
                               int64_t new_batch_pitch, void* stream) {
  using namespace hdit;
  if (kv_cache == nullptr || new_k == nullptr || new_v == nullptr) return set_error(HDIT_ERR_BAD_ARG, "null pointer");
  if (batch < 0 || n_tokens < 0 || row_bytes < 0 || token_start < 0 || token_start + n_tokens > cache_tokens)
    return set_error(HDIT_ERR_SHAPE, "token range [%lld, %lld) outside the cache of %lld tokens",
                     (long long)token_start, (long long)(token_start + n_tokens), (long long)cache_tokens);
  hdit_copy_piece pc[2];
  for (int i = 0; i < 2; ++i) {
    pc[i].src = (i == 0) ? new_k : new_v;
    pc[i].dst = static_cast<char*>(kv_cache) + token_start * 2 * row_bytes + i * row_bytes;
    pc[i].n_outer = batch;
    pc[i].src_outer_pitch = new_batch_pitch;
    pc[i].dst_outer_pitch = cache_tokens * 2 * row_bytes;
    pc[i].rows = n_tokens;
    pc[i].src_pitch = new_token_pitch;
    pc[i].dst_pitch = 2 * row_bytes;
    pc[i].row_bytes = row_bytes;
  }
  return hdit_copy_pieces(pc, 2, stream);
}
