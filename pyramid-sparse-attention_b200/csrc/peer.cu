// Peer-memory exchange for head-sharded runs on the GPUs of one node.
//
// A sequence-parallel model keeps activations as [tokens/P][heads][D] per rank; the attention layer wants
// [heads/P][tokens][D].  Instead of an all-to-all collective, every rank maps its peers' buffers (CUDA IPC) and
//   * pulls the rows of its heads straight out of the peers' q/k/v buffers (plain 16-byte loads over NVLink), and
//   * lets the attention kernel store its output rows straight into the owning peer's buffer (plain stores).
// Nothing here waits on another GPU from inside a kernel: the host orders the steps (a barrier before the pull, one
// after the forward), so no kernel ever spins on a flag a peer writes.  No TMA touches peer memory.
//
// HBM/NVLink-bound byte movement: every element crosses NVLink at most once.
#include <cstring>

#include "psa_common.cuh"
#include "fwd.h"

namespace psa {

struct PullArgs {
  const uint4* src[kMaxPeers];   // peer buffers [tokens_per_rank][heads_total][row16] in 16-byte units
  uint4* dst;                    // [heads_local][tokens][row16]
  int n_peers, heads_total, head0, heads_local, row16;
  int64_t tokens_per_rank, tokens, rot;   // rot: token offset at which this rank starts its walk over the peers
};

// One 16-byte word per thread and load, eight independent loads in flight per thread (peer loads are latency-bound:
// a few microseconds each).  Consecutive threads read consecutive words of a token's rows (all local heads).  The grid is kept
// small when the copy runs under compute kernels: a resident copy CTA keeps a register-hungry compute CTA off its SM.
constexpr int kPullUnroll = 8;
__global__ void __launch_bounds__(512) pull_heads_kernel(const PullArgs a) {
  const int64_t total = (int64_t)a.heads_local * a.tokens * a.row16;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t per_token = (int64_t)a.row16 * a.heads_local;
  int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; w + (kPullUnroll - 1) * stride < total; w += kPullUnroll * stride) {
    uint4 v[kPullUnroll];
    int64_t d[kPullUnroll];
#pragma unroll
    for (int u = 0; u < kPullUnroll; ++u) {
      const int64_t i = w + u * stride;
      // token-major walk: the rows of all local heads of one token are one contiguous range of the peer's buffer
      const int64_t tw = i / per_token;
      const int rem = (int)(i - tw * per_token);
      const int h = rem / a.row16;
      const int c = rem - h * a.row16;
      int64_t t = tw + a.rot;
      t = t >= a.tokens ? t - a.tokens : t;
      const int owner = (int)(t / a.tokens_per_rank);
      const int64_t local = t - owner * a.tokens_per_rank;
      v[u] = a.src[owner][(local * a.heads_total + a.head0 + h) * a.row16 + c];
      d[u] = (h * a.tokens + t) * a.row16 + c;
    }
#pragma unroll
    for (int u = 0; u < kPullUnroll; ++u) a.dst[d[u]] = v[u];
  }
  for (; w < total; w += stride) {
    const int64_t tw = w / per_token;
    const int rem = (int)(w - tw * per_token);
    const int h = rem / a.row16;
    const int c = rem - h * a.row16;
    int64_t t = tw + a.rot;
    t = t >= a.tokens ? t - a.tokens : t;
    const int owner = (int)(t / a.tokens_per_rank);
    const int64_t local = t - owner * a.tokens_per_rank;
    a.dst[(h * a.tokens + t) * a.row16 + c] = a.src[owner][(local * a.heads_total + a.head0 + h) * a.row16 + c];
  }
}

// The opposite direction: every rank sends the rows of its own tokens to the ranks that own the heads.  Reads are one
// sequential pass over the local buffer; the remote side sees posted 16-byte stores that fill whole 256-byte rows.
struct PushArgs {
  const uint4* src;          // [tokens_per_rank][heads_total][row16]
  uint4* dst[kMaxPeers];     // peer r: [heads_per_rank][tokens][row16], holding heads [r*heads_per_rank, ...)
  int n_peers, heads_total, heads_per_rank, row16, self_rank;
  int64_t tokens_per_rank, tokens;
};

__global__ void __launch_bounds__(512) push_heads_kernel(const PushArgs a) {
  const int64_t per_token = (int64_t)a.heads_total * a.row16;
  const int64_t total = a.tokens_per_rank * per_token;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t t0 = (int64_t)a.self_rank * a.tokens_per_rank;
  int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; w + (kPullUnroll - 1) * stride < total; w += kPullUnroll * stride) {
    uint4 v[kPullUnroll];
#pragma unroll
    for (int u = 0; u < kPullUnroll; ++u) v[u] = a.src[w + u * stride];
#pragma unroll
    for (int u = 0; u < kPullUnroll; ++u) {
      const int64_t i = w + u * stride;
      const int64_t t = i / per_token;
      const int rem = (int)(i - t * per_token);
      const int h = rem / a.row16, c = rem - h * a.row16;
      const int owner = h / a.heads_per_rank, hl = h - owner * a.heads_per_rank;
      a.dst[owner][((int64_t)hl * a.tokens + t0 + t) * a.row16 + c] = v[u];
    }
  }
  for (; w < total; w += stride) {
    const int64_t t = w / per_token;
    const int rem = (int)(w - t * per_token);
    const int h = rem / a.row16, c = rem - h * a.row16;
    const int owner = h / a.heads_per_rank, hl = h - owner * a.heads_per_rank;
    a.dst[owner][((int64_t)hl * a.tokens + t0 + t) * a.row16 + c] = a.src[w];
  }
}

// Sampled rows only (what the block-score stage reads): row i of head h's compacted sample matrix is token
// min((ic / keep) * block + idx[h][ic % keep], seq - 1), ic = min(i, n_valid - 1); the rank that owns that token stores
// it into the head owner's sample matrix [heads_per_rank][n_out][row16].
struct PushSampleArgs {
  const uint4* src;          // [tokens_per_rank][heads_total][row16]
  const int32_t* idx;        // [heads_total][keep]
  uint4* dst[kMaxPeers];
  int n_peers, heads_total, heads_per_rank, row16, self_rank, block, keep, n_valid, n_out;
  int64_t tokens_per_rank, seq;
};

__global__ void __launch_bounds__(256) push_samples_kernel(const PushSampleArgs a) {
  const int64_t total = (int64_t)a.heads_total * a.n_out * a.row16;
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(w % a.row16);
    const int64_t hi = w / a.row16;
    const int i = (int)(hi % a.n_out), h = (int)(hi / a.n_out);
    const int ic = i < a.n_valid ? i : a.n_valid - 1;
    int64_t tok = (int64_t)(ic / a.keep) * a.block + a.idx[h * a.keep + (ic % a.keep)];
    tok = tok < a.seq ? tok : a.seq - 1;
    const int64_t local = tok - (int64_t)a.self_rank * a.tokens_per_rank;
    if (local < 0 || local >= a.tokens_per_rank) continue;
    const int owner = h / a.heads_per_rank, hl = h - owner * a.heads_per_rank;
    a.dst[owner][((int64_t)hl * a.n_out + i) * a.row16 + c] = a.src[(local * a.heads_total + h) * a.row16 + c];
  }
}

}  // namespace psa

extern "C" int psa_push_samples(const void* src, const int32_t* idx, void* const* peer_dst, int n_peers, int64_t tokens_per_rank,
                                int heads_total, int head_dim, int elem_bytes, int block, int keep, int64_t n_valid, int64_t n_out,
                                int self_rank, void* stream) {
  using namespace psa;
  PSA_REQUIRE(src && idx && peer_dst, PSA_ERR_ARG, "psa_push_samples: null pointer");
  PSA_REQUIRE(n_peers >= 1 && n_peers <= kMaxPeers && self_rank >= 0 && self_rank < n_peers, PSA_ERR_ARG,
              "psa_push_samples: rank %d of %d (at most %d)", self_rank, n_peers, kMaxPeers);
  PSA_REQUIRE(tokens_per_rank > 0 && heads_total > 0 && heads_total % n_peers == 0, PSA_ERR_ARG,
              "psa_push_samples: %d heads do not divide over %d ranks", heads_total, n_peers);
  PSA_REQUIRE(block > 0 && keep > 0 && n_valid > 0 && n_out >= n_valid && n_out < (1ll << 31), PSA_ERR_ARG,
              "psa_push_samples: bad sample geometry");
  PSA_REQUIRE(head_dim > 0 && (elem_bytes == 2 || elem_bytes == 4) && (head_dim * elem_bytes) % 16 == 0, PSA_ERR_ARG,
              "psa_push_samples: rows must be a multiple of 16 bytes");
  PushSampleArgs a;
  a.src = (const uint4*)src; a.idx = idx;
  for (int i = 0; i < kMaxPeers; ++i) {
    a.dst[i] = i < n_peers ? (uint4*)peer_dst[i] : nullptr;
    if (i < n_peers) PSA_REQUIRE(peer_dst[i] && ((uintptr_t)peer_dst[i] & 15) == 0, PSA_ERR_ARG, "psa_push_samples: peer %d pointer", i);
  }
  a.n_peers = n_peers; a.heads_total = heads_total; a.heads_per_rank = heads_total / n_peers;
  a.row16 = head_dim * elem_bytes / 16; a.self_rank = self_rank; a.block = block; a.keep = keep;
  a.n_valid = (int)n_valid; a.n_out = (int)n_out;
  a.tokens_per_rank = tokens_per_rank; a.seq = tokens_per_rank * n_peers;
  const int64_t total = (int64_t)heads_total * n_out * a.row16;
  int64_t blocks = cdiv64(total, 256 * 4);
  if (blocks > 148 * 8) blocks = 148 * 8;
  push_samples_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(a);
  PSA_CHECK_LAUNCH("psa_push_samples");
  return PSA_OK;
}

extern "C" int psa_push_heads(const void* src, void* const* peer_dst, int n_peers, int64_t tokens_per_rank, int heads_total,
                              int head_dim, int elem_bytes, int self_rank, int max_blocks, void* stream) {
  using namespace psa;
  PSA_REQUIRE(src && peer_dst, PSA_ERR_ARG, "psa_push_heads: null pointer");
  PSA_REQUIRE(n_peers >= 1 && n_peers <= kMaxPeers && self_rank >= 0 && self_rank < n_peers, PSA_ERR_ARG,
              "psa_push_heads: rank %d of %d (at most %d)", self_rank, n_peers, kMaxPeers);
  PSA_REQUIRE(tokens_per_rank > 0 && heads_total > 0 && heads_total % n_peers == 0, PSA_ERR_ARG,
              "psa_push_heads: %d heads do not divide over %d ranks", heads_total, n_peers);
  PSA_REQUIRE(head_dim > 0 && (elem_bytes == 2 || elem_bytes == 4) && (head_dim * elem_bytes) % 16 == 0 && max_blocks >= 0, PSA_ERR_ARG,
              "psa_push_heads: rows must be a multiple of 16 bytes");
  PSA_REQUIRE(((uintptr_t)src & 15) == 0, PSA_ERR_ARG, "psa_push_heads: src must be 16-byte aligned");
  PushArgs a;
  a.src = (const uint4*)src;
  for (int i = 0; i < kMaxPeers; ++i) {
    a.dst[i] = i < n_peers ? (uint4*)peer_dst[i] : nullptr;
    if (i < n_peers) PSA_REQUIRE(peer_dst[i] && ((uintptr_t)peer_dst[i] & 15) == 0, PSA_ERR_ARG, "psa_push_heads: peer %d pointer", i);
  }
  a.n_peers = n_peers; a.heads_total = heads_total; a.heads_per_rank = heads_total / n_peers;
  a.row16 = head_dim * elem_bytes / 16; a.self_rank = self_rank;
  a.tokens_per_rank = tokens_per_rank; a.tokens = tokens_per_rank * n_peers;
  const int64_t total = tokens_per_rank * heads_total * a.row16;
  int64_t blocks = cdiv64(total, 512 * kPullUnroll);
  const int64_t cap = max_blocks > 0 ? max_blocks : 148 * 2;
  if (blocks > cap) blocks = cap;
  push_heads_kernel<<<(unsigned)blocks, 512, 0, (cudaStream_t)stream>>>(a);
  PSA_CHECK_LAUNCH("psa_push_heads");
  return PSA_OK;
}

extern "C" int psa_peer_alloc(size_t bytes, void** ptr, void* handle64) {
  using namespace psa;
  PSA_REQUIRE(ptr && handle64 && bytes > 0, PSA_ERR_ARG, "psa_peer_alloc: bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_peer_alloc: cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    PSA_REQUIRE(false, PSA_ERR_CUDA, "psa_peer_alloc: cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
  }
  memcpy(handle64, &h, 64);
  *ptr = p;
  return PSA_OK;
}

extern "C" int psa_peer_open(const void* handle64, void** ptr) {
  using namespace psa;
  PSA_REQUIRE(ptr && handle64, PSA_ERR_ARG, "psa_peer_open: bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_peer_open: cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
  *ptr = p;
  return PSA_OK;
}

extern "C" int psa_peer_close(void* ptr) {
  using namespace psa;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_peer_close: %s", cudaGetErrorString(e));
  return PSA_OK;
}

extern "C" int psa_peer_free(void* ptr) {
  using namespace psa;
  cudaError_t e = cudaFree(ptr);
  PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_peer_free: %s", cudaGetErrorString(e));
  return PSA_OK;
}

extern "C" int psa_pull_heads(const void* const* peer_src, int n_peers, void* dst, int64_t tokens_per_rank, int heads_total,
                              int head0, int heads_local, int head_dim, int elem_bytes, int max_blocks, int self_rank, void* stream) {
  using namespace psa;
  PSA_REQUIRE(peer_src && dst, PSA_ERR_ARG, "psa_pull_heads: null pointer");
  PSA_REQUIRE(n_peers >= 1 && n_peers <= kMaxPeers, PSA_ERR_ARG, "psa_pull_heads: n_peers=%d (1..%d)", n_peers, kMaxPeers);
  PSA_REQUIRE(tokens_per_rank > 0 && heads_total > 0 && head0 >= 0 && heads_local > 0 && head0 + heads_local <= heads_total,
              PSA_ERR_ARG, "psa_pull_heads: bad head range [%d, %d) of %d", head0, head0 + heads_local, heads_total);
  PSA_REQUIRE(head_dim > 0 && (elem_bytes == 2 || elem_bytes == 4) && (head_dim * elem_bytes) % 16 == 0, PSA_ERR_ARG,
              "psa_pull_heads: rows must be a multiple of 16 bytes");
  PullArgs a;
  for (int i = 0; i < kMaxPeers; ++i) {
    a.src[i] = i < n_peers ? (const uint4*)peer_src[i] : nullptr;
    if (i < n_peers) PSA_REQUIRE(peer_src[i] && ((uintptr_t)peer_src[i] & 15) == 0, PSA_ERR_ARG, "psa_pull_heads: peer %d pointer", i);
  }
  PSA_REQUIRE(((uintptr_t)dst & 15) == 0, PSA_ERR_ARG, "psa_pull_heads: dst must be 16-byte aligned");
  a.dst = (uint4*)dst;
  a.n_peers = n_peers; a.heads_total = heads_total; a.head0 = head0; a.heads_local = heads_local;
  a.row16 = head_dim * elem_bytes / 16;
  PSA_REQUIRE(self_rank >= 0 && self_rank < n_peers, PSA_ERR_ARG, "psa_pull_heads: self_rank=%d of %d", self_rank, n_peers);
  a.tokens_per_rank = tokens_per_rank; a.tokens = tokens_per_rank * n_peers;
  a.rot = (int64_t)((self_rank + 1) % n_peers) * tokens_per_rank;
  const int64_t total = (int64_t)heads_local * a.tokens * a.row16;
  PSA_REQUIRE(max_blocks >= 0, PSA_ERR_ARG, "psa_pull_heads: max_blocks=%d", max_blocks);
  int64_t blocks = cdiv64(total, 512 * kPullUnroll);
  const int64_t cap = max_blocks > 0 ? max_blocks : 148 * 2;
  if (blocks > cap) blocks = cap;
  pull_heads_kernel<<<(unsigned)blocks, 512, 0, (cudaStream_t)stream>>>(a);
  PSA_CHECK_LAUNCH("psa_pull_heads");
  return PSA_OK;
}
