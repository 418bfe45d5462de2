// Pyramid K/V builder: levels 2/4/8 of the mean-pooled K and V in ONE pass over HBM.
//
// HBM-bound.  Algorithmic bytes per call: read K and V once (2*N*e), write levels 2, 4, 8
// (2*N*e*(1/2+1/4+1/8)) = 3.75*N*e with N = BH*S*D elements of e bytes.
//
// Each thread owns one 16-byte channel chunk of 8 consecutive tokens: it loads 8 x 16 B (rows 8j..8j+7,
// clamped to S-1 = replicate padding), forms level 2 (4 rows), level 4 (2 rows) and level 8 (1 row) in
// registers, rounding to the element type after every level exactly like a chain of means over a
// size-2 dimension does, and stores 7 x 16 B.  Consecutive threads take consecutive 16-byte chunks of
// the same token group, so every warp access covers whole 128-byte lines.
#include "psa_common.cuh"
#include "fwd.h"

namespace psa {

template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void pair_mean(const uint4& a, const uint4& b, uint4& o) {
  constexpr int N = Vec16<T>::N;
  const T* pa = reinterpret_cast<const T*>(&a);
  const T* pb = reinterpret_cast<const T*>(&b);
  T* po = reinterpret_cast<T*>(&o);
#pragma unroll
  for (int i = 0; i < N; ++i) po[i] = Elem<T>::from_f((Elem<T>::to_f(pa[i]) + Elem<T>::to_f(pb[i])) * 0.5f);
}

// grid.x: chunks of work items; grid.y: 0 = K, 1 = V.
template <typename T>
__global__ void __launch_bounds__(256) pyramid_kernel(const T* __restrict__ k, const T* __restrict__ v,
                                                      T* __restrict__ k2, T* __restrict__ k4, T* __restrict__ k8,
                                                      T* __restrict__ v2, T* __restrict__ v4, T* __restrict__ v8,
                                                      int64_t bh, int64_t S, int64_t n8, int cpr /*16B chunks per row*/) {
  const T* x = blockIdx.y ? v : k;
  T* x2 = blockIdx.y ? v2 : k2;
  T* x4 = blockIdx.y ? v4 : k4;
  T* x8 = blockIdx.y ? v8 : k8;
  const int64_t total = bh * n8 * cpr;
  const int64_t row_u4 = cpr;  // uint4 per token row
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(w % cpr);
    const int64_t g = w / cpr;  // token group index over all heads
    const int64_t head = g / n8;
    const int64_t j = g % n8;
    const uint4* src = reinterpret_cast<const uint4*>(x) + head * S * row_u4 + c;
    uint4 r[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      int64_t tok = j * 8 + t;
      tok = tok < S ? tok : S - 1;
      r[t] = __ldg(src + tok * row_u4);
    }
    uint4 a[4], b[2], d;
#pragma unroll
    for (int t = 0; t < 4; ++t) pair_mean<T>(r[2 * t], r[2 * t + 1], a[t]);
    pair_mean<T>(a[0], a[1], b[0]);
    pair_mean<T>(a[2], a[3], b[1]);
    pair_mean<T>(b[0], b[1], d);
    uint4* d2 = reinterpret_cast<uint4*>(x2) + (head * n8 * 4 + j * 4) * row_u4 + c;
    uint4* d4 = reinterpret_cast<uint4*>(x4) + (head * n8 * 2 + j * 2) * row_u4 + c;
    uint4* d8 = reinterpret_cast<uint4*>(x8) + (head * n8 + j) * row_u4 + c;
#pragma unroll
    for (int t = 0; t < 4; ++t) d2[t * row_u4] = a[t];
    d4[0] = b[0];
    d4[row_u4] = b[1];
    d8[0] = d;
  }
}

template <typename T>
static int launch_pyramid(const void* k, const void* v, void* k2, void* k4, void* k8, void* v2, void* v4, void* v8,
                          int64_t bh, int64_t S, int D, int block_n, cudaStream_t st) {
  const int64_t s_pad = cdiv64(S, block_n) * block_n;
  const int64_t n8 = s_pad / 8;
  const int cpr = D * (int)sizeof(T) / 16;
  const int64_t total = bh * n8 * cpr;
  int64_t blocks = cdiv64(total, 256);
  const int64_t cap = 148 * 16;  // a few resident CTAs per SM, grid-stride beyond that
  if (blocks > cap) blocks = cap;
  dim3 grid((unsigned)blocks, 2);
  pyramid_kernel<T><<<grid, 256, 0, st>>>((const T*)k, (const T*)v, (T*)k2, (T*)k4, (T*)k8, (T*)v2, (T*)v4, (T*)v8,
                                          bh, S, n8, cpr);
  PSA_CHECK_LAUNCH("psa_pyramid_kv");
  return PSA_OK;
}

}  // namespace psa

extern "C" int psa_pyramid_kv(const void* k, const void* v, void* k2, void* k4, void* k8, void* v2, void* v4,
                              void* v8, int64_t bh, int64_t seq, int head_dim, int block_n, int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(k && v && k2 && k4 && k8 && v2 && v4 && v8, PSA_ERR_ARG, "psa_pyramid_kv: null pointer");
  PSA_REQUIRE(bh > 0 && seq > 0, PSA_ERR_ARG, "psa_pyramid_kv: empty tensor (bh=%lld seq=%lld)", (long long)bh,
              (long long)seq);
  PSA_REQUIRE(block_n > 0 && block_n % 8 == 0, PSA_ERR_ARG, "psa_pyramid_kv: block_n=%d must be a multiple of 8", block_n);
  PSA_REQUIRE(head_dim > 0 && head_dim % 8 == 0, PSA_ERR_ARG, "psa_pyramid_kv: head_dim=%d must be a multiple of 8",
              head_dim);
  const void* ptrs[8] = {k, v, k2, k4, k8, v2, v4, v8};
  for (int i = 0; i < 8; ++i)
    PSA_REQUIRE(((uintptr_t)ptrs[i] & 15) == 0, PSA_ERR_ARG, "psa_pyramid_kv: pointer %d is not 16-byte aligned", i);
  cudaStream_t st = (cudaStream_t)stream;
  PSA_DISPATCH_DTYPE(dtype, T, return launch_pyramid<T>(k, v, k2, k4, k8, v2, v4, v8, bh, seq, head_dim, block_n, st));
  return PSA_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Tile-image variant for the tensor-core forward (16-bit element types).
//
// The forward gathers blocks of P = block_n/level pooled rows into 128-byte-swizzled shared-memory tiles.  Fetching a
// block from a row-major tensor needs one tensor-map TMA operation per 64-channel slab, and the TMA issue rate (about
// one operation per 100 cycles per SM) bounds tiles made of narrow blocks.  Here every level - level 1 included - is
// written in HBM exactly as its shared-memory image: groups of 8 rows, each group = [slab][8 rows][128 B] with the
// 16-byte chunks of a row XOR-ed by (row & 7).  A block then is one contiguous range of P*D*2 bytes and one linear
// bulk copy.  Algorithmic bytes: read K,V once (2 N e), write levels 1,2,4,8 (3.75 N e).
namespace psa {

template <typename T>
__device__ __forceinline__ void img_store(unsigned char* base, int64_t bh, int64_t groups, int slabs, int64_t row, int c, const uint4& val) {
  const int64_t g = row >> 3;
  const int r = (int)(row & 7);
  unsigned char* p = base + ((bh * groups + g) * slabs + (c >> 3)) * 1024 + r * 128 + (((c & 7) ^ r) << 4);
  *reinterpret_cast<uint4*>(p) = val;
}

template <typename T, bool ROPE>
__global__ void __launch_bounds__(256) pyramid_img_kernel(const RowSource k, const RowSource v, unsigned char* __restrict__ kimg,
                                                          unsigned char* __restrict__ vimg, ImgLevels L, int64_t bh, int64_t S, int64_t n8,
                                                          int cpr, const RopeTables rope) {
  const RowSource& x = blockIdx.y ? v : k;
  unsigned char* img = blockIdx.y ? vimg : kimg;
  const int slabs = cpr / 8;
  const int64_t total = bh * n8 * cpr;
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(w % cpr);
    const int64_t g = w / cpr;
    const int64_t head = g / n8;
    const int64_t j = g % n8;
    uint4 r[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      int64_t tok = j * 8 + t;
      tok = tok < S ? tok : S - 1;
      r[t] = (ROPE && blockIdx.y == 0) ? load_row_word<true>(x, rope, head, S, tok, cpr, c) : *row_word(x, head, S, tok, cpr, c);
    }
    uint4 a[4], b[2], d;
#pragma unroll
    for (int t = 0; t < 4; ++t) pair_mean<T>(r[2 * t], r[2 * t + 1], a[t]);
    pair_mean<T>(a[0], a[1], b[0]);
    pair_mean<T>(a[2], a[3], b[1]);
    pair_mean<T>(b[0], b[1], d);
#pragma unroll
    for (int t = 0; t < 8; ++t) img_store<T>(img + L.off[0], head, L.groups[0], slabs, j * 8 + t, c, r[t]);
#pragma unroll
    for (int t = 0; t < 4; ++t) img_store<T>(img + L.off[1], head, L.groups[1], slabs, j * 4 + t, c, a[t]);
    img_store<T>(img + L.off[2], head, L.groups[2], slabs, j * 2, c, b[0]);
    img_store<T>(img + L.off[2], head, L.groups[2], slabs, j * 2 + 1, c, b[1]);
    img_store<T>(img + L.off[3], head, L.groups[3], slabs, j, c, d);
  }
}

}  // namespace psa

extern "C" size_t psa_kv_image_bytes(int64_t bh, int64_t seq, int head_dim, int block_n) {
  if (bh <= 0 || seq <= 0 || (head_dim != 64 && head_dim != 128) || block_n < 64 || block_n % 64) return 0;
  psa::ImgLevels L = psa::make_img_levels(bh, seq, head_dim, block_n);
  return (size_t)(L.off[3] + bh * L.groups[3] * (head_dim / 64) * 1024);
}

namespace psa {
static int launch_pyramid_images(const RowSource& k, const RowSource& v, void* kimg, void* vimg, int64_t bh, int64_t seq, int head_dim,
                                 int block_n, int dtype, int max_blocks, cudaStream_t st, const RopeTables& rope = RopeTables{}) {
  const ImgLevels L = make_img_levels(bh, seq, head_dim, block_n);
  const int64_t s_pad = cdiv64(seq, block_n) * block_n;
  const int64_t n8 = s_pad / 8;
  const int cpr = head_dim * 2 / 16;
  int64_t blocks = cdiv64(bh * n8 * cpr, 256);
  const int64_t cap = max_blocks > 0 ? max_blocks : 148 * 16;
  if (blocks > cap) blocks = cap;
  dim3 grid((unsigned)blocks, 2);
  if (dtype == PSA_F16) {
    if (rope.a) pyramid_img_kernel<__half, true><<<grid, 256, 0, st>>>(k, v, (unsigned char*)kimg, (unsigned char*)vimg, L, bh, seq, n8, cpr, rope);
    else pyramid_img_kernel<__half, false><<<grid, 256, 0, st>>>(k, v, (unsigned char*)kimg, (unsigned char*)vimg, L, bh, seq, n8, cpr, rope);
  } else {
    if (rope.a) pyramid_img_kernel<__nv_bfloat16, true><<<grid, 256, 0, st>>>(k, v, (unsigned char*)kimg, (unsigned char*)vimg, L, bh, seq, n8, cpr, rope);
    else pyramid_img_kernel<__nv_bfloat16, false><<<grid, 256, 0, st>>>(k, v, (unsigned char*)kimg, (unsigned char*)vimg, L, bh, seq, n8, cpr, rope);
  }
  PSA_CHECK_LAUNCH("psa_pyramid_kv_images");
  return PSA_OK;
}
}  // namespace psa

extern "C" int psa_pyramid_kv_images(const void* k, const void* v, void* kimg, void* vimg, int64_t bh, int64_t seq, int head_dim,
                                     int block_n, int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(k && v && kimg && vimg, PSA_ERR_ARG, "psa_pyramid_kv_images: null pointer");
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "psa_pyramid_kv_images: 16-bit element types only");
  PSA_REQUIRE(psa_kv_image_bytes(bh, seq, head_dim, block_n) > 0, PSA_ERR_ARG,
              "psa_pyramid_kv_images: needs head_dim 64/128 and block_n a multiple of 64 (got %d, %d)", head_dim, block_n);
  // the swizzle phase of an image row depends only on its offset inside the image, so 16 bytes (bulk-copy source
  // alignment) is all the base needs
  PSA_REQUIRE((((uintptr_t)k | (uintptr_t)v | (uintptr_t)kimg | (uintptr_t)vimg) & 15) == 0, PSA_ERR_ARG,
              "psa_pyramid_kv_images: k, v and the images must be 16-byte aligned");
  return launch_pyramid_images(local_rows(k), local_rows(v), kimg, vimg, bh, seq, head_dim, block_n, dtype, 0, (cudaStream_t)stream);
}

extern "C" int psa_pyramid_kv_images_perm(const void* k, const void* v, const int32_t* perm, void* kimg, void* vimg, int64_t bh,
                                          int64_t seq, int head_dim, int block_n, int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(k && v && perm && kimg && vimg, PSA_ERR_ARG, "psa_pyramid_kv_images_perm: null pointer");
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "psa_pyramid_kv_images_perm: 16-bit element types only");
  PSA_REQUIRE(seq < ((int64_t)1 << 31), PSA_ERR_ARG, "psa_pyramid_kv_images_perm: seq=%lld does not fit the int32 order table",
              (long long)seq);
  PSA_REQUIRE(psa_kv_image_bytes(bh, seq, head_dim, block_n) > 0, PSA_ERR_ARG,
              "psa_pyramid_kv_images_perm: needs head_dim 64/128 and block_n a multiple of 64 (got %d, %d)", head_dim, block_n);
  PSA_REQUIRE((((uintptr_t)k | (uintptr_t)v | (uintptr_t)kimg | (uintptr_t)vimg) & 15) == 0, PSA_ERR_ARG,
              "psa_pyramid_kv_images_perm: k, v and the images must be 16-byte aligned");
  RowSource ks = local_rows(k), vs = local_rows(v);
  ks.perm = vs.perm = perm;
  return launch_pyramid_images(ks, vs, kimg, vimg, bh, seq, head_dim, block_n, dtype, 0, (cudaStream_t)stream);
}

extern "C" int psa_pyramid_kv_images_perm_rope(const void* k, const void* v, const int32_t* perm, const float* rope_a,
                                               const float* rope_b, int64_t rope_first, void* kimg, void* vimg, int64_t bh, int64_t seq,
                                               int head_dim, int block_n, int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(k && v && kimg && vimg && rope_a && rope_b, PSA_ERR_ARG, "psa_pyramid_kv_images_perm_rope: null pointer");
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "psa_pyramid_kv_images_perm_rope: 16-bit element types only");
  PSA_REQUIRE(seq < ((int64_t)1 << 31) && rope_first >= 0 && rope_first <= seq, PSA_ERR_ARG, "psa_pyramid_kv_images_perm_rope: bad shape");
  PSA_REQUIRE(psa_kv_image_bytes(bh, seq, head_dim, block_n) > 0, PSA_ERR_ARG,
              "psa_pyramid_kv_images_perm_rope: needs head_dim 64/128 and block_n a multiple of 64 (got %d, %d)", head_dim, block_n);
  PSA_REQUIRE((((uintptr_t)k | (uintptr_t)v | (uintptr_t)kimg | (uintptr_t)vimg | (uintptr_t)rope_a | (uintptr_t)rope_b) & 15) == 0,
              PSA_ERR_ARG, "psa_pyramid_kv_images_perm_rope: k, v, the images and the tables must be 16-byte aligned");
  RowSource ks = local_rows(k), vs = local_rows(v);
  ks.perm = vs.perm = perm;      // may be null: stored order
  const RopeTables rope = {rope_a, rope_b, rope_first, dtype == PSA_BF16};   // applied to the keys only
  return launch_pyramid_images(ks, vs, kimg, vimg, bh, seq, head_dim, block_n, dtype, 0, (cudaStream_t)stream, rope);
}

static int pyramid_kv_images_tm(const void* k, const void* v, const int32_t* perm, const float* rope_a, const float* rope_b,
                                int64_t rope_first, void* kimg, void* vimg, int heads, int64_t seq, int head_dim, int block_n,
                                int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(k && v && kimg && vimg, PSA_ERR_ARG, "psa_pyramid_kv_images_tm: null pointer");
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "psa_pyramid_kv_images_tm: 16-bit element types only");
  PSA_REQUIRE(heads > 0 && seq > 0 && seq < ((int64_t)1 << 31), PSA_ERR_ARG, "psa_pyramid_kv_images_tm: bad shape");
  PSA_REQUIRE(psa_kv_image_bytes(heads, seq, head_dim, block_n) > 0, PSA_ERR_ARG,
              "psa_pyramid_kv_images_tm: needs head_dim 64/128 and block_n a multiple of 64 (got %d, %d)", head_dim, block_n);
  PSA_REQUIRE((((uintptr_t)k | (uintptr_t)v | (uintptr_t)kimg | (uintptr_t)vimg) & 15) == 0, PSA_ERR_ARG,
              "psa_pyramid_kv_images_tm: k, v and the images must be 16-byte aligned");
  RowSource ks = {}, vs = {};
  ks.peer[0] = k; vs.peer[0] = v;
  ks.n_peers = vs.n_peers = 1;
  ks.heads_total = vs.heads_total = heads;
  ks.tokens_per_rank = vs.tokens_per_rank = seq;
  ks.perm = vs.perm = perm;
  const RopeTables rope = {rope_a, rope_b, rope_first, dtype == PSA_BF16};   // applied to the keys only
  return launch_pyramid_images(ks, vs, kimg, vimg, heads, seq, head_dim, block_n, dtype, 0, (cudaStream_t)stream, rope);
}

extern "C" int psa_pyramid_kv_images_tm(const void* k, const void* v, const int32_t* perm, void* kimg, void* vimg, int heads,
                                        int64_t seq, int head_dim, int block_n, int dtype, void* stream) {
  return pyramid_kv_images_tm(k, v, perm, nullptr, nullptr, 0, kimg, vimg, heads, seq, head_dim, block_n, dtype, stream);
}

extern "C" int psa_pyramid_kv_images_tm_rope(const void* k, const void* v, const int32_t* perm, const float* rope_a,
                                             const float* rope_b, int64_t rope_first, void* kimg, void* vimg, int heads, int64_t seq,
                                             int head_dim, int block_n, int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(rope_a && rope_b && rope_first >= 0 && rope_first <= seq, PSA_ERR_ARG, "psa_pyramid_kv_images_tm_rope: bad rotary tables");
  PSA_REQUIRE((((uintptr_t)rope_a | (uintptr_t)rope_b) & 15) == 0, PSA_ERR_ARG,
              "psa_pyramid_kv_images_tm_rope: tables must be 16-byte aligned");
  return pyramid_kv_images_tm(k, v, perm, rope_a, rope_b, rope_first, kimg, vimg, heads, seq, head_dim, block_n, dtype, stream);
}

extern "C" int psa_pyramid_kv_images_peers(const void* const* peer_k, const void* const* peer_v, int n_peers, int64_t tokens_per_rank,
                                           int heads_total, int head0, void* kimg, void* vimg, int64_t heads_local, int head_dim,
                                           int block_n, int dtype, int max_blocks, void* stream) {
  using namespace psa;
  PSA_REQUIRE(peer_k && peer_v && kimg && vimg, PSA_ERR_ARG, "psa_pyramid_kv_images_peers: null pointer");
  PSA_REQUIRE(n_peers >= 1 && n_peers <= kMaxPeers, PSA_ERR_ARG, "psa_pyramid_kv_images_peers: n_peers=%d (1..%d)", n_peers, kMaxPeers);
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "psa_pyramid_kv_images_peers: 16-bit element types only");
  PSA_REQUIRE(heads_local > 0 && head0 >= 0 && head0 + heads_local <= heads_total && tokens_per_rank > 0 && max_blocks >= 0,
              PSA_ERR_ARG, "psa_pyramid_kv_images_peers: bad head range, shard size or grid cap");
  const int64_t seq = tokens_per_rank * n_peers;
  PSA_REQUIRE(psa_kv_image_bytes(heads_local, seq, head_dim, block_n) > 0, PSA_ERR_ARG,
              "psa_pyramid_kv_images_peers: needs head_dim 64/128 and block_n a multiple of 64 (got %d, %d)", head_dim, block_n);
  PSA_REQUIRE((((uintptr_t)kimg | (uintptr_t)vimg) & 15) == 0, PSA_ERR_ARG, "psa_pyramid_kv_images_peers: images must be 16-byte aligned");
  RowSource k = {}, v = {};
  for (int i = 0; i < n_peers; ++i) {
    PSA_REQUIRE(peer_k[i] && peer_v[i] && (((uintptr_t)peer_k[i] | (uintptr_t)peer_v[i]) & 15) == 0, PSA_ERR_ARG,
                "psa_pyramid_kv_images_peers: peer %d pointer", i);
    k.peer[i] = peer_k[i];
    v.peer[i] = peer_v[i];
  }
  k.n_peers = v.n_peers = n_peers;
  k.heads_total = v.heads_total = heads_total;
  k.head0 = v.head0 = head0;
  k.tokens_per_rank = v.tokens_per_rank = tokens_per_rank;
  return launch_pyramid_images(k, v, kimg, vimg, heads_local, seq, head_dim, block_n, dtype, max_blocks, (cudaStream_t)stream);
}
