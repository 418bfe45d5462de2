// Antidiagonal block-importance estimate of the causal (vision-language) call site.
//
// Tokens are grouped by `stride`; the logit of (query group i, key group j) is the sum of the stride antidiagonal dot
// products q[i*stride + stride-1-s] . k[j*stride + s], i.e. ONE dense GEMM of the two [n, stride*D] matrices whose rows
// are the groups (the query side with its tokens in reverse order).  Neither matrix is materialised: a K-chunk of 64
// channels of a group row is 128 contiguous bytes of one token of q or k.  Then a row softmax (causal: groups j <= i)
// and the sum of the probabilities over (block/stride x block/stride) cells give the mass per (query block, key block).
//
// Lengths that are a multiple of the stride take the tcgen05 route (antidiag_tc.cu: GEMM with a partial softmax in its
// epilogue + a combine kernel, no logits in HBM).  Other lengths run the two kernels of this file:
// Kernel 1, warp-level mma.sync: 128x128 logit
// tiles, 8 warps of 32x64, K streamed in chunks of 64 through registers into padded shared-memory tiles; it writes the
// logits as fp32, already multiplied by log2(e)/sqrt(D)/stride, and skips the tiles above the diagonal when causal.
// Kernel 2 (HBM-bound: reads the logits once per pass): one CTA per query block, a warp per group row: maximum, sum
// of exp2, then the cell sums, accumulated per warp in shared memory in a fixed order (deterministic).
#include "mma_sync.cuh"

namespace psa {
bool antidiag_tc_supported(int64_t seq, int head_dim, int stride, int n, int dtype);
int launch_antidiag_tc(const void* q, const void* k, void* out, float* scratch, int64_t bh, int64_t seq, int head_dim, int stride, int n,
                       int n_valid, int rb, int nb, int causal, float scale_log2, int dtype, int32_t* status, cudaStream_t st);
namespace {

constexpr int kTile = 128;       // groups per CTA tile, both ways
constexpr int kBK = 64;          // channels per K-chunk
constexpr int kRowHalves = 72;   // shared-memory row pitch in 16-bit elements (64 + 8: conflict-free fragment loads)

struct AdParams {
  int64_t seq;      // valid tokens
  int n;            // groups of the padded length
  int stride, D;
  int causal;
  float scale_log2;
};

// 16-byte word `c` (0..7) of K-chunk `kc` of group row `g`: query side reads its tokens in reverse order.
template <bool QUERY>
__device__ __forceinline__ uint4 load_chunk_word(const uint4* __restrict__ base, const AdParams& p, int g, int kc, int c) {
  const int chunks_per_token = p.D / kBK;
  const int s = kc / chunks_per_token, d0 = (kc - s * chunks_per_token) * kBK;
  const int64_t tok = (int64_t)g * p.stride + (QUERY ? p.stride - 1 - s : s);
  if (g >= p.n || tok >= p.seq) return make_uint4(0u, 0u, 0u, 0u);
  return base[(tok * p.D + d0) / 8 + c];
}

template <typename T>
__global__ void __launch_bounds__(256) antidiag_logits_kernel(const T* __restrict__ q, const T* __restrict__ k, float* __restrict__ logits,
                                                             AdParams p) {
  const int jt = blockIdx.x, it = blockIdx.y;
  if (p.causal && jt > it) return;
  const int64_t bh = blockIdx.z;
  __shared__ __align__(16) unsigned short As[kTile * kRowHalves];
  __shared__ __align__(16) unsigned short Bs[kTile * kRowHalves];
  const uint4* qb = reinterpret_cast<const uint4*>(q + bh * p.seq * p.D);
  const uint4* kb = reinterpret_cast<const uint4*>(k + bh * p.seq * p.D);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int wm = (warp & 3) * 32, wn = (warp >> 2) * 64;   // warp tile origin inside the CTA tile
  const int i0 = it * kTile, j0 = jt * kTile;

  float acc[2][8][4];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;

  // each thread moves 4 words of A and 4 of B per chunk: word w = tid + 256*x -> row w / 8, word-in-row w % 8
  uint4 ra[4], rb[4];
  const int n_chunks = p.stride * p.D / kBK;
#pragma unroll
  for (int x = 0; x < 4; ++x) {
    const int w = tid + 256 * x;
    ra[x] = load_chunk_word<true>(qb, p, i0 + (w >> 3), 0, w & 7);
    rb[x] = load_chunk_word<false>(kb, p, j0 + (w >> 3), 0, w & 7);
  }
  for (int kc = 0; kc < n_chunks; ++kc) {
    __syncthreads();   // the previous chunk's fragments have been read
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int w = tid + 256 * x;
      *reinterpret_cast<uint4*>(&As[(w >> 3) * kRowHalves + (w & 7) * 8]) = ra[x];
      *reinterpret_cast<uint4*>(&Bs[(w >> 3) * kRowHalves + (w & 7) * 8]) = rb[x];
    }
    __syncthreads();
    if (kc + 1 < n_chunks) {
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int w = tid + 256 * x;
        ra[x] = load_chunk_word<true>(qb, p, i0 + (w >> 3), kc + 1, w & 7);
        rb[x] = load_chunk_word<false>(kb, p, j0 + (w >> 3), kc + 1, w & 7);
      }
    }
#pragma unroll
    for (int ks = 0; ks < kBK; ks += 16) {
      uint32_t af[2][4];
#pragma unroll
      for (int a = 0; a < 2; ++a) {
        const unsigned short* r0 = &As[(wm + a * 16 + g) * kRowHalves + ks + tig * 2];
        const unsigned short* r1 = r0 + 8 * kRowHalves;
        af[a][0] = *reinterpret_cast<const uint32_t*>(r0);
        af[a][1] = *reinterpret_cast<const uint32_t*>(r1);
        af[a][2] = *reinterpret_cast<const uint32_t*>(r0 + 8);
        af[a][3] = *reinterpret_cast<const uint32_t*>(r1 + 8);
      }
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        const unsigned short* c0 = &Bs[(wn + b * 8 + g) * kRowHalves + ks + tig * 2];
        uint32_t bf[2];
        bf[0] = *reinterpret_cast<const uint32_t*>(c0);
        bf[1] = *reinterpret_cast<const uint32_t*>(c0 + 8);
        MmaOp<T>::run(acc[0][b], af[0], bf);
        MmaOp<T>::run(acc[1][b], af[1], bf);
      }
    }
  }
  float* out = logits + bh * (int64_t)p.n * p.n;
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const int col = j0 + wn + b * 8 + tig * 2;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = i0 + wm + a * 16 + g + h * 8;
        if (row < p.n && col < p.n) {   // n is even (a multiple of block/stride >= 2), so col + 1 < n as well
          float2 v = make_float2(acc[a][b][h * 2] * p.scale_log2, acc[a][b][h * 2 + 1] * p.scale_log2);
          *reinterpret_cast<float2*>(&out[(int64_t)row * p.n + col]) = v;
        }
      }
    }
}

// One CTA per query block; rb = groups per block (power of two, 2..32).  part: [8 warps][n / rb] floats.
template <typename T>
__global__ void __launch_bounds__(256) antidiag_softmax_cells_kernel(const float* __restrict__ logits, T* __restrict__ out, int n,
                                                                    int n_valid, int rb, int nb, int causal) {
  extern __shared__ float part[];
  const int qb = blockIdx.x;
  const int64_t bh = blockIdx.y;
  const int nkb = n / rb;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < 8 * nkb; e += blockDim.x) part[e] = 0.f;
  __syncthreads();
  float* mine = part + warp * nkb;
  for (int r = warp; r < rb; r += 8) {
    const int i = qb * rb + r;
    if (i >= n_valid) continue;   // groups without a valid query token contribute nothing
    const int ncols = causal ? i + 1 : n;
    const float* x = logits + (bh * n + i) * (int64_t)n;
    float m = -INFINITY;
    for (int j = lane; j < ncols; j += 32) m = fmaxf(m, x[j]);
    for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    float l = 0.f;
    for (int j = lane; j < ncols; j += 32) l += exp2f(x[j] - m);
    for (int off = 16; off; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
    const float inv = 1.0f / l;
    const int span = (ncols + 31) & ~31;
    for (int j = lane; j < span; j += 32) {
      float pj = j < ncols ? exp2f(x[j] - m) * inv : 0.f;
      for (int off = 1; off < rb; off <<= 1) pj += __shfl_xor_sync(0xffffffffu, pj, off);
      if ((lane & (rb - 1)) == 0 && j < n) mine[j / rb] += pj;
    }
    __syncwarp();
  }
  __syncthreads();
  T* dst = out + (bh * nb + qb) * (int64_t)nb;
  for (int c = threadIdx.x; c < nb; c += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += part[w * nkb + c];
    dst[c] = Elem<T>::from_f(s);
  }
}

struct AdDims {
  int64_t padded;
  int n, n_valid, rb, nb;
};

int make_dims(AdDims& d, int64_t seq, int head_dim, int block_size, int stride, int chunk_size) {
  PSA_REQUIRE(seq > 0 && seq < ((int64_t)1 << 30), PSA_ERR_ARG, "antidiagonal estimate: seq=%lld out of range", (long long)seq);
  PSA_REQUIRE(head_dim == 64 || head_dim == 128, PSA_ERR_ARG, "antidiagonal estimate: head_dim=%d (64/128)", head_dim);
  PSA_REQUIRE(stride >= 1 && block_size > 0 && block_size % stride == 0, PSA_ERR_ARG,
              "antidiagonal estimate: block_size=%d must be a multiple of stride=%d", block_size, stride);
  const int rb = block_size / stride;
  PSA_REQUIRE(rb >= 2 && rb <= 32 && (rb & (rb - 1)) == 0, PSA_ERR_UNSUPPORTED,
              "antidiagonal estimate: block_size/stride=%d must be a power of two in 2..32", rb);
  PSA_REQUIRE(chunk_size > 0 && chunk_size % block_size == 0, PSA_ERR_ARG,
              "antidiagonal estimate: chunk_size=%d must be a multiple of block_size=%d", chunk_size, block_size);
  d.padded = cdiv64(seq, chunk_size) * chunk_size;
  d.n = (int)(d.padded / stride);
  d.n_valid = (int)cdiv64(seq, stride);
  d.rb = rb;
  d.nb = (int)cdiv64(seq, block_size);
  PSA_REQUIRE(d.n / rb <= 1024, PSA_ERR_UNSUPPORTED, "antidiagonal estimate: %d key blocks (at most 1024)", d.n / rb);
  return PSA_OK;
}

}  // namespace
}  // namespace psa

// bytes either route needs: the fp32 logits (mma.sync route), or per row one maximum per column tile and one sum per key
// block of whole tiles (tcgen05 route)
static size_t antidiag_scratch_need(int64_t bh, const psa::AdDims& d) {
  const size_t logits = (size_t)bh * d.n * d.n * sizeof(float);
  const size_t tiles = (size_t)(d.n + 127) / 128;
  const size_t partial = (size_t)bh * d.n * tiles * (1 + 128 / d.rb) * sizeof(float);
  return logits > partial ? logits : partial;
}

extern "C" size_t psa_antidiag_scratch_bytes(int64_t bh, int64_t seq, int head_dim, int block_size, int stride, int chunk_size) {
  psa::AdDims d;
  if (bh <= 0 || psa::make_dims(d, seq, head_dim, block_size, stride, chunk_size) != PSA_OK) return 0;
  return antidiag_scratch_need(bh, d);
}

extern "C" int psa_antidiag_scores(const void* q, const void* k, void* out, void* scratch, size_t scratch_bytes, int64_t bh,
                                   int64_t seq, int head_dim, int block_size, int stride, int chunk_size, int causal, int dtype,
                                   void* stream) {
  return psa_antidiag_scores_impl(q, k, out, scratch, scratch_bytes, bh, seq, head_dim, block_size, stride, chunk_size, causal, dtype,
                                  0, nullptr, stream);
}

extern "C" int psa_antidiag_scores_impl(const void* q, const void* k, void* out, void* scratch, size_t scratch_bytes, int64_t bh,
                                        int64_t seq, int head_dim, int block_size, int stride, int chunk_size, int causal, int dtype,
                                        int impl, int32_t* status, void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && k && out && scratch, PSA_ERR_ARG, "psa_antidiag_scores: null pointer");
  PSA_REQUIRE(impl == 0 || impl == 2 || impl == 3, PSA_ERR_ARG, "psa_antidiag_scores: impl=%d (0 pick, 2 tcgen05, 3 mma.sync)", impl);
  PSA_REQUIRE(bh > 0 && bh < 65536, PSA_ERR_ARG, "psa_antidiag_scores: bh=%lld out of range", (long long)bh);
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "psa_antidiag_scores: f16/bf16 only");
  PSA_REQUIRE((((uintptr_t)q | (uintptr_t)k | (uintptr_t)scratch) & 15) == 0, PSA_ERR_ARG,
              "psa_antidiag_scores: q, k and scratch must be 16-byte aligned");
  AdDims d;
  int rc = make_dims(d, seq, head_dim, block_size, stride, chunk_size);
  if (rc != PSA_OK) return rc;
  PSA_REQUIRE(scratch_bytes >= antidiag_scratch_need(bh, d), PSA_ERR_ARG, "psa_antidiag_scores: scratch too small (%zu bytes)",
              scratch_bytes);
  AdParams p;
  p.seq = seq; p.n = d.n; p.stride = stride; p.D = head_dim; p.causal = causal ? 1 : 0;
  p.scale_log2 = (float)(1.4426950408889634 / sqrt((double)head_dim) / (double)stride);
  cudaStream_t st = (cudaStream_t)stream;
  const int row_tiles = (d.n_valid + kTile - 1) / kTile;
  const int col_tiles = causal ? row_tiles : (d.n + kTile - 1) / kTile;
  dim3 grid((unsigned)col_tiles, (unsigned)row_tiles, (unsigned)bh);
  const size_t smem = (size_t)8 * (d.n / d.rb) * sizeof(float);
  dim3 grid2((unsigned)d.nb, (unsigned)bh);
  const bool tc_ok = antidiag_tc_supported(seq, head_dim, stride, d.n, dtype);
  PSA_REQUIRE(impl != 2 || tc_ok, PSA_ERR_UNSUPPORTED,
              "psa_antidiag_scores: the tcgen05 kernel needs a length that is a multiple of the stride (seq=%lld, stride=%d)",
              (long long)seq, stride);
  const bool use_tc = tc_ok && impl != 3;
  if (use_tc)      // GEMM with a partial softmax in its epilogue, then a small combine kernel: no logits in HBM
    return launch_antidiag_tc(q, k, out, (float*)scratch, bh, seq, head_dim, stride, d.n, d.n_valid, d.rb, d.nb, p.causal, p.scale_log2,
                              dtype, status, st);
  if (dtype == PSA_F16) {
    antidiag_logits_kernel<__half><<<grid, 256, 0, st>>>((const __half*)q, (const __half*)k, (float*)scratch, p);
    PSA_CHECK_LAUNCH("psa_antidiag_scores(logits)");
    antidiag_softmax_cells_kernel<__half><<<grid2, 256, smem, st>>>((const float*)scratch, (__half*)out, d.n, d.n_valid, d.rb, d.nb, p.causal);
  } else {
    antidiag_logits_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (float*)scratch, p);
    PSA_CHECK_LAUNCH("psa_antidiag_scores(logits)");
    antidiag_softmax_cells_kernel<__nv_bfloat16><<<grid2, 256, smem, st>>>((const float*)scratch, (__nv_bfloat16*)out, d.n, d.n_valid, d.rb,
                                                                            d.nb, p.causal);
  }
  PSA_CHECK_LAUNCH("psa_antidiag_scores(cells)");
  return PSA_OK;
}
