// K-similarity cap: per key block, the mean cosine similarity of token pairs (2i,2i+1), (4i,4i+3) and
// (8i,8i+7) decides the coarsest pyramid level the block may be pooled to.
//
// HBM-bound: K is read once (N*e bytes), one int32 per block is written.
// One warp per key block; the warp walks the block 8 tokens at a time, lanes split the channels.
#include "psa_common.cuh"

namespace psa {

template <typename T>
__global__ void __launch_bounds__(128) ksim_kernel(const T* __restrict__ k, const int32_t* __restrict__ perm, int32_t* __restrict__ out,
                                                   int64_t seq, int D, int bn, int nblk, float t2, float t4, float t8) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int blk = blockIdx.x * 4 + warp;
  if (blk >= nblk) return;
  const int64_t bh = blockIdx.y;
  const T* kh = k + bh * seq * D;
  float c2 = 0.f, c4 = 0.f, c8 = 0.f;
  for (int g0 = 0; g0 < bn; g0 += 8) {
    float nn[8], d2[4], d4[2], d8;
#pragma unroll
    for (int t = 0; t < 8; ++t) nn[t] = 0.f;
#pragma unroll
    for (int t = 0; t < 4; ++t) d2[t] = 0.f;
    d4[0] = d4[1] = 0.f; d8 = 0.f;
    for (int c = lane; c < D; c += 32) {
      float x[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        int64_t tok = (int64_t)blk * bn + g0 + t;
        tok = tok < seq ? tok : seq - 1;
        if (perm) tok = perm[tok];              // token `tok` of the reordered sequence is stored row perm[tok]
        x[t] = Elem<T>::to_f(kh[tok * D + c]);
        nn[t] = fmaf(x[t], x[t], nn[t]);
      }
#pragma unroll
      for (int t = 0; t < 4; ++t) d2[t] = fmaf(x[2 * t], x[2 * t + 1], d2[t]);
      d4[0] = fmaf(x[0], x[3], d4[0]);
      d4[1] = fmaf(x[4], x[7], d4[1]);
      d8 = fmaf(x[0], x[7], d8);
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) {
#pragma unroll
      for (int t = 0; t < 8; ++t) nn[t] += __shfl_xor_sync(0xffffffffu, nn[t], off);
#pragma unroll
      for (int t = 0; t < 4; ++t) d2[t] += __shfl_xor_sync(0xffffffffu, d2[t], off);
      d4[0] += __shfl_xor_sync(0xffffffffu, d4[0], off);
      d4[1] += __shfl_xor_sync(0xffffffffu, d4[1], off);
      d8 += __shfl_xor_sync(0xffffffffu, d8, off);
    }
#pragma unroll
    for (int t = 0; t < 8; ++t) nn[t] = sqrtf(nn[t] + 1e-12f);
#pragma unroll
    for (int t = 0; t < 4; ++t) c2 += d2[t] / (nn[2 * t] * nn[2 * t + 1] + 1e-6f);
    c4 += d4[0] / (nn[0] * nn[3] + 1e-6f) + d4[1] / (nn[4] * nn[7] + 1e-6f);
    c8 += d8 / (nn[0] * nn[7] + 1e-6f);
  }
  if (lane == 0) {
    const float s2 = c2 / (float)(bn / 2), s4 = c4 / (float)(bn / 4), s8 = c8 / (float)(bn / 8);
    int r = 1;
    if (s2 > t2) r = 2;
    if (s4 > t4) r = 4;
    if (s8 > t8) r = 8;
    out[bh * nblk + blk] = r;
  }
}

}  // namespace psa

static int ksim_launch(const void* k, const int32_t* perm, int32_t* out, int64_t bh, int64_t seq, int head_dim, int block_n, float t2,
                       float t4, float t8, int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(k && out, PSA_ERR_ARG, "psa_ksim: null pointer");
  PSA_REQUIRE(bh > 0 && bh < 65536 && seq > 0, PSA_ERR_ARG, "psa_ksim: bad shape");
  PSA_REQUIRE(block_n >= 8 && block_n % 8 == 0, PSA_ERR_ARG, "psa_ksim: blocksize must be divisible by 8");
  const int nblk = (int)cdiv64(seq, block_n);
  dim3 grid((nblk + 3) / 4, (unsigned)bh);
  cudaStream_t st = (cudaStream_t)stream;
  PSA_DISPATCH_DTYPE(dtype, T, (ksim_kernel<T><<<grid, 128, 0, st>>>((const T*)k, perm, out, seq, head_dim, block_n, nblk, t2, t4, t8)));
  PSA_CHECK_LAUNCH("psa_ksim");
  return PSA_OK;
}

extern "C" int psa_ksim(const void* k, int32_t* out, int64_t bh, int64_t seq, int head_dim, int block_n, float t2,
                        float t4, float t8, int dtype, void* stream) {
  return ksim_launch(k, nullptr, out, bh, seq, head_dim, block_n, t2, t4, t8, dtype, stream);
}

extern "C" int psa_ksim_perm(const void* k, const int32_t* perm, int32_t* out, int64_t bh, int64_t seq, int head_dim, int block_n,
                             float t2, float t4, float t8, int dtype, void* stream) {
  PSA_REQUIRE(perm, PSA_ERR_ARG, "psa_ksim_perm: null pointer");
  return ksim_launch(k, perm, out, bh, seq, head_dim, block_n, t2, t4, t8, dtype, stream);
}
