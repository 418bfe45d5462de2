// Token reordering (space-filling-curve order of the video tokens) folded into the attention kernels.
//
// The reference reorders q, k, v with three index_select copies before the attention and the output with a fourth one
// after it (src/psa_triton/utils/rearranger.py:69-132).  Here one int32 table `perm` [seq] (token t of the attention's
// sequence = row perm[t] of the stored tensor) is read by the kernels that touch the rows anyway: the tile-image builder
// and the sample gather of the block scores read k, v (and the sampled quarter of q) through it, and the forward's
// epilogue stores output row t at row perm[t].  Only q needs a copy of its own (the forward fetches query tiles with
// one bulk tensor copy per tile), which is the kernel in this file.
#include "psa_common.cuh"
#include "fwd.h"

namespace psa {
namespace {

// dst[bh][t][:] = src[bh][perm[t]][:], rows of cpr 16-byte words.
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ perm,
                                                          uint4* __restrict__ dst, int64_t seq, int cpr) {
  const int64_t bh = blockIdx.y;
  const uint4* s = src + bh * seq * cpr;
  uint4* d = dst + bh * seq * cpr;
  const int64_t total = seq * cpr;
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = w / cpr;
    const int c = (int)(w - t * cpr);
    d[w] = s[(int64_t)perm[t] * cpr + c];
  }
}

// dst[h][t][:] = src[perm ? perm[t] : t][h][:]: token-major rows regrouped by head (and reordered) in one pass.
__global__ void __launch_bounds__(256) gather_heads_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ perm,
                                                           uint4* __restrict__ dst, int64_t seq, int heads, int cpr) {
  const int64_t h = blockIdx.y;
  uint4* d = dst + h * seq * cpr;
  const int64_t total = seq * cpr;
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = w / cpr;
    const int c = (int)(w - t * cpr);
    const int64_t row = perm ? (int64_t)perm[t] : t;
    d[w] = src[(row * heads + h) * cpr + c];
  }
}

// dst[bh][t][:] = rotated src[bh][perm ? perm[t] : t][:] (16-bit rows; see RopeTables in fwd.h for the arithmetic).
__global__ void __launch_bounds__(256) gather_rows_rope_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ perm,
                                                               uint4* __restrict__ dst, int64_t seq, int cpr,
                                                               const float* __restrict__ rope_a, const float* __restrict__ rope_b,
                                                               int64_t rope_first, int bf16) {
  const int64_t bh = blockIdx.y;
  const uint4* s = src + bh * seq * cpr;
  uint4* d = dst + bh * seq * cpr;
  const int64_t total = seq * cpr;
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = w / cpr;
    const int c = (int)(w - t * cpr);
    const int64_t row = perm ? (int64_t)perm[t] : t;
    uint4 x = s[row * cpr + c];
    if (row >= rope_first) {
      const int64_t off = ((row - rope_first) * cpr + c) * 8;
      x = rotate_word(x, rope_a + off, rope_b + off, bf16 != 0);
    }
    d[w] = x;
  }
}

// The same with every row rotated on the way (16-bit rows; see RopeTables in fwd.h for the arithmetic).
__global__ void __launch_bounds__(256) gather_heads_rope_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ perm,
                                                                uint4* __restrict__ dst, int64_t seq, int heads, int cpr,
                                                                const float* __restrict__ rope_a, const float* __restrict__ rope_b,
                                                                int64_t rope_first, int bf16) {
  const int64_t h = blockIdx.y;
  uint4* d = dst + h * seq * cpr;
  const int64_t total = seq * cpr;
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = w / cpr;
    const int c = (int)(w - t * cpr);
    const int64_t row = perm ? (int64_t)perm[t] : t;
    uint4 x = src[(row * heads + h) * cpr + c];
    if (row >= rope_first) {
      const int64_t off = ((row - rope_first) * cpr + c) * 8;
      x = rotate_word(x, rope_a + off, rope_b + off, bf16 != 0);
    }
    d[w] = x;
  }
}

}  // namespace
}  // namespace psa

extern "C" int psa_gather_rows(const void* src, const int32_t* perm, void* dst, int64_t bh, int64_t seq, int head_dim,
                               int elem_bytes, void* stream) {
  using namespace psa;
  PSA_REQUIRE(src && perm && dst, PSA_ERR_ARG, "psa_gather_rows: null pointer");
  PSA_REQUIRE(src != dst, PSA_ERR_ARG, "psa_gather_rows: cannot reorder in place");
  PSA_REQUIRE(bh > 0 && bh < 65536 && seq > 0 && seq < ((int64_t)1 << 31), PSA_ERR_ARG, "psa_gather_rows: bad shape");
  PSA_REQUIRE(elem_bytes == 2 || elem_bytes == 4, PSA_ERR_ARG, "psa_gather_rows: elem_bytes=%d (2 or 4)", elem_bytes);
  PSA_REQUIRE(head_dim > 0 && (head_dim * elem_bytes) % 16 == 0, PSA_ERR_ARG,
              "psa_gather_rows: rows of %d bytes are not a multiple of 16", head_dim * elem_bytes);
  PSA_REQUIRE((((uintptr_t)src | (uintptr_t)dst) & 15) == 0, PSA_ERR_ARG, "psa_gather_rows: src and dst must be 16-byte aligned");
  const int cpr = head_dim * elem_bytes / 16;
  int64_t blocks = cdiv64(seq * cpr, 256);
  // enough CTAs to cover the machine several times over once the heads (grid.y) are counted in
  const int64_t cap = cdiv64(148 * 16, bh);
  if (blocks > cap) blocks = cap;
  dim3 grid((unsigned)blocks, (unsigned)bh);
  gather_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, perm, (uint4*)dst, seq, cpr);
  PSA_CHECK_LAUNCH("psa_gather_rows");
  return PSA_OK;
}

extern "C" int psa_gather_heads(const void* src, const int32_t* perm, void* dst, int heads, int64_t seq, int head_dim,
                                int elem_bytes, void* stream) {
  using namespace psa;
  PSA_REQUIRE(src && dst, PSA_ERR_ARG, "psa_gather_heads: null pointer");
  PSA_REQUIRE(src != dst, PSA_ERR_ARG, "psa_gather_heads: cannot regroup in place");
  PSA_REQUIRE(heads > 0 && heads < 65536 && seq > 0 && seq < ((int64_t)1 << 31), PSA_ERR_ARG, "psa_gather_heads: bad shape");
  PSA_REQUIRE(elem_bytes == 2 || elem_bytes == 4, PSA_ERR_ARG, "psa_gather_heads: elem_bytes=%d (2 or 4)", elem_bytes);
  PSA_REQUIRE(head_dim > 0 && (head_dim * elem_bytes) % 16 == 0, PSA_ERR_ARG,
              "psa_gather_heads: rows of %d bytes are not a multiple of 16", head_dim * elem_bytes);
  PSA_REQUIRE((((uintptr_t)src | (uintptr_t)dst) & 15) == 0, PSA_ERR_ARG, "psa_gather_heads: src and dst must be 16-byte aligned");
  const int cpr = head_dim * elem_bytes / 16;
  int64_t blocks = cdiv64(seq * cpr, 256);
  const int64_t cap = cdiv64(148 * 16, heads);
  if (blocks > cap) blocks = cap;
  dim3 grid((unsigned)blocks, (unsigned)heads);
  gather_heads_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, perm, (uint4*)dst, seq, heads, cpr);
  PSA_CHECK_LAUNCH("psa_gather_heads");
  return PSA_OK;
}

extern "C" int psa_gather_heads_rope(const void* src, const int32_t* perm, const float* rope_a, const float* rope_b,
                                     int64_t rope_first, void* dst, int heads, int64_t seq, int head_dim, int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(src && dst && rope_a && rope_b, PSA_ERR_ARG, "psa_gather_heads_rope: null pointer");
  PSA_REQUIRE(src != dst, PSA_ERR_ARG, "psa_gather_heads_rope: cannot regroup in place");
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "psa_gather_heads_rope: f16/bf16 only");
  PSA_REQUIRE(heads > 0 && heads < 65536 && seq > 0 && seq < ((int64_t)1 << 31) && rope_first >= 0 && rope_first <= seq, PSA_ERR_ARG,
              "psa_gather_heads_rope: bad shape");
  PSA_REQUIRE(head_dim > 0 && head_dim % 8 == 0, PSA_ERR_ARG, "psa_gather_heads_rope: head_dim=%d is not a multiple of 8", head_dim);
  PSA_REQUIRE((((uintptr_t)src | (uintptr_t)dst | (uintptr_t)rope_a | (uintptr_t)rope_b) & 15) == 0, PSA_ERR_ARG,
              "psa_gather_heads_rope: src, dst and the tables must be 16-byte aligned");
  const int cpr = head_dim * 2 / 16;
  int64_t blocks = cdiv64(seq * cpr, 256);
  const int64_t cap = cdiv64(148 * 16, heads);
  if (blocks > cap) blocks = cap;
  dim3 grid((unsigned)blocks, (unsigned)heads);
  gather_heads_rope_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, perm, (uint4*)dst, seq, heads, cpr, rope_a, rope_b,
                                                                    rope_first, dtype == PSA_BF16);
  PSA_CHECK_LAUNCH("psa_gather_heads_rope");
  return PSA_OK;
}

extern "C" int psa_gather_rows_rope(const void* src, const int32_t* perm, const float* rope_a, const float* rope_b, int64_t rope_first,
                                    void* dst, int64_t bh, int64_t seq, int head_dim, int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(src && dst && rope_a && rope_b, PSA_ERR_ARG, "psa_gather_rows_rope: null pointer");
  PSA_REQUIRE(src != dst, PSA_ERR_ARG, "psa_gather_rows_rope: cannot reorder in place");
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "psa_gather_rows_rope: f16/bf16 only");
  PSA_REQUIRE(bh > 0 && bh < 65536 && seq > 0 && seq < ((int64_t)1 << 31) && rope_first >= 0 && rope_first <= seq, PSA_ERR_ARG,
              "psa_gather_rows_rope: bad shape");
  PSA_REQUIRE(head_dim > 0 && head_dim % 8 == 0, PSA_ERR_ARG, "psa_gather_rows_rope: head_dim=%d is not a multiple of 8", head_dim);
  PSA_REQUIRE((((uintptr_t)src | (uintptr_t)dst | (uintptr_t)rope_a | (uintptr_t)rope_b) & 15) == 0, PSA_ERR_ARG,
              "psa_gather_rows_rope: src, dst and the tables must be 16-byte aligned");
  const int cpr = head_dim * 2 / 16;
  int64_t blocks = cdiv64(seq * cpr, 256);
  const int64_t cap = cdiv64(148 * 16, bh);
  if (blocks > cap) blocks = cap;
  dim3 grid((unsigned)blocks, (unsigned)bh);
  gather_rows_rope_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, perm, (uint4*)dst, seq, cpr, rope_a, rope_b, rope_first,
                                                                   dtype == PSA_BF16);
  PSA_CHECK_LAUNCH("psa_gather_rows_rope");
  return PSA_OK;
}
