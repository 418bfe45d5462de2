// Legacy (old mask format) forward on the tensor-core kernel.
//
// The old format stores one level per (query block, key block of 128): 0 = skipped, l in {1,2,4,8} = attend the
// 128/l pooled tokens of level l with logit + ln l (psa_kernel_legacy.py:34-101, 580-799).  That is the separator-format
// forward with block_n = 128 and no compatibility extras - causal rows stop at the diagonal block (:584-586), inside
// which pooled token j of level l is visible iff (j+1)*l - 1 <= query position (:78-81) - so the dense level row is
// regrouped into an index row (level-1 blocks, -1, level-2 blocks, -1, level-4, -1, level-8, -1) and the tcgen05 kernel
// runs on it; the kernel also writes the log-sum-exp the backward needs and gives 0 / -inf for rows without any
// visible key, as the legacy kernel does.
#include "psa_common.cuh"
#include "fwd.h"

namespace psa {

// One warp per mask row: four ordered compaction passes with ballots.
__global__ void __launch_bounds__(256) old_mask_to_index_rows(const int32_t* __restrict__ old_mask, int32_t* __restrict__ rows,
                                                              int64_t n_rows, int mask_cols, int nk, int causal) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int32_t* src = old_mask + row * mask_cols;
  int32_t* dst = rows + row * (nk + 5);
  const int end = causal ? (int)(row % nk) + 1 : nk;     // causal rows only walk key blocks up to the diagonal
  int pos = 0;
  for (int level = 1; level <= 8; level <<= 1) {
    for (int c0 = 0; c0 < end; c0 += 32) {
      const int c = c0 + lane;
      const bool hit = c < end && src[c] == level;
      const unsigned bits = __ballot_sync(0xffffffffu, hit);
      if (hit) dst[pos + __popc(bits & ((1u << lane) - 1))] = c;
      pos += __popc(bits);
    }
    if (lane == 0) dst[pos] = -1;
    ++pos;
  }
  for (int c = pos + lane; c < nk + 5; c += 32) dst[c] = 0;
}

}  // namespace psa

extern "C" size_t psa_legacy_index_bytes(int64_t bh, int64_t seq) {
  if (bh <= 0 || seq <= 0) return 0;
  const int64_t n = (seq + 127) / 128;
  return (size_t)(bh * n * (n + 5) * (int64_t)sizeof(int32_t));
}

static int legacy_fwd_images(const void* q, const void* kimg, const void* vimg, const int32_t* mask, int32_t* index_scratch,
                             void* out, float* lse, const int32_t* out_perm, int64_t bh, int64_t seq, int head_dim, int mask_cols,
                             float sm_scale, int causal, int dtype, int32_t* status, void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && kimg && vimg && mask && index_scratch && out, PSA_ERR_ARG, "psa_legacy_fwd_images: null pointer");
  PSA_REQUIRE(bh > 0 && bh < 65536 && seq > 0, PSA_ERR_ARG, "psa_legacy_fwd_images: bad shape");
  const int nk = (int)cdiv64(seq, 128);
  PSA_REQUIRE(mask_cols >= nk, PSA_ERR_ARG, "psa_legacy_fwd_images: mask has %d columns, needs %d", mask_cols, nk);
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t n_rows = bh * nk;
  old_mask_to_index_rows<<<(unsigned)cdiv64(n_rows, 8), 256, 0, st>>>(mask, index_scratch, n_rows, mask_cols, nk, causal);
  PSA_CHECK_LAUNCH("psa_legacy_fwd_images(index rows)");
  const int64_t s_pad = (int64_t)nk * 128;
  FwdArgs a;
  a.q = q; a.mask = index_scratch; a.out = out; a.status = status; a.kimg = kimg; a.vimg = vimg;
  const int64_t nl[4] = {seq, s_pad / 2, s_pad / 4, s_pad / 8};
  for (int i = 0; i < 4; ++i) { a.k[i] = q; a.v[i] = q; a.n[i] = nl[i]; }
  a.bh = bh; a.seq_q = seq; a.seq_k = seq; a.D = head_dim; a.bm = 128; a.bn = 128; a.tn = 32;
  a.width = nk + 5; a.scale = sm_scale; a.quirk = 0; a.dtype = dtype;
  a.lse = lse; a.legacy = 1; a.causal = causal ? 1 : 0;
  a.scatter.row_perm = out_perm;
  PSA_REQUIRE(fwd_tc_supported(a), PSA_ERR_UNSUPPORTED,
              "psa_legacy_fwd_images: needs f16/bf16, head_dim 64/128 and at most 1467 key blocks");
  return fwd_tc_launch(a, st);
}

extern "C" int psa_legacy_fwd_images(const void* q, const void* kimg, const void* vimg, const int32_t* mask, int32_t* index_scratch,
                                     void* out, float* lse, int64_t bh, int64_t seq, int head_dim, int mask_cols, float sm_scale,
                                     int causal, int dtype, int32_t* status, void* stream) {
  return legacy_fwd_images(q, kimg, vimg, mask, index_scratch, out, lse, nullptr, bh, seq, head_dim, mask_cols, sm_scale, causal, dtype,
                           status, stream);
}

extern "C" int psa_legacy_fwd_images_perm(const void* q, const void* kimg, const void* vimg, const int32_t* mask, int32_t* index_scratch,
                                          void* out, const int32_t* out_perm, int64_t bh, int64_t seq, int head_dim, int mask_cols,
                                          float sm_scale, int dtype, int32_t* status, void* stream) {
  PSA_REQUIRE(out_perm, PSA_ERR_ARG, "psa_legacy_fwd_images_perm: null pointer");
  return legacy_fwd_images(q, kimg, vimg, mask, index_scratch, out, nullptr, out_perm, bh, seq, head_dim, mask_cols, sm_scale, 0, dtype,
                           status, stream);
}
