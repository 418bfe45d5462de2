// extern "C" surface shared by all kernels: error text, build info and the attention entry points that
// choose between the scalar and the tcgen05 kernels.
#include <stdarg.h>
#include <string.h>

#include "psa_common.cuh"
#include "fwd.h"

namespace psa {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

}  // namespace psa

extern "C" const char* psa_last_error_string(void) { return psa::g_err; }

extern "C" const char* psa_build_info(void) {
  return "psa_b200 sm_100a (pyramid, block scores, level assignment, multi-level forward, legacy fwd/bwd); "
         "built " __DATE__ " " __TIME__;
}

extern "C" int psa_fwd(const void* q, const void* k, const void* v, const void* k2, const void* k4, const void* k8,
                       const void* v2, const void* v4, const void* v8, const int32_t* mask, void* out, int64_t bh,
                       int64_t seq_q, int64_t seq_k, int head_dim, int block_m, int block_n, int tile_n, int mask_width,
                       float sm_scale, int compat_quirk, int impl, int dtype, int32_t* status, void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && k && v && k2 && k4 && k8 && v2 && v4 && v8 && mask && out, PSA_ERR_ARG, "psa_fwd: null pointer");
  PSA_REQUIRE(head_dim == 64 || head_dim == 128, PSA_ERR_ARG, "psa_fwd: head_dim=%d (must be 64 or 128)", head_dim);
  PSA_REQUIRE(block_n == 32 || block_n == 64 || block_n == 128, PSA_ERR_ARG, "psa_fwd: block_n=%d (32/64/128)", block_n);
  PSA_REQUIRE(tile_n == 32, PSA_ERR_UNSUPPORTED, "psa_fwd: tile_n=%d (only 32, the value every preset uses)", tile_n);
  PSA_REQUIRE(block_m == 32 || block_m == 64 || block_m == 128, PSA_ERR_ARG, "psa_fwd: block_m=%d (32/64/128)", block_m);
  PSA_REQUIRE(bh > 0 && bh < 65536 && seq_q > 0 && seq_k > 0, PSA_ERR_ARG, "psa_fwd: bad shape");
  PSA_REQUIRE(mask_width >= 1 && mask_width <= 16384, PSA_ERR_ARG, "psa_fwd: mask_width=%d", mask_width);
  PSA_REQUIRE(impl >= 0 && impl <= 2, PSA_ERR_ARG, "psa_fwd: impl=%d", impl);
  const int64_t s_pad = cdiv64(seq_k, block_n) * block_n;
  const void* kl[4] = {k, k2, k4, k8};
  const void* vl[4] = {v, v2, v4, v8};
  const int64_t nl[4] = {seq_k, s_pad / 2, s_pad / 4, s_pad / 8};
  cudaStream_t st = (cudaStream_t)stream;
  FwdArgs a;
  a.q = q; a.mask = mask; a.out = out; a.status = status; a.kimg = nullptr; a.vimg = nullptr;
  for (int i = 0; i < 4; ++i) { a.k[i] = kl[i]; a.v[i] = vl[i]; a.n[i] = nl[i]; }
  a.bh = bh; a.seq_q = seq_q; a.seq_k = seq_k; a.D = head_dim; a.bm = block_m; a.bn = block_n; a.tn = tile_n;
  a.width = mask_width; a.scale = sm_scale; a.quirk = compat_quirk; a.dtype = dtype;
  const bool tc_ok = fwd_tc_supported(a);
  if (impl == 2) PSA_REQUIRE(tc_ok, PSA_ERR_UNSUPPORTED, "psa_fwd: the tcgen05 kernel needs f16/bf16, block_m=128");
  if (impl == 2 || (impl == 0 && tc_ok)) return fwd_tc_launch(a, st);
  return fwd_simt_dispatch(q, kl, vl, nl, mask, out, bh, seq_q, head_dim, block_m, block_n, tile_n, mask_width, sm_scale,
                           compat_quirk, dtype, st);
}

extern "C" int psa_legacy_fwd(const void* q, const void* k, const void* v, const void* k2, const void* k4,
                              const void* k8, const void* v2, const void* v4, const void* v8, const int32_t* mask,
                              void* out, float* lse, int64_t bh, int64_t seq, int head_dim, int mask_cols, float sm_scale,
                              int causal, int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && k && v && k2 && k4 && k8 && v2 && v4 && v8 && mask && out, PSA_ERR_ARG, "psa_legacy_fwd: null pointer");
  PSA_REQUIRE(head_dim == 64 || head_dim == 128, PSA_ERR_ARG, "psa_legacy_fwd: head_dim=%d (must be 64 or 128)", head_dim);
  PSA_REQUIRE(bh > 0 && bh < 65536 && seq > 0, PSA_ERR_ARG, "psa_legacy_fwd: bad shape");
  PSA_REQUIRE(mask_cols >= cdiv64(seq, 128), PSA_ERR_ARG, "psa_legacy_fwd: mask has %d columns, needs %lld", mask_cols,
              (long long)cdiv64(seq, 128));
  const int64_t s_pad = cdiv64(seq, 128) * 128;
  const void* kl[4] = {k, k2, k4, k8};
  const void* vl[4] = {v, v2, v4, v8};
  const int64_t nl[4] = {seq, s_pad / 2, s_pad / 4, s_pad / 8};
  return legacy_fwd_simt_dispatch(q, kl, vl, nl, mask, out, lse, bh, seq, head_dim, mask_cols, sm_scale, causal, dtype,
                                  (cudaStream_t)stream);
}

extern "C" int psa_fwd_images(const void* q, const void* kimg, const void* vimg, const int32_t* mask, void* out, int64_t bh,
                              int64_t seq_q, int64_t seq_k, int head_dim, int block_m, int block_n, int tile_n, int mask_width,
                              float sm_scale, int compat_quirk, int dtype, int32_t* status, void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && kimg && vimg && mask && out, PSA_ERR_ARG, "psa_fwd_images: null pointer");
  PSA_REQUIRE(bh > 0 && bh < 65536 && seq_q > 0 && seq_k > 0, PSA_ERR_ARG, "psa_fwd_images: bad shape");
  PSA_REQUIRE(block_n == 64 || block_n == 128, PSA_ERR_UNSUPPORTED, "psa_fwd_images: block_n=%d (64/128)", block_n);
  PSA_REQUIRE(mask_width >= 1, PSA_ERR_ARG, "psa_fwd_images: mask_width=%d", mask_width);
  const int64_t s_pad = cdiv64(seq_k, block_n) * block_n;
  FwdArgs a;
  a.q = q; a.mask = mask; a.out = out; a.status = status; a.kimg = kimg; a.vimg = vimg;
  const int64_t nl[4] = {seq_k, s_pad / 2, s_pad / 4, s_pad / 8};
  for (int i = 0; i < 4; ++i) { a.k[i] = q; a.v[i] = q; a.n[i] = nl[i]; }   // row-major levels are not read in image mode
  a.bh = bh; a.seq_q = seq_q; a.seq_k = seq_k; a.D = head_dim; a.bm = block_m; a.bn = block_n; a.tn = tile_n;
  a.width = mask_width; a.scale = sm_scale; a.quirk = compat_quirk; a.dtype = dtype;
  PSA_REQUIRE(fwd_tc_supported(a), PSA_ERR_UNSUPPORTED,
              "psa_fwd_images: needs f16/bf16, block_m=128, tile_n=32, head_dim 64/128, mask width <= 1472");
  return fwd_tc_launch(a, (cudaStream_t)stream);
}

extern "C" int psa_fwd_images_perm(const void* q, const void* kimg, const void* vimg, const int32_t* mask, void* out,
                                  const int32_t* out_perm, int64_t bh, int64_t seq_q, int64_t seq_k, int head_dim, int block_m,
                                  int block_n, int tile_n, int mask_width, float sm_scale, int compat_quirk, int dtype,
                                  int32_t* status, void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && kimg && vimg && mask && out && out_perm, PSA_ERR_ARG, "psa_fwd_images_perm: null pointer");
  PSA_REQUIRE(bh > 0 && bh < 65536 && seq_q > 0 && seq_k > 0 && seq_q < ((int64_t)1 << 31), PSA_ERR_ARG,
              "psa_fwd_images_perm: bad shape");
  PSA_REQUIRE(block_n == 64 || block_n == 128, PSA_ERR_UNSUPPORTED, "psa_fwd_images_perm: block_n=%d (64/128)", block_n);
  PSA_REQUIRE(mask_width >= 1, PSA_ERR_ARG, "psa_fwd_images_perm: mask_width=%d", mask_width);
  const int64_t s_pad = cdiv64(seq_k, block_n) * block_n;
  FwdArgs a;
  a.q = q; a.mask = mask; a.out = out; a.status = status; a.kimg = kimg; a.vimg = vimg;
  const int64_t nl[4] = {seq_k, s_pad / 2, s_pad / 4, s_pad / 8};
  for (int i = 0; i < 4; ++i) { a.k[i] = q; a.v[i] = q; a.n[i] = nl[i]; }   // row-major levels are not read in image mode
  a.bh = bh; a.seq_q = seq_q; a.seq_k = seq_k; a.D = head_dim; a.bm = block_m; a.bn = block_n; a.tn = tile_n;
  a.width = mask_width; a.scale = sm_scale; a.quirk = compat_quirk; a.dtype = dtype;
  a.scatter.row_perm = out_perm;
  PSA_REQUIRE(fwd_tc_supported(a), PSA_ERR_UNSUPPORTED,
              "psa_fwd_images_perm: needs f16/bf16, block_m=128, tile_n=32, head_dim 64/128, mask width <= 1472");
  return fwd_tc_launch(a, (cudaStream_t)stream);
}

extern "C" int psa_fwd_images_tm(const void* q, const void* kimg, const void* vimg, const int32_t* mask, void* out,
                                const int32_t* out_perm, int heads, int64_t seq, int head_dim, int block_m, int block_n, int tile_n,
                                int mask_width, float sm_scale, int compat_quirk, int dtype, int32_t* status, void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && kimg && vimg && mask && out, PSA_ERR_ARG, "psa_fwd_images_tm: null pointer");
  PSA_REQUIRE(heads > 0 && heads < 65536 && seq > 0 && seq < ((int64_t)1 << 31), PSA_ERR_ARG, "psa_fwd_images_tm: bad shape");
  PSA_REQUIRE(block_n == 64 || block_n == 128, PSA_ERR_UNSUPPORTED, "psa_fwd_images_tm: block_n=%d (64/128)", block_n);
  PSA_REQUIRE(mask_width >= 1, PSA_ERR_ARG, "psa_fwd_images_tm: mask_width=%d", mask_width);
  PSA_REQUIRE(((uintptr_t)out & 15) == 0, PSA_ERR_ARG, "psa_fwd_images_tm: out must be 16-byte aligned");
  const int64_t s_pad = cdiv64(seq, block_n) * block_n;
  FwdArgs a;
  a.q = q; a.mask = mask; a.out = nullptr; a.status = status; a.kimg = kimg; a.vimg = vimg;
  const int64_t nl[4] = {seq, s_pad / 2, s_pad / 4, s_pad / 8};
  for (int i = 0; i < 4; ++i) { a.k[i] = q; a.v[i] = q; a.n[i] = nl[i]; }   // row-major levels are not read in image mode
  a.bh = heads; a.seq_q = seq; a.seq_k = seq; a.D = head_dim; a.bm = block_m; a.bn = block_n; a.tn = tile_n;
  a.width = mask_width; a.scale = sm_scale; a.quirk = compat_quirk; a.dtype = dtype;
  a.scatter.peer_out[0] = out;
  a.scatter.n_peers = 1; a.scatter.heads_total = heads; a.scatter.head0 = 0; a.scatter.tokens_per_rank = seq;
  a.scatter.row_perm = out_perm;
  PSA_REQUIRE(fwd_tc_supported(a), PSA_ERR_UNSUPPORTED,
              "psa_fwd_images_tm: needs f16/bf16, block_m=128, tile_n=32, head_dim 64/128, mask width <= 1472");
  return fwd_tc_launch(a, (cudaStream_t)stream);
}

extern "C" int psa_fwd_images_scatter(const void* q, const void* kimg, const void* vimg, const int32_t* mask, void* const* peer_out,
                                      int n_peers, int64_t tokens_per_rank, int heads_total, int head0, int64_t bh, int64_t seq_q,
                                      int64_t seq_k, int head_dim, int block_m, int block_n, int tile_n, int mask_width,
                                      float sm_scale, int compat_quirk, int dtype, int32_t* status, void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && kimg && vimg && mask && peer_out, PSA_ERR_ARG, "psa_fwd_images_scatter: null pointer");
  PSA_REQUIRE(n_peers >= 1 && n_peers <= kMaxPeers, PSA_ERR_ARG, "psa_fwd_images_scatter: n_peers=%d (1..%d)", n_peers, kMaxPeers);
  PSA_REQUIRE(bh > 0 && bh < 65536 && seq_q > 0 && seq_k > 0, PSA_ERR_ARG, "psa_fwd_images_scatter: bad shape");
  PSA_REQUIRE(tokens_per_rank > 0 && tokens_per_rank * n_peers >= seq_q, PSA_ERR_ARG,
              "psa_fwd_images_scatter: %d peers x %lld tokens do not cover %lld query rows", n_peers, (long long)tokens_per_rank,
              (long long)seq_q);
  PSA_REQUIRE(head0 >= 0 && head0 + bh <= heads_total, PSA_ERR_ARG, "psa_fwd_images_scatter: heads [%d, %lld) of %d", head0,
              (long long)(head0 + bh), heads_total);
  PSA_REQUIRE(block_n == 64 || block_n == 128, PSA_ERR_UNSUPPORTED, "psa_fwd_images_scatter: block_n=%d (64/128)", block_n);
  PSA_REQUIRE(mask_width >= 1, PSA_ERR_ARG, "psa_fwd_images_scatter: mask_width=%d", mask_width);
  const int64_t s_pad = cdiv64(seq_k, block_n) * block_n;
  FwdArgs a;
  a.q = q; a.mask = mask; a.out = const_cast<void*>(q); a.status = status; a.kimg = kimg; a.vimg = vimg;   // out unused
  const int64_t nl[4] = {seq_k, s_pad / 2, s_pad / 4, s_pad / 8};
  for (int i = 0; i < 4; ++i) { a.k[i] = q; a.v[i] = q; a.n[i] = nl[i]; }
  a.bh = bh; a.seq_q = seq_q; a.seq_k = seq_k; a.D = head_dim; a.bm = block_m; a.bn = block_n; a.tn = tile_n;
  a.width = mask_width; a.scale = sm_scale; a.quirk = compat_quirk; a.dtype = dtype;
  for (int i = 0; i < kMaxPeers; ++i) {
    a.scatter.peer_out[i] = i < n_peers ? peer_out[i] : nullptr;
    if (i < n_peers) PSA_REQUIRE(peer_out[i] && ((uintptr_t)peer_out[i] & 15) == 0, PSA_ERR_ARG, "psa_fwd_images_scatter: peer %d", i);
  }
  a.scatter.n_peers = n_peers; a.scatter.heads_total = heads_total; a.scatter.head0 = head0;
  a.scatter.tokens_per_rank = tokens_per_rank;
  PSA_REQUIRE(fwd_tc_supported(a), PSA_ERR_UNSUPPORTED,
              "psa_fwd_images_scatter: needs f16/bf16, block_m=128, tile_n=32, head_dim 64/128, mask width <= 1472");
  return fwd_tc_launch(a, (cudaStream_t)stream);
}
