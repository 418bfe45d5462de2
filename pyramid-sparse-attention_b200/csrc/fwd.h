// Argument bundle and dispatch hooks of the attention forward kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace psa {

struct FwdArgs {
  const void* q;
  const void* k[4];  // levels 1, 2, 4, 8
  const void* v[4];
  int64_t n[4];      // tokens per head at each level
  const int32_t* mask;
  void* out;
  int32_t* status;
  int64_t bh, seq_q, seq_k;
  int D, bm, bn, tn, width, quirk, dtype;
  float scale;
};

int fwd_simt_dispatch(const void* q, const void* const* kl, const void* const* vl, const int64_t* nl, const int32_t* mask,
                      void* out, int64_t bh, int64_t seq_q, int D, int bm, int bn, int tn, int width, float scale,
                      int quirk, int dtype, cudaStream_t st);
int legacy_fwd_simt_dispatch(const void* q, const void* const* kl, const void* const* vl, const int64_t* nl,
                             const int32_t* mask, void* out, float* lse, int64_t bh, int64_t seq, int D, int mask_cols,
                             float scale, int causal, int dtype, cudaStream_t st);

// tcgen05 forward (fwd_tc.cu)
bool fwd_tc_supported(const FwdArgs& a);
int fwd_tc_launch(const FwdArgs& a, cudaStream_t st);

}  // namespace psa
