// Scalar legacy forward on the dense old-format mask (optional causal); see fwd_simt.cu for the layout.
#include "psa_common.cuh"
#include "fwd_simt_core.cuh"
#include "fwd.h"

namespace psa {

// ----------------------------------------------------------------- dense old-format mask ----------
template <typename T, int D>
__global__ void __launch_bounds__(512) psa_legacy_fwd_simt_kernel(const T* __restrict__ q, LevelPtrs lp, const int32_t* __restrict__ mask,
                                           T* __restrict__ out, float* __restrict__ lse, int64_t seq, int mask_cols,
                                           int mq, float scale, int causal) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float(*Ks)[D] = reinterpret_cast<float(*)[D]>(smem_raw);
  float(*Vs)[D] = Ks + 32;
  int32_t* row = reinterpret_cast<int32_t*>(Vs + 32);

  const int m = blockIdx.x;
  const int64_t bh = blockIdx.y;
  const int g = threadIdx.x & 3;
  const int64_t qrow = (int64_t)m * 128 + (threadIdx.x >> 2);
  const bool valid = qrow < seq;
  const int32_t* mrow = mask + (bh * mq + m) * (int64_t)mask_cols;
  int nblk = (int)((seq + 127) / 128);
  int end = causal ? (nblk < m + 1 ? nblk : m + 1) : nblk;
  end = end < mask_cols ? end : mask_cols;
  for (int i = threadIdx.x; i < end; i += blockDim.x) row[i] = mrow[i];

  FwdCore<T, D> st;
  st.init(q + (bh * seq + (valid ? qrow : 0)) * D, valid, g);
  __syncthreads();

  for (int pb = 0; pb < end; ++pb) {
    const int level = row[pb];
    int li;
    if (level == 1) li = 0; else if (level == 2) li = 1; else if (level == 4) li = 2; else if (level == 8) li = 3; else continue;
    const int P = 128 / level;
    const int C = P < 32 ? P : 32;
    const T* Kl = (const T*)lp.k[li] + bh * lp.n[li] * D;
    const T* Vl = (const T*)lp.v[li] + bh * lp.n[li] * D;
    const float bias = logf((float)level);
    for (int c0 = 0; c0 < P; c0 += C) {
      const int64_t t0 = (int64_t)pb * P + c0;
      int64_t nv = lp.n[li] - t0; nv = nv < 0 ? 0 : (nv > C ? C : nv);
      st.chunk(Kl, Vl, t0, C, (int)nv, bias, scale, Ks, Vs, g, causal ? level : 0, qrow);
    }
  }
  if (valid) {
    const float l_safe = fmaxf(st.l, 1e-8f);
    const float inv = 1.0f / l_safe;
    T* o = out + (bh * seq + qrow) * D;
#pragma unroll
    for (int d = 0; d < FwdCore<T, D>::DPT; ++d) o[d * 4 + g] = Elem<T>::from_f(st.acc[d] * inv);
    if (lse && g == 0) lse[bh * seq + qrow] = st.m + logf(l_safe);
  }
}

template <typename T, int D>
static int launch_legacy_fwd_simt(const void* q, const LevelPtrs& lp, const int32_t* mask, void* out, float* lse,
                                  int64_t bh, int64_t seq, int mask_cols, float scale, int causal, cudaStream_t st) {
  const int mq = (int)cdiv64(seq, 128);
  size_t smem = 2 * 32 * D * sizeof(float) + (size_t)mask_cols * 4;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(psa_legacy_fwd_simt_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_legacy_fwd: smem opt-in failed: %s", cudaGetErrorString(e));
  }
  dim3 grid(mq, (unsigned)bh);
  psa_legacy_fwd_simt_kernel<T, D><<<grid, 512, smem, st>>>((const T*)q, lp, mask, (T*)out, lse, seq, mask_cols, mq,
                                                            scale, causal);
  PSA_CHECK_LAUNCH("psa_legacy_fwd(scalar)");
  return PSA_OK;
}

int legacy_fwd_simt_dispatch(const void* q, const void* const* kl, const void* const* vl, const int64_t* nl,
                             const int32_t* mask, void* out, float* lse, int64_t bh, int64_t seq, int D, int mask_cols,
                             float scale, int causal, int dtype, cudaStream_t st) {
  LevelPtrs lp;
  for (int i = 0; i < 4; ++i) { lp.k[i] = kl[i]; lp.v[i] = vl[i]; lp.n[i] = nl[i]; }
  PSA_DISPATCH_DTYPE(dtype, T, {
    if (D == 64) return launch_legacy_fwd_simt<T, 64>(q, lp, mask, out, lse, bh, seq, mask_cols, scale, causal, st);
    return launch_legacy_fwd_simt<T, 128>(q, lp, mask, out, lse, bh, seq, mask_cols, scale, causal, st);
  });
  return PSA_OK;
}

}  // namespace psa
