// Scalar (CUDA-core, fp32) multi-level block-sparse attention forward, for both mask formats.
//
// This is the any-dtype path: it serves float32 inputs (exact fp32 dot products) and is the on-device
// cross-check of the tcgen05 kernel.  One CTA per (query block, batch*head); 4 threads share a query row,
// each owning the channels d with d % 4 == its quarter, so that shared-memory reads of a key row are
// conflict-free.  Keys/values are staged 32 tokens at a time as fp32 in shared memory; softmax is the
// usual running max / running sum, natural exponent, with the probabilities rounded to the element type
// before they multiply V (as the tensor-core kernels do).
#include "psa_common.cuh"
#include "fwd_simt_core.cuh"
#include "fwd.h"

namespace psa {

// ----------------------------------------------------------------- separator-format mask ---------
template <typename T, int D>
__global__ void __launch_bounds__(512) psa_fwd_simt_kernel(const T* __restrict__ q, LevelPtrs lp, const int32_t* __restrict__ mask,
                                    T* __restrict__ out, int64_t seq_q, int bm, int bn, int tn, int width, int mq,
                                    float scale, int quirk) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float(*Ks)[D] = reinterpret_cast<float(*)[D]>(smem_raw);
  float(*Vs)[D] = Ks + 32;
  int32_t* row = reinterpret_cast<int32_t*>(Vs + 32);

  const int m = blockIdx.x;
  const int64_t bh = blockIdx.y;
  const int g = threadIdx.x & 3;
  const int64_t qrow = (int64_t)m * bm + (threadIdx.x >> 2);
  const bool valid = qrow < seq_q;
  const int32_t* mrow = mask + (bh * mq + m) * (int64_t)width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) row[i] = mrow[i];

  FwdCore<T, D> st;
  st.init(q + (bh * seq_q + (valid ? qrow : 0)) * D, valid, g);
  __syncthreads();

  int pos = 0;
  for (int li = 0; li < 4 && pos < width; ++li) {
    const int level = 1 << li;
    const int P = bn / level;
    const T* Kl = (const T*)lp.k[li] + bh * lp.n[li] * D;
    const T* Vl = (const T*)lp.v[li] + bh * lp.n[li] * D;
    const int64_t nl = lp.n[li];
    const float bias = logf((float)level);
    const int C = P < 32 ? P : 32;
    int count = 0;
    while (pos < width && row[pos] != -1) {
      const int64_t a = row[pos];
      for (int c0 = 0; c0 < P; c0 += C) {
        const int64_t t0 = a * P + c0;
        int64_t nv = nl - t0; nv = nv < 0 ? 0 : (nv > C ? C : nv);
        st.chunk(Kl, Vl, t0, C, (int)nv, bias, scale, Ks, Vs, g, 0, 0);
      }
      ++pos; ++count;
    }
    if (quirk && P < tn && count >= 2) {
      // every merged pair of this level also saw pooled tokens [2P, tn): the same columns count/2 times
      const float qbias = bias + logf((float)(count / 2));
      for (int j = 2; j < tn / P; ++j) {
        const int64_t t0 = (int64_t)j * P;
        int64_t nv = nl - t0; nv = nv < 0 ? 0 : (nv > C ? C : nv);
        st.chunk(Kl, Vl, t0, C, (int)nv, qbias, scale, Ks, Vs, g, 0, 0);
      }
    }
    ++pos;  // separator
  }
  if (valid) {
    T* o = out + (bh * seq_q + qrow) * D;
    const float inv = 1.0f / st.l;   // an empty row gives 0/0 like the reference
#pragma unroll
    for (int d = 0; d < FwdCore<T, D>::DPT; ++d) o[d * 4 + g] = Elem<T>::from_f(st.acc[d] * inv);
  }
}

template <typename T, int D>
static int launch_fwd_simt(const void* q, const LevelPtrs& lp, const int32_t* mask, void* out, int64_t bh, int64_t seq_q,
                           int bm, int bn, int tn, int width, float scale, int quirk, cudaStream_t st) {
  const int mq = (int)cdiv64(seq_q, bm);
  size_t smem = 2 * 32 * D * sizeof(float) + (size_t)width * 4;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(psa_fwd_simt_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_fwd: smem opt-in failed: %s", cudaGetErrorString(e));
  }
  dim3 grid(mq, (unsigned)bh);
  psa_fwd_simt_kernel<T, D><<<grid, bm * 4, smem, st>>>((const T*)q, lp, mask, (T*)out, seq_q, bm, bn, tn, width, mq,
                                                         scale, quirk);
  PSA_CHECK_LAUNCH("psa_fwd(scalar)");
  return PSA_OK;
}

int fwd_simt_dispatch(const void* q, const void* const* kl, const void* const* vl, const int64_t* nl, const int32_t* mask,
                      void* out, int64_t bh, int64_t seq_q, int D, int bm, int bn, int tn, int width, float scale,
                      int quirk, int dtype, cudaStream_t st) {
  LevelPtrs lp;
  for (int i = 0; i < 4; ++i) { lp.k[i] = kl[i]; lp.v[i] = vl[i]; lp.n[i] = nl[i]; }
  PSA_DISPATCH_DTYPE(dtype, T, {
    if (D == 64) return launch_fwd_simt<T, 64>(q, lp, mask, out, bh, seq_q, bm, bn, tn, width, scale, quirk, st);
    return launch_fwd_simt<T, 128>(q, lp, mask, out, bh, seq_q, bm, bn, tn, width, scale, quirk, st);
  });
  return PSA_OK;
}

}  // namespace psa
