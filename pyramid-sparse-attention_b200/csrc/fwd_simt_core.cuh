// Per-row state and the 32-token chunk step shared by the scalar forward kernels.
#pragma once
#include "psa_common.cuh"

namespace psa {

template <typename T, int D>
struct FwdCore {
  static constexpr int DPT = D / 4;
  float q[DPT], acc[DPT];
  float m, l;

  __device__ __forceinline__ void init(const T* qrow, bool valid, int g) {
#pragma unroll
    for (int d = 0; d < DPT; ++d) { q[d] = valid ? Elem<T>::to_f(qrow[d * 4 + g]) : 0.f; acc[d] = 0.f; }
    m = -INFINITY; l = 0.f;
  }

  // Attend to C (<= 32) consecutive pooled tokens [t0, t0+C) of one level; only the first nv exist.
  // causal_level > 0: pooled token j is visible iff (j+1)*causal_level - 1 <= qpos.
  __device__ __forceinline__ void chunk(const T* __restrict__ Kl, const T* __restrict__ Vl, int64_t t0, int C, int nv,
                                        float bias, float scale, float (*Ks)[D], float (*Vs)[D], int g,
                                        int causal_level, int64_t qpos) {
    __syncthreads();
    for (int e = threadIdx.x; e < C * D; e += blockDim.x) {
      int r = e / D, c = e % D;
      bool ok = r < nv;
      Ks[r][c] = ok ? Elem<T>::to_f(Kl[(t0 + r) * D + c]) : 0.f;
      Vs[r][c] = ok ? Elem<T>::to_f(Vl[(t0 + r) * D + c]) : 0.f;
    }
    __syncthreads();
    // 8 tokens per softmax step keeps the scores in registers without unrolling the whole chunk
    for (int c0 = 0; c0 < C; c0 += 8) {
      float s[8];
      float mx = -INFINITY;
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {
        const int c = c0 + cc;
        float part = 0.f;
        if (c < C) {
#pragma unroll
          for (int d = 0; d < DPT; ++d) part = fmaf(q[d], Ks[c][d * 4 + g], part);
        }
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        bool vis = c < nv && (causal_level == 0 || ((t0 + c + 1) * causal_level - 1 <= qpos));
        s[cc] = vis ? part * scale + bias : -INFINITY;
        mx = fmaxf(mx, s[cc]);
      }
      const float m_new = fmaxf(m, mx);
      if (m_new == -INFINITY) continue;   // nothing visible yet for this row
      const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
      float lsum = 0.f;
#pragma unroll
      for (int d = 0; d < DPT; ++d) acc[d] *= alpha;
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {
        const int c = c0 + cc;
        if (c < C) {
          float p = s[cc] == -INFINITY ? 0.f : expf(s[cc] - m_new);
          lsum += p;
          float pr = Elem<T>::round(p);
#pragma unroll
          for (int d = 0; d < DPT; ++d) acc[d] = fmaf(pr, Vs[c][d * 4 + g], acc[d]);
        }
      }
      l = l * alpha + lsum;
      m = m_new;
    }
  }
};

struct LevelPtrs {
  const void* k[4];
  const void* v[4];
  int64_t n[4];  // tokens per head at levels 1,2,4,8
};

}  // namespace psa
