// Legacy (old-format mask) attention backward: dQ, dK, dV.  Scalar fp32 kernels, any dtype.
//
// The reference expands every pooled level back to original key positions (repeat_l(avgpool_l(K))), runs one dQ and
// one dK/dV kernel per level on 64x64 tiles and folds the repeated gradients back.  All l copies of a pooled token t
// carry the same key/value, so for query row i they contribute c_t(i) * ds_it where ds_it = p_it (dO_i.v_t - delta_i),
// p_it = exp(q_i.k_t * scale - lse_i) and c_t(i) = number of the group's ORIGINAL positions j that exist (j < L_K) and
// are visible (causal: j <= i, on original positions - the reference's backward rule).  Hence, without expanding
// anything in HBM:
//   dQ_i        = scale * sum_t c_t(i) ds_it k_t
//   dK_j (j in t) += scale / l * sum_i c_t(i) ds_it q_i          dV_j (j in t) += 1 / l * sum_i c_t(i) p_it dO_i
// and positions j >= S of the replicate-padded tail add their share to token S-1.
//
// Kernels: delta = rowsum(O * dO); dQ: one CTA per 128 query rows (4 threads per row); dK/dV: one CTA per 128-key
// block, 4 threads per pooled token, fp32 block accumulators in shared memory.
#include "psa_common.cuh"

namespace psa {

struct BwdLevels {
  const void* k[4];
  const void* v[4];
  int64_t n[4];
};

template <typename T>
__global__ void __launch_bounds__(256) bwd_delta_kernel(const T* __restrict__ o, const T* __restrict__ dout, float* __restrict__ delta,
                                                       int64_t rows, int D) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row >= rows) return;
  float acc = 0.f;
  for (int c = lane; c < D; c += 32) acc = fmaf(Elem<T>::to_f(o[row * D + c]), Elem<T>::to_f(dout[row * D + c]), acc);
  for (int off = 16; off; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[row] = acc;
}

__device__ __forceinline__ int visible_count(int64_t j0, int level, int64_t l_k, bool causal, int64_t qpos) {
  int64_t hi = l_k;
  if (causal && qpos + 1 < hi) hi = qpos + 1;
  int64_t c = hi - j0;
  return c < 0 ? 0 : (c > level ? level : (int)c);
}

// ------------------------------------------------------------------------------------------ dQ
template <typename T, int D>
__global__ void __launch_bounds__(512) bwd_dq_kernel(const T* __restrict__ q, BwdLevels lv, const int32_t* __restrict__ mask,
                                                    const float* __restrict__ lse, const float* __restrict__ delta,
                                                    const T* __restrict__ dout, T* __restrict__ dq, int64_t seq, int mask_cols,
                                                    int mq, float scale, int causal) {
  constexpr int DPT = D / 4;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float(*Ks)[D] = reinterpret_cast<float(*)[D]>(smem_raw);
  float(*Vs)[D] = Ks + 32;
  const int m = blockIdx.x;
  const int64_t bh = blockIdx.y;
  const int g = threadIdx.x & 3;
  const int64_t qrow = (int64_t)m * 128 + (threadIdx.x >> 2);
  const bool valid = qrow < seq;
  const int64_t s_pad = (seq + 127) / 128 * 128;
  float qv[DPT], dov[DPT], acc[DPT];
  const T* qp = q + (bh * seq + (valid ? qrow : 0)) * D;
  const T* dp_ = dout + (bh * seq + (valid ? qrow : 0)) * D;
#pragma unroll
  for (int d = 0; d < DPT; ++d) {
    qv[d] = valid ? Elem<T>::to_f(qp[d * 4 + g]) : 0.f;
    dov[d] = valid ? Elem<T>::to_f(dp_[d * 4 + g]) : 0.f;
    acc[d] = 0.f;
  }
  const float my_lse = valid ? lse[bh * seq + qrow] : 0.f;
  const float my_delta = valid ? delta[bh * seq + qrow] : 0.f;
  const int32_t* mrow = mask + (bh * mq + m) * (int64_t)mask_cols;
  const int nblk = (int)(s_pad / 128);
  for (int pb = 0; pb < nblk && pb < mask_cols; ++pb) {
    const int level = mrow[pb];
    int li;
    if (level == 1) li = 0; else if (level == 2) li = 1; else if (level == 4) li = 2; else if (level == 8) li = 3; else continue;
    if (causal && (int64_t)pb * 128 > (int64_t)m * 128 + 127) continue;   // nothing visible
    const int P = 128 / level;
    const int C = P < 32 ? P : 32;
    const T* Kl = (const T*)lv.k[li] + bh * lv.n[li] * D;
    const T* Vl = (const T*)lv.v[li] + bh * lv.n[li] * D;
    const int64_t l_k = level == 1 ? seq : s_pad;
    for (int c0 = 0; c0 < P; c0 += C) {
      const int64_t t0 = (int64_t)pb * P + c0;
      __syncthreads();
      for (int e = threadIdx.x; e < C * D; e += blockDim.x) {
        const int r = e / D, c = e % D;
        const bool ok = t0 + r < lv.n[li];
        Ks[r][c] = ok ? Elem<T>::to_f(Kl[(t0 + r) * D + c]) : 0.f;
        Vs[r][c] = ok ? Elem<T>::to_f(Vl[(t0 + r) * D + c]) : 0.f;
      }
      __syncthreads();
      for (int c = 0; c < C; ++c) {
        float s = 0.f, dpv = 0.f;
#pragma unroll
        for (int d = 0; d < DPT; ++d) {
          s = fmaf(qv[d], Ks[c][d * 4 + g], s);
          dpv = fmaf(dov[d], Vs[c][d * 4 + g], dpv);
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        dpv += __shfl_xor_sync(0xffffffffu, dpv, 1);
        dpv += __shfl_xor_sync(0xffffffffu, dpv, 2);
        const int cnt = valid ? visible_count((t0 + c) * level, level, l_k, causal != 0, qrow) : 0;
        if (cnt > 0) {
          const float pij = expf(s * scale - my_lse);
          const float ds = Elem<T>::round(pij * (dpv - my_delta)) * (float)cnt;
#pragma unroll
          for (int d = 0; d < DPT; ++d) acc[d] = fmaf(ds, Ks[c][d * 4 + g], acc[d]);
        }
      }
    }
  }
  if (valid) {
    T* o = dq + (bh * seq + qrow) * D;
#pragma unroll
    for (int d = 0; d < DPT; ++d) o[d * 4 + g] = Elem<T>::from_f(acc[d] * scale);
  }
}

// ------------------------------------------------------------------------------------------ dK, dV
// One CTA per 128-key block; 256 threads = 64 pooled tokens x 4 channel quarters per pass.
template <typename T, int D>
__global__ void __launch_bounds__(256) bwd_dkdv_kernel(const T* __restrict__ q, BwdLevels lv, const int32_t* __restrict__ mask,
                                                      const float* __restrict__ lse, const float* __restrict__ delta,
                                                      const T* __restrict__ dout, T* __restrict__ dk, T* __restrict__ dv,
                                                      int64_t seq, int mask_cols, int mq, float scale, int causal) {
  constexpr int DPT = D / 4;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float(*dKs)[D] = reinterpret_cast<float(*)[D]>(smem_raw);      // [128][D] gradients of the block's ORIGINAL positions
  float(*dVs)[D] = dKs + 128;
  float(*Qs)[D] = dVs + 128;                                       // [32][D] staged query rows
  float(*Ds)[D] = Qs + 32;                                         // [32][D] staged dO rows
  float* Ls = reinterpret_cast<float*>(Ds + 32);                   // [32] lse, [32] delta
  const int pb = blockIdx.x;
  const int64_t bh = blockIdx.y;
  const int g = threadIdx.x & 3, tl = threadIdx.x >> 2;           // token slot 0..63
  const int64_t s_pad = (seq + 127) / 128 * 128;
  for (int e = threadIdx.x; e < 128 * D; e += blockDim.x) { dKs[0][e] = 0.f; dVs[0][e] = 0.f; }
  const int32_t* mcol = mask + bh * mq * (int64_t)mask_cols + pb;

  for (int li = 0; li < 4; ++li) {
    const int level = 1 << li, P = 128 / level;
    // does any query block use this level for this key block?
    int any = 0;
    for (int m = threadIdx.x; m < mq; m += blockDim.x) any |= (mcol[(int64_t)m * mask_cols] == level);
    any = __syncthreads_or(any);
    if (!any) continue;
    const T* Kl = (const T*)lv.k[li] + bh * lv.n[li] * D;
    const T* Vl = (const T*)lv.v[li] + bh * lv.n[li] * D;
    const int64_t l_k = level == 1 ? seq : s_pad;
    for (int tp = 0; tp < P; tp += 64) {            // passes of 64 pooled tokens
      const int tloc = tp + tl;                     // pooled token inside the block
      const int64_t t = (int64_t)pb * P + tloc;
      const bool tok_ok = tloc < P && t < lv.n[li];
      float kv[DPT], vv[DPT], A[DPT], B[DPT];
#pragma unroll
      for (int d = 0; d < DPT; ++d) {
        kv[d] = tok_ok ? Elem<T>::to_f(Kl[t * D + d * 4 + g]) : 0.f;
        vv[d] = tok_ok ? Elem<T>::to_f(Vl[t * D + d * 4 + g]) : 0.f;
        A[d] = 0.f; B[d] = 0.f;
      }
      for (int m = 0; m < mq; ++m) {
        if (mcol[(int64_t)m * mask_cols] != level) continue;
        if (causal && (int64_t)m * 128 + 127 < (int64_t)pb * 128) continue;
        for (int r0 = 0; r0 < 128; r0 += 32) {
          const int64_t row0 = (int64_t)m * 128 + r0;
          if (row0 >= seq) break;
          __syncthreads();
          for (int e = threadIdx.x; e < 32 * D; e += blockDim.x) {
            const int r = e / D, c = e % D;
            const bool ok = row0 + r < seq;
            Qs[r][c] = ok ? Elem<T>::to_f(q[(bh * seq + row0 + r) * D + c]) : 0.f;
            Ds[r][c] = ok ? Elem<T>::to_f(dout[(bh * seq + row0 + r) * D + c]) : 0.f;
          }
          if (threadIdx.x < 32) {
            const bool ok = row0 + threadIdx.x < seq;
            Ls[threadIdx.x] = ok ? lse[bh * seq + row0 + threadIdx.x] : INFINITY;   // exp(-inf) = 0 for missing rows
            Ls[32 + threadIdx.x] = ok ? delta[bh * seq + row0 + threadIdx.x] : 0.f;
          }
          __syncthreads();
          for (int r = 0; r < 32; ++r) {
            float s = 0.f, dpv = 0.f;
#pragma unroll
            for (int d = 0; d < DPT; ++d) {
              s = fmaf(kv[d], Qs[r][d * 4 + g], s);
              dpv = fmaf(vv[d], Ds[r][d * 4 + g], dpv);
            }
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            dpv += __shfl_xor_sync(0xffffffffu, dpv, 1);
            dpv += __shfl_xor_sync(0xffffffffu, dpv, 2);
            const int cnt = (tok_ok && row0 + r < seq) ? visible_count(t * level, level, l_k, causal != 0, row0 + r) : 0;
            if (cnt > 0) {
              const float pij = expf(s * scale - Ls[r]);
              const float pc = Elem<T>::round(pij) * (float)cnt;
              const float ds = Elem<T>::round(pij * (dpv - Ls[32 + r])) * (float)cnt;
#pragma unroll
              for (int d = 0; d < DPT; ++d) {
                A[d] = fmaf(ds, Qs[r][d * 4 + g], A[d]);
                B[d] = fmaf(pc, Ds[r][d * 4 + g], B[d]);
              }
            }
          }
        }
      }
      // spread the pooled token's gradient over its l original positions (mean-pool backward)
      __syncthreads();
      if (tok_ok) {
        const float wk = scale / (float)level, wv = 1.0f / (float)level;
        for (int jj = 0; jj < level; ++jj) {
          const int jloc = tloc * level + jj;      // original position inside the block
#pragma unroll
          for (int d = 0; d < DPT; ++d) {
            dKs[jloc][d * 4 + g] += A[d] * wk;
            dVs[jloc][d * 4 + g] += B[d] * wv;
          }
        }
      }
      __syncthreads();
    }
  }
  __syncthreads();
  // replicate-pad tail: positions >= seq hand their gradient to token seq-1 (which lives in this block)
  const int64_t j0 = (int64_t)pb * 128;
  if (j0 + 128 > seq && j0 < seq) {
    const int last = (int)(seq - 1 - j0);
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      float ak = 0.f, av = 0.f;
      for (int jl = last + 1; jl < 128; ++jl) { ak += dKs[jl][c]; av += dVs[jl][c]; }
      dKs[last][c] += ak;
      dVs[last][c] += av;
    }
    __syncthreads();
  }
  for (int e = threadIdx.x; e < 128 * D; e += blockDim.x) {
    const int jl = e / D, c = e % D;
    if (j0 + jl < seq) {
      dk[(bh * seq + j0 + jl) * D + c] = Elem<T>::from_f(dKs[jl][c]);
      dv[(bh * seq + j0 + jl) * D + c] = Elem<T>::from_f(dVs[jl][c]);
    }
  }
}

template <typename T, int D>
static int launch_bwd(const void* q, const BwdLevels& lv, const int32_t* mask, const void* out, const float* lse, const void* dout,
                      void* dq, void* dk, void* dv, float* delta, int64_t bh, int64_t seq, int mask_cols, float scale, int causal,
                      cudaStream_t st) {
  const int mq = (int)cdiv64(seq, 128);
  const int64_t rows = bh * seq;
  bwd_delta_kernel<T><<<(unsigned)cdiv64(rows, 8), 256, 0, st>>>((const T*)out, (const T*)dout, delta, rows, D);
  PSA_CHECK_LAUNCH("psa_legacy_bwd(delta)");
  {
    const size_t smem = 2 * 32 * D * sizeof(float);
    dim3 grid(mq, (unsigned)bh);
    bwd_dq_kernel<T, D><<<grid, 512, smem, st>>>((const T*)q, lv, mask, lse, delta, (const T*)dout, (T*)dq, seq, mask_cols, mq, scale,
                                                  causal);
    PSA_CHECK_LAUNCH("psa_legacy_bwd(dq)");
  }
  {
    const size_t smem = (size_t)(2 * 128 + 2 * 32) * D * sizeof(float) + 64 * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(bwd_dkdv_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_legacy_bwd: smem opt-in failed: %s", cudaGetErrorString(e));
    dim3 grid(mq, (unsigned)bh);      // key blocks of 128 = same count as query blocks
    bwd_dkdv_kernel<T, D><<<grid, 256, smem, st>>>((const T*)q, lv, mask, lse, delta, (const T*)dout, (T*)dk, (T*)dv, seq, mask_cols,
                                                    mq, scale, causal);
    PSA_CHECK_LAUNCH("psa_legacy_bwd(dkdv)");
  }
  return PSA_OK;
}

}  // namespace psa

extern "C" int psa_legacy_bwd(const void* q, const void* k, const void* v, const void* k2, const void* k4, const void* k8,
                              const void* v2, const void* v4, const void* v8, const int32_t* mask, const void* out,
                              const float* lse, const void* dout, void* dq, void* dk, void* dv, float* delta, int64_t bh,
                              int64_t seq, int head_dim, int mask_cols, float sm_scale, int causal, int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && k && v && k2 && k4 && k8 && v2 && v4 && v8 && mask && out && lse && dout && dq && dk && dv && delta, PSA_ERR_ARG,
              "psa_legacy_bwd: null pointer");
  PSA_REQUIRE(head_dim == 64 || head_dim == 128, PSA_ERR_ARG, "psa_legacy_bwd: head_dim=%d (must be 64 or 128)", head_dim);
  PSA_REQUIRE(bh > 0 && bh < 65536 && seq > 0, PSA_ERR_ARG, "psa_legacy_bwd: bad shape");
  PSA_REQUIRE(mask_cols >= cdiv64(seq, 128), PSA_ERR_ARG, "psa_legacy_bwd: mask has %d columns, needs %lld", mask_cols,
              (long long)cdiv64(seq, 128));
  const int64_t s_pad = cdiv64(seq, 128) * 128;
  BwdLevels lv;
  const void* kl[4] = {k, k2, k4, k8};
  const void* vl[4] = {v, v2, v4, v8};
  const int64_t nl[4] = {seq, s_pad / 2, s_pad / 4, s_pad / 8};
  for (int i = 0; i < 4; ++i) { lv.k[i] = kl[i]; lv.v[i] = vl[i]; lv.n[i] = nl[i]; }
  cudaStream_t st = (cudaStream_t)stream;
  PSA_DISPATCH_DTYPE(dtype, T, {
    if (head_dim == 64)
      return launch_bwd<T, 64>(q, lv, mask, out, lse, dout, dq, dk, dv, delta, bh, seq, mask_cols, sm_scale, causal, st);
    return launch_bwd<T, 128>(q, lv, mask, out, lse, dout, dq, dk, dv, delta, bh, seq, mask_cols, sm_scale, causal, st);
  });
  return PSA_OK;
}
