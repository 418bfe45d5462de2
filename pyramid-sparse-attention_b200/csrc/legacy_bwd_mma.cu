// Legacy (old-format mask) attention backward on tensor cores (warp-level mma.sync, f16/bf16 operands, fp32
// accumulation).  Same mathematics as the scalar kernels in legacy_bwd.cu, whose header derives it: a pooled token t of
// level l stands for l identical expanded keys, of which c_t(i) exist and are visible to query row i, so
//   ds_it = round(p_it (dO_i.v_t - delta_i)) c_t(i),   pc_it = round(p_it) c_t(i),   p_it = exp(q_i.k_t scale - lse_i)
//   dQ_i = scale sum_t ds_it k_t,   dK_j (j in t) += scale / l sum_i ds_it q_i,   dV_j (j in t) += 1 / l sum_i pc_it dO_i
// with round() to the element type where the reference casts before its products.  (The products ds c and p c are
// rounded once more when they become tensor-core operands; that only changes values where c is 3, 5, 6 or 7, i.e. on
// the causal diagonal and in the replicate-padded tail.)
//
// dQ: one CTA per 128 query rows, a warp per 16 rows with its Q and dO fragments in registers; the selected key blocks
// stream through 32 pooled tokens at a time (copied asynchronously, double-buffered).  dK/dV: one CTA per 128-key block; per level the block's pooled K and V sit in shared
// memory, a warp owns 16 pooled tokens and keeps their dK and dV in registers while the query rows of every block that
// selected this level stream through in chunks of 16 (copied asynchronously, double-buffered); the result is spread over the original positions in fp32 shared
// memory (mean-pool backward), the replicate-padded tail is folded into the last token, one rounding at the end.
#include "mma_sync.cuh"

namespace psa {
namespace {

struct BwdLv {
  const void* k[4];
  const void* v[4];
  int64_t n[4];
};

__device__ __forceinline__ int visible_cnt(int64_t j0, int level, int64_t l_k, bool causal, int64_t qpos) {
  int64_t hi = l_k;
  if (causal && qpos + 1 < hi) hi = qpos + 1;
  const int64_t c = hi - j0;
  return c < 0 ? 0 : (c > level ? level : (int)c);
}

// Stage `rows` rows of D 16-bit channels ([r][D+8] in shared memory); rows failing ok(r) are zero.
template <int D, typename F>
__device__ __forceinline__ void stage_rows(unsigned short* dst, const unsigned short* __restrict__ src, int rows, F ok) {
  constexpr int PITCH = D + 8, WPR = D / 8;
  for (int e = threadIdx.x; e < rows * WPR; e += blockDim.x) {
    const int r = e / WPR, c = e - r * WPR;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (ok(r)) val = *reinterpret_cast<const uint4*>(src + (int64_t)r * D + c * 8);
    *reinterpret_cast<uint4*>(dst + r * PITCH + c * 8) = val;
  }
}

// The same with asynchronous copies (cp.async, zero fill for the rows failing ok(r)); `safe` is any valid address of the
// source tensor.  The caller commits the group and waits for it before the rows are read.
template <int D, typename F>
__device__ __forceinline__ void stage_rows_async(unsigned short* dst, const unsigned short* __restrict__ src,
                                                 const unsigned short* __restrict__ safe, int rows, F ok) {
  constexpr int PITCH = D + 8, WPR = D / 8;
  for (int e = threadIdx.x; e < rows * WPR; e += blockDim.x) {
    const int r = e / WPR, c = e - r * WPR;
    const bool v = ok(r);
    const unsigned short* from = v ? src + (int64_t)r * D + c * 8 : safe;
    const uint32_t to = (uint32_t)__cvta_generic_to_shared(dst + r * PITCH + c * 8);
    const int bytes = v ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(to), "l"(from), "r"(bytes) : "memory");
  }
}
__device__ __forceinline__ void async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// C = A(16 x D, rows g / g+8 of `a_rows`) . B^T(8 tokens x D, row g of `b_rows`), both [row][D+8] in shared memory.
template <typename T, int D>
__device__ __forceinline__ void dot_rows(float (&c)[4], const unsigned short* a_rows, const unsigned short* b_row, int tig) {
  constexpr int PITCH = D + 8;
#pragma unroll
  for (int k0 = 0; k0 < D; k0 += 16) {
    uint32_t a[4], b[2];
    const unsigned short* ap = a_rows + k0 + tig * 2;
    a[0] = *reinterpret_cast<const uint32_t*>(ap);
    a[1] = *reinterpret_cast<const uint32_t*>(ap + 8 * PITCH);
    a[2] = *reinterpret_cast<const uint32_t*>(ap + 8);
    a[3] = *reinterpret_cast<const uint32_t*>(ap + 8 * PITCH + 8);
    const unsigned short* bp = b_row + k0 + tig * 2;
    b[0] = *reinterpret_cast<const uint32_t*>(bp);
    b[1] = *reinterpret_cast<const uint32_t*>(bp + 8);
    MmaOp<T>::run(c, a, b);
  }
}

// ------------------------------------------------------------------------------------------ dQ
template <typename T, int D>
__global__ void __launch_bounds__(256) bwd_dq_mma_kernel(const T* __restrict__ q, BwdLv lv, const int32_t* __restrict__ mask,
                                                        const float* __restrict__ lse, const float* __restrict__ delta,
                                                        const T* __restrict__ dout, T* __restrict__ dq, int64_t seq, int mask_cols,
                                                        int mq, float scale, int causal) {
  constexpr int PITCH = D + 8, KS = D / 16, ND = D / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned short* Ks = reinterpret_cast<unsigned short*>(smem_raw);   // [2 buffers][32][PITCH]
  unsigned short* Vs = Ks + 2 * 32 * PITCH;
  const int m = blockIdx.x;
  const int64_t bh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int64_t s_pad = (seq + 127) / 128 * 128;
  const int64_t row0 = (int64_t)m * 128 + warp * 16 + g, row1 = row0 + 8;
  const bool ok0 = row0 < seq, ok1 = row1 < seq;

  // A fragments of this warp's 16 query rows and their dO rows, straight from global memory
  uint32_t qa[KS][4], da[KS][4];
  {
    const unsigned short* q0 = reinterpret_cast<const unsigned short*>(q) + (bh * seq + (ok0 ? row0 : 0)) * D;
    const unsigned short* q1 = reinterpret_cast<const unsigned short*>(q) + (bh * seq + (ok1 ? row1 : 0)) * D;
    const unsigned short* d0 = reinterpret_cast<const unsigned short*>(dout) + (bh * seq + (ok0 ? row0 : 0)) * D;
    const unsigned short* d1 = reinterpret_cast<const unsigned short*>(dout) + (bh * seq + (ok1 ? row1 : 0)) * D;
#pragma unroll
    for (int k = 0; k < KS; ++k) {
      const int c = k * 16 + tig * 2;
      qa[k][0] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + c) : 0u;
      qa[k][1] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + c) : 0u;
      qa[k][2] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + c + 8) : 0u;
      qa[k][3] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + c + 8) : 0u;
      da[k][0] = ok0 ? *reinterpret_cast<const uint32_t*>(d0 + c) : 0u;
      da[k][1] = ok1 ? *reinterpret_cast<const uint32_t*>(d1 + c) : 0u;
      da[k][2] = ok0 ? *reinterpret_cast<const uint32_t*>(d0 + c + 8) : 0u;
      da[k][3] = ok1 ? *reinterpret_cast<const uint32_t*>(d1 + c + 8) : 0u;
    }
  }
  const float lse0 = ok0 ? lse[bh * seq + row0] : 0.f, lse1 = ok1 ? lse[bh * seq + row1] : 0.f;
  const float del0 = ok0 ? delta[bh * seq + row0] : 0.f, del1 = ok1 ? delta[bh * seq + row1] : 0.f;
  float acc[ND][4];
#pragma unroll
  for (int n = 0; n < ND; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;

  const int32_t* mrow = mask + (bh * mq + m) * (int64_t)mask_cols;
  const int nblk = (int)(s_pad / 128);
  // The selected key blocks form one stream of 32-token chunks; chunk i+1 is copied (cp.async) while chunk i is used.
  struct Chunk { int pb, c0, level, li; };
  auto find_chunk = [&](int pb, int c0, Chunk& ch) -> bool {
    for (; pb < nblk && pb < mask_cols; ++pb, c0 = 0) {
      const int level = mrow[pb];
      int li;
      if (level == 1) li = 0; else if (level == 2) li = 1; else if (level == 4) li = 2; else if (level == 8) li = 3; else continue;
      if (causal && (int64_t)pb * 128 > (int64_t)m * 128 + 127) continue;   // nothing visible
      if (c0 >= 128 / level) continue;
      ch.pb = pb; ch.c0 = c0; ch.level = level; ch.li = li;
      return true;
    }
    return false;
  };
  auto issue = [&](const Chunk& ch, int buf) {
    const int P = 128 / ch.level;
    const unsigned short* Kl = reinterpret_cast<const unsigned short*>(lv.k[ch.li]) + bh * lv.n[ch.li] * D;
    const unsigned short* Vl = reinterpret_cast<const unsigned short*>(lv.v[ch.li]) + bh * lv.n[ch.li] * D;
    const int64_t t0 = (int64_t)ch.pb * P + ch.c0, n_l = lv.n[ch.li];
    const int c0 = ch.c0;
    auto tok_ok = [&](int r) { return c0 + r < P && t0 + r < n_l; };
    stage_rows_async<D>(Ks + buf * 32 * PITCH, Kl + t0 * D, Kl, 32, tok_ok);
    stage_rows_async<D>(Vs + buf * 32 * PITCH, Vl + t0 * D, Vl, 32, tok_ok);
  };
  Chunk cur, nxt;
  bool has = find_chunk(0, 0, cur);
  if (has) issue(cur, 0);
  async_commit();
  for (int buf = 0; has; buf ^= 1) {
    const bool has_next = find_chunk(cur.pb, cur.c0 + 32, nxt);
    async_wait_all();
    __syncthreads();   // chunk `cur` has landed for everyone, and everyone is done with the other buffer
    if (has_next) issue(nxt, buf ^ 1);
    async_commit();
    {
      const int level = cur.level, P = 128 / level, c0 = cur.c0;
      const int64_t l_k = level == 1 ? seq : s_pad;
      const int64_t t0 = (int64_t)cur.pb * P + c0, n_l = lv.n[cur.li];
      auto tok_ok = [&](int r) { return c0 + r < P && t0 + r < n_l; };
      const unsigned short* Kb = Ks + buf * 32 * PITCH;
      const unsigned short* Vb = Vs + buf * 32 * PITCH;
      // CTA-uniform: the chunk holds 32 existing pooled tokens whose original positions all exist and lie before the
      // first row of this query block (or the call is not causal), and the query block has no missing rows
      const bool whole = (!causal || cur.pb < m) && c0 + 32 <= P && t0 + 32 <= n_l && (t0 + 32) * level <= l_k &&
                         (int64_t)m * 128 + 128 <= seq;
      // S = Q K^T and dP = dO V^T for 16 rows x 32 tokens, then ds in the accumulator layout
      uint32_t dsa[2][4];
      // the eight products (4 token tiles x {S, dP}) advance together: independent accumulators keep the pipe busy
      float s4[4][4], dp4[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) { s4[nt][e] = 0.f; dp4[nt][e] = 0.f; }
#pragma unroll
      for (int k = 0; k < KS; ++k)
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          uint32_t b[2];
          const unsigned short* kp = Kb + (nt * 8 + g) * PITCH + k * 16 + tig * 2;
          b[0] = *reinterpret_cast<const uint32_t*>(kp);
          b[1] = *reinterpret_cast<const uint32_t*>(kp + 8);
          MmaOp<T>::run(s4[nt], qa[k], b);
          const unsigned short* vp = Vb + (nt * 8 + g) * PITCH + k * 16 + tig * 2;
          b[0] = *reinterpret_cast<const uint32_t*>(vp);
          b[1] = *reinterpret_cast<const uint32_t*>(vp + 8);
          MmaOp<T>::run(dp4[nt], da[k], b);
        }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const float(&s)[4] = s4[nt];
        const float(&dp)[4] = dp4[nt];
        float val[4];
        if (whole) {
          // every copy of every token of the chunk exists and is visible to every row of this query block
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const bool hi = e >= 2;
            const float pij = expf(s[e] * scale - (hi ? lse1 : lse0));
            val[e] = Elem<T>::round(pij * (dp[e] - (hi ? del1 : del0))) * (float)level;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int tok = nt * 8 + tig * 2 + (e & 1);
            const bool hi = e >= 2;
            const bool rok = hi ? ok1 : ok0;
            const int cnt = (rok && tok_ok(tok)) ? visible_cnt((t0 + tok) * level, level, l_k, causal != 0, hi ? row1 : row0) : 0;
            float x = 0.f;
            if (cnt > 0) {
              const float pij = expf(s[e] * scale - (hi ? lse1 : lse0));
              x = Elem<T>::round(pij * (dp[e] - (hi ? del1 : del0))) * (float)cnt;
            }
            val[e] = x;
          }
        }
        // two neighbouring 8-token tiles form the A fragment of one 16-token k-step
        dsa[nt >> 1][(nt & 1) * 2 + 0] = MmaOp<T>::pack(val[0], val[1]);
        dsa[nt >> 1][(nt & 1) * 2 + 1] = MmaOp<T>::pack(val[2], val[3]);
      }
      // dQ += ds K  (K as [token][channel]: transposed fragment loads)
#pragma unroll
      for (int ks = 0; ks < 2; ++ks)
#pragma unroll
        for (int n = 0; n < ND; ++n) {
          uint32_t b[2];
          ldsm_x2_trans(b, Kb + (ks * 16 + (lane & 15)) * PITCH + n * 8);
          MmaOp<T>::run(acc[n], dsa[ks], b);
        }
    }
    cur = nxt;
    has = has_next;
  }
  unsigned short* o0 = reinterpret_cast<unsigned short*>(dq) + (bh * seq + row0) * D;
  unsigned short* o1 = reinterpret_cast<unsigned short*>(dq) + (bh * seq + row1) * D;
#pragma unroll
  for (int n = 0; n < ND; ++n) {
    if (ok0) *reinterpret_cast<uint32_t*>(o0 + n * 8 + tig * 2) = MmaOp<T>::pack(acc[n][0] * scale, acc[n][1] * scale);
    if (ok1) *reinterpret_cast<uint32_t*>(o1 + n * 8 + tig * 2) = MmaOp<T>::pack(acc[n][2] * scale, acc[n][3] * scale);
  }
}

// ------------------------------------------------------------------------------------------ dK, dV
template <typename T, int D>
__global__ void __launch_bounds__(256) bwd_dkdv_mma_kernel(const T* __restrict__ q, BwdLv lv, const int32_t* __restrict__ mask,
                                                          const float* __restrict__ lse, const float* __restrict__ delta,
                                                          const T* __restrict__ dout, T* __restrict__ dk, T* __restrict__ dv,
                                                          int64_t seq, int mask_cols, int mq, float scale, int causal) {
  constexpr int PITCH = D + 8, ND = D / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float(*dKs)[D] = reinterpret_cast<float(*)[D]>(smem_raw);      // [128][D] gradients of the block's ORIGINAL positions
  float(*dVs)[D] = dKs + 128;
  unsigned short* Kls = reinterpret_cast<unsigned short*>(dVs + 128);   // [128][PITCH] pooled K of the current level
  unsigned short* Vls = Kls + 128 * PITCH;
  constexpr int RC = 16;                                                 // query rows per staged chunk
  unsigned short* Qs = Vls + 128 * PITCH;                                // [2 buffers][RC][PITCH] staged query rows
  unsigned short* Ds = Qs + 2 * RC * PITCH;                              // [2 buffers][RC][PITCH] staged dO rows
  float* Ls = reinterpret_cast<float*>(Ds + 2 * RC * PITCH);             // [2 buffers]: [RC] lse, [RC] delta
  unsigned char* flags = reinterpret_cast<unsigned char*>(Ls + 4 * RC);  // [mq] query blocks that use the current level
  const int pb = blockIdx.x;
  const int64_t bh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tig = lane & 3;
  const int64_t s_pad = (seq + 127) / 128 * 128;
  for (int e = threadIdx.x; e < 128 * D; e += blockDim.x) { dKs[0][e] = 0.f; dVs[0][e] = 0.f; }
  const int32_t* mcol = mask + bh * mq * (int64_t)mask_cols + pb;
  const unsigned short* qg = reinterpret_cast<const unsigned short*>(q) + bh * seq * D;
  const unsigned short* dg = reinterpret_cast<const unsigned short*>(dout) + bh * seq * D;

  for (int li = 0; li < 4; ++li) {
    const int level = 1 << li, P = 128 / level;
    // which query blocks selected this level for this key block (one pass over the mask column, kept in shared memory)
    int any = 0;
    for (int mm = threadIdx.x; mm < mq; mm += blockDim.x) {
      const bool f = mcol[(int64_t)mm * mask_cols] == level && !(causal && (int64_t)mm * 128 + 127 < (int64_t)pb * 128);
      flags[mm] = f ? 1 : 0;
      any |= f ? 1 : 0;
    }
    any = __syncthreads_or(any);
    if (!any) continue;
    const unsigned short* Kl = reinterpret_cast<const unsigned short*>(lv.k[li]) + bh * lv.n[li] * D;
    const unsigned short* Vl = reinterpret_cast<const unsigned short*>(lv.v[li]) + bh * lv.n[li] * D;
    const int64_t l_k = level == 1 ? seq : s_pad;
    const int64_t t0 = (int64_t)pb * P, n_l = lv.n[li];
    auto tok_ok = [&](int r) { return r < P && t0 + r < n_l; };
    stage_rows<D>(Kls, Kl + t0 * D, 128, tok_ok);
    stage_rows<D>(Vls, Vl + t0 * D, 128, tok_ok);
    const bool active = warp * 16 < P;                      // this warp's 16 pooled tokens exist at this level
    const int tk0 = warp * 16 + g, tk1 = tk0 + 8;           // my two token rows
    float aK[ND][4], aV[ND][4];
#pragma unroll
    for (int n = 0; n < ND; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) { aK[n][e] = 0.f; aV[n][e] = 0.f; }

    // The query rows of every block that selected this level form one stream of RC-row chunks; chunk i+1 is copied
    // (cp.async) while chunk i is used.
    struct RowChunk { int mm, r0; };
    auto find_rows = [&](int mm, int r0, RowChunk& c) -> bool {
      for (; mm < mq; ++mm, r0 = 0) {
        if (!flags[mm]) continue;
        if (r0 >= 128 || (int64_t)mm * 128 + r0 >= seq) continue;
        c.mm = mm; c.r0 = r0;
        return true;
      }
      return false;
    };
    auto issue = [&](const RowChunk& c, int buf) {
      const int64_t row0 = (int64_t)c.mm * 128 + c.r0;
      auto row_ok = [&](int r) { return row0 + r < seq; };
      stage_rows_async<D>(Qs + buf * RC * PITCH, qg + row0 * D, qg, RC, row_ok);
      stage_rows_async<D>(Ds + buf * RC * PITCH, dg + row0 * D, dg, RC, row_ok);
      if (threadIdx.x < RC) {
        const bool ok = row0 + threadIdx.x < seq;
        Ls[buf * 2 * RC + threadIdx.x] = ok ? lse[bh * seq + row0 + threadIdx.x] : INFINITY;   // exp(-inf) = 0 for missing rows
        Ls[buf * 2 * RC + RC + threadIdx.x] = ok ? delta[bh * seq + row0 + threadIdx.x] : 0.f;
      }
    };
    RowChunk cur, nxt;
    bool has = find_rows(0, 0, cur);
    if (has) issue(cur, 0);
    async_commit();
    for (int buf = 0; has; buf ^= 1) {
      const bool has_next = find_rows(cur.mm, cur.r0 + RC, nxt);
      async_wait_all();
      __syncthreads();   // chunk `cur` (and, first time, the level's K/V) is in place; the other buffer is free
      if (has_next) issue(nxt, buf ^ 1);
      async_commit();
      if (active) {
        const int64_t row0 = (int64_t)cur.mm * 128 + cur.r0;
        auto row_ok = [&](int r) { return row0 + r < seq; };
        const unsigned short* Qb = Qs + buf * RC * PITCH;
        const unsigned short* Db = Ds + buf * RC * PITCH;
        const float* Lb = Ls + buf * 2 * RC;
        // CTA-uniform: the key block is complete (no padded positions) and lies before the query block (or the call is
        // not causal), and the chunk has no missing rows
        const bool whole = (!causal || cur.mm > pb) && (int64_t)pb * 128 + 128 <= seq && row0 + RC <= seq;
        // S^T = K Q^T and dP^T = V dO^T for 16 tokens x RC query rows
        uint32_t pa[RC / 16][4], dsa[RC / 16][4];
        float s2[RC / 8][4], dp2[RC / 8][4];
#pragma unroll
        for (int nt = 0; nt < RC / 8; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) { s2[nt][e] = 0.f; dp2[nt][e] = 0.f; }
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16) {
          uint32_t ak[4], av[4];
          const unsigned short* kp = Kls + tk0 * PITCH + k0 + tig * 2;
          const unsigned short* vp = Vls + tk0 * PITCH + k0 + tig * 2;
          ak[0] = *reinterpret_cast<const uint32_t*>(kp);
          ak[1] = *reinterpret_cast<const uint32_t*>(kp + 8 * PITCH);
          ak[2] = *reinterpret_cast<const uint32_t*>(kp + 8);
          ak[3] = *reinterpret_cast<const uint32_t*>(kp + 8 * PITCH + 8);
          av[0] = *reinterpret_cast<const uint32_t*>(vp);
          av[1] = *reinterpret_cast<const uint32_t*>(vp + 8 * PITCH);
          av[2] = *reinterpret_cast<const uint32_t*>(vp + 8);
          av[3] = *reinterpret_cast<const uint32_t*>(vp + 8 * PITCH + 8);
#pragma unroll
          for (int nt = 0; nt < RC / 8; ++nt) {
            uint32_t b[2];
            const unsigned short* qp = Qb + (nt * 8 + g) * PITCH + k0 + tig * 2;
            b[0] = *reinterpret_cast<const uint32_t*>(qp);
            b[1] = *reinterpret_cast<const uint32_t*>(qp + 8);
            MmaOp<T>::run(s2[nt], ak, b);
            const unsigned short* dp_ = Db + (nt * 8 + g) * PITCH + k0 + tig * 2;
            b[0] = *reinterpret_cast<const uint32_t*>(dp_);
            b[1] = *reinterpret_cast<const uint32_t*>(dp_ + 8);
            MmaOp<T>::run(dp2[nt], av, b);
          }
        }
#pragma unroll
        for (int nt = 0; nt < RC / 8; ++nt) {
          const float(&s)[4] = s2[nt];
          const float(&dp)[4] = dp2[nt];
          float pv[4], dv_[4];
          if (whole) {
            // all copies of the block's tokens exist and are visible to all rows of the chunk
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int r = nt * 8 + tig * 2 + (e & 1);
              const float pij = expf(s[e] * scale - Lb[r]);
              pv[e] = Elem<T>::round(pij) * (float)level;
              dv_[e] = Elem<T>::round(pij * (dp[e] - Lb[RC + r])) * (float)level;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int r = nt * 8 + tig * 2 + (e & 1);       // query row inside the chunk
              const int tk = e >= 2 ? tk1 : tk0;
              const int cnt = (tok_ok(tk) && row_ok(r)) ? visible_cnt((t0 + tk) * level, level, l_k, causal != 0, row0 + r) : 0;
              float x = 0.f, y = 0.f;
              if (cnt > 0) {
                const float pij = expf(s[e] * scale - Lb[r]);
                x = Elem<T>::round(pij) * (float)cnt;
                y = Elem<T>::round(pij * (dp[e] - Lb[RC + r])) * (float)cnt;
              }
              pv[e] = x; dv_[e] = y;
            }
          }
          pa[nt >> 1][(nt & 1) * 2 + 0] = MmaOp<T>::pack(pv[0], pv[1]);
          pa[nt >> 1][(nt & 1) * 2 + 1] = MmaOp<T>::pack(pv[2], pv[3]);
          dsa[nt >> 1][(nt & 1) * 2 + 0] = MmaOp<T>::pack(dv_[0], dv_[1]);
          dsa[nt >> 1][(nt & 1) * 2 + 1] = MmaOp<T>::pack(dv_[2], dv_[3]);
        }
        // dV_l += p^T dO,  dK_l += ds^T Q  (k = the RC query rows)
#pragma unroll
        for (int ks = 0; ks < RC / 16; ++ks)
#pragma unroll
          for (int n = 0; n < ND; ++n) {
            uint32_t b[2];
            ldsm_x2_trans(b, Db + (ks * 16 + (lane & 15)) * PITCH + n * 8);
            MmaOp<T>::run(aV[n], pa[ks], b);
            ldsm_x2_trans(b, Qb + (ks * 16 + (lane & 15)) * PITCH + n * 8);
            MmaOp<T>::run(aK[n], dsa[ks], b);
          }
      }
      cur = nxt;
      has = has_next;
    }
    // spread the pooled tokens' gradients over their l original positions (mean-pool backward)
    __syncthreads();
    if (active) {
      const float wk = scale / (float)level, wv = 1.0f / (float)level;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int tk = h ? tk1 : tk0;
        if (tok_ok(tk)) {
          for (int jj = 0; jj < level; ++jj) {
            const int jloc = tk * level + jj;
#pragma unroll
            for (int n = 0; n < ND; ++n) {
              const int c = n * 8 + tig * 2;
              dKs[jloc][c] += aK[n][h * 2] * wk;
              dKs[jloc][c + 1] += aK[n][h * 2 + 1] * wk;
              dVs[jloc][c] += aV[n][h * 2] * wv;
              dVs[jloc][c + 1] += aV[n][h * 2 + 1] * wv;
            }
          }
        }
      }
    }
    __syncthreads();
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

template <typename T>
__global__ void __launch_bounds__(256) bwd_delta_mma_kernel(const T* __restrict__ o, const T* __restrict__ dout, float* __restrict__ delta,
                                                           int64_t rows, int D) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;
  if (row >= rows) return;
  float acc = 0.f;
  for (int c = lane; c < D; c += 32) acc = fmaf(Elem<T>::to_f(o[row * D + c]), Elem<T>::to_f(dout[row * D + c]), acc);
  for (int off = 16; off; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[row] = acc;
}

template <typename T, int D>
int launch_bwd_mma(const void* q, const BwdLv& lv, const int32_t* mask, const void* out, const float* lse, const void* dout, void* dq,
                   void* dk, void* dv, float* delta, int64_t bh, int64_t seq, int mask_cols, float scale, int causal, cudaStream_t st) {
  constexpr int PITCH = D + 8;
  const int mq = (int)cdiv64(seq, 128);
  const int64_t rows = bh * seq;
  bwd_delta_mma_kernel<T><<<(unsigned)cdiv64(rows, 8), 256, 0, st>>>((const T*)out, (const T*)dout, delta, rows, D);
  PSA_CHECK_LAUNCH("psa_legacy_bwd_tc(delta)");
  dim3 grid(mq, (unsigned)bh);
  {
    const size_t smem = (size_t)2 * 2 * 32 * PITCH * 2;
    bwd_dq_mma_kernel<T, D><<<grid, 256, smem, st>>>((const T*)q, lv, mask, lse, delta, (const T*)dout, (T*)dq, seq, mask_cols, mq,
                                                      scale, causal);
    PSA_CHECK_LAUNCH("psa_legacy_bwd_tc(dq)");
  }
  {
    const size_t smem = (size_t)2 * 128 * D * sizeof(float) + (size_t)(2 * 128 + 2 * 32) * PITCH * 2 + 64 * sizeof(float) +
                        (((size_t)mq + 15) & ~(size_t)15);
    PSA_REQUIRE(smem <= 227 * 1024, PSA_ERR_UNSUPPORTED, "psa_legacy_bwd_tc: %d query blocks exceed the kernel's shared memory", mq);
    cudaError_t e = cudaFuncSetAttribute(bwd_dkdv_mma_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_legacy_bwd_tc: smem opt-in failed: %s", cudaGetErrorString(e));
    bwd_dkdv_mma_kernel<T, D><<<grid, 256, smem, st>>>((const T*)q, lv, mask, lse, delta, (const T*)dout, (T*)dk, (T*)dv, seq,
                                                        mask_cols, mq, scale, causal);
    PSA_CHECK_LAUNCH("psa_legacy_bwd_tc(dkdv)");
  }
  return PSA_OK;
}

}  // namespace
}  // namespace psa

extern "C" int psa_legacy_bwd_tc(const void* q, const void* k, const void* v, const void* k2, const void* k4, const void* k8,
                                 const void* v2, const void* v4, const void* v8, const int32_t* mask, const void* out,
                                 const float* lse, const void* dout, void* dq, void* dk, void* dv, float* delta, int64_t bh,
                                 int64_t seq, int head_dim, int mask_cols, float sm_scale, int causal, int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && k && v && k2 && k4 && k8 && v2 && v4 && v8 && mask && out && lse && dout && dq && dk && dv && delta, PSA_ERR_ARG,
              "psa_legacy_bwd_tc: null pointer");
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "psa_legacy_bwd_tc: f16/bf16 only");
  PSA_REQUIRE(head_dim == 64 || head_dim == 128, PSA_ERR_ARG, "psa_legacy_bwd_tc: head_dim=%d (must be 64 or 128)", head_dim);
  PSA_REQUIRE(bh > 0 && bh < 65536 && seq > 0, PSA_ERR_ARG, "psa_legacy_bwd_tc: bad shape");
  PSA_REQUIRE(mask_cols >= cdiv64(seq, 128), PSA_ERR_ARG, "psa_legacy_bwd_tc: mask has %d columns, needs %lld", mask_cols,
              (long long)cdiv64(seq, 128));
  const void* all[] = {q, k, v, k2, k4, k8, v2, v4, v8, dout, dq};
  for (const void* ptr : all) PSA_REQUIRE(((uintptr_t)ptr & 15) == 0, PSA_ERR_ARG, "psa_legacy_bwd_tc: tensors must be 16-byte aligned");
  const int64_t s_pad = cdiv64(seq, 128) * 128;
  BwdLv lv;
  const void* kl[4] = {k, k2, k4, k8};
  const void* vl[4] = {v, v2, v4, v8};
  const int64_t nl[4] = {seq, s_pad / 2, s_pad / 4, s_pad / 8};
  for (int i = 0; i < 4; ++i) { lv.k[i] = kl[i]; lv.v[i] = vl[i]; lv.n[i] = nl[i]; }
  cudaStream_t st = (cudaStream_t)stream;
#define PSA_BWD_TC(TT)                                                                                                        \
  (head_dim == 64 ? launch_bwd_mma<TT, 64>(q, lv, mask, out, lse, dout, dq, dk, dv, delta, bh, seq, mask_cols, sm_scale, causal, st) \
                  : launch_bwd_mma<TT, 128>(q, lv, mask, out, lse, dout, dq, dk, dv, delta, bh, seq, mask_cols, sm_scale, causal, st))
  return dtype == PSA_F16 ? PSA_BWD_TC(__half) : PSA_BWD_TC(__nv_bfloat16);
#undef PSA_BWD_TC
}
