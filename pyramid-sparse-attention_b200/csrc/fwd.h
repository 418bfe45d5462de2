// Argument bundle and dispatch hooks of the attention forward kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace psa {

// Placement of the four levels inside one operand's tile-image buffer (see pyramid.cu): level li starts at off[li] and
// holds, per (batch*head), groups[li] groups of 8 rows, each group = [64-channel slab][8 rows][128 B].
struct ImgLevels {
  int64_t off[4];
  int64_t groups[4];
};

inline ImgLevels make_img_levels(int64_t bh, int64_t seq, int D, int block_n) {
  ImgLevels L;
  const int64_t s_pad = (seq + block_n - 1) / block_n * block_n;
  int64_t off = 0;
  for (int li = 0; li < 4; ++li) {
    const int64_t rows = s_pad >> li;
    L.groups[li] = (rows + 7) / 8;
    L.off[li] = off;
    off += bh * L.groups[li] * (int64_t)(D / 64) * 1024;
  }
  return L;
}

// Output scatter for head-sharded runs: the rank computes heads [head0, head0+bh) of all tokens, and token s belongs to
// rank s / tokens_per_rank, whose output buffer is laid out [tokens_per_rank][heads_total][D].  n_peers == 0: plain
// local output [bh][seq_q][D].  row_perm != null: query row s is stored as token row_perm[s] (of its head, or of the
// token-major buffers), which undoes a token reordering applied on the way in (int32 [seq_q], a permutation).
constexpr int kMaxPeers = 8;
struct OutScatter {
  void* peer_out[kMaxPeers];
  int n_peers;
  int heads_total, head0;
  int64_t tokens_per_rank;
  const int32_t* row_perm;
};

// Where a row-major operand [bh][seq][D] lives.  n_peers == 0: one local tensor.  n_peers > 0 (head-sharded run, one
// batch): token t of local head h is row (t % tokens_per_rank) of peer t / tokens_per_rank, whose buffer is laid out
// [tokens_per_rank][heads_total][D]; kernels read it with plain loads.  perm != null: the operand is read in a reordered
// token sequence, token t of the sequence being row perm[t] of the stored tensor (int32 [seq]).
struct RowSource {
  const void* base;
  const void* peer[kMaxPeers];
  int n_peers;
  int heads_total, head0;
  int64_t tokens_per_rank;
  const int32_t* perm;
};

// Rotary tables for rows that are rotated while they are read (16-bit operands), as the attention processors of the
// diffusion transformers do before the attention call (modify_diffusers.py:260-281 for Wan, :363-369 for CogVideoX).
// Stored token s >= first uses row s - first of the two fp32 tables [.., D]; channel pair (x0, x1) becomes
// (x0*a[even] - x1*b[even], x1*a[odd] + x0*b[odd]), every product and sum rounded to fp32 on its own (no fused
// multiply-add) and the result rounded once to the element type - bit for bit what the framework's element-wise ops give.
// a == null: no rotation (kernels are then instantiated without the rotary code).
struct RopeTables {
  const float* a;
  const float* b;
  int64_t first;
  int bf16;   // element type of the rows: 1 bf16, 0 f16
};

inline RowSource local_rows(const void* base) {
  RowSource r = {};
  r.base = base;
  return r;
}

#ifdef __CUDACC__
// 16-byte word `c` of the row of token `tok` of local head `bh` (row16 words per row)
__device__ __forceinline__ const uint4* row_word(const RowSource& s, int64_t bh, int64_t seq, int64_t tok, int row16, int c) {
  if (s.perm) tok = s.perm[tok];
  if (s.n_peers == 0) return reinterpret_cast<const uint4*>(s.base) + (bh * seq + tok) * row16 + c;
  const int64_t owner = tok / s.tokens_per_rank, local = tok - owner * s.tokens_per_rank;
  return reinterpret_cast<const uint4*>(s.peer[owner]) + (local * s.heads_total + s.head0 + bh) * row16 + c;
}

// Eight 16-bit channels (four pairs) turned by the table entries a[0..7], b[0..7].
__device__ __forceinline__ uint4 rotate_word(uint4 w, const float* __restrict__ a, const float* __restrict__ b, bool bf16) {
  const float4 a0 = *reinterpret_cast<const float4*>(a), a1 = *reinterpret_cast<const float4*>(a + 4);
  const float4 b0 = *reinterpret_cast<const float4*>(b), b1 = *reinterpret_cast<const float4*>(b + 4);
  const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
  const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
  uint32_t in[4] = {w.x, w.y, w.z, w.w}, out[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float x0, x1;
    if (bf16) {
      x0 = __uint_as_float(in[i] << 16);
      x1 = __uint_as_float(in[i] & 0xffff0000u);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&in[i]);
      x0 = __low2float(h);
      x1 = __high2float(h);
    }
    const float y0 = __fsub_rn(__fmul_rn(x0, av[2 * i]), __fmul_rn(x1, bv[2 * i]));
    const float y1 = __fadd_rn(__fmul_rn(x1, av[2 * i + 1]), __fmul_rn(x0, bv[2 * i + 1]));
    if (bf16) {
      const __nv_bfloat162 o = __floats2bfloat162_rn(y0, y1);
      out[i] = *reinterpret_cast<const uint32_t*>(&o);
    } else {
      const __half2 o = __floats2half2_rn(y0, y1);
      out[i] = *reinterpret_cast<const uint32_t*>(&o);
    }
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

// 16-byte word `c` of the row of token `tok` of local head `bh`; with ROPE, rotated by the tables (if they are set).
template <bool ROPE>
__device__ __forceinline__ uint4 load_row_word(const RowSource& s, const RopeTables& rope, int64_t bh, int64_t seq, int64_t tok,
                                               int row16, int c) {
  if (!ROPE) return *row_word(s, bh, seq, tok, row16, c);
  const int64_t stored = s.perm ? (int64_t)s.perm[tok] : tok;
  uint4 w = *row_word(s, bh, seq, tok, row16, c);
  if (rope.a && stored >= rope.first) {
    const int64_t off = ((stored - rope.first) * row16 + c) * 8;    // row16 * 8 channels per table row
    w = rotate_word(w, rope.a + off, rope.b + off, rope.bf16 != 0);
  }
  return w;
}
#endif

struct FwdArgs {
  const void* q;
  const void* k[4];  // levels 1, 2, 4, 8
  const void* v[4];
  int64_t n[4];      // tokens per head at each level
  const void* kimg;  // tile images of K and V (all four levels), or null
  const void* vimg;
  const int32_t* mask;
  void* out;
  int32_t* status;
  int64_t bh, seq_q, seq_k;
  int D, bm, bn, tn, width, quirk, dtype;
  float scale;
  OutScatter scatter = {};   // n_peers == 0 unless the output goes to peer buffers
  float* lse = nullptr;      // optional [bh][seq_q]: log-sum-exp of every row (natural log)
  int legacy = 0;            // legacy semantics: a row without any visible key gives 0 (lse -inf) instead of 0/0
  int causal = 0;            // legacy causal rule: pooled token j of level l is visible iff (j+1)*l - 1 <= query position
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
