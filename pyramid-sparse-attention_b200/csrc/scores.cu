// Block-importance scores on sampled tokens.
//
// Stage A (cell maxima): for every sampled query row i and every K cell c (block_n/4 consecutive sampled
// key rows) R[i,c] = max_{j in c}(q_i . k_j) * (D^-0.5 * log2 e), stored in the element type, and the row
// maximum m_i of the UNROUNDED values.  The sampled rows are gathered on the fly from Q/K through the
// per-head index lists (token = min(block*blk + idx[t], S-1): replicate padding of the tail block; sample
// rows past the end replicate the last sample: the reference pads the sample matrices to a multiple of 64).
// Stage B (pooling + normalisation): Po[r,c] = max_{i in group r} exp2(R[i,c] - m_i) rounded to the element
// type, divided by the row sum over ALL cells (padded cells included), sliced to [Mq, Nk].
//
// This file holds the scalar fp32 stage A (any dtype; exact fp32 dot products) and stage B.  The tcgen05
// stage A for f16/bf16 lives in scores_tc.cu.
#include <mutex>

#include "psa_common.cuh"
#include "scores.h"

namespace psa {

// ---------------------------------------------------------------- stage A, scalar -----------------
// CTA: 64 sampled q rows x all K cells; 256 threads as 16x16, each 4x4 outputs of a 64x64 tile.
template <typename T>
__global__ void __launch_bounds__(256) scores_cellmax_simt(const T* __restrict__ q, const T* __restrict__ k,
                                                           const int32_t* __restrict__ idx_q,
                                                           const int32_t* __restrict__ idx_k, T* __restrict__ R,
                                                           float* __restrict__ rowmax, ScoreDims d) {
  __shared__ float Qs[64][33];
  __shared__ float Ks[64][33];
  __shared__ int64_t qtok[64];
  __shared__ int64_t ktok[64];
  const int bh = blockIdx.y;
  const int row0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const T* qh = q + (int64_t)bh * d.seq_q * d.D;
  const T* kh = k + (int64_t)bh * d.seq_k * d.D;
  if (threadIdx.x < 64) {
    int i = row0 + threadIdx.x;
    i = i < d.nq_s ? i : d.nq_s - 1;
    int64_t tok = (int64_t)(i / d.kq) * d.bm + idx_q[bh * d.kq + (i % d.kq)];
    qtok[threadIdx.x] = tok < d.seq_q ? tok : d.seq_q - 1;
  }
  float run_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  const int cells_per_tile = 64 / d.kk;
  for (int col0 = 0; col0 < d.nk_cols; col0 += 64) {
    __syncthreads();
    if (threadIdx.x < 64) {
      int j = col0 + threadIdx.x;
      j = j < d.nk_s ? j : d.nk_s - 1;
      int64_t tok = (int64_t)(j / d.kk) * d.bn + idx_k[bh * d.kk + (j % d.kk)];
      ktok[threadIdx.x] = tok < d.seq_k ? tok : d.seq_k - 1;
    }
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
    for (int d0 = 0; d0 < d.D; d0 += 32) {
      __syncthreads();
      for (int e = threadIdx.x; e < 64 * 32; e += 256) {
        int r = e >> 5, c = e & 31;
        Qs[r][c] = Elem<T>::to_f(qh[qtok[r] * d.D + d0 + c]);
        Ks[r][c] = Elem<T>::to_f(kh[ktok[r] * d.D + d0 + c]);
      }
      __syncthreads();
#pragma unroll 8
      for (int c = 0; c < 32; ++c) {
        float qa[4], kb[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) qa[a] = Qs[ty * 4 + a][c];
#pragma unroll
        for (int b = 0; b < 4; ++b) kb[b] = Ks[tx * 4 + b][c];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(qa[a], kb[b], acc[a][b]);
      }
    }
    // cell maxima: a thread's 4 columns sit inside one cell (kk is a multiple of 4); reduce over the
    // kk/4 neighbouring tx lanes.
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      float mx = fmaxf(fmaxf(acc[a][0], acc[a][1]), fmaxf(acc[a][2], acc[a][3]));
      for (int off = 1; off < d.kk / 4; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      mx *= d.qk_scale;
      run_max[a] = fmaxf(run_max[a], mx);
      const int row = row0 + ty * 4 + a;
      if ((tx % (d.kk / 4)) == 0 && row < d.nq_s) {
        const int cell = col0 / d.kk + (tx * 4) / d.kk;
        if (cell < d.n_d) R[((int64_t)bh * d.nq_s + row) * d.n_d + cell] = Elem<T>::from_f(mx);
      }
    }
    (void)cells_per_tile;
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    float mx = run_max[a];
    for (int off = 1; off < 16; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    const int row = row0 + ty * 4 + a;
    if (tx == 0 && row < d.nq_s) rowmax[(int64_t)bh * d.nq_s + row] = mx;
  }
}

// ---------------------------------------------------------------- stage B -------------------------
// CTA per (query block r, bh).  Dynamic smem: n_d floats.
template <typename T, int VEC>
struct alignas(VEC * sizeof(T)) CellPack { T e[VEC]; };

// VEC neighbouring cells per thread and load; the launcher picks the widest VEC (<= 8 bytes) that divides n_d.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) scores_pool_normalise(const T* __restrict__ R, const float* __restrict__ rowmax,
                                                            T* __restrict__ po, ScoreDims d) {
  extern __shared__ float sm_po[];
  __shared__ float red[8];
  __shared__ float s_rowmax[64];
  const int r = blockIdx.x, bh = blockIdx.y;
  const int64_t rbase = (int64_t)bh * d.nq_s + (int64_t)r * d.kq;
  if (threadIdx.x < d.kq) s_rowmax[threadIdx.x] = rowmax[rbase + threadIdx.x];
  __syncthreads();
  // exp2 is monotone, so the pooled maximum of exp2(x - m_t) is exp2 of the maximum of (x - m_t): one exp2 per cell.
  // A thread owns VEC neighbouring cells and walks the block's sampled rows.
  using Pack = CellPack<T, VEC>;
  float part = 0.f;
  for (int c = threadIdx.x * VEC; c < d.n_d; c += blockDim.x * VEC) {
    float best[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) best[v] = -INFINITY;
    const T* col = R + rbase * d.n_d + c;
    int t = 0;
    for (; t + 8 <= d.kq; t += 8) {
      Pack raw[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) raw[u] = *reinterpret_cast<const Pack*>(col + (int64_t)(t + u) * d.n_d);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float m = s_rowmax[t + u];
#pragma unroll
        for (int v = 0; v < VEC; ++v) best[v] = fmaxf(best[v], Elem<T>::to_f(raw[u].e[v]) - m);
      }
    }
    for (; t < d.kq; ++t) {
      const Pack raw = *reinterpret_cast<const Pack*>(col + (int64_t)t * d.n_d);
      const float m = s_rowmax[t];
#pragma unroll
      for (int v = 0; v < VEC; ++v) best[v] = fmaxf(best[v], Elem<T>::to_f(raw.e[v]) - m);
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      const float b = Elem<T>::round(exp2f(best[v]));
      sm_po[c + v] = b;
      part += b;
    }
  }
  for (int off = 16; off; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
  __syncthreads();
  float sum = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) sum += red[w];
  sum = Elem<T>::round(sum);
  T* dst = po + ((int64_t)bh * d.Mq + r) * d.Nk;
  for (int c = threadIdx.x; c < d.Nk; c += blockDim.x) dst[c] = Elem<T>::from_f(sm_po[c] / sum);
}

template <typename T>
static int launch_scores(const RowSource& q, const RowSource& k, const int32_t* idx_q, const int32_t* idx_k, void* po,
                         void* scratch, const ScoreDims& d, int64_t bh, int impl, cudaStream_t st,
                         const RopeTables& rope = RopeTables{}) {
  T* R = (T*)scratch;
  const size_t r_bytes = ((size_t)bh * d.nq_s * d.n_d * sizeof(T) + 255) & ~(size_t)255;
  float* rowmax = (float*)((char*)scratch + r_bytes);
  const size_t m_bytes = ((size_t)bh * d.nq_s * sizeof(float) + 255) & ~(size_t)255;
  void* extra = (char*)scratch + r_bytes + m_bytes;
  bool use_tc = (impl == 2) || (impl == 0 && sizeof(T) == 2 && scores_tc_supported(d));
  if (use_tc) {
    int rc = launch_scores_cellmax_tc(q, k, idx_q, idx_k, R, rowmax, extra, d, bh, sizeof(T) == 4 ? PSA_F32 :
                                      (std::is_same<T, __half>::value ? PSA_F16 : PSA_BF16), st, rope);
    if (rc != PSA_OK) return rc;
  } else {
    PSA_REQUIRE(q.n_peers == 0 && k.n_peers == 0 && !rope.a, PSA_ERR_UNSUPPORTED, "the scalar score kernel reads local tensors only");
    dim3 grid((unsigned)cdiv64(d.nq_s, 64), (unsigned)bh);
    scores_cellmax_simt<T><<<grid, 256, 0, st>>>((const T*)q.base, (const T*)k.base, idx_q, idx_k, R, rowmax, d);
    PSA_CHECK_LAUNCH("psa_block_scores(stage A)");
  }
  dim3 gridb((unsigned)d.Mq, (unsigned)bh);
  // n_d is a multiple of 64 / (block_n / 4), i.e. of 2 at least; R itself is 256-byte aligned
  constexpr int kWide = 8 / (int)sizeof(T);
  if (d.n_d % kWide == 0) scores_pool_normalise<T, kWide><<<gridb, 256, d.n_d * sizeof(float), st>>>(R, rowmax, (T*)po, d);
  else if (d.n_d % 2 == 0) scores_pool_normalise<T, 2><<<gridb, 256, d.n_d * sizeof(float), st>>>(R, rowmax, (T*)po, d);
  else scores_pool_normalise<T, 1><<<gridb, 256, d.n_d * sizeof(float), st>>>(R, rowmax, (T*)po, d);
  PSA_CHECK_LAUNCH("psa_block_scores(stage B)");
  return PSA_OK;
}

int make_score_dims(ScoreDims& d, int64_t seq_q, int64_t seq_k, int D, int bm, int bn) {
  PSA_REQUIRE(bm >= 16 && bm <= 256 && bm % 16 == 0, PSA_ERR_ARG, "block_m=%d unsupported (16..256, multiple of 16)", bm);
  PSA_REQUIRE(bn == 32 || bn == 64 || bn == 128, PSA_ERR_ARG, "block_n=%d unsupported (32/64/128)", bn);
  PSA_REQUIRE(D == 64 || D == 128, PSA_ERR_ARG, "head_dim=%d unsupported (64/128)", D);
  PSA_REQUIRE(seq_q > 0 && seq_k > 0, PSA_ERR_ARG, "empty sequence");
  d.seq_q = seq_q; d.seq_k = seq_k; d.D = D; d.bm = bm; d.bn = bn;
  d.kq = bm / 4; d.kk = bn / 4;
  d.Mq = (int)cdiv64(seq_q, bm); d.Nk = (int)cdiv64(seq_k, bn);
  d.nq_s = d.Mq * d.kq; d.nk_s = d.Nk * d.kk;
  d.nk_cols = (int)(cdiv64(d.nk_s, 64) * 64);
  d.n_d = d.nk_cols / d.kk;
  PSA_REQUIRE(d.kq <= 64, PSA_ERR_ARG, "block_m too large");
  const float sm_scale = (float)(1.0 / sqrt((double)D));
  d.qk_scale = sm_scale * 1.44269504f;
  return PSA_OK;
}

}  // namespace psa

namespace psa {
// Scratch a call really uses: R, the row maxima and (16-bit inputs) the compacted sample matrices of its head_dim.
static size_t score_scratch_bytes(int64_t bh, int64_t seq_q, int64_t seq_k, int head_dim, int block_m, int block_n, int dtype) {
  ScoreDims d;
  if (make_score_dims(d, seq_q, seq_k, head_dim, block_m, block_n) != PSA_OK) return 0;
  const size_t es = dtype == PSA_F32 ? 4 : 2;
  const size_t r_bytes = ((size_t)bh * d.nq_s * d.n_d * es + 255) & ~(size_t)255;
  const size_t m_bytes = ((size_t)bh * d.nq_s * sizeof(float) + 255) & ~(size_t)255;
  const size_t extra = dtype == PSA_F32 ? 0 : scores_tc_extra_scratch(d, bh);
  return r_bytes + m_bytes + extra;
}
}  // namespace psa

// The public bound does not know the head_dim: it is sized for 128, the larger of the two supported widths.
extern "C" size_t psa_block_scores_scratch_bytes(int64_t bh, int64_t seq_q, int64_t seq_k, int block_m, int block_n,
                                                 int dtype) {
  return psa::score_scratch_bytes(bh, seq_q, seq_k, 128, block_m, block_n, dtype);
}

extern "C" int psa_block_scores(const void* q, const void* k, const int32_t* idx_q, const int32_t* idx_k, void* po,
                                void* scratch, size_t scratch_bytes, int64_t bh, int64_t seq_q, int64_t seq_k,
                                int head_dim, int block_m, int block_n, int dtype, int impl, void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && k && idx_q && idx_k && po && scratch, PSA_ERR_ARG, "psa_block_scores: null pointer");
  PSA_REQUIRE(bh > 0 && bh < 65536, PSA_ERR_ARG, "psa_block_scores: bh=%lld out of range", (long long)bh);
  PSA_REQUIRE(((uintptr_t)scratch & 255) == 0, PSA_ERR_ARG, "psa_block_scores: scratch must be 256-byte aligned");
  ScoreDims d;
  int rc = make_score_dims(d, seq_q, seq_k, head_dim, block_m, block_n);
  if (rc != PSA_OK) return rc;
  PSA_REQUIRE(scratch_bytes >= psa_block_scores_scratch_bytes(bh, seq_q, seq_k, block_m, block_n, dtype), PSA_ERR_ARG,
              "psa_block_scores: scratch too small (%zu bytes)", scratch_bytes);
  PSA_REQUIRE(impl >= 0 && impl <= 2, PSA_ERR_ARG, "psa_block_scores: impl=%d", impl);
  cudaStream_t st = (cudaStream_t)stream;
  PSA_DISPATCH_DTYPE(dtype, T, return launch_scores<T>(local_rows(q), local_rows(k), idx_q, idx_k, po, scratch, d, bh, impl, st));
  return PSA_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Allocation-free variant.  Some hosts of this library may not allocate device memory at call time: code that
// runs with a fixed memory budget handed out at start-up (an inference server that has given every byte to its own
// pools), a plug-in that is only given input and output buffers, or a caller inside a region where cudaMalloc is
// forbidden.  For them the stage-A/stage-B scratch lives in this file-scope device array, which every GPU that loads
// the library keeps until the process exits.
namespace psa {

constexpr size_t kStaticScratchBytes = PSA_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scores_scratch[kStaticScratchBytes];

// Device address of the array, resolved once per device.  In host code the array's name is only a handle for the
// runtime, not a device address, so it must go through cudaGetSymbolAddress with the target device current.
static int static_scratch_ptr(void** out) {
  constexpr int kMaxDevices = 64;
  static void* cached[kMaxDevices] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  PSA_REQUIRE(e == cudaSuccess && dev >= 0 && dev < kMaxDevices, PSA_ERR_CUDA, "psa_block_scores_static: cudaGetDevice failed: %s",
              cudaGetErrorString(e));
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scores_scratch);
    PSA_REQUIRE(e == cudaSuccess && ptr != nullptr, PSA_ERR_CUDA,
                "psa_block_scores_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return PSA_OK;
}

}  // namespace psa

extern "C" size_t psa_block_scores_static_capacity(void) { return psa::kStaticScratchBytes; }

extern "C" int psa_block_scores_static(const void* q, const void* k, const int32_t* idx_q, const int32_t* idx_k, void* po,
                                       int64_t bh, int64_t seq_q, int64_t seq_k, int head_dim, int block_m, int block_n,
                                       int dtype, int impl, void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && k && idx_q && idx_k && po, PSA_ERR_ARG, "psa_block_scores_static: null pointer");
  PSA_REQUIRE(bh > 0 && bh < 65536, PSA_ERR_ARG, "psa_block_scores_static: bh=%lld out of range", (long long)bh);
  PSA_REQUIRE(impl >= 0 && impl <= 2, PSA_ERR_ARG, "psa_block_scores_static: impl=%d", impl);
  ScoreDims d;
  int rc = make_score_dims(d, seq_q, seq_k, head_dim, block_m, block_n);
  if (rc != PSA_OK) return rc;
  const size_t need = score_scratch_bytes(bh, seq_q, seq_k, head_dim, block_m, block_n, dtype);   // of this head_dim
  PSA_REQUIRE(need <= kStaticScratchBytes, PSA_ERR_ARG,
              "psa_block_scores_static: this call needs %zu bytes of scratch but the built-in scratch holds %zu; "
              "split the call over fewer heads or use psa_block_scores with caller-provided scratch",
              need, kStaticScratchBytes);
  void* scratch = nullptr;
  rc = static_scratch_ptr(&scratch);
  if (rc != PSA_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  PSA_DISPATCH_DTYPE(dtype, T, return launch_scores<T>(local_rows(q), local_rows(k), idx_q, idx_k, po, scratch, d, bh, impl, st));
  return PSA_OK;
}

static int block_scores_perm(const void* q, const void* k, const int32_t* perm_q, const int32_t* perm_k, const psa::RopeTables& rope,
                             const int32_t* idx_q, const int32_t* idx_k, void* po, void* scratch, size_t scratch_bytes, int64_t bh,
                             int64_t seq_q, int64_t seq_k, int head_dim, int block_m, int block_n, int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && k && (rope.a || (perm_q && perm_k)) && idx_q && idx_k && po && scratch, PSA_ERR_ARG, "psa_block_scores_perm: null pointer");
  PSA_REQUIRE(bh > 0 && bh < 65536, PSA_ERR_ARG, "psa_block_scores_perm: bh=%lld out of range", (long long)bh);
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "psa_block_scores_perm: f16/bf16 only");
  PSA_REQUIRE(((uintptr_t)scratch & 255) == 0 && (((uintptr_t)q | (uintptr_t)k) & 15) == 0, PSA_ERR_ARG,
              "psa_block_scores_perm: scratch must be 256-byte aligned, q and k 16-byte aligned");
  ScoreDims d;
  int rc = make_score_dims(d, seq_q, seq_k, head_dim, block_m, block_n);
  if (rc != PSA_OK) return rc;
  PSA_REQUIRE(scores_tc_supported(d), PSA_ERR_UNSUPPORTED, "psa_block_scores_perm: block sizes not covered by the tcgen05 path");
  PSA_REQUIRE(scratch_bytes >= psa_block_scores_scratch_bytes(bh, seq_q, seq_k, block_m, block_n, dtype), PSA_ERR_ARG,
              "psa_block_scores_perm: scratch too small (%zu bytes)", scratch_bytes);
  RowSource qs = local_rows(q), ks = local_rows(k);
  qs.perm = perm_q;
  ks.perm = perm_k;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == PSA_F16) return launch_scores<__half>(qs, ks, idx_q, idx_k, po, scratch, d, bh, 2, st, rope);
  return launch_scores<__nv_bfloat16>(qs, ks, idx_q, idx_k, po, scratch, d, bh, 2, st, rope);
}

extern "C" int psa_block_scores_perm(const void* q, const void* k, const int32_t* perm_q, const int32_t* perm_k,
                                     const int32_t* idx_q, const int32_t* idx_k, void* po, void* scratch, size_t scratch_bytes,
                                     int64_t bh, int64_t seq_q, int64_t seq_k, int head_dim, int block_m, int block_n, int dtype,
                                     void* stream) {
  return block_scores_perm(q, k, perm_q, perm_k, psa::RopeTables{}, idx_q, idx_k, po, scratch, scratch_bytes, bh, seq_q, seq_k, head_dim,
                           block_m, block_n, dtype, stream);
}

extern "C" int psa_block_scores_perm_rope(const void* q, const void* k, const int32_t* perm, const float* rope_a, const float* rope_b,
                                          int64_t rope_first, const int32_t* idx_q, const int32_t* idx_k, void* po, void* scratch,
                                          size_t scratch_bytes, int64_t bh, int64_t seq, int head_dim, int block_m, int block_n,
                                          int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(rope_a && rope_b && rope_first >= 0 && rope_first <= seq, PSA_ERR_ARG, "psa_block_scores_perm_rope: bad rotary tables");
  PSA_REQUIRE((((uintptr_t)rope_a | (uintptr_t)rope_b) & 15) == 0, PSA_ERR_ARG, "psa_block_scores_perm_rope: tables must be 16-byte aligned");
  const RopeTables rope = {rope_a, rope_b, rope_first, dtype == PSA_BF16};
  return block_scores_perm(q, k, perm, perm, rope, idx_q, idx_k, po, scratch, scratch_bytes, bh, seq, seq, head_dim, block_m, block_n,
                           dtype, stream);
}

static int block_scores_tm(const void* q, const void* k, const int32_t* perm, const float* rope_a, const float* rope_b,
                           int64_t rope_first, const int32_t* idx_q, const int32_t* idx_k, void* po, void* scratch,
                           size_t scratch_bytes, int heads, int64_t seq, int head_dim, int block_m, int block_n, int dtype,
                           void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && k && idx_q && idx_k && po && scratch, PSA_ERR_ARG, "psa_block_scores_tm: null pointer");
  PSA_REQUIRE(heads > 0 && heads < 65536 && seq > 0 && seq < ((int64_t)1 << 31), PSA_ERR_ARG, "psa_block_scores_tm: bad shape");
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "psa_block_scores_tm: f16/bf16 only");
  PSA_REQUIRE(((uintptr_t)scratch & 255) == 0 && (((uintptr_t)q | (uintptr_t)k) & 15) == 0, PSA_ERR_ARG,
              "psa_block_scores_tm: scratch must be 256-byte aligned, q and k 16-byte aligned");
  ScoreDims d;
  int rc = make_score_dims(d, seq, seq, head_dim, block_m, block_n);
  if (rc != PSA_OK) return rc;
  PSA_REQUIRE(scores_tc_supported(d), PSA_ERR_UNSUPPORTED, "psa_block_scores_tm: block sizes not covered by the tcgen05 path");
  PSA_REQUIRE(scratch_bytes >= psa_block_scores_scratch_bytes(heads, seq, seq, block_m, block_n, dtype), PSA_ERR_ARG,
              "psa_block_scores_tm: scratch too small (%zu bytes)", scratch_bytes);
  RowSource qs = {}, ks = {};
  qs.peer[0] = q; ks.peer[0] = k;
  qs.n_peers = ks.n_peers = 1;
  qs.heads_total = ks.heads_total = heads;
  qs.tokens_per_rank = ks.tokens_per_rank = seq;
  qs.perm = ks.perm = perm;
  const RopeTables rope = {rope_a, rope_b, rope_first, dtype == PSA_BF16};
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == PSA_F16) return launch_scores<__half>(qs, ks, idx_q, idx_k, po, scratch, d, heads, 2, st, rope);
  return launch_scores<__nv_bfloat16>(qs, ks, idx_q, idx_k, po, scratch, d, heads, 2, st, rope);
}

extern "C" int psa_block_scores_tm(const void* q, const void* k, const int32_t* perm, const int32_t* idx_q, const int32_t* idx_k,
                                   void* po, void* scratch, size_t scratch_bytes, int heads, int64_t seq, int head_dim, int block_m,
                                   int block_n, int dtype, void* stream) {
  return block_scores_tm(q, k, perm, nullptr, nullptr, 0, idx_q, idx_k, po, scratch, scratch_bytes, heads, seq, head_dim, block_m,
                         block_n, dtype, stream);
}

extern "C" int psa_block_scores_tm_rope(const void* q, const void* k, const int32_t* perm, const float* rope_a, const float* rope_b,
                                        int64_t rope_first, const int32_t* idx_q, const int32_t* idx_k, void* po, void* scratch,
                                        size_t scratch_bytes, int heads, int64_t seq, int head_dim, int block_m, int block_n,
                                        int dtype, void* stream) {
  using namespace psa;
  PSA_REQUIRE(rope_a && rope_b && rope_first >= 0 && rope_first <= seq, PSA_ERR_ARG, "psa_block_scores_tm_rope: bad rotary tables");
  PSA_REQUIRE((((uintptr_t)rope_a | (uintptr_t)rope_b) & 15) == 0, PSA_ERR_ARG, "psa_block_scores_tm_rope: tables must be 16-byte aligned");
  return block_scores_tm(q, k, perm, rope_a, rope_b, rope_first, idx_q, idx_k, po, scratch, scratch_bytes, heads, seq, head_dim,
                         block_m, block_n, dtype, stream);
}

extern "C" int psa_block_scores_peers(const void* const* peer_q, const void* const* peer_k, int n_peers, int64_t tokens_per_rank,
                                      int heads_total, int head0, const int32_t* idx_q, const int32_t* idx_k, void* po, void* scratch,
                                      size_t scratch_bytes, int64_t heads_local, int head_dim, int block_m, int block_n, int dtype,
                                      void* stream) {
  using namespace psa;
  PSA_REQUIRE(peer_q && peer_k && idx_q && idx_k && po && scratch, PSA_ERR_ARG, "psa_block_scores_peers: null pointer");
  PSA_REQUIRE(n_peers >= 1 && n_peers <= kMaxPeers, PSA_ERR_ARG, "psa_block_scores_peers: n_peers=%d (1..%d)", n_peers, kMaxPeers);
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "psa_block_scores_peers: f16/bf16 only");
  PSA_REQUIRE(heads_local > 0 && head0 >= 0 && head0 + heads_local <= heads_total && tokens_per_rank > 0, PSA_ERR_ARG,
              "psa_block_scores_peers: bad head range or shard size");
  PSA_REQUIRE(((uintptr_t)scratch & 255) == 0, PSA_ERR_ARG, "psa_block_scores_peers: scratch must be 256-byte aligned");
  const int64_t seq = tokens_per_rank * n_peers;
  ScoreDims d;
  int rc = make_score_dims(d, seq, seq, head_dim, block_m, block_n);
  if (rc != PSA_OK) return rc;
  PSA_REQUIRE(scores_tc_supported(d), PSA_ERR_UNSUPPORTED, "psa_block_scores_peers: block sizes not covered by the tcgen05 path");
  PSA_REQUIRE(scratch_bytes >= psa_block_scores_scratch_bytes(heads_local, seq, seq, block_m, block_n, dtype), PSA_ERR_ARG,
              "psa_block_scores_peers: scratch too small (%zu bytes)", scratch_bytes);
  RowSource q = {}, k = {};
  for (int i = 0; i < n_peers; ++i) {
    PSA_REQUIRE(peer_q[i] && peer_k[i] && (((uintptr_t)peer_q[i] | (uintptr_t)peer_k[i]) & 15) == 0, PSA_ERR_ARG,
                "psa_block_scores_peers: peer %d pointer", i);
    q.peer[i] = peer_q[i];
    k.peer[i] = peer_k[i];
  }
  q.n_peers = k.n_peers = n_peers;
  q.heads_total = k.heads_total = heads_total;
  q.head0 = k.head0 = head0;
  q.tokens_per_rank = k.tokens_per_rank = tokens_per_rank;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == PSA_F16) return launch_scores<__half>(q, k, idx_q, idx_k, po, scratch, d, heads_local, 2, st);
  return launch_scores<__nv_bfloat16>(q, k, idx_q, idx_k, po, scratch, d, heads_local, 2, st);
}

// Rows of the compacted sample matrices of one block-score call: queries nq (= ceil(seq/block_m) * block_m/4), keys nk
// (the same for block_n, padded up to a multiple of 64 rows; rows past the last valid sample repeat it).
extern "C" int psa_sample_rows(int64_t seq_q, int64_t seq_k, int block_m, int block_n, int64_t* nq, int64_t* nk_valid, int64_t* nk) {
  using namespace psa;
  ScoreDims d;
  int rc = make_score_dims(d, seq_q, seq_k, 128, block_m, block_n);
  if (rc != PSA_OK) return rc;
  if (nq) *nq = d.nq_s;
  if (nk_valid) *nk_valid = d.nk_s;
  if (nk) *nk = d.nk_cols;
  return PSA_OK;
}

extern "C" int psa_block_scores_samples(const void* qs, const void* ks, void* po, void* scratch, size_t scratch_bytes, int64_t bh,
                                        int64_t seq_q, int64_t seq_k, int head_dim, int block_m, int block_n, int dtype,
                                        void* stream) {
  using namespace psa;
  PSA_REQUIRE(qs && ks && po && scratch, PSA_ERR_ARG, "psa_block_scores_samples: null pointer");
  PSA_REQUIRE(bh > 0 && bh < 65536, PSA_ERR_ARG, "psa_block_scores_samples: bh=%lld out of range", (long long)bh);
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "psa_block_scores_samples: f16/bf16 only");
  PSA_REQUIRE(((uintptr_t)scratch & 255) == 0 && (((uintptr_t)qs | (uintptr_t)ks) & 15) == 0, PSA_ERR_ARG,
              "psa_block_scores_samples: scratch must be 256-byte aligned, samples 16-byte aligned");
  ScoreDims d;
  int rc = make_score_dims(d, seq_q, seq_k, head_dim, block_m, block_n);
  if (rc != PSA_OK) return rc;
  PSA_REQUIRE(scratch_bytes >= psa_block_scores_scratch_bytes(bh, seq_q, seq_k, block_m, block_n, dtype), PSA_ERR_ARG,
              "psa_block_scores_samples: scratch too small (%zu bytes)", scratch_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  const size_t es = 2;
  void* R = scratch;
  const size_t r_bytes = ((size_t)bh * d.nq_s * d.n_d * es + 255) & ~(size_t)255;
  float* rowmax = (float*)((char*)scratch + r_bytes);
  rc = launch_scores_cellmax_tc_samples(qs, ks, R, rowmax, d, bh, dtype, st);
  if (rc != PSA_OK) return rc;
  dim3 gridb((unsigned)d.Mq, (unsigned)bh);
  if (dtype == PSA_F16) {
    if (d.n_d % 4 == 0) scores_pool_normalise<__half, 4><<<gridb, 256, d.n_d * sizeof(float), st>>>((const __half*)R, rowmax, (__half*)po, d);
    else scores_pool_normalise<__half, 2><<<gridb, 256, d.n_d * sizeof(float), st>>>((const __half*)R, rowmax, (__half*)po, d);
  } else {
    if (d.n_d % 4 == 0)
      scores_pool_normalise<__nv_bfloat16, 4><<<gridb, 256, d.n_d * sizeof(float), st>>>((const __nv_bfloat16*)R, rowmax, (__nv_bfloat16*)po, d);
    else
      scores_pool_normalise<__nv_bfloat16, 2><<<gridb, 256, d.n_d * sizeof(float), st>>>((const __nv_bfloat16*)R, rowmax, (__nv_bfloat16*)po, d);
  }
  PSA_CHECK_LAUNCH("psa_block_scores_samples(stage B)");
  return PSA_OK;
}
