// Block-score stage A on tcgen05 tensor cores (f16/bf16).
//
// 1. gather_samples_kernel compacts the sampled query / key rows (block/4 per block, replicate-padded) into dense
//    [BH, rows, D] buffers inside the caller's scratch (HBM-bound, 16-byte vector copies).
// 2. scores_cellmax_tc_kernel: one CTA per (128 sampled query rows, batch*head) streams all sampled key rows in
//    128-row tiles with TMA (128-byte swizzle, no multicast), S = Qs Ks^T by tcgen05.mma into a double-buffered TMEM
//    accumulator, and 4 epilogue warps (thread = row) reduce every cell of block_n/4 columns to its maximum,
//    scale it, keep the running row maximum of the unrounded values and store R in the element type.
//    256 TMEM columns and ~100 KB of shared memory per CTA, so two CTAs share an SM and one's epilogue overlaps
//    the other's MMAs.
// Tensor-bound: F_est = 2*BH*(Sq/4)*(Sk/4)*D per call.  Every mbarrier wait is bounded.
#include <algorithm>
#include <cmath>

#include "psa_common.cuh"
#include "scores.h"
#include "tc_common.cuh"

namespace psa {

namespace {

constexpr int kSlabBytes = 128 * 128;
constexpr int kThreads = 192;
constexpr int kStages = 2;

template <typename T, bool ROPE>
__global__ void __launch_bounds__(256) gather_samples_kernel(const RowSource x, const int32_t* __restrict__ idx,
                                                             T* __restrict__ out, int64_t seq, int D, int block, int keep,
                                                             int n_valid, int n_out, const RopeTables rope) {
  const int cpr = D * (int)sizeof(T) / 16;
  const int64_t bh = blockIdx.y;
  uint4* dst = reinterpret_cast<uint4*>(out + bh * (int64_t)n_out * D);
  const int64_t total = (int64_t)n_out * cpr;
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (int64_t)gridDim.x * blockDim.x) {
    int i = (int)(w / cpr);
    const int c = (int)(w % cpr);
    const int ic = i < n_valid ? i : n_valid - 1;
    int64_t tok = (int64_t)(ic / keep) * block + idx[bh * keep + (ic % keep)];
    tok = tok < seq ? tok : seq - 1;
    dst[(int64_t)i * cpr + c] = load_row_word<ROPE>(x, rope, bh, seq, tok, cpr, c);
  }
}

struct Ctrl {
  uint64_t full[kStages], empty[kStages], s_full[2], s_empty[2], q_full;
  uint32_t tmem_base;
  int abort_flag;
};

struct Params {
  void* R;
  float* rowmax;
  int nq_s, n_d, kk, n_tiles;
  int ksplit;          // CTAs per query tile, each with a contiguous share of the key tiles (grid.z)
  float qk_scale;
};

// max of floats through integer atomics; *addr must start at -inf
__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  v += 0.0f;   // -0 -> +0
  if (v >= 0.f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

__global__ void fill_neg_inf(float* x, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) x[i] = -INFINITY;
}

template <int D, int FMT>
__global__ void __launch_bounds__(kThreads, 2) scores_cellmax_tc_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                                       const __grid_constant__ CUtensorMap tm_k, const Params p) {
  constexpr int SLABS = D / 64;
  constexpr int TILE_BYTES = SLABS * kSlabBytes;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = smem;
  unsigned char* sK = smem + TILE_BYTES;
  Ctrl* ctl = reinterpret_cast<Ctrl*>(smem + TILE_BYTES * (1 + kStages));
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, bh = blockIdx.y;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) { tc::mbar_init(&ctl->full[i], 1); tc::mbar_init(&ctl->empty[i], 1); }
    for (int i = 0; i < 2; ++i) { tc::mbar_init(&ctl->s_full[i], 1); tc::mbar_init(&ctl->s_empty[i], 128); }
    tc::mbar_init(&ctl->q_full, 1);
    ctl->abort_flag = 0;
    tc::fence_mbar_init();
  }
  __syncthreads();
  if (warp == 1) {
    tc::tmem_alloc(&ctl->tmem_base, 256);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  // this CTA's share of the key tiles: [j0, j0 + n_tiles)
  const int per = (p.n_tiles + p.ksplit - 1) / p.ksplit;
  const int j0 = (int)blockIdx.z * per;
  const int n_tiles = p.n_tiles - j0 < per ? (p.n_tiles - j0 > 0 ? p.n_tiles - j0 : 0) : per;

  if (warp == 0) {
    if (lane == 0) {
      for (int s = 0; s < SLABS; ++s) tc::tma_load_3d(sQ + s * kSlabBytes, &tm_q, &ctl->q_full, s * 64, qt * 128, bh);
      tc::mbar_arrive_expect_tx(&ctl->q_full, TILE_BYTES);
      for (int j = 0; j < n_tiles; ++j) {
        const int stage = j % kStages;
        if (!tc::mbar_wait(&ctl->empty[stage], ((j / kStages) & 1) ^ 1, abort_flag)) break;
        for (int s = 0; s < SLABS; ++s)
          tc::tma_load_3d(sK + stage * TILE_BYTES + s * kSlabBytes, &tm_k, &ctl->full[stage], s * 64, (j0 + j) * 128, bh);
        tc::mbar_arrive_expect_tx(&ctl->full[stage], TILE_BYTES);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = tc::mbar_wait(&ctl->q_full, 0, abort_flag);
      const uint32_t idesc = tc::make_idesc(FMT, 128, 128, 0, 0);
      const uint32_t q_addr = tc::smem_u32(sQ);
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int stage = j % kStages, b = j & 1;
        ok = tc::mbar_wait(&ctl->full[stage], (j / kStages) & 1, abort_flag);
        if (!ok) break;
        ok = tc::mbar_wait(&ctl->s_empty[b], ((j >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        tc::tc_fence_after();
        const uint32_t k_addr = tc::smem_u32(sK + stage * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * kSlabBytes + (ks & 3) * 32;
          tc::umma_ss(tmem + b * 128, tc::make_smem_desc(q_addr + off, 16, 1024), tc::make_smem_desc(k_addr + off, 16, 1024),
                      idesc, ks > 0);
        }
        tc::umma_commit(&ctl->empty[stage]);
        tc::umma_commit(&ctl->s_full[b]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int row = qt * 128 + r;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int cells_per_tile = 128 / p.kk;
    float run_max = -INFINITY;
    uint16_t* Rrow = reinterpret_cast<uint16_t*>(p.R) + ((int64_t)bh * p.nq_s + (row < p.nq_s ? row : 0)) * p.n_d;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int b = j & 1;
      ok = tc::mbar_wait(&ctl->s_full[b], (j >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc::tc_fence_after();
      uint32_t packed[8];     // up to 16 cells of a tile (kk = 8), two per word
      const int cell0 = (j0 + j) * cells_per_tile;
#pragma unroll
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t v[32];
        tc::tmem_ld32(tmem + b * 128 + lane_base + c0, v);
        tc::tmem_wait_ld();
        // maxima of groups of 8 columns, then merge up to the cell width
        float g[4];
#pragma unroll
        for (int q8 = 0; q8 < 4; ++q8) {
          float mx = __uint_as_float(v[q8 * 8]);
#pragma unroll
          for (int i = 1; i < 8; ++i) mx = fmaxf(mx, __uint_as_float(v[q8 * 8 + i]));
          g[q8] = mx;
        }
        float cm[4];
        int ncell;
        if (p.kk == 8) { ncell = 4; cm[0] = g[0]; cm[1] = g[1]; cm[2] = g[2]; cm[3] = g[3]; }
        else if (p.kk == 16) { ncell = 2; cm[0] = fmaxf(g[0], g[1]); cm[1] = fmaxf(g[2], g[3]); cm[2] = cm[3] = 0.f; }
        else { ncell = 1; cm[0] = fmaxf(fmaxf(g[0], g[1]), fmaxf(g[2], g[3])); cm[1] = cm[2] = cm[3] = 0.f; }
        const int cbase = (c0 / 32) * ncell;          // first cell of this 32-column chunk inside the tile
        float sc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          sc[i] = cm[i] * p.qk_scale;
          if (i < ncell && cell0 + cbase + i < p.n_d) run_max = fmaxf(run_max, sc[i]);
        }
        // pack this chunk's cells (element type) into the tile's output words
        if (p.kk == 8) {
          packed[(c0 / 32) * 2] = FMT ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(sc[0])) |
                                            ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(sc[1])) << 16)
                                      : (uint32_t)__half_as_ushort(__float2half_rn(sc[0])) |
                                            ((uint32_t)__half_as_ushort(__float2half_rn(sc[1])) << 16);
          packed[(c0 / 32) * 2 + 1] = FMT ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(sc[2])) |
                                                ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(sc[3])) << 16)
                                          : (uint32_t)__half_as_ushort(__float2half_rn(sc[2])) |
                                                ((uint32_t)__half_as_ushort(__float2half_rn(sc[3])) << 16);
        } else if (p.kk == 16) {
          packed[c0 / 32] = FMT ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(sc[0])) |
                                      ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(sc[1])) << 16)
                                : (uint32_t)__half_as_ushort(__float2half_rn(sc[0])) |
                                      ((uint32_t)__half_as_ushort(__float2half_rn(sc[1])) << 16);
        } else {
          const uint32_t h = FMT ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(sc[0]))
                                 : (uint32_t)__half_as_ushort(__float2half_rn(sc[0]));
          if ((c0 / 32) & 1) packed[c0 / 64] |= h << 16; else packed[c0 / 64] = h;
        }
      }
      tc::tc_fence_before();
      tc::mbar_arrive(&ctl->s_empty[b]);
      if (row < p.nq_s) {
        // cells_per_tile 16-bit values, i.e. cells_per_tile/2 words; n_d and cell0 are even, so words stay aligned
        const int nwords = cells_per_tile / 2;
        uint32_t* dst = reinterpret_cast<uint32_t*>(Rrow + cell0);
        const int valid_cells = p.n_d - cell0 < cells_per_tile ? p.n_d - cell0 : cells_per_tile;
        if (valid_cells == cells_per_tile && nwords == 4 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
          *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        } else {
#pragma unroll
          for (int w = 0; w < 8; ++w)
            if (w < nwords && 2 * w < valid_cells) dst[w] = packed[w];
        }
      }
    }
    if (ok && row < p.nq_s) {
      if (p.ksplit == 1) p.rowmax[(int64_t)bh * p.nq_s + row] = run_max;
      else atomic_max_float(&p.rowmax[(int64_t)bh * p.nq_s + row], run_max);
    }
  }

  tc::tc_fence_before();
  __syncthreads();
  if (ctl->abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, 256);
  }
}

template <int D, int FMT>
int launch_cellmax(const void* qs, const void* ks, void* R, float* rowmax, const ScoreDims& d, int64_t bh, cudaStream_t st) {
  CUtensorMap tq, tk;
  int rc = encode_tmap_3d(&tq, qs, 2, FMT, D, d.nq_s, bh, 128);
  if (rc != PSA_OK) return rc;
  rc = encode_tmap_3d(&tk, ks, 2, FMT, D, d.nk_cols, bh, 128);
  if (rc != PSA_OK) return rc;
  Params p;
  p.R = R; p.rowmax = rowmax; p.nq_s = d.nq_s; p.n_d = d.n_d; p.kk = d.kk;
  p.n_tiles = (d.nk_cols + 127) / 128;
  p.qk_scale = d.qk_scale;
  const int smem = (D / 64) * kSlabBytes * (1 + kStages) + 256 + 1024;
  cudaError_t e = cudaFuncSetAttribute(scores_cellmax_tc_kernel<D, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_block_scores: shared-memory opt-in failed: %s", cudaGetErrorString(e));
  // Two CTAs share an SM.  When the query tiles do not fill whole waves (few heads per GPU), the key range of every
  // query tile is split over 2 or 4 CTAs; their row maxima meet through atomics.
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const double slots = 2.0 * (sms > 0 ? sms : 148);
  const int64_t ctas = (int64_t)((d.nq_s + 127) / 128) * bh;
  int ksplit = 1;
  double best = 0.0;
  for (int ks = 1; ks <= 4 && ks <= p.n_tiles; ks *= 2) {
    const double waves = (double)(ctas * ks) / slots;
    const double eff = waves / ceil(waves) - 0.01 * (ks - 1);      // a split costs a little (query tile loaded again)
    if (eff > best + 1e-9) { best = eff; ksplit = ks; }
  }
  p.ksplit = ksplit;
  if (ksplit > 1) {
    const int64_t n = bh * (int64_t)d.nq_s;
    fill_neg_inf<<<(unsigned)std::min<int64_t>((n + 255) / 256, 1024), 256, 0, st>>>(rowmax, n);
  }
  dim3 grid((d.nq_s + 127) / 128, (unsigned)bh, (unsigned)ksplit);
  scores_cellmax_tc_kernel<D, FMT><<<grid, kThreads, smem, st>>>(tq, tk, p);
  PSA_CHECK_LAUNCH("psa_block_scores(tcgen05 stage A)");
  return PSA_OK;
}

}  // namespace

bool scores_tc_supported(const ScoreDims& d) {
  return (d.D == 64 || d.D == 128) && (d.kk == 8 || d.kk == 16 || d.kk == 32) && d.kq >= 1 && (d.n_d % 2 == 0);
}

size_t scores_tc_extra_scratch(const ScoreDims& d, int64_t bh) {
  const size_t qb = ((size_t)bh * d.nq_s * d.D * 2 + 255) & ~(size_t)255;
  const size_t kb = ((size_t)bh * d.nk_cols * d.D * 2 + 255) & ~(size_t)255;
  return qb + kb;
}

int launch_scores_cellmax_tc(const RowSource& q, const RowSource& k, const int32_t* idx_q, const int32_t* idx_k, void* R,
                             float* rowmax, void* extra, const ScoreDims& d, int64_t bh, int dtype, cudaStream_t st,
                             const RopeTables& rope) {
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "the tcgen05 score kernel needs f16/bf16 inputs");
  PSA_REQUIRE(scores_tc_supported(d), PSA_ERR_UNSUPPORTED, "the tcgen05 score kernel does not cover this block size");
  const size_t qb = ((size_t)bh * d.nq_s * d.D * 2 + 255) & ~(size_t)255;
  void* qs = extra;
  void* ks = (char*)extra + qb;
  {
    const int cpr = d.D * 2 / 16;
    dim3 gq((unsigned)std::min<int64_t>(cdiv64((int64_t)d.nq_s * cpr, 256), 148 * 8), (unsigned)bh);
    dim3 gk((unsigned)std::min<int64_t>(cdiv64((int64_t)d.nk_cols * cpr, 256), 148 * 8), (unsigned)bh);
    if (rope.a) {
      gather_samples_kernel<uint16_t, true><<<gq, 256, 0, st>>>(q, idx_q, (uint16_t*)qs, d.seq_q, d.D, d.bm, d.kq, d.nq_s, d.nq_s, rope);
      gather_samples_kernel<uint16_t, true><<<gk, 256, 0, st>>>(k, idx_k, (uint16_t*)ks, d.seq_k, d.D, d.bn, d.kk, d.nk_s, d.nk_cols, rope);
    } else {
      gather_samples_kernel<uint16_t, false><<<gq, 256, 0, st>>>(q, idx_q, (uint16_t*)qs, d.seq_q, d.D, d.bm, d.kq, d.nq_s, d.nq_s, rope);
      gather_samples_kernel<uint16_t, false><<<gk, 256, 0, st>>>(k, idx_k, (uint16_t*)ks, d.seq_k, d.D, d.bn, d.kk, d.nk_s, d.nk_cols, rope);
    }
    PSA_CHECK_LAUNCH("psa_block_scores(gather)");
  }
  const int fmt = dtype == PSA_BF16;
  if (d.D == 64) return fmt ? launch_cellmax<64, 1>(qs, ks, R, rowmax, d, bh, st) : launch_cellmax<64, 0>(qs, ks, R, rowmax, d, bh, st);
  return fmt ? launch_cellmax<128, 1>(qs, ks, R, rowmax, d, bh, st) : launch_cellmax<128, 0>(qs, ks, R, rowmax, d, bh, st);
}

int launch_scores_cellmax_tc_samples(const void* qs, const void* ks, void* R, float* rowmax, const ScoreDims& d, int64_t bh,
                                     int dtype, cudaStream_t st) {
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "the tcgen05 score kernel needs f16/bf16 inputs");
  PSA_REQUIRE(scores_tc_supported(d), PSA_ERR_UNSUPPORTED, "the tcgen05 score kernel does not cover this block size");
  const int fmt = dtype == PSA_BF16;
  if (d.D == 64) return fmt ? launch_cellmax<64, 1>(qs, ks, R, rowmax, d, bh, st) : launch_cellmax<64, 0>(qs, ks, R, rowmax, d, bh, st);
  return fmt ? launch_cellmax<128, 1>(qs, ks, R, rowmax, d, bh, st) : launch_cellmax<128, 0>(qs, ks, R, rowmax, d, bh, st);
}

}  // namespace psa
