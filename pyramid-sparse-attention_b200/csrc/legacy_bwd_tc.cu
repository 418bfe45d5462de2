// Legacy (old-format mask) attention backward on tcgen05 tensor cores (f16/bf16, head_dim 64/128).
//
// Mathematics (the scalar kernels in legacy_bwd.cu derive it; reference: psa_kernel_legacy.py:947-1320): a pooled token t
// of level l stands for l identical expanded keys, of which c_t(i) exist and are visible to query row i, so with
// p_it = exp(q_i.k_t scale - lse_i):
//   ds_it = round(p_it (dO_i.v_t - delta_i)) c_t(i),   pc_it = round(p_it) c_t(i)
//   dQ_i = scale sum_t ds_it k_t,   dK_j (j in t) += scale / l sum_i ds_it q_i,   dV_j (j in t) += 1 / l sum_i pc_it dO_i
// Two kernels share one skeleton: a STATIONARY pair of 128-row operand tiles in shared memory, a STREAM of 128-row
// operand tiles through a two-stage ring, both products of a stream tile computed in 64-column halves into
// double-buffered TMEM (S and dP), one thread per accumulator row turning them into the 16-bit operand of the
// accumulating products IN PLACE in TMEM, and a single MMA-issuing thread that runs the fixed order
//   acc(half 0, tile t)  S/dP(half 0, tile t+1)  acc(half 1, tile t)  S/dP(half 1, tile t+1) ...
// so the element-wise work of one half always runs under the tensor work of the other.
//
//   bwd_dq_tc_kernel    stationary: Q and dO of one query block (rows = queries).  Stream: the selected key blocks of
//                       all levels, PACKED back to back into 128-token K and V tiles (tile images, one linear bulk copy
//                       per block and operand).  S = Q K^T, dP = dO V^T, dS over dP, dQ += dS K (K read MN-major from
//                       the same tile).  Per-column metadata (copies, first original position) comes from the producer.
//   bwd_dkdv_tc_kernel  stationary: 128 consecutive pooled K and V rows of ONE level (= l consecutive key blocks),
//                       rows = pooled keys.  Stream: Q and dO tiles of every query block that selected that level for at
//                       least one of those key blocks (rows whose block was not selected get zeros).  S^T = K Q^T,
//                       dP^T = V dO^T, P^T over S^T, dS^T over dP^T, dV += P^T dO, dK += dS^T Q.  The fp32 sums of the
//                       pooled rows go to scratch; bwd_fold_kernel spreads them over the original positions
//                       (mean-pool backward), folds the replicate-padded tail into the last token and rounds once.
// Every wait is bounded; on expiry the CTA records PSA_ERR_TIMEOUT, lets copies in flight land, frees TMEM and returns.
#include <cstddef>

#include "psa_common.cuh"
#include "fwd.h"
#include "tc_common.cuh"

namespace psa {
namespace {

constexpr int kSlab = 128 * 128;          // 128 rows x 128 B (64 16-bit channels)
constexpr int kThreadsBwd = 576;          // warp 0 producer, warp 1 MMA issuer, warps 2-17 element-wise (four groups)
constexpr int kEwWarps = 16;
constexpr int kMaxBlocks = 1472;          // key / query blocks per head the lists are sized for

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <int FMT> __device__ __forceinline__ uint32_t pack16(float a, float b);
template <> __device__ __forceinline__ uint32_t pack16<1>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack16<0>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <int FMT> __device__ __forceinline__ float round16(float x);
template <> __device__ __forceinline__ float round16<1>(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
template <> __device__ __forceinline__ float round16<0>(float x) { return __half2float(__float2half_rn(x)); }

// Visible copies of the pooled token whose first original position is j0, for the query at qpos.
__device__ __forceinline__ int copies(int64_t j0, int level, int64_t l_k, int causal, int64_t qpos) {
  int64_t hi = l_k;
  if (causal && qpos + 1 < hi) hi = qpos + 1;
  const int64_t c = hi - j0;
  return c < 0 ? 0 : (c > level ? level : (int)c);
}

struct BwdParams {
  const int32_t* mask;       // [bh][mq][mask_cols] levels
  const unsigned char* kimg; // tile images (block 128) of K and V, all levels
  const unsigned char* vimg;
  ImgLevels img;
  const float* stat;         // [bh][s_pad / 2][4]: (-lse0, -lse1, -delta0, -delta1) of two rows, lse in log2 units; rows >= seq: (-inf, 0)
  void* dq;                  // [bh][seq][D]
  float* dkp[4];             // pooled fp32 sums per level: [bh][s_pad / l][D]
  float* dvp[4];
  const int2* items;         // dK/dV work list: (level index, group), heavy first
  int n_entries;             // entries of `items` (per head)
  int* counter;              // zero at launch: work beyond the first item of every CTA is claimed from it
  int32_t* status;
  int64_t seq, s_pad, bh;
  int mq, mask_cols, causal;
  float scale, scale_log2;
};

struct TmapQD {
  CUtensorMap q, d;          // {64 channels, 128 rows} boxes of Q and dO, [bh][seq][D]
};

template <int D> struct BCfg {
  static constexpr int SLABS = D / 64;
  static constexpr int TILE = SLABS * kSlab;
  static constexpr int OFF_A0 = 0;                      // stationary tile 0 (K or Q)
  static constexpr int OFF_A1 = TILE;                   // stationary tile 1 (V or dO)
  static constexpr int OFF_B0 = 2 * TILE;               // stream ring, operand 0 (Q or K): 2 stages
  static constexpr int OFF_B1 = 4 * TILE;               // stream ring, operand 1 (dO or V): 2 stages
  static constexpr int OFF_META = 6 * TILE;             // per stage 128 x 16 B (dK/dV: 128 x float2 row statistics)
  static constexpr int OFF_LC = OFF_META + 2 * 2048;    // dQ: per stage 128 floats, log2(copies) of every column (-inf: none)
  static constexpr int OFF_LIST = OFF_LC + 2 * 512;     // work lists: 3 x kMaxBlocks words
  static constexpr int OFF_CTRL = OFF_LIST + 3 * kMaxBlocks * 4;
  static constexpr int SMEM = OFF_CTRL + 512 + 1024;    // control block + alignment slack
};

struct BCtrl {
  uint64_t a_full, a_free;               // stationary tiles loaded / all products that read them complete
  uint64_t b_full[2], b0_free[2], b1_free[2];
  uint64_t s_full, p_full;               // S and dP of a tile ready / their 16-bit operands written
  uint64_t acc_full, acc_free;
  uint64_t job_ready[3], job_done[3];
  int job_id[3], job_n[3], job_last[3];  // id < 0: no more work; n = stream tiles; last = columns of the last tile (dQ) / head (dK/dV)
  int tile_flag[2];                      // dQ: the stage's tile holds the block on the causal diagonal
  uint32_t tmem_base;
  int abort_flag;
};

// ------------------------------------------------------------------------------------------------------------------
// dK / dV
// ------------------------------------------------------------------------------------------------------------------
template <int D, int FMT>
__global__ void __launch_bounds__(kThreadsBwd, 1) bwd_dkdv_tc_kernel(const __grid_constant__ TmapQD maps, const BwdParams p) {
  using C = BCfg<D>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  BCtrl* ctl = reinterpret_cast<BCtrl*>(smem + C::OFF_CTRL);
  uint32_t* lists = reinterpret_cast<uint32_t*>(smem + C::OFF_LIST);
  volatile int* abort_flag = &ctl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tc::mbar_init(&ctl->a_full, 1); tc::mbar_init(&ctl->a_free, 1);
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&ctl->b_full[i], 1); tc::mbar_init(&ctl->b0_free[i], 1); tc::mbar_init(&ctl->b1_free[i], 1);
    }
    tc::mbar_init(&ctl->s_full, 1); tc::mbar_init(&ctl->p_full, kEwWarps);
    tc::mbar_init(&ctl->acc_full, 1); tc::mbar_init(&ctl->acc_free, kEwWarps);
    for (int i = 0; i < 3; ++i) { tc::mbar_init(&ctl->job_ready[i], 1); tc::mbar_init(&ctl->job_done[i], kEwWarps + 1); }
    ctl->abort_flag = 0;
    tc::fence_mbar_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(&ctl->tmem_base, 512);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  const int nk = p.mq;                                      // key blocks = query blocks
  const int64_t total_jobs = (int64_t)p.n_entries * p.bh;
  // TMEM columns: dK [0,D), dV [128,128+D), S^T [256,384), dP^T [384,512)
  constexpr uint32_t kAccK = 0, kAccV = 128, kST = 256, kDP = 384;

  if (warp == 0) {
    // ================================================================ producer
    bool ok = true;
    int gp = 0, ic = 0;                                    // stream tiles issued so far / jobs with work so far
    int64_t job = blockIdx.x;
    for (int it = 0; ok; ++it) {
      const int slot = it % 3;
      if (it >= 3) {
        ok = tc::mbar_wait(&ctl->job_done[slot], ((it / 3) - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      if (job >= total_jobs) {
        if (lane == 0) { ctl->job_id[slot] = -1; __threadfence_block(); tc::mbar_arrive(&ctl->job_ready[slot]); }
        break;
      }
      // head-major order: the CTAs running at the same time stream the Q and dO rows of the same head (they stay in L2)
      const int2 e = p.items[job % p.n_entries];
      const int64_t bh = job / p.n_entries;
      const int li = e.x, g = e.y, l = 1 << li;
      const int n0 = g * l;                                // first key block of the group
      const int nsub = min(l, nk - n0);
      uint32_t* list = lists + slot * kMaxBlocks;
      // query blocks that selected level l for at least one of the group's key blocks, with the sub-block bits
      int n_pairs = 0;
      const int m_lo = p.causal ? n0 : 0;
      const int32_t* mbase = p.mask + (bh * p.mq) * (int64_t)p.mask_cols + n0;
      for (int m0 = m_lo; m0 < p.mq; m0 += 32) {
        const int m = m0 + lane;
        uint32_t bits = 0;
        if (m < p.mq) {
          const int32_t* row = mbase + (int64_t)m * p.mask_cols;
          for (int i = 0; i < nsub; ++i)
            if (row[i] == l && (!p.causal || n0 + i <= m)) bits |= 1u << i;
        }
        const unsigned hit = __ballot_sync(0xffffffffu, bits != 0);
        if (bits) list[n_pairs + __popc(hit & ((1u << lane) - 1))] = (uint32_t)m | bits << 16;
        n_pairs += __popc(hit);
      }
      __syncwarp();
      if (lane == 0) {
        ctl->job_id[slot] = (int)job; ctl->job_n[slot] = n_pairs; ctl->job_last[slot] = (int)bh;
        __threadfence_block();
        tc::mbar_arrive(&ctl->job_ready[slot]);
      }
      // next job (claimed now, so that the atomic's latency is hidden)
      int next = 0;
      if (lane == 0) next = atomicAdd(p.counter, 1);
      next = __shfl_sync(0xffffffffu, next, 0);
      job = (int64_t)gridDim.x + next;
      if (n_pairs == 0) continue;
      // stationary K and V rows [g*128, g*128+128) of level li (fewer at the end of the level)
      ok = tc::mbar_wait(&ctl->a_free, (ic & 1) ^ 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) {
        const int64_t n_l = p.s_pad >> li;
        const int rows = (int)min((int64_t)128, n_l - (int64_t)g * 128);
        const int64_t off = p.img.off[li] + (((int64_t)bh * p.img.groups[li] + (int64_t)g * 16) * C::SLABS << 10);
        const uint32_t bytes = (uint32_t)rows * D * 2;
        tc::bulk_load_a(tc::smem_u32(smem + C::OFF_A0), p.kimg + off, bytes, tc::smem_u32(&ctl->a_full));
        tc::bulk_load_a(tc::smem_u32(smem + C::OFF_A1), p.vimg + off, bytes, tc::smem_u32(&ctl->a_full));
        tc::mbar_arrive_expect_tx(&ctl->a_full, 2 * bytes);
      }
      ++ic;
      for (int pi = 0; pi < n_pairs && ok; ++pi, ++gp) {
        const int st = gp & 1;
        // a stage is free when both accumulating products of its previous tile have completed
        ok = tc::mbar_wait(&ctl->b0_free[st], ((gp >> 1) & 1) ^ 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane == 0) {
          const int m = (int)(list[pi] & 0xffffu);
          unsigned char* sq = smem + C::OFF_B0 + st * C::TILE;
          unsigned char* sd = smem + C::OFF_B1 + st * C::TILE;
          for (int s = 0; s < C::SLABS; ++s) {
            tc::tma_load_3d(sq + s * kSlab, &maps.q, &ctl->b_full[st], s * 64, m * 128, (int)bh);
            tc::tma_load_3d(sd + s * kSlab, &maps.d, &ctl->b_full[st], s * 64, m * 128, (int)bh);
          }
          tc::bulk_load_a(tc::smem_u32(smem + C::OFF_META + st * 2048), p.stat + (bh * p.s_pad + (int64_t)m * 128) * 2, 1024,
                          tc::smem_u32(&ctl->b_full[st]));
          tc::mbar_arrive_expect_tx(&ctl->b_full[st], 2 * C::TILE + 1024);
        }
      }
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    if (lane == 0) {
      bool ok = true;
      const uint32_t idesc_s = tc::make_idesc(FMT, 128, 128, 0, 0);
      const uint32_t idesc_acc = tc::make_idesc(FMT, 128, D, 0, 1);
      const uint64_t kdesc = tc::make_smem_desc(tc::smem_u32(smem + C::OFF_A0), 16, C::SLABS * 1024);
      const uint64_t vdesc = tc::make_smem_desc(tc::smem_u32(smem + C::OFF_A1), 16, C::SLABS * 1024);
      const uint64_t qk0 = tc::make_smem_desc(tc::smem_u32(smem + C::OFF_B0), 16, 1024);      // stream tiles as K-major B
      const uint64_t dk0 = tc::make_smem_desc(tc::smem_u32(smem + C::OFF_B1), 16, 1024);
      const uint64_t qm0 = tc::make_smem_desc(tc::smem_u32(smem + C::OFF_B0), kSlab, 1024);   // ... and as MN-major B
      const uint64_t dm0 = tc::make_smem_desc(tc::smem_u32(smem + C::OFF_B1), kSlab, 1024);
      const uint32_t ctl_a = tc::smem_u32(ctl);
      const uint32_t s_full_a = ctl_a + (uint32_t)offsetof(BCtrl, s_full), p_full_a = ctl_a + (uint32_t)offsetof(BCtrl, p_full);
      const uint32_t b_full_a = ctl_a + (uint32_t)offsetof(BCtrl, b_full);
      int gp = 0, ic = 0;
      // S^T = K Q^T and dP^T = V dO^T of the tile in stage st (N = 128 query rows); one commit for both
      auto issue_s = [&](int st) {
        const uint64_t off = (uint64_t)((uint32_t)(st * C::TILE) >> 4);
        const uint64_t qd = qk0 + off, dd = dk0 + off;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          tc::umma_ss(tmem + kST, kdesc + (uint64_t)(((ks >> 2) * 1024 + (ks & 3) * 32) >> 4),
                      qd + (uint64_t)(((ks >> 2) * kSlab + (ks & 3) * 32) >> 4), idesc_s, ks > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          tc::umma_ss(tmem + kDP, vdesc + (uint64_t)(((ks >> 2) * 1024 + (ks & 3) * 32) >> 4),
                      dd + (uint64_t)(((ks >> 2) * kSlab + (ks & 3) * 32) >> 4), idesc_s, ks > 0 ? 1u : 0u);
        tc::umma_commit_a(s_full_a);
      };
      // dV += P^T dO and dK += dS^T Q.  k-step ks = query rows [16 ks, 16 ks + 16); its 16-bit operand sits at column
      // 32 (ks / 2) + 8 (ks % 2) of the buffer the fp32 values came from
      auto issue_acc = [&](int st, bool first) {
        const uint64_t off = (uint64_t)((uint32_t)(st * C::TILE) >> 4);
        const uint64_t qd = qm0 + off, dd = dm0 + off;
        tc::umma_ts(tmem + kAccV, tmem + kST, dd, idesc_acc, first ? 0u : 1u);
#pragma unroll
        for (int ks = 1; ks < 8; ++ks)
          tc::umma_ts(tmem + kAccV, tmem + kST + (ks >> 1) * 32 + (ks & 1) * 8, dd + (uint64_t)(ks * (2048 >> 4)), idesc_acc, 1u);
        tc::umma_ts(tmem + kAccK, tmem + kDP, qd, idesc_acc, first ? 0u : 1u);
#pragma unroll
        for (int ks = 1; ks < 8; ++ks)
          tc::umma_ts(tmem + kAccK, tmem + kDP + (ks >> 1) * 32 + (ks & 1) * 8, qd + (uint64_t)(ks * (2048 >> 4)), idesc_acc, 1u);
      };
      for (int it = 0; ok; ++it) {
        const int slot = it % 3;
        ok = tc::mbar_wait(&ctl->job_ready[slot], (it / 3) & 1, abort_flag);
        if (!ok || ctl->job_id[slot] < 0) break;
        const int n = ctl->job_n[slot];
        if (n == 0) { tc::mbar_arrive(&ctl->job_done[slot]); continue; }
        ok = tc::mbar_wait(&ctl->a_full, ic & 1, abort_flag);
        if (ok) ok = tc::mbar_wait_a(b_full_a + (gp & 1) * 8, (gp >> 1) & 1, abort_flag);
        if (!ok) break;
        tc::tc_fence_after();
        issue_s(gp & 1);
        for (int pi = 0; pi < n && ok; ++pi, ++gp) {
          const int st = gp & 1;
          ok = tc::mbar_wait_a(p_full_a, gp & 1, abort_flag);
          if (ok && pi == 0 && ic > 0) ok = tc::mbar_wait(&ctl->acc_free, (ic - 1) & 1, abort_flag);
          if (!ok) break;
          tc::tc_fence_after();
          issue_acc(st, pi == 0);
          if (pi + 1 < n) {
            ok = tc::mbar_wait_a(b_full_a + (st ^ 1) * 8, ((gp + 1) >> 1) & 1, abort_flag);
            if (!ok) break;
            tc::tc_fence_after();
            issue_s(st ^ 1);      // its commit also says that both accumulating products above are complete
          }
        }
        if (!ok) break;
        tc::umma_commit(&ctl->acc_full);
        tc::umma_commit(&ctl->a_free);
        tc::mbar_arrive(&ctl->job_done[slot]);
        ++ic;
      }
    }
  } else {
    // ================================================================ element-wise warps: one thread per pooled key row
    // four groups of four warps; group cg works on query columns [32 cg, 32 cg + 32) of the tile
    const int quarter = warp & 3, cg = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tST = tmem + kST + cg * 32 + lane_base, tDP = tmem + kDP + cg * 32 + lane_base;
    const bool relay = warp == 2 && lane == 0;                 // tells the producer which stream stages are free again
    bool ok = true;
    int gp = 0, ic = 0;
    for (int it = 0; ok; ++it) {
      const int slot = it % 3;
      ok = tc::mbar_wait(&ctl->job_ready[slot], (it / 3) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int job = ctl->job_id[slot];
      if (job < 0) break;
      const int n = ctl->job_n[slot];
      const int64_t bh = ctl->job_last[slot];
      const int2 e = p.items[job % p.n_entries];
      const int li = e.x, g = e.y, l = 1 << li;
      const int n0 = g * l;
      const int64_t n_l = p.s_pad >> li;
      const int64_t t = (int64_t)g * 128 + r;                 // pooled row of this thread
      const bool exists = t < n_l;
      const int sub = (r << li) >> 7;                        // key block of the group this row belongs to
      const int64_t j0 = t * l, l_k = li == 0 ? p.seq : p.s_pad;
      const float c_static = (float)copies(j0, l, l_k, 0, 0);
      const float log2c = (float)li;                          // c_static is l = 2^li wherever it is not 0 (level 1: 1)
      // the sums of this row: groups 0, 1 store the two halves of the dK channels, groups 2, 3 those of dV
      constexpr int HD = D / 2;
      float* dst = (cg < 2 ? p.dkp[li] : p.dvp[li]) + (bh * n_l + t) * D + (cg & 1) * HD;
      if (n == 0) {
        if (exists)
          for (int c = 0; c < HD; c += 4) *reinterpret_cast<float4*>(dst + c) = make_float4(0.f, 0.f, 0.f, 0.f);
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&ctl->job_done[slot]);
        continue;
      }
      const uint32_t* list = lists + slot * kMaxBlocks;
      for (int pi = 0; pi < n && ok; ++pi, ++gp) {
        const int st = gp & 1;
        const uint32_t ent = list[pi];
        const int m = (int)(ent & 0xffffu);
        const bool act = exists && ((ent >> (16 + sub)) & 1u);
        const bool diag = p.causal && act && (n0 + sub == m);
        ok = tc::mbar_wait(&ctl->b_full[st], (gp >> 1) & 1, abort_flag);      // the row statistics of this tile
        if (ok) ok = tc::mbar_wait(&ctl->s_full, gp & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        // S^T and dP^T of this tile are complete, hence also both accumulating products of the previous tile: its stage
        // may be refilled
        if (relay && pi > 0) tc::mbar_arrive(&ctl->b0_free[st ^ 1]);
        tc::tc_fence_after();
        const float4* stat2 = reinterpret_cast<const float4*>(smem + C::OFF_META + st * 2048) + cg * 16;   // two columns each
        const bool slow = __any_sync(0xffffffffu, diag);
        const int64_t qbase = (int64_t)m * 128 + cg * 32;
        // this thread's 32 columns in two chunks of 16 (one after the other: the element-wise warps are bound by their
        // arithmetic, not by TMEM latency, and fewer live registers spare them spills).  The packed 16-bit results go back
        // IN PLACE into columns this thread has read itself - chunk c into [8 c, 8 c + 8) of its group's columns - because
        // the other groups work on the same buffers at the same time; the MMA takes every 16-element k-step from its own
        // TMEM address, so the operand need not be contiguous.
        uint32_t sa[16], da[16];
        auto chunk = [&](const uint32_t (&sv)[16], const uint32_t (&dv)[16], int c) {
          uint32_t pp[8], pd[8];
          if (!slow) {
            // every copy that exists is visible: the count c is a power of two (or 0), so it goes into the exponent -
            // p c = 2^(s scale - lse + log2 c), exact scaling - and one rounding after the product equals the reference's
            // rounding before it.  c = 0 (row not selected by this query block, or no copy exists): log2 c = -inf gives
            // p = 0 and ds = 0 * finite.  Two columns at a time on the packed fp32 pipe.
            const float lc = (act && c_static > 0.f) ? log2c : -INFINITY;
            const float2 lc2 = make_float2(lc, lc), sl2 = make_float2(p.scale_log2, p.scale_log2);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float4 s2 = stat2[c * 8 + k];                     // (-lse0, -lse1, -delta0, -delta1) of the two query columns
              const float2 x = __ffma2_rn(make_float2(__uint_as_float(sv[2 * k]), __uint_as_float(sv[2 * k + 1])), sl2,
                                          __fadd2_rn(lc2, make_float2(s2.x, s2.y)));
              const float2 pc = make_float2(ex2f(x.x), ex2f(x.y));
              const float2 y = __fmul2_rn(pc, __fadd2_rn(make_float2(__uint_as_float(dv[2 * k]), __uint_as_float(dv[2 * k + 1])),
                                                         make_float2(s2.z, s2.w)));
              pp[k] = pack16<FMT>(pc.x, pc.y);
              pd[k] = pack16<FMT>(y.x, y.y);
            }
          } else {
            // a key block on the causal diagonal: the copies a query sees depend on its position
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float4 s2 = stat2[c * 8 + k];
              const int64_t q0 = qbase + c * 16 + 2 * k;
              const float c0 = act ? (float)copies(j0, l, l_k, 1, q0) : 0.f, c1 = act ? (float)copies(j0, l, l_k, 1, q0 + 1) : 0.f;
              const float p0 = ex2f(fmaf(__uint_as_float(sv[2 * k]), p.scale_log2, s2.x));
              const float p1 = ex2f(fmaf(__uint_as_float(sv[2 * k + 1]), p.scale_log2, s2.y));
              const float y0 = p0 * (__uint_as_float(dv[2 * k]) + s2.z), y1 = p1 * (__uint_as_float(dv[2 * k + 1]) + s2.w);
              pp[k] = pack16<FMT>(c0 > 0.f ? round16<FMT>(p0) * c0 : 0.f, c1 > 0.f ? round16<FMT>(p1) * c1 : 0.f);
              pd[k] = pack16<FMT>(c0 > 0.f ? round16<FMT>(y0) * c0 : 0.f, c1 > 0.f ? round16<FMT>(y1) * c1 : 0.f);
            }
          }
          tc::tmem_st8(tST + 8 * c, pp);
          tc::tmem_st8(tDP + 8 * c, pd);
        };
        tc::tmem_ld16(tST, sa); tc::tmem_ld16(tDP, da);
        tc::tmem_wait_ld();
        chunk(sa, da, 0);
        tc::tmem_ld16(tST + 16, sa); tc::tmem_ld16(tDP + 16, da);
        tc::tmem_wait_ld();
        chunk(sa, da, 1);
        tc::tmem_wait_st();
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&ctl->p_full);
      }
      if (!ok) break;
      // ---- the pooled rows' sums
      ok = tc::mbar_wait(&ctl->acc_full, ic & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (relay) tc::mbar_arrive(&ctl->b0_free[(gp - 1) & 1]);   // the last tile's stage
      tc::tc_fence_after();
      const uint32_t tAcc = tmem + (cg < 2 ? kAccK : kAccV) + (cg & 1) * HD + lane_base;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t a[32];
        tc::tmem_ld32(tAcc + c0, a);
        tc::tmem_wait_ld();
        if (exists) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(dst + c0 + i) = make_float4(__uint_as_float(a[i]), __uint_as_float(a[i + 1]),
                                                                    __uint_as_float(a[i + 2]), __uint_as_float(a[i + 3]));
        }
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) { tc::mbar_arrive(&ctl->acc_free); tc::mbar_arrive(&ctl->job_done[slot]); }
      ++ic;
    }
  }

  tc::tc_fence_before();
  __syncthreads();
  if (ctl->abort_flag) {
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, PSA_ERR_TIMEOUT);
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------------------------------
template <int D, int FMT>
__global__ void __launch_bounds__(kThreadsBwd, 1) bwd_dq_tc_kernel(const __grid_constant__ TmapQD maps, const BwdParams p) {
  using C = BCfg<D>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  BCtrl* ctl = reinterpret_cast<BCtrl*>(smem + C::OFF_CTRL);
  uint32_t* items = reinterpret_cast<uint32_t*>(smem + C::OFF_LIST);      // selected blocks of the row being streamed
  volatile int* abort_flag = &ctl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tc::mbar_init(&ctl->a_full, 1); tc::mbar_init(&ctl->a_free, 1);
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&ctl->b_full[i], 2);            // one arrival for the V copies of the tile, one for its K copies
      tc::mbar_init(&ctl->b0_free[i], 1); tc::mbar_init(&ctl->b1_free[i], 1);
    }
    tc::mbar_init(&ctl->s_full, 1); tc::mbar_init(&ctl->p_full, kEwWarps);
    tc::mbar_init(&ctl->acc_full, 1); tc::mbar_init(&ctl->acc_free, kEwWarps);
    for (int i = 0; i < 3; ++i) { tc::mbar_init(&ctl->job_ready[i], 1); tc::mbar_init(&ctl->job_done[i], kEwWarps + 1); }
    ctl->abort_flag = 0;
    tc::fence_mbar_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(&ctl->tmem_base, 512);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  const int nk = p.mq;
  const int64_t total_rows = (int64_t)p.mq * p.bh;
  // TMEM columns: dQ [0,D), S of even tiles [128,256), S of odd tiles [256,384), dP [384,512)
  constexpr uint32_t kAcc = 0, kS = 128, kDP = 384;
  constexpr int kGroup = C::SLABS * 1024;          // 8 rows of a tile image

  if (warp == 0) {
    // ================================================================ producer
    bool ok = true;
    int gt = 0, rc = 0;                                    // stream tiles issued so far / rows with work so far
    int64_t R = blockIdx.x;
    for (int it = 0; ok; ++it) {
      const int slot = it % 3;
      if (it >= 3) {
        ok = tc::mbar_wait(&ctl->job_done[slot], ((it / 3) - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      if (R >= total_rows) {
        if (lane == 0) { ctl->job_id[slot] = -1; __threadfence_block(); tc::mbar_arrive(&ctl->job_ready[slot]); }
        break;
      }
      // head-major order (the CTAs running at the same time stream the K/V images of the same head: they stay in L2);
      // within a head the causal rows are walked from the last query block down, the long ones first
      const int m = p.causal ? p.mq - 1 - (int)(R % p.mq) : (int)(R % p.mq);
      const int64_t bh = R / p.mq;
      // the row's blocks, level by level (ordered compaction of the dense level row); entry: block | level index << 12 |
      // first column (in units of 16 tokens) << 16
      const int32_t* mrow = p.mask + (bh * p.mq + m) * (int64_t)p.mask_cols;
      const int end = p.causal ? min(nk, m + 1) : nk;
      int n_items = 0, tokens = 0;
      for (int li = 0; li < 4; ++li) {
        const int level = 1 << li, P = 128 >> li;
        for (int c0 = 0; c0 < end; c0 += 32) {
          const int c = c0 + lane;
          const bool hit = c < end && mrow[c] == level;
          const unsigned bits = __ballot_sync(0xffffffffu, hit);
          const int before = __popc(bits & ((1u << lane) - 1));
          if (hit) items[n_items + before] = (uint32_t)c | (uint32_t)li << 12 | (uint32_t)((tokens + before * P) >> 4) << 16;
          n_items += __popc(bits);
          tokens += __popc(bits) * P;
        }
      }
      __syncwarp();
      const int n_tiles = (tokens + 127) >> 7;
      const int last_cols = tokens - (n_tiles - 1) * 128;
      if (lane == 0) {
        ctl->job_id[slot] = (int)R; ctl->job_n[slot] = n_tiles; ctl->job_last[slot] = last_cols;
        __threadfence_block();
        tc::mbar_arrive(&ctl->job_ready[slot]);
      }
      int next = 0;
      if (lane == 0) next = atomicAdd(p.counter, 1);
      next = __shfl_sync(0xffffffffu, next, 0);
      R = (int64_t)gridDim.x + next;
      if (n_tiles == 0) continue;
      // stationary Q and dO tiles of the query block
      ok = tc::mbar_wait(&ctl->a_free, (rc & 1) ^ 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) {
        for (int s = 0; s < C::SLABS; ++s) {
          tc::tma_load_3d(smem + C::OFF_A0 + s * kSlab, &maps.q, &ctl->a_full, s * 64, m * 128, (int)bh);
          tc::tma_load_3d(smem + C::OFF_A1 + s * kSlab, &maps.d, &ctl->a_full, s * 64, m * 128, (int)bh);
        }
        tc::mbar_arrive_expect_tx(&ctl->a_full, 2 * C::TILE);
      }
      ++rc;
      int ki = 0;
      for (int t = 0; t < n_tiles && ok; ++t, ++gt) {
        const int st = gt & 1;
        const int probe = ki + lane;
        const int in_tile = __popc(__ballot_sync(0xffffffffu, probe < n_items && (int)(items[probe < n_items ? probe : 0] >> 19) == t));
        const uint32_t x = lane < in_tile ? items[ki + lane] : 0u;
        const int li = (x >> 12) & 3, blk = x & 0xfff, P = 128 >> li, col = ((int)(x >> 16) << 4) & 127;
        const int64_t off = p.img.off[li] + (((int64_t)bh * p.img.groups[li] + (((int64_t)blk * P) >> 3)) * C::SLABS << 10);
        const uint32_t dstoff = (uint32_t)(col >> 3) * kGroup;
        const uint32_t my_bytes = lane < in_tile ? (uint32_t)(P * D * 2) : 0u;
        const uint32_t bytes = __reduce_add_sync(0xffffffffu, my_bytes);
        // V of the stage's previous tile is free as soon as its dP is complete: the V copies leave first
        ok = tc::mbar_wait(&ctl->b1_free[st], ((gt >> 1) & 1) ^ 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane < in_tile)
          tc::bulk_load_a(tc::smem_u32(smem + C::OFF_B1 + st * C::TILE) + dstoff, p.vimg + off, my_bytes, tc::smem_u32(&ctl->b_full[st]));
        __syncwarp();
        if (lane == 0) tc::mbar_arrive_expect_tx(&ctl->b_full[st], bytes);
        // K is read last (by dQ += dS K): its release also says that the metadata of the stage are no longer needed
        ok = tc::mbar_wait(&ctl->b0_free[st], ((gt >> 1) & 1) ^ 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane < in_tile)
          tc::bulk_load_a(tc::smem_u32(smem + C::OFF_B0 + st * C::TILE) + dstoff, p.kimg + off, my_bytes, tc::smem_u32(&ctl->b_full[st]));
        // per-column metadata, written by the whole warp block after block: (first original position, positions that
        // exist from there, level, copies when nothing hides them); absent columns: zeros
        int4* meta = reinterpret_cast<int4*>(smem + C::OFF_META + st * 2048);
        float* lcol = reinterpret_cast<float*>(smem + C::OFF_LC + st * 512);
        int flag_diag = 0;
        for (int b = 0; b < in_tile; ++b) {
          const int b_li = __shfl_sync(0xffffffffu, li, b), b_blk = __shfl_sync(0xffffffffu, blk, b);
          const int b_col = __shfl_sync(0xffffffffu, col, b);
          const int b_l = 1 << b_li, b_P = 128 >> b_li;
          const int64_t l_k = b_li == 0 ? p.seq : p.s_pad;
          for (int c = lane; c < b_P; c += 32) {
            const int64_t j0 = ((int64_t)b_blk * b_P + c) * b_l;
            const int64_t avail = l_k - j0;
            const int cs = avail < 0 ? 0 : (avail > b_l ? b_l : (int)avail);
            meta[b_col + c] = make_int4((int)j0, (int)min(avail, (int64_t)1 << 30), b_l, 0);
            lcol[b_col + c] = cs > 0 ? (float)b_li : -INFINITY;      // cs is 0 or the level 2^li
          }
          if (p.causal && b_blk == m) flag_diag = 1;
        }
        const int used = t == n_tiles - 1 ? last_cols : 128;
        for (int c = used + lane; c < 128; c += 32) { meta[c] = make_int4(0, 0, 0, 0); lcol[c] = -INFINITY; }
        if (lane == 0) ctl->tile_flag[st] = flag_diag;
        ki += in_tile;
        __syncwarp();
        if (lane == 0) tc::mbar_arrive_expect_tx(&ctl->b_full[st], bytes);
      }
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    if (lane == 0) {
      bool ok = true;
      const uint32_t idesc_acc = tc::make_idesc(FMT, 128, D, 0, 1);
      const uint32_t idesc_full = tc::make_idesc(FMT, 128, 128, 0, 0);
      const uint64_t qdesc = tc::make_smem_desc(tc::smem_u32(smem + C::OFF_A0), 16, 1024);
      const uint64_t ddesc = tc::make_smem_desc(tc::smem_u32(smem + C::OFF_A1), 16, 1024);
      const uint64_t kk0 = tc::make_smem_desc(tc::smem_u32(smem + C::OFF_B0), 16, kGroup);     // stream tiles as K-major B
      const uint64_t vk0 = tc::make_smem_desc(tc::smem_u32(smem + C::OFF_B1), 16, kGroup);
      const uint64_t km0 = tc::make_smem_desc(tc::smem_u32(smem + C::OFF_B0), 1024, kGroup);   // K tile as MN-major B
      const uint32_t ctl_a = tc::smem_u32(ctl);
      const uint32_t s_full_a = ctl_a + (uint32_t)offsetof(BCtrl, s_full), p_full_a = ctl_a + (uint32_t)offsetof(BCtrl, p_full);
      const uint32_t b_full_a = ctl_a + (uint32_t)offsetof(BCtrl, b_full);
      int g0 = 0, rc = 0;                                   // stream tiles of the rows before this one / rows with work
      // S = Q K^T of tile u of the row (stage and score buffer by the running tile count), N = its columns
      auto issue_S = [&](int gu, int cols) {
        const uint64_t kd = kk0 + (uint64_t)((uint32_t)((gu & 1) * C::TILE) >> 4);
        const uint32_t idesc = cols == 128 ? idesc_full : tc::make_idesc(FMT, 128, cols, 0, 0);
        const uint32_t ts = tmem + kS + (gu & 1) * 128;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          tc::umma_ss(ts, qdesc + (uint64_t)(((ks >> 2) * kSlab + (ks & 3) * 32) >> 4),
                      kd + (uint64_t)(((ks >> 2) * 1024 + (ks & 3) * 32) >> 4), idesc, ks > 0 ? 1u : 0u);
      };
      // dP = dO V^T of the same tile; its commit covers every product issued before it
      auto issue_dP = [&](int gu, int cols) {
        const uint64_t vd = vk0 + (uint64_t)((uint32_t)((gu & 1) * C::TILE) >> 4);
        const uint32_t idesc = cols == 128 ? idesc_full : tc::make_idesc(FMT, 128, cols, 0, 0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          tc::umma_ss(tmem + kDP, ddesc + (uint64_t)(((ks >> 2) * kSlab + (ks & 3) * 32) >> 4),
                      vd + (uint64_t)(((ks >> 2) * 1024 + (ks & 3) * 32) >> 4), idesc, ks > 0 ? 1u : 0u);
        tc::umma_commit_a(s_full_a);
      };
      // dQ += dS K; k-step ks = columns [16 ks, 16 ks + 16) of the tile, whose 16-bit operand sits at column
      // 32 (ks / 2) + 8 (ks % 2) of the dP buffer
      auto issue_acc = [&](int gu, int cols, bool first) {
        const uint64_t kd = km0 + (uint64_t)((uint32_t)((gu & 1) * C::TILE) >> 4);
        if (cols == 128) {
          tc::umma_ts(tmem + kAcc, tmem + kDP, kd, idesc_acc, first ? 0u : 1u);
#pragma unroll
          for (int ks = 1; ks < 8; ++ks)
            tc::umma_ts(tmem + kAcc, tmem + kDP + (ks >> 1) * 32 + (ks & 1) * 8, kd + (uint64_t)(ks * ((2 * kGroup) >> 4)), idesc_acc, 1u);
        } else {
          for (int ks = 0; ks < cols / 16; ++ks)
            tc::umma_ts(tmem + kAcc, tmem + kDP + (ks >> 1) * 32 + (ks & 1) * 8, kd + (uint64_t)(ks * ((2 * kGroup) >> 4)), idesc_acc,
                        (first && ks == 0) ? 0u : 1u);
        }
      };
      for (int it = 0; ok; ++it) {
        const int slot = it % 3;
        ok = tc::mbar_wait(&ctl->job_ready[slot], (it / 3) & 1, abort_flag);
        if (!ok || ctl->job_id[slot] < 0) break;
        const int n = ctl->job_n[slot], last_cols = ctl->job_last[slot];
        if (n == 0) { tc::mbar_arrive(&ctl->job_done[slot]); continue; }
        auto cols_of = [&](int u) { return u == n - 1 ? last_cols : 128; };
        ok = tc::mbar_wait(&ctl->a_full, rc & 1, abort_flag);
        if (ok) ok = tc::mbar_wait_a(b_full_a + (g0 & 1) * 8, (g0 >> 1) & 1, abort_flag);
        if (!ok) break;
        tc::tc_fence_after();
        issue_S(g0, cols_of(0));
        issue_dP(g0, cols_of(0));
        // S of tile u+1 is issued as soon as its operands are there, dQ of tile u and dP of tile u+1 when the element-wise
        // warps are done with tile u: the issuer polls for whichever comes first
        int s_issued = 1, t = 0;
        uint32_t idle = 0;
        while (ok && t < n) {
          bool progressed = false;
          if (s_issued < n && s_issued <= t + 1 && tc::mbar_test_wait_a(b_full_a + ((g0 + s_issued) & 1) * 8, ((g0 + s_issued) >> 1) & 1)) {
            tc::tc_fence_after();
            issue_S(g0 + s_issued, cols_of(s_issued));
            ++s_issued;
            progressed = true;
          }
          if (tc::mbar_test_wait_a(p_full_a, (g0 + t) & 1)) {
            if (t == 0 && rc > 0) {
              ok = tc::mbar_wait(&ctl->acc_free, (rc - 1) & 1, abort_flag);
              if (!ok) break;
            }
            tc::tc_fence_after();
            issue_acc(g0 + t, cols_of(t), t == 0);
            if (t + 1 < n) {
              if (s_issued == t + 1) {      // its K/V stage has not landed yet
                ok = tc::mbar_wait_a(b_full_a + ((g0 + t + 1) & 1) * 8, ((g0 + t + 1) >> 1) & 1, abort_flag);
                if (!ok) break;
                tc::tc_fence_after();
                issue_S(g0 + t + 1, cols_of(t + 1));
                ++s_issued;
              }
              issue_dP(g0 + t + 1, cols_of(t + 1));
            }
            ++t;
            progressed = true;
          }
          if (progressed) {
            idle = 0;
          } else if (++idle > (1u << 24) || ((idle & 1023) == 1023 && *abort_flag)) {
            *abort_flag = 1;
            ok = false;
          }
        }
        if (!ok) break;
        tc::umma_commit(&ctl->acc_full);
        tc::umma_commit(&ctl->a_free);
        tc::mbar_arrive(&ctl->job_done[slot]);
        ++rc;
        g0 += n;
      }
    }
  } else {
    // ================================================================ element-wise warps: one thread per query row
    // four groups of four warps; group cg works on columns [32 cg, 32 cg + 32) of the tile
    const int quarter = warp & 3, cg = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tDP = tmem + kDP + cg * 32 + lane_base;
    const bool relay = warp == 2 && lane == 0;                 // tells the producer which stream stages are free again
    bool ok = true;
    int gt = 0, rc = 0;
    for (int it = 0; ok; ++it) {
      const int slot = it % 3;
      ok = tc::mbar_wait(&ctl->job_ready[slot], (it / 3) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int64_t R = ctl->job_id[slot];
      if (R < 0) break;
      const int n = ctl->job_n[slot], last_cols = ctl->job_last[slot];
      const int m = p.causal ? p.mq - 1 - (int)(R % p.mq) : (int)(R % p.mq);
      const int64_t bh = R / p.mq;
      const int64_t qpos = (int64_t)m * 128 + r;
      constexpr int QD = D / 4;                               // channels of the row each group stores
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.dq) + ((int64_t)bh * p.seq + qpos) * D + cg * QD;
      if (n == 0) {
        if (qpos < p.seq)
          for (int c = 0; c < QD; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0u, 0u, 0u, 0u);
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&ctl->job_done[slot]);
        continue;
      }
      // (-lse * log2 e, -delta) of this row; -inf for rows past the end
      const float* my_pair = p.stat + ((bh * p.s_pad + qpos) >> 1) * 4 + (qpos & 1);
      const float2 my = make_float2(my_pair[0], my_pair[2]);
      for (int t = 0; t < n && ok; ++t, ++gt) {
        const int st = gt & 1;
        const int used = t == n - 1 ? last_cols : 128;
        ok = tc::mbar_wait(&ctl->s_full, gt & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        // S and dP of this tile are complete, and so is dQ of the previous tile: V of this tile and K of the previous one
        // may be replaced
        if (relay) {
          tc::mbar_arrive(&ctl->b1_free[st]);
          if (t > 0) tc::mbar_arrive(&ctl->b0_free[st ^ 1]);
        }
        if (cg * 32 < used) {
          tc::tc_fence_after();
          const uint32_t tS = tmem + kS + st * 128 + cg * 32 + lane_base;
          const int4* meta = reinterpret_cast<const int4*>(smem + C::OFF_META + st * 2048) + cg * 32;
          const float2* lc2 = reinterpret_cast<const float2*>(smem + C::OFF_LC + st * 512) + cg * 16;
          const bool slow = ctl->tile_flag[st] != 0;
          const float2 sl2 = make_float2(p.scale_log2, p.scale_log2), nlse2 = make_float2(my.x, my.x), ndel2 = make_float2(my.y, my.y);
          uint32_t sa[16], da[16];
          auto chunk = [&](const uint32_t (&sv)[16], const uint32_t (&dv)[16], int c) {
            uint32_t pd[8];
            if (!slow) {
              // the copy count of a column is a power of two (or 0): it goes into the exponent, p c = 2^(s scale - lse +
              // log2 c), so one rounding after the product equals the reference's rounding before it; log2 c = -inf
              // (no copy exists) gives 0.  Two columns at a time on the packed fp32 pipe.
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const float2 x = __ffma2_rn(make_float2(__uint_as_float(sv[2 * k]), __uint_as_float(sv[2 * k + 1])), sl2,
                                            __fadd2_rn(lc2[c * 8 + k], nlse2));
                const float2 pc = make_float2(ex2f(x.x), ex2f(x.y));
                const float2 y = __fmul2_rn(pc, __fadd2_rn(make_float2(__uint_as_float(dv[2 * k]), __uint_as_float(dv[2 * k + 1])), ndel2));
                pd[k] = pack16<FMT>(y.x, y.y);
              }
            } else {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const int4 m0 = meta[c * 16 + 2 * k], m1 = meta[c * 16 + 2 * k + 1];
                const int v0 = min(m0.y, (int)min(qpos + 1 - (int64_t)m0.x, (int64_t)1 << 30));
                const int v1 = min(m1.y, (int)min(qpos + 1 - (int64_t)m1.x, (int64_t)1 << 30));
                const float c0 = (float)max(0, min(v0, m0.z)), c1 = (float)max(0, min(v1, m1.z));
                const float p0 = ex2f(fmaf(__uint_as_float(sv[2 * k]), p.scale_log2, my.x));
                const float p1 = ex2f(fmaf(__uint_as_float(sv[2 * k + 1]), p.scale_log2, my.x));
                const float y0 = p0 * (__uint_as_float(dv[2 * k]) + my.y), y1 = p1 * (__uint_as_float(dv[2 * k + 1]) + my.y);
                pd[k] = pack16<FMT>(c0 > 0.f ? round16<FMT>(y0) * c0 : 0.f, c1 > 0.f ? round16<FMT>(y1) * c1 : 0.f);
              }
            }
            tc::tmem_st8(tDP + 8 * c, pd);
          };
          // this thread's 32 columns in two chunks of 16, one after the other; the packed results go back in place into
          // columns of the dP buffer the thread has read itself (chunk c into [8 c, 8 c + 8) of its group's columns),
          // because the other groups work on the same buffer at the same time.  Columns past the tile's end hold stale
          // bits and are never read by a product.
          tc::tmem_ld16(tS, sa); tc::tmem_ld16(tDP, da);
          tc::tmem_wait_ld();
          chunk(sa, da, 0);
          tc::tmem_ld16(tS + 16, sa); tc::tmem_ld16(tDP + 16, da);
          tc::tmem_wait_ld();
          chunk(sa, da, 1);
          tc::tmem_wait_st();
          tc::tc_fence_before();
        }
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&ctl->p_full);
      }
      if (!ok) break;
      // ---- dQ rows: each group stores a quarter of the channels
      ok = tc::mbar_wait(&ctl->acc_full, rc & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (relay) tc::mbar_arrive(&ctl->b0_free[(gt - 1) & 1]);   // K of the row's last tile
      tc::tc_fence_after();
      const uint32_t tAcc = tmem + kAcc + cg * QD + lane_base;
#pragma unroll
      for (int c0 = 0; c0 < QD; c0 += 16) {
        uint32_t a[16];
        tc::tmem_ld16(tAcc + c0, a);
        tc::tmem_wait_ld();
        if (qpos < p.seq) {
#pragma unroll
          for (int i = 0; i < 16; i += 8)
            *reinterpret_cast<uint4*>(orow + c0 + i) =
                make_uint4(pack16<FMT>(__uint_as_float(a[i]) * p.scale, __uint_as_float(a[i + 1]) * p.scale),
                           pack16<FMT>(__uint_as_float(a[i + 2]) * p.scale, __uint_as_float(a[i + 3]) * p.scale),
                           pack16<FMT>(__uint_as_float(a[i + 4]) * p.scale, __uint_as_float(a[i + 5]) * p.scale),
                           pack16<FMT>(__uint_as_float(a[i + 6]) * p.scale, __uint_as_float(a[i + 7]) * p.scale));
        }
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) { tc::mbar_arrive(&ctl->acc_free); tc::mbar_arrive(&ctl->job_done[slot]); }
      ++rc;
    }
  }

  tc::tc_fence_before();
  __syncthreads();
  if (ctl->abort_flag) {
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, PSA_ERR_TIMEOUT);
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Small kernels around the two: row statistics, the dK/dV work list, the fold of the pooled sums.
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) bwd_stat_kernel(const T* __restrict__ o, const T* __restrict__ dout, const float* __restrict__ lse,
                                                       float* __restrict__ stat, int64_t bh, int64_t seq, int64_t s_pad, int D) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;       // over bh * s_pad
  if (row >= bh * s_pad) return;
  const int64_t b = row / s_pad, t = row - b * s_pad;
  float* dst = stat + (row >> 1) * 4 + (row & 1);           // per pair of rows: (-lse0, -lse1, -delta0, -delta1)
  if (t >= seq) {
    if (lane == 0) { dst[0] = -INFINITY; dst[2] = 0.f; }
    return;
  }
  const int64_t src = (b * seq + t) * D;
  float acc = 0.f;
  for (int c = lane * 2; c < D; c += 64) {
    acc = fmaf(Elem<T>::to_f(o[src + c]), Elem<T>::to_f(dout[src + c]), acc);
    acc = fmaf(Elem<T>::to_f(o[src + c + 1]), Elem<T>::to_f(dout[src + c + 1]), acc);
  }
  for (int off = 16; off; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const float l = lse[b * seq + t];
    // a row that saw no key has lse = -inf; its probabilities are taken as 0 (the reference leaves them undefined)
    dst[0] = l == -INFINITY ? -INFINITY : -l * 1.4426950408889634f;
    dst[2] = -acc;
  }
}

// Work list of the dK/dV kernel: every (level, group of 128 pooled rows), ordered by the group's first key block, so
// that under a causal mask the groups with the most query blocks come first.
__global__ void bwd_items_kernel(int2* __restrict__ items, int nk) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int n = 0;
  for (int blk = 0; blk < nk; ++blk)
    for (int li = 0; li < 4; ++li)
      if ((blk & ((1 << li) - 1)) == 0) items[n++] = make_int2(li, blk >> li);
}

// dK[j] = scale * sum_l dKp_l[j / l] / l, dV[j] = sum_l dVp_l[j / l] / l; the replicate-padded positions [seq, s_pad)
// hand their share to token seq - 1.  One thread per (head, token, 4 channels).
template <typename T, int D>
__global__ void __launch_bounds__(256) bwd_fold_kernel(BwdParams p, T* __restrict__ dk, T* __restrict__ dv) {
  constexpr int CH = D / 4;
  const int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (w >= p.bh * p.seq * CH) return;
  const int c = (int)(w % CH) * 4;
  const int64_t tok = (w / CH) % p.seq, bh = w / ((int64_t)CH * p.seq);
  float4 k4 = make_float4(0.f, 0.f, 0.f, 0.f), v4 = k4;
  auto add = [&](int64_t j) {
#pragma unroll
    for (int li = 0; li < 4; ++li) {
      const int64_t n_l = p.s_pad >> li;
      const float w_l = 1.0f / (float)(1 << li);
      const float4 a = *reinterpret_cast<const float4*>(p.dkp[li] + (bh * n_l + (j >> li)) * D + c);
      const float4 b = *reinterpret_cast<const float4*>(p.dvp[li] + (bh * n_l + (j >> li)) * D + c);
      k4.x = fmaf(a.x, w_l, k4.x); k4.y = fmaf(a.y, w_l, k4.y); k4.z = fmaf(a.z, w_l, k4.z); k4.w = fmaf(a.w, w_l, k4.w);
      v4.x = fmaf(b.x, w_l, v4.x); v4.y = fmaf(b.y, w_l, v4.y); v4.z = fmaf(b.z, w_l, v4.z); v4.w = fmaf(b.w, w_l, v4.w);
    }
  };
  add(tok);
  if (tok == p.seq - 1)
    for (int64_t j = p.seq; j < p.s_pad; ++j) add(j);
  const int64_t dst = (bh * p.seq + tok) * D + c;
  dk[dst] = Elem<T>::from_f(k4.x * p.scale); dk[dst + 1] = Elem<T>::from_f(k4.y * p.scale);
  dk[dst + 2] = Elem<T>::from_f(k4.z * p.scale); dk[dst + 3] = Elem<T>::from_f(k4.w * p.scale);
  dv[dst] = Elem<T>::from_f(v4.x); dv[dst + 1] = Elem<T>::from_f(v4.y);
  dv[dst + 2] = Elem<T>::from_f(v4.z); dv[dst + 3] = Elem<T>::from_f(v4.w);
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

struct Scratch {
  size_t stat, pooled[8], items, counters, total;
};

Scratch scratch_layout(int64_t bh, int64_t seq, int D) {
  Scratch s;
  const int64_t nk = cdiv64(seq, 128), s_pad = nk * 128;
  size_t off = 0;
  s.stat = off; off += align256((size_t)bh * s_pad * sizeof(float2));
  for (int i = 0; i < 8; ++i) {
    s.pooled[i] = off;
    off += align256((size_t)bh * (s_pad >> (i & 3)) * D * sizeof(float));
  }
  s.items = off; off += align256((size_t)2 * nk * sizeof(int2));
  s.counters = off; off += 256;
  s.total = off;
  return s;
}

template <typename T, int D, int FMT>
int launch_bwd_tc(const void* q, const void* kimg, const void* vimg, const int32_t* mask, const void* out, const float* lse,
                  const void* dout, void* dq, void* dk, void* dv, unsigned char* scratch, int64_t bh, int64_t seq, int mask_cols,
                  float scale, int causal, int32_t* status, cudaStream_t st) {
  using C = BCfg<D>;
  const int nk = (int)cdiv64(seq, 128);
  const int64_t s_pad = (int64_t)nk * 128;
  const Scratch L = scratch_layout(bh, seq, D);
  BwdParams p;
  p.mask = mask; p.kimg = (const unsigned char*)kimg; p.vimg = (const unsigned char*)vimg;
  p.img = make_img_levels(bh, seq, D, 128);
  p.stat = reinterpret_cast<const float*>(scratch + L.stat);
  p.dq = dq;
  for (int i = 0; i < 4; ++i) {
    p.dkp[i] = reinterpret_cast<float*>(scratch + L.pooled[i]);
    p.dvp[i] = reinterpret_cast<float*>(scratch + L.pooled[4 + i]);
  }
  p.items = reinterpret_cast<const int2*>(scratch + L.items);
  int n_entries = 0;
  for (int li = 0; li < 4; ++li) n_entries += (nk + (1 << li) - 1) >> li;
  p.n_entries = n_entries;
  p.status = status; p.seq = seq; p.s_pad = s_pad; p.bh = bh; p.mq = nk; p.mask_cols = mask_cols; p.causal = causal ? 1 : 0;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  int* counters = reinterpret_cast<int*>(scratch + L.counters);
  cudaError_t e = cudaMemsetAsync(counters, 0, 256, st);
  PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_legacy_bwd_tcgen05: cudaMemsetAsync failed: %s", cudaGetErrorString(e));

  bwd_stat_kernel<T><<<(unsigned)cdiv64(bh * s_pad, 8), 256, 0, st>>>((const T*)out, (const T*)dout, lse,
                                                                     reinterpret_cast<float*>(scratch + L.stat), bh, seq, s_pad, D);
  PSA_CHECK_LAUNCH("psa_legacy_bwd_tcgen05(row statistics)");
  bwd_items_kernel<<<1, 32, 0, st>>>(reinterpret_cast<int2*>(scratch + L.items), nk);
  PSA_CHECK_LAUNCH("psa_legacy_bwd_tcgen05(work list)");

  TmapQD maps;
  int rc = encode_tmap_3d(&maps.q, q, 2, FMT == 1, D, seq, bh, 128);
  if (rc != PSA_OK) return rc;
  rc = encode_tmap_3d(&maps.d, dout, 2, FMT == 1, D, seq, bh, 128);
  if (rc != PSA_OK) return rc;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  PSA_REQUIRE(sms > 0, PSA_ERR_CUDA, "psa_legacy_bwd_tcgen05: cannot read the SM count");
  {
    e = cudaFuncSetAttribute(bwd_dq_tc_kernel<D, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_legacy_bwd_tcgen05: shared-memory opt-in (%d B) failed: %s", C::SMEM, cudaGetErrorString(e));
    const int64_t rows = (int64_t)nk * bh;
    p.counter = counters;
    bwd_dq_tc_kernel<D, FMT><<<(unsigned)(rows < sms ? rows : sms), kThreadsBwd, C::SMEM, st>>>(maps, p);
    PSA_CHECK_LAUNCH("psa_legacy_bwd_tcgen05(dq)");
  }
  {
    e = cudaFuncSetAttribute(bwd_dkdv_tc_kernel<D, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_legacy_bwd_tcgen05: shared-memory opt-in (%d B) failed: %s", C::SMEM, cudaGetErrorString(e));
    const int64_t jobs = (int64_t)n_entries * bh;
    p.counter = counters + 16;
    bwd_dkdv_tc_kernel<D, FMT><<<(unsigned)(jobs < sms ? jobs : sms), kThreadsBwd, C::SMEM, st>>>(maps, p);
    PSA_CHECK_LAUNCH("psa_legacy_bwd_tcgen05(dk, dv)");
  }
  const int64_t work = bh * seq * (D / 4);
  bwd_fold_kernel<T, D><<<(unsigned)cdiv64(work, 256), 256, 0, st>>>(p, (T*)dk, (T*)dv);
  PSA_CHECK_LAUNCH("psa_legacy_bwd_tcgen05(fold)");
  return PSA_OK;
}

}  // namespace
}  // namespace psa

extern "C" size_t psa_legacy_bwd_scratch_bytes(int64_t bh, int64_t seq, int head_dim) {
  if (bh <= 0 || seq <= 0 || (head_dim != 64 && head_dim != 128)) return 0;
  return psa::scratch_layout(bh, seq, head_dim).total;
}

extern "C" int psa_legacy_bwd_tcgen05(const void* q, const void* kimg, const void* vimg, const int32_t* mask, const void* out,
                                      const float* lse, const void* dout, void* dq, void* dk, void* dv, void* scratch,
                                      size_t scratch_bytes, int64_t bh, int64_t seq, int head_dim, int mask_cols, float sm_scale,
                                      int causal, int dtype, int32_t* status, void* stream) {
  using namespace psa;
  PSA_REQUIRE(q && kimg && vimg && mask && out && lse && dout && dq && dk && dv && scratch, PSA_ERR_ARG,
              "psa_legacy_bwd_tcgen05: null pointer");
  PSA_REQUIRE(dtype == PSA_F16 || dtype == PSA_BF16, PSA_ERR_UNSUPPORTED, "psa_legacy_bwd_tcgen05: f16/bf16 only");
  PSA_REQUIRE(head_dim == 64 || head_dim == 128, PSA_ERR_ARG, "psa_legacy_bwd_tcgen05: head_dim=%d (must be 64 or 128)", head_dim);
  PSA_REQUIRE(bh > 0 && bh < 65536 && seq > 0, PSA_ERR_ARG, "psa_legacy_bwd_tcgen05: bad shape");
  const int64_t nk = cdiv64(seq, 128);
  PSA_REQUIRE(nk <= kMaxBlocks, PSA_ERR_UNSUPPORTED, "psa_legacy_bwd_tcgen05: %lld key blocks, at most %d", (long long)nk, kMaxBlocks);
  PSA_REQUIRE(mask_cols >= nk, PSA_ERR_ARG, "psa_legacy_bwd_tcgen05: mask has %d columns, needs %lld", mask_cols, (long long)nk);
  PSA_REQUIRE(sm_scale > 0.f, PSA_ERR_ARG, "psa_legacy_bwd_tcgen05: sm_scale must be positive");
  PSA_REQUIRE(2 * nk * bh < ((int64_t)1 << 31), PSA_ERR_UNSUPPORTED, "psa_legacy_bwd_tcgen05: too many (head, block) pairs");
  const void* all[] = {q, kimg, vimg, dout, dq, dk, dv};
  for (const void* ptr : all) PSA_REQUIRE(((uintptr_t)ptr & 15) == 0, PSA_ERR_ARG, "psa_legacy_bwd_tcgen05: tensors must be 16-byte aligned");
  PSA_REQUIRE(((uintptr_t)scratch & 255) == 0, PSA_ERR_ARG, "psa_legacy_bwd_tcgen05: scratch must be 256-byte aligned");
  PSA_REQUIRE(scratch_bytes >= psa_legacy_bwd_scratch_bytes(bh, seq, head_dim), PSA_ERR_ARG,
              "psa_legacy_bwd_tcgen05: scratch too small (%zu bytes)", scratch_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  unsigned char* sc = (unsigned char*)scratch;
#define PSA_BWD(TT, FMT)                                                                                                              \
  (head_dim == 64 ? launch_bwd_tc<TT, 64, FMT>(q, kimg, vimg, mask, out, lse, dout, dq, dk, dv, sc, bh, seq, mask_cols, sm_scale, causal, \
                                               status, st)                                                                            \
                  : launch_bwd_tc<TT, 128, FMT>(q, kimg, vimg, mask, out, lse, dout, dq, dk, dv, sc, bh, seq, mask_cols, sm_scale,     \
                                                causal, status, st))
  return dtype == PSA_F16 ? PSA_BWD(__half, 0) : PSA_BWD(__nv_bfloat16, 1);
#undef PSA_BWD
}
