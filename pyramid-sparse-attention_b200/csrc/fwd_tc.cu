// Multi-level block-sparse flash-attention forward on tcgen05 tensor cores (f16/bf16, block_m = 128).
//
// One CTA per (128-row query block, batch*head), 12 warps:
//   warps 0-2   producers: decode the block's index list into a flat item table, then gather the selected K/V blocks of
//               every pyramid level into 128-token tiles, PACKING blocks of different levels into the same tile.  A
//               block is P = block_n/level contiguous pooled rows.  From tile images it is ONE linear bulk copy per
//               operand; from row-major tensors one TMA box {64 ch, P rows} per 64-channel slab (128-byte swizzle).
//               Never multicast.  A copy costs its issuing thread 150-200 cycles whatever its size, so the blocks of a
//               tile are spread over the lanes of all three warps (lane l of warp w takes block 3l+w), which decode and
//               issue side by side.  K tiles and V tiles live in separate rings (K is released after S = Q K^T, V after
//               O += P V) and K runs one tile ahead of V.  The producers also write the logit bias of the tile's
//               columns (log2 of the level, -inf for columns that do not exist), per column and per group of 4 columns.
//   warp 3      MMA issuer (one thread): S = Q K^T (operands in shared memory) into one of two TMEM score buffers, and
//               O += P V with P read from TMEM and V read MN-major from its swizzled tile.  Descriptors are built once;
//               per MMA only an immediate is added.  It polls (non-blocking) for whichever product is ready and issues in
//               the fixed order QK0 QK1 PV0 QK2 PV1 ...; the tensor pipe runs in issue order, so "S of tile t ready" also
//               says that P V of tile t-2 is done with the buffer.
//   warps 4-11  softmax: two groups of four warps, ONE thread per query row.  Group g owns tiles g, g+2, g+4, ... with
//               its own running maximum, running sum and output accumulator (a split-KV inside the CTA), so no thread
//               needs another thread's partial result and the two warps on a scheduler work on different tiles.  Two
//               passes over the score tile in TMEM, 32 columns at a time with the next chunk's load in flight: maximum,
//               then exp2 / sum / round to the element type, written back IN PLACE over the scores.  The running
//               maximum is only raised when the new one exceeds it by more than 2^8 ("lazy" rescale of the accumulator).
//               Epilogue: the groups exchange (max, sum), hand each other half of their partial output through shared
//               memory and write O / sum.
// TMEM (512 columns): S0/P0 [0,128), S1/P1 [128,256), O of even tiles [256,256+D), O of odd tiles [384,384+D).
//
// Every mbarrier wait is bounded; on expiry the CTA records PSA_ERR_TIMEOUT in the status word, lets copies in
// flight land, frees its TMEM and returns.
#include <cstddef>

#include "psa_common.cuh"
#include "fwd.h"
#include "tc_common.cuh"

namespace psa {

namespace {

constexpr int kMaxWidth = 4064;        // longest index list (entries) the kernel handles
constexpr int kMaxItems = 4096;        // item table capacity (entries + extra + padding blocks)
constexpr int kSlabBytes = 128 * 128;  // 128 rows x 128 B (64 16-bit channels)
constexpr int kProducerWarps = 3;
constexpr int kProducerThreads = kProducerWarps * 32;
constexpr int kSoftmaxThreads = 256;
constexpr int kThreads = kProducerThreads + 32 + kSoftmaxThreads;   // 384
constexpr int kBiasSlots = 8;

struct TmapPack {
  CUtensorMap q;
  CUtensorMap k[4];   // levels 1, 2, 4, 8
  CUtensorMap v[4];
};

struct TcParams {
  const int32_t* mask;
  void* out;
  int32_t* status;
  int64_t seq_q;
  int64_t n[4];
  int mq, bn, tn, width, quirk;
  float scale_log2;   // sm_scale * log2(e)
  // tile-image mode: K/V of all levels pre-laid-out as shared-memory images (one linear bulk copy per block)
  const unsigned char* kimg;
  const unsigned char* vimg;
  ImgLevels img;
  OutScatter scatter;   // n_peers > 0: rows go to the peer that owns the token (plain stores over NVLink)
};

template <int D> struct Cfg {
  static constexpr int SLABS = D / 64;
  static constexpr int NK = D == 64 ? 4 : 3;   // K-tile ring
  static constexpr int NV = D == 64 ? 4 : 2;   // V-tile ring
  static constexpr int TILE_BYTES = SLABS * kSlabBytes;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + TILE_BYTES;
  static constexpr int OFF_V = OFF_K + NK * TILE_BYTES;
  static constexpr int OFF_BIAS = OFF_V + NV * TILE_BYTES;
  static constexpr int OFF_BIASG = OFF_BIAS + kBiasSlots * 128 * 4;   // one bias word per 4 columns + per-warp tile flags
  static constexpr int OFF_XCH = OFF_BIASG + kBiasSlots * (32 + 4) * 4;
  static constexpr int OFF_ROW = OFF_XCH + 2 * 2 * 128 * 4;
  static constexpr int OFF_CTRL = OFF_ROW + kMaxItems * 4;
  static constexpr int SMEM_BYTES = OFF_CTRL + 1024 + 1024;   // control block + alignment slack
};

struct Ctrl {
  uint64_t k_full[4], k_empty[4], v_full[4], v_empty[4];
  uint64_t s_full[2], p_full[2], pv_done[2], q_full;
  uint32_t tmem_base;
  int abort_flag;
  int n_sep;
  int sep[16];
  int n_tiles, last_cols, n_items;
  int seg_start[4], seg_cnt[4], item_base[4], tok_base[4];
  float qbias2[4];
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int FMT> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<1>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<0>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Item table entry (one gathered block): bits 0-11 block index, 12-13 level index, 14 extra block of a narrow level
// (reference compatibility), 15 inert padding block, 16-31 first tile column of the block counted from the start
// of the row's token stream, in units of 4 tokens.
constexpr uint32_t kItemQuirk = 1u << 14, kItemPad = 1u << 15;

#ifdef PSA_FWD_PROFILE
}  // namespace
__device__ long long g_prof[64];
__device__ long long g_trace[16 * 64];
namespace {
#define TRACE(row, t) do { if (blockIdx.x == 3 && blockIdx.y == 0 && (t) < 64) g_trace[(row) * 64 + (t)] = clock64(); } while (0)
#define PROF_T0() long long prof_t0 = clock64()
#define PROF_ADD(slot) do { long long t1 = clock64(); prof_acc[slot] += t1 - prof_t0; prof_t0 = t1; } while (0)
#else
#define PROF_T0()
#define PROF_ADD(slot)
#define TRACE(row, t)
#endif

// IMG = true: K/V tiles use the image layout [8-row group][slab][8 rows][128 B] and are filled by linear bulk copies from
// the tile-image buffers; IMG = false: [slab][128 rows][128 B] filled by tensor-map TMA boxes from row-major tensors.
template <int D, int FMT, bool IMG>
__global__ void __launch_bounds__(kThreads, 1) psa_fwd_tc_kernel(const __grid_constant__ TmapPack maps, const TcParams p) {
  using C = Cfg<D>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = smem + C::OFF_Q;
  unsigned char* sK = smem + C::OFF_K;
  unsigned char* sV = smem + C::OFF_V;
  float* sBias = reinterpret_cast<float*>(smem + C::OFF_BIAS);
  float* sBiasG = reinterpret_cast<float*>(smem + C::OFF_BIASG);   // [slot][32 group words | 3 producer flags | pad]
  float* sXch = reinterpret_cast<float*>(smem + C::OFF_XCH);      // [group][max | sum][row]
  uint32_t* sItems = reinterpret_cast<uint32_t*>(smem + C::OFF_ROW);
  Ctrl* ctl = reinterpret_cast<Ctrl*>(smem + C::OFF_CTRL);
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x;
  const int bh = blockIdx.y;
#ifdef PSA_FWD_PROFILE
  if (threadIdx.x == 0 && blockIdx.x == 3 && blockIdx.y == 0) g_prof[48] = clock64();
#endif
  const int32_t* mrow = p.mask + ((int64_t)bh * p.mq + m) * p.width;

  // ---------------------------------------------------------------- setup
  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) {
      tc::mbar_init(&ctl->k_full[i], kProducerWarps); tc::mbar_init(&ctl->k_empty[i], 1);
      tc::mbar_init(&ctl->v_full[i], kProducerWarps); tc::mbar_init(&ctl->v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&ctl->s_full[i], 1);
      tc::mbar_init(&ctl->p_full[i], 4);   // one arrival per softmax warp of the group
      tc::mbar_init(&ctl->pv_done[i], 1);
    }
    tc::mbar_init(&ctl->q_full, 1);
    ctl->abort_flag = 0;
    ctl->n_sep = 0;
    tc::fence_mbar_init();
    // the query tile does not depend on the index list: fetch it while the list is decoded
    tc::tma_prefetch_desc(&maps.q);
    for (int s = 0; s < C::SLABS; ++s) tc::tma_load_3d(sQ + s * kSlabBytes, &maps.q, &ctl->q_full, s * 64, m * 128, bh);
    tc::mbar_arrive_expect_tx(&ctl->q_full, C::TILE_BYTES);
  }
  // the raw index list is staged in the (still unused) K ring; the item table built from it stays resident
  int32_t* sTmp = reinterpret_cast<int32_t*>(sK);
  for (int i = threadIdx.x; i < p.width; i += kThreads) sTmp[i] = mrow[i];
  __syncthreads();
  if (warp == 3) {
    tc::tmem_alloc(&ctl->tmem_base, 512);
    tc::tmem_relinquish();
  }
  // separators of the index list (their order is recovered by a tiny sort)
  for (int i = threadIdx.x; i < p.width; i += kThreads)
    if (sTmp[i] == -1) {
      int slot = atomicAdd(&ctl->n_sep, 1);
      if (slot < 16) ctl->sep[slot] = i;
    }
  __syncthreads();
  if (threadIdx.x == 0) {
    int ns = ctl->n_sep < 16 ? ctl->n_sep : 16;
    for (int a = 1; a < ns; ++a) {   // insertion sort, <= 16 entries
      int v = ctl->sep[a], b = a - 1;
      while (b >= 0 && ctl->sep[b] > v) { ctl->sep[b + 1] = ctl->sep[b]; --b; }
      ctl->sep[b + 1] = v;
    }
    int prev = -1, tokens = 0, n_items = 0, last_P = p.bn;
    for (int li = 0; li < 4; ++li) {
      int end = li < ns ? ctl->sep[li] : p.width;
      int start = prev + 1;
      int cnt = end > start ? end - start : 0;      // a row that ended early leaves later segments empty
      ctl->seg_start[li] = start;
      ctl->seg_cnt[li] = cnt;
      ctl->item_base[li] = n_items;
      ctl->tok_base[li] = tokens;
      const int P = p.bn >> li;
      int items = cnt;
      const bool quirk = p.quirk && P < p.tn && cnt >= 2;
      if (quirk) items += p.tn / P - 2;
      ctl->qbias2[li] = quirk ? (float)li + log2f((float)(cnt / 2)) : 0.f;
      if (items > 0) last_P = P;
      tokens += items * P;
      n_items += items;
      prev = end;
    }
    // inert padding blocks (block 0 of the last used level, bias -inf) up to a multiple of 16 columns
    const int padded = (tokens + 15) & ~15;
    const int last_li = 31 - __clz(p.bn / last_P);
    for (int t = tokens; t < padded; t += last_P)
      sItems[n_items++] = (uint32_t)last_li << 12 | kItemPad | ((uint32_t)(t >> 2) << 16);
    ctl->n_items = n_items;
    ctl->n_tiles = (padded + 127) / 128;
    ctl->last_cols = padded - (ctl->n_tiles - 1) * 128;
  }
  __syncthreads();
  for (int li = 0; li < 4; ++li) {
    const int P = p.bn >> li, cnt = ctl->seg_cnt[li], start = ctl->seg_start[li];
    const int ib = ctl->item_base[li], tb = ctl->tok_base[li];
    for (int e = threadIdx.x; e < cnt; e += kThreads)
      sItems[ib + e] = ((uint32_t)sTmp[start + e] & 0xfffu) | (uint32_t)li << 12 | ((uint32_t)((tb + e * P) >> 2) << 16);
    if (p.quirk && P < p.tn && cnt >= 2)
      for (int j = 2 + threadIdx.x; j < p.tn / P; j += kThreads)
        sItems[ib + cnt + j - 2] = (uint32_t)j | (uint32_t)li << 12 | kItemQuirk | ((uint32_t)((tb + (cnt + j - 2) * P) >> 2) << 16);
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
#ifdef PSA_FWD_PROFILE
  if (threadIdx.x == 0 && blockIdx.x == 3 && blockIdx.y == 0) g_prof[49] = clock64();   // item table ready
#endif
  const int n_tiles = ctl->n_tiles;
  const int last_cols = ctl->last_cols;
  const uint32_t tmem = ctl->tmem_base;

  if (n_tiles > 0) {
    if (warp < kProducerWarps) {
      // ============================================================ producers
      const int n_items = ctl->n_items;
#ifdef PSA_FWD_PROFILE
      long long prof_acc[4] = {0, 0, 0, 0};
#endif
      PROF_T0();
      // everything the per-block issue needs, as plain 32-bit shared addresses / 64-bit map addresses
      const uint32_t ctl_a = tc::smem_u32(ctl);
      const uint32_t k_full_a = ctl_a + (uint32_t)offsetof(Ctrl, k_full), k_empty_a = ctl_a + (uint32_t)offsetof(Ctrl, k_empty);
      const uint32_t v_full_a = ctl_a + (uint32_t)offsetof(Ctrl, v_full), v_empty_a = ctl_a + (uint32_t)offsetof(Ctrl, v_empty);
      const uint32_t sK_a = tc::smem_u32(sK), sV_a = tc::smem_u32(sV);
      const uint64_t kmap0 = reinterpret_cast<uint64_t>(&maps.k[0]), vmap0 = reinterpret_cast<uint64_t>(&maps.v[0]);
      const int n0 = (int)p.n[0], n1 = (int)p.n[1], n2 = (int)p.n[2], n3 = (int)p.n[3];
      const float qb0 = ctl->qbias2[0], qb1 = ctl->qbias2[1], qb2 = ctl->qbias2[2], qb3 = ctl->qbias2[3];
      // The items of a tile are consecutive table entries (at most 32: blocks are at least 4 tokens wide).  Lane l of
      // producer warp w takes entry first + 3*l + w, so address arithmetic, bias and copy issue of all the blocks of a
      // tile run side by side instead of one block after the other.
      int ki = 0, vi = 0;              // first item of the next K tile / V tile
      bool ok = true;
      // step s gathers K tile s and then V tile s-1: K runs one tile ahead of V
      for (int step = 0; ok && step <= n_tiles; ++step) {
        if (step < n_tiles) {
          const int t = step, stage = t % C::NK, slot = t % kBiasSlots;
          ok = tc::mbar_wait_a(k_empty_a + stage * 8, ((t / C::NK) & 1) ^ 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          PROF_ADD(0);
          const uint32_t tile_a = sK_a + stage * C::TILE_BYTES, bar_a = k_full_a + stage * 8;
          float* bias_row = sBias + slot * 128;
          float* biasg_row = sBiasG + slot * 36;
          const int probe = ki + lane;
          const int in_tile = __popc(__ballot_sync(0xffffffffu, probe < n_items && (int)(sItems[probe < n_items ? probe : 0] >> 21) == t));
          const bool active = 3 * lane + warp < in_tile;
          const uint32_t x = active ? sItems[ki + 3 * lane + warp] : 0u;
          const int li = (x >> 12) & 3, blk = x & 0xfff, P = p.bn >> li, col = ((int)(x >> 16) << 2) & 127, row0 = blk * P;
          // logit bias of the block's columns
          const int nl = li == 0 ? n0 : (li == 1 ? n1 : (li == 2 ? n2 : n3));
          const float qb = li == 0 ? qb0 : (li == 1 ? qb1 : (li == 2 ? qb2 : qb3));
          const float bias2 = (x & kItemPad) ? -INFINITY : ((x & kItemQuirk) ? qb : (float)li);
          const int nvalid = nl - row0;
          uint32_t my_bytes = 0;
          if (active) {
            if (IMG) {
              const unsigned char* src = p.kimg + p.img.off[li] + (((int64_t)bh * p.img.groups[li] + (row0 >> 3)) * C::SLABS << 10);
              tc::bulk_load_a(tile_a + (col >> 3) * (C::SLABS * 1024), src, (uint32_t)(P * D * 2), bar_a);
            } else {
#pragma unroll
              for (int sl = 0; sl < C::SLABS; ++sl)
                tc::tma_load_3d_a(tile_a + sl * kSlabBytes + col * 128, kmap0 + (uint64_t)li * sizeof(CUtensorMap), bar_a, sl * 64, row0, bh);
            }
            my_bytes = (uint32_t)C::SLABS * P * 128u;
            if (P <= 16) {   // narrow block: its lane writes the few bias words itself
              float4* dst = reinterpret_cast<float4*>(bias_row + col);
              for (int c = 0; c < P; c += 4) {
                dst[c >> 2] = make_float4(c < nvalid ? bias2 : -INFINITY, c + 1 < nvalid ? bias2 : -INFINITY,
                                          c + 2 < nvalid ? bias2 : -INFINITY, c + 3 < nvalid ? bias2 : -INFINITY);
                biasg_row[(col + c) >> 2] = c < nvalid ? bias2 : -INFINITY;
              }
            }
          }
          // a block that ends inside a group of 4 columns makes the tile take the per-column path of the softmax
          const bool odd_edge = active && nvalid > 0 && nvalid < P && (nvalid & 3) != 0;
          const bool any_odd = __any_sync(0xffffffffu, odd_edge);
          if (lane == 0) reinterpret_cast<int*>(biasg_row)[32 + warp] = any_odd ? 1 : 0;
          // wide blocks (at most 4 per tile): the whole warp writes the bias, 4 columns per lane
          unsigned wide = __ballot_sync(0xffffffffu, active && P > 16);
          while (wide) {
            const int src_lane = __ffs(wide) - 1;
            wide &= wide - 1;
            const int w_col = __shfl_sync(0xffffffffu, col, src_lane), w_P = __shfl_sync(0xffffffffu, P, src_lane);
            const int w_nv = __shfl_sync(0xffffffffu, nvalid, src_lane);
            const float w_b = __shfl_sync(0xffffffffu, bias2, src_lane);
            const int c = lane * 4;
            if (c < w_P) {
              *reinterpret_cast<float4*>(bias_row + w_col + c) =
                  make_float4(c < w_nv ? w_b : -INFINITY, c + 1 < w_nv ? w_b : -INFINITY, c + 2 < w_nv ? w_b : -INFINITY,
                              c + 3 < w_nv ? w_b : -INFINITY);
              biasg_row[(w_col + c) >> 2] = c < w_nv ? w_b : -INFINITY;
            }
          }
          ki += in_tile;
          // the bias of this tile must be complete before the tile is announced: the softmax warps read it once the
          // scores are ready, and "scores ready" follows "K tile full" through the MMA issuer
          if (t == n_tiles - 1 && warp == 0)
            for (int c = last_cols + lane; c < 128; c += 32) { bias_row[c] = -INFINITY; biasg_row[c >> 2] = -INFINITY; }
          const uint32_t bytes = __reduce_add_sync(0xffffffffu, my_bytes);
          if (lane == 0) tc::mbar_arrive_expect_tx_a(bar_a, bytes);
          if (warp == 0 && lane == 0) TRACE(6, t);
          PROF_ADD(1);
        }
        if (step > 0) {
          const int t = step - 1, stage = t % C::NV;
          ok = tc::mbar_wait_a(v_empty_a + stage * 8, ((t / C::NV) & 1) ^ 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          PROF_ADD(2);
          const uint32_t tile_a = sV_a + stage * C::TILE_BYTES, bar_a = v_full_a + stage * 8;
          const int probe = vi + lane;
          const int in_tile = __popc(__ballot_sync(0xffffffffu, probe < n_items && (int)(sItems[probe < n_items ? probe : 0] >> 21) == t));
          const int mine = vi + 3 * lane + warp;
          uint32_t my_bytes = 0;
          if (3 * lane + warp < in_tile) {
            const uint32_t x = sItems[mine];
            const int li = (x >> 12) & 3, blk = x & 0xfff, P = p.bn >> li, col = ((int)(x >> 16) << 2) & 127;
            if (IMG) {
              const unsigned char* src = p.vimg + p.img.off[li] + (((int64_t)bh * p.img.groups[li] + ((blk * P) >> 3)) * C::SLABS << 10);
              tc::bulk_load_a(tile_a + (col >> 3) * (C::SLABS * 1024), src, (uint32_t)(P * D * 2), bar_a);
            } else {
#pragma unroll
              for (int sl = 0; sl < C::SLABS; ++sl)
                tc::tma_load_3d_a(tile_a + sl * kSlabBytes + col * 128, vmap0 + (uint64_t)li * sizeof(CUtensorMap), bar_a, sl * 64, blk * P, bh);
            }
            my_bytes = (uint32_t)C::SLABS * P * 128u;
          }
          vi += in_tile;
          const uint32_t bytes = __reduce_add_sync(0xffffffffu, my_bytes);
          if (lane == 0) tc::mbar_arrive_expect_tx_a(bar_a, bytes);
          if (warp == 0 && lane == 0) TRACE(7, t);
          PROF_ADD(3);
        }
      }
#ifdef PSA_FWD_PROFILE
      if (lane == 0 && blockIdx.x == 3 && blockIdx.y == 0) for (int i = 0; i < 4; ++i) g_prof[warp * 4 + i] = prof_acc[i];
#endif
    } else if (warp == 3) {
      // ============================================================ MMA issuer
      if (lane == 0) {
        bool ok = tc::mbar_wait(&ctl->q_full, 0, abort_flag);
        // ready-made descriptors: per tile only the stage offset is added, per MMA only an immediate
        const uint32_t idesc_pv = tc::make_idesc(FMT, 128, D, 0, 1);
        const uint32_t idesc_qk_full = tc::make_idesc(FMT, 128, 128, 0, 0);
        const uint64_t qdesc = tc::make_smem_desc(tc::smem_u32(sQ), 16, 1024);
        // image layout: 8-row groups are SLABS KiB apart and the slabs of a group follow each other
        constexpr uint32_t kGroupStride = IMG ? C::SLABS * 1024 : 1024;
        constexpr uint32_t kSlabStride = IMG ? 1024 : kSlabBytes;
        const uint64_t kdesc0 = tc::make_smem_desc(tc::smem_u32(sK), 16, kGroupStride);
        const uint64_t vdesc0 = tc::make_smem_desc(tc::smem_u32(sV), kSlabStride, kGroupStride);
        const uint32_t ctl_a = tc::smem_u32(ctl);
        const uint32_t k_full_a = ctl_a + (uint32_t)offsetof(Ctrl, k_full), k_empty_a = ctl_a + (uint32_t)offsetof(Ctrl, k_empty);
        const uint32_t v_full_a = ctl_a + (uint32_t)offsetof(Ctrl, v_full), v_empty_a = ctl_a + (uint32_t)offsetof(Ctrl, v_empty);
        const uint32_t s_full_a = ctl_a + (uint32_t)offsetof(Ctrl, s_full);
        const uint32_t p_full_a = ctl_a + (uint32_t)offsetof(Ctrl, p_full), pv_done_a = ctl_a + (uint32_t)offsetof(Ctrl, pv_done);
        int qk_next = 0, pv_next = 0;
        uint32_t idle = 0;
#ifdef PSA_FWD_PROFILE
        long long prof_acc[4] = {0, 0, 0, 0};
        long long n_idle = 0;
#endif
        PROF_T0();
        while (ok && pv_next < n_tiles) {
          bool progressed = false;
          if (pv_next < qk_next) {
            const int t = pv_next, b = t & 1, stage = t % C::NV;
            if (tc::mbar_test_wait_a(p_full_a + b * 8, (t >> 1) & 1) && tc::mbar_test_wait_a(v_full_a + stage * 8, (t / C::NV) & 1)) {
              tc::tc_fence_after();
              TRACE(0, t);
              const uint64_t vdesc = vdesc0 + (uint64_t)(stage * (C::TILE_BYTES >> 4));
              const uint32_t tP = tmem + b * 128;            // probabilities overwrite the scores they came from
              const uint32_t tO = tmem + 256 + b * 128;      // even and odd tiles accumulate separately
              if (t < n_tiles - 1 || last_cols == 128) {
                tc::umma_ts(tO, tP, vdesc, idesc_pv, t > 1 ? 1u : 0u);
#pragma unroll
                for (int ks = 1; ks < 8; ++ks) tc::umma_ts(tO, tP + ks * 8, vdesc + (uint64_t)(ks * ((2 * kGroupStride) >> 4)), idesc_pv, 1u);
              } else {
                for (int ks = 0; ks < last_cols / 16; ++ks)
                  tc::umma_ts(tO, tP + ks * 8, vdesc + (uint64_t)(ks * ((2 * kGroupStride) >> 4)), idesc_pv, (t > 1 || ks > 0) ? 1u : 0u);
              }
              tc::umma_commit_a(v_empty_a + stage * 8);   // V tile may be refilled
              tc::umma_commit_a(pv_done_a + b * 8);       // accumulator b is consistent again
              TRACE(1, t);
              ++pv_next;
              progressed = true;
              PROF_ADD(0);
            }
          }
          // S = Q K^T of tile t is only issued once P V of tile t-2 has been: the tensor pipe runs in issue order, so
          // "S_t ready" then also means that P V of tile t-2 has finished reading the probabilities that were written over
          // the scores of buffer t&1
          if (qk_next < n_tiles && qk_next <= pv_next + 1) {
            const int t = qk_next, b = t & 1, stage = t % C::NK;
            if (tc::mbar_test_wait_a(k_full_a + stage * 8, (t / C::NK) & 1)) {
              tc::tc_fence_after();
              TRACE(2, t);
              const uint64_t kdesc = kdesc0 + (uint64_t)(stage * (C::TILE_BYTES >> 4));
              const uint32_t idesc_qk = t == n_tiles - 1 ? tc::make_idesc(FMT, 128, last_cols, 0, 0) : idesc_qk_full;
              const uint32_t tSb = tmem + b * 128;
#pragma unroll
              for (int ks = 0; ks < D / 16; ++ks) {
                constexpr int dummy = 0; (void)dummy;
                const uint32_t qoff = (uint32_t)(((ks >> 2) * kSlabBytes + (ks & 3) * 32) >> 4);
                const uint32_t koff = (uint32_t)(((ks >> 2) * kSlabStride + (ks & 3) * 32) >> 4);
                tc::umma_ss(tSb, qdesc + qoff, kdesc + koff, idesc_qk, ks > 0 ? 1u : 0u);
              }
              tc::umma_commit_a(k_empty_a + stage * 8);   // K tile may be refilled
              tc::umma_commit_a(s_full_a + b * 8);
              TRACE(3, t);
              ++qk_next;
              progressed = true;
              PROF_ADD(1);
            }
          }
          if (progressed) {
            idle = 0;
          } else if (++idle > (1u << 24) || ((idle & 255) == 255 && *abort_flag)) {
            *abort_flag = 1;
            ok = false;
          }
#ifdef PSA_FWD_PROFILE
          if (!progressed) {
            const bool pv_possible = pv_next < qk_next;
            int slot = 2;
            if (pv_possible && !tc::mbar_try_wait(&ctl->p_full[pv_next & 1], (pv_next >> 1) & 1)) slot = 2;
            else if (pv_possible && !tc::mbar_try_wait(&ctl->v_full[pv_next % C::NV], (pv_next / C::NV) & 1)) slot = 3;
            if (qk_next < n_tiles && !tc::mbar_try_wait(&ctl->k_full[qk_next % C::NK], (qk_next / C::NK) & 1)) ++n_idle;
            PROF_ADD(slot);
          }
#endif
        }
#ifdef PSA_FWD_PROFILE
        if (blockIdx.x == 3 && blockIdx.y == 0) { for (int i = 0; i < 4; ++i) g_prof[16 + i] = prof_acc[i]; g_prof[20] = n_idle; g_prof[21] = n_tiles; g_prof[22] = ctl->n_items; }
#endif
      }
    } else {
      // ============================================================ softmax / epilogue
      // Two groups of four warps, one thread per query row each.  Group g owns the tiles t = g, g+2, g+4, ... with its
      // own running maximum, running sum and output accumulator, so the two warps that share a scheduler are in
      // different phases of different tiles (one on the ex2 pipe while the other scales and searches the maximum) and
      // no thread ever needs its neighbour's partial result.  The two partial outputs are merged once, at the end.
      const int quarter = warp & 3;                 // TMEM lanes this warp may touch
      const int g = (warp - 4) >> 2;                // softmax group = tile parity = score buffer = accumulator
      const int r = quarter * 32 + lane;            // row inside the query block
      const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
      const uint32_t tS = tmem + g * 128 + lane_base;         // scores of my tiles; probabilities go back in place
      const uint32_t tO = tmem + 256 + g * 128 + lane_base;   // my accumulator
      float m_run = -INFINITY, l_run = 0.f;
      bool ok = true;
#ifdef PSA_FWD_PROFILE
      long long sprof[6] = {0, 0, 0, 0, 0, 0};
      long long sprof_t = clock64();
#define SPROF(i) do { long long t1_ = clock64(); sprof[i] += t1_ - sprof_t; sprof_t = t1_; } while (0)
#else
#define SPROF(i)
#endif
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
      for (int j = g; j < n_tiles; j += 2) {
        const int slot = j % kBiasSlots, it = j >> 1;
        ok = tc::mbar_wait(&ctl->s_full[g], it & 1, abort_flag);   // scores ready (and the tile's bias words visible)
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        SPROF(0);
        if (r == 0) TRACE(4, j);
        if (lane == 0) TRACE(12 + quarter, j);
        tc::tc_fence_after();
        const bool ragged = j == n_tiles - 1 && last_cols < 128;   // columns the MMA did not write hold stale bits
        const float4* bias4 = reinterpret_cast<const float4*>(sBias + slot * 128);
        const float4* bg4 = reinterpret_cast<const float4*>(sBiasG + slot * 36);     // one bias word per 4 columns
        const int* flagw = reinterpret_cast<const int*>(sBiasG + slot * 36) + 32;
        // Fast path: the bias is uniform inside every aligned group of 4 columns (blocks are at least 4 wide), so the
        // maximum is taken on raw scores per group and the bias enters once per group.  A tile with a block that ends
        // inside a group, or with unwritten columns, takes the per-column path.
        const bool slow = ragged || (flagw[0] | flagw[1] | flagw[2]) != 0;
        uint32_t va[32], vb[32];      // two chunks of 32 score columns in flight
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
        if (!slow) {
          // pass 1: running maximum; the load of the next chunk is issued before the current one is used
#define PSA_MAX_CHUNK(v, c)                                                                                                  \
  do {                                                                                                                       \
    const float4 ga = bg4[2 * (c)], gb = bg4[2 * (c) + 1];                                                                   \
    const float* f = reinterpret_cast<const float*>(v);                                                                      \
    mx0 = fmaxf(mx0, fmaf(fmaxf(fmaxf(f[0], f[1]), fmaxf(f[2], f[3])), p.scale_log2, ga.x));                                 \
    mx1 = fmaxf(mx1, fmaf(fmaxf(fmaxf(f[4], f[5]), fmaxf(f[6], f[7])), p.scale_log2, ga.y));                                 \
    mx2 = fmaxf(mx2, fmaf(fmaxf(fmaxf(f[8], f[9]), fmaxf(f[10], f[11])), p.scale_log2, ga.z));                               \
    mx3 = fmaxf(mx3, fmaf(fmaxf(fmaxf(f[12], f[13]), fmaxf(f[14], f[15])), p.scale_log2, ga.w));                             \
    mx0 = fmaxf(mx0, fmaf(fmaxf(fmaxf(f[16], f[17]), fmaxf(f[18], f[19])), p.scale_log2, gb.x));                             \
    mx1 = fmaxf(mx1, fmaf(fmaxf(fmaxf(f[20], f[21]), fmaxf(f[22], f[23])), p.scale_log2, gb.y));                             \
    mx2 = fmaxf(mx2, fmaf(fmaxf(fmaxf(f[24], f[25]), fmaxf(f[26], f[27])), p.scale_log2, gb.z));                             \
    mx3 = fmaxf(mx3, fmaf(fmaxf(fmaxf(f[28], f[29]), fmaxf(f[30], f[31])), p.scale_log2, gb.w));                             \
  } while (0)
          tc::tmem_ld32(tS, va);
          tc::tmem_wait_ld(); tc::tmem_ld32(tS + 32, vb); PSA_MAX_CHUNK(va, 0);
          tc::tmem_wait_ld(); tc::tmem_ld32(tS + 64, va); PSA_MAX_CHUNK(vb, 1);
          tc::tmem_wait_ld(); tc::tmem_ld32(tS + 96, vb); PSA_MAX_CHUNK(va, 2);
          tc::tmem_wait_ld(); tc::tmem_ld32(tS, va);      PSA_MAX_CHUNK(vb, 3);   // chunk 0 again, for pass 2
#undef PSA_MAX_CHUNK
        } else {
#pragma unroll 1
          for (int h = 0; h < 4; ++h) {
            tc::tmem_ld32(tS + h * 32, va);
            tc::tmem_wait_ld();
            if (ragged) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (h * 32 + i >= last_cols) va[i] = 0u;
            }
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) {
              const float4 ba = bias4[h * 8 + q4];
              mx0 = fmaxf(mx0, fmaf(__uint_as_float(va[4 * q4 + 0]), p.scale_log2, ba.x));
              mx1 = fmaxf(mx1, fmaf(__uint_as_float(va[4 * q4 + 1]), p.scale_log2, ba.y));
              mx2 = fmaxf(mx2, fmaf(__uint_as_float(va[4 * q4 + 2]), p.scale_log2, ba.z));
              mx3 = fmaxf(mx3, fmaf(__uint_as_float(va[4 * q4 + 3]), p.scale_log2, ba.w));
            }
          }
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        SPROF(1);
        // raise the running maximum only when it is far off (or still unset)
        float alpha = 1.f;
        const bool raise = mx > m_run + 8.f;
        if (raise) {
          alpha = m_run == -INFINITY ? 0.f : ex2(m_run - mx);
          m_run = mx;
          l_run *= alpha;
        }
        if (it > 0 && __any_sync(0xffffffffu, raise)) {
          // the accumulator may only be touched between two of its P V products: wait for the one of tile j-2
          ok = tc::mbar_wait(&ctl->pv_done[g], (it - 1) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc::tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            tc::tmem_ld32(tO + c0, vb);
            tc::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) vb[i] = __float_as_uint(__uint_as_float(vb[i]) * alpha);
            tc::tmem_st32(tO + c0, vb);
          }
          tc::tmem_wait_st();
        }
        SPROF(2);
        // pass 2: probabilities (rounded to the element type) written over the scores, running sum.  Chunk c reads score
        // columns [32c, 32c+32) and writes packed columns [16c, 16c+16): always columns that were read before.
        const float m_use = m_run == -INFINITY ? 0.f : m_run;
        float2 ls_a = make_float2(0.f, 0.f), ls_b = make_float2(0.f, 0.f);
        if (!slow) {
#define PSA_EXP_GROUP(f, cg, k, acc)                                                                                          \
  do {                                                                                                                       \
    const float2 cc = make_float2(cg, cg);                                                                                   \
    const float2 x01 = __ffma2_rn(make_float2(f[4 * (k)], f[4 * (k) + 1]), scale2, cc);                                      \
    const float2 x23 = __ffma2_rn(make_float2(f[4 * (k) + 2], f[4 * (k) + 3]), scale2, cc);                                  \
    const float2 e01 = make_float2(ex2(x01.x), ex2(x01.y)), e23 = make_float2(ex2(x23.x), ex2(x23.y));                       \
    acc = __fadd2_rn(acc, __fadd2_rn(e01, e23));                                                                             \
    pk[2 * (k)] = pack2<FMT>(e01.x, e01.y);                                                                                  \
    pk[2 * (k) + 1] = pack2<FMT>(e23.x, e23.y);                                                                              \
  } while (0)
#define PSA_EXP_CHUNK(v, c)                                                                                                  \
  do {                                                                                                                       \
    const float4 ga = bg4[2 * (c)], gb = bg4[2 * (c) + 1];                                                                   \
    const float* f = reinterpret_cast<const float*>(v);                                                                      \
    uint32_t pk[16];                                                                                                         \
    PSA_EXP_GROUP(f, ga.x - m_use, 0, ls_a); PSA_EXP_GROUP(f, ga.y - m_use, 1, ls_b);                                        \
    PSA_EXP_GROUP(f, ga.z - m_use, 2, ls_a); PSA_EXP_GROUP(f, ga.w - m_use, 3, ls_b);                                        \
    PSA_EXP_GROUP(f, gb.x - m_use, 4, ls_a); PSA_EXP_GROUP(f, gb.y - m_use, 5, ls_b);                                        \
    PSA_EXP_GROUP(f, gb.z - m_use, 6, ls_a); PSA_EXP_GROUP(f, gb.w - m_use, 7, ls_b);                                        \
    tc::tmem_st16(tS + 16 * (c), pk);                                                                                        \
  } while (0)
          tc::tmem_wait_ld(); tc::tmem_ld32(tS + 32, vb); PSA_EXP_CHUNK(va, 0);
          tc::tmem_wait_ld(); tc::tmem_ld32(tS + 64, va); PSA_EXP_CHUNK(vb, 1);
          tc::tmem_wait_ld(); tc::tmem_ld32(tS + 96, vb); PSA_EXP_CHUNK(va, 2);
          tc::tmem_wait_ld();                             PSA_EXP_CHUNK(vb, 3);
#undef PSA_EXP_CHUNK
#undef PSA_EXP_GROUP
        } else {
#pragma unroll 1
          for (int h = 0; h < 4; ++h) {
            tc::tmem_ld32(tS + h * 32, va);
            tc::tmem_wait_ld();
            if (ragged) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (h * 32 + i >= last_cols) va[i] = 0u;
            }
            uint32_t pk[16];
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) {
              const float4 ba = bias4[h * 8 + q4];
              const float a0 = ex2(fmaf(__uint_as_float(va[4 * q4 + 0]), p.scale_log2, ba.x) - m_use);
              const float a1 = ex2(fmaf(__uint_as_float(va[4 * q4 + 1]), p.scale_log2, ba.y) - m_use);
              const float a2 = ex2(fmaf(__uint_as_float(va[4 * q4 + 2]), p.scale_log2, ba.z) - m_use);
              const float a3 = ex2(fmaf(__uint_as_float(va[4 * q4 + 3]), p.scale_log2, ba.w) - m_use);
              ls_a.x += a0 + a1;
              ls_b.x += a2 + a3;
              pk[2 * q4] = pack2<FMT>(a0, a1);
              pk[2 * q4 + 1] = pack2<FMT>(a2, a3);
            }
            tc::tmem_st16(tS + h * 16, pk);
          }
        }
        l_run += (ls_a.x + ls_a.y) + (ls_b.x + ls_b.y);
        tc::tmem_wait_st();
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&ctl->p_full[g]);   // one arrival per warp
        if (r == 0) TRACE(5, j);
        if (lane == 0) TRACE(8 + quarter, j);
        SPROF(3);
      }
#ifdef PSA_FWD_PROFILE
      if (threadIdx.x == 128 && blockIdx.x == 3 && blockIdx.y == 0) for (int i = 0; i < 6; ++i) g_prof[32 + i] = sprof[i];
#endif
      // ---- epilogue: merge the two groups' partial results
      const int my_tiles = (n_tiles - g + 1) >> 1;
      if (ok && my_tiles > 0) {
        ok = tc::mbar_wait(&ctl->pv_done[g], (my_tiles - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
      }
#ifdef PSA_FWD_PROFILE
      if (threadIdx.x == 128 && blockIdx.x == 3 && blockIdx.y == 0) g_prof[50] = clock64();   // group 0 through its last P V
#endif
      // group g publishes (maximum, sum); both groups then agree on the weights.  An aborting group still joins the
      // barriers so that the other one is not left waiting.
      sXch[g * 256 + r] = m_run;
      sXch[g * 256 + 128 + r] = l_run;
      tc::named_bar_sync(1, kSoftmaxThreads);
      const float m_o = sXch[(g ^ 1) * 256 + r], l_o = sXch[(g ^ 1) * 256 + 128 + r];
      const float m_all = fmaxf(m_run, m_o);
      const float w_me = m_run == -INFINITY ? 0.f : ex2(m_run - m_all);
      const float w_ot = m_o == -INFINITY ? 0.f : ex2(m_o - m_all);
      const float inv = 1.0f / (l_run * w_me + l_o * w_ot);     // empty row: 0/0 like the reference
      const float w = w_me * inv;
      // each group finishes half of the channels: it hands the other half of its partial output over through shared
      // memory (the K ring is idle by now), transposed so that a warp's 32 rows are 32 consecutive words
      constexpr int HALF = D / 2;
      float* stage = reinterpret_cast<float*>(sK);
      tc::tc_fence_after();
      if (ok && my_tiles > 0) {
#pragma unroll 1
        for (int c0 = 0; c0 < HALF; c0 += 32) {
          uint32_t v[32];
          tc::tmem_ld32(tO + (g ^ 1) * HALF + c0, v);
          tc::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) stage[(g * HALF + c0 + i) * 128 + r] = __uint_as_float(v[i]) * w;
        }
      }
      tc::named_bar_sync(2, kSoftmaxThreads);
      if (ok) {
        const bool other_has = n_tiles - my_tiles > 0;
        const int64_t qrow = (int64_t)m * 128 + r;
        uint16_t* orow;
        if (p.scatter.n_peers > 0 && qrow < p.seq_q) {
          const int64_t owner = qrow / p.scatter.tokens_per_rank, local = qrow - owner * p.scatter.tokens_per_rank;
          orow = reinterpret_cast<uint16_t*>(p.scatter.peer_out[owner]) +
                 (local * p.scatter.heads_total + p.scatter.head0 + bh) * D + g * HALF;
        } else {
          orow = reinterpret_cast<uint16_t*>(p.out) + ((int64_t)bh * p.seq_q + qrow) * D + g * HALF;
        }
#pragma unroll 1
        for (int c0 = 0; c0 < HALF; c0 += 32) {
          uint32_t v[32];
          if (my_tiles > 0) {
            tc::tmem_ld32(tO + g * HALF + c0, v);
            tc::tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
          }
          float f[32];
#pragma unroll
          for (int i = 0; i < 32; ++i)
            f[i] = __uint_as_float(v[i]) * w + (other_has ? stage[((g ^ 1) * HALF + c0 + i) * 128 + r] : 0.f);
          if (qrow < p.seq_q) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 o;
              o.x = pack2<FMT>(f[i], f[i + 1]);
              o.y = pack2<FMT>(f[i + 2], f[i + 3]);
              o.z = pack2<FMT>(f[i + 4], f[i + 5]);
              o.w = pack2<FMT>(f[i + 6], f[i + 7]);
              *reinterpret_cast<uint4*>(orow + c0 + i) = o;
            }
          }
        }
      }
    }
  } else if (warp >= 4) {
    // no block selected at all: the reference divides 0 by 0
    const int half = (warp - 4) >> 2;
    const int64_t qrow = (int64_t)m * 128 + (warp & 3) * 32 + lane;
    if (qrow < p.seq_q) {
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + ((int64_t)bh * p.seq_q + qrow) * D + half * (D / 2);
      if (p.scatter.n_peers > 0) {
        const int64_t owner = qrow / p.scatter.tokens_per_rank, local = qrow - owner * p.scatter.tokens_per_rank;
        orow = reinterpret_cast<uint16_t*>(p.scatter.peer_out[owner]) +
               (local * p.scatter.heads_total + p.scatter.head0 + bh) * D + half * (D / 2);
      }
      const uint32_t nan2 = pack2<FMT>(__int_as_float(0x7fc00000), __int_as_float(0x7fc00000));
      for (int c = 0; c < D / 2; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(nan2, nan2, nan2, nan2);
    }
  }

  // ---------------------------------------------------------------- teardown
  if (n_tiles == 0 && threadIdx.x == 0) tc::mbar_wait(&ctl->q_full, 0, abort_flag);   // the early query fetch must land first
  tc::tc_fence_before();
  __syncthreads();
#ifdef PSA_FWD_PROFILE
  if (threadIdx.x == 0 && blockIdx.x == 3 && blockIdx.y == 0) g_prof[51] = clock64();
#endif
  if (ctl->abort_flag) {
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, PSA_ERR_TIMEOUT);
    for (int i = 0; i < 64; ++i) __nanosleep(1000);   // let copies in flight land before the CTA retires
    __syncthreads();
  }
  if (warp == 3) {
    __syncwarp();
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, 512);
  }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time dependency on libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

}  // namespace

int encode_tmap_3d(CUtensorMap* map, const void* base, int elem_bytes, int is_bf16, int64_t channels, int64_t tokens,
                   int64_t bh, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  PSA_REQUIRE(fn != nullptr, PSA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {(cuuint64_t)channels, (cuuint64_t)tokens, (cuuint64_t)bh};
  cuuint64_t strides[2] = {(cuuint64_t)channels * elem_bytes, (cuuint64_t)tokens * channels * elem_bytes};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base),
                  dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PSA_REQUIRE(r == CUDA_SUCCESS, PSA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (tokens=%lld box_rows=%d)", (int)r,
              (long long)tokens, box_rows);
  return PSA_OK;
}

bool fwd_tc_supported(const FwdArgs& a) {
  if (a.dtype != PSA_F16 && a.dtype != PSA_BF16) return false;
  if (a.bm != 128 || a.tn != 32) return false;
  if (a.D != 64 && a.D != 128) return false;
  if (a.width > kMaxWidth) return false;
  if (a.bh > 65535) return false;
  if (!(a.scale > 0.f)) return false;
  const void* ptrs[] = {a.q, a.out, a.k[0], a.k[1], a.k[2], a.k[3], a.v[0], a.v[1], a.v[2], a.v[3]};
  for (const void* ptr : ptrs)
    if ((uintptr_t)ptr & 15) return false;
  return true;
}

template <int D, int FMT, bool IMG>
static int launch_tc(const FwdArgs& a, cudaStream_t st) {
  using C = Cfg<D>;
  TmapPack maps;
  const int is_bf16 = FMT == 1;
  int rc = encode_tmap_3d(&maps.q, a.q, 2, is_bf16, D, a.seq_q, a.bh, 128);
  if (rc != PSA_OK) return rc;
  for (int li = 0; li < 4 && !IMG; ++li) {
    const int P = a.bn >> li;
    rc = encode_tmap_3d(&maps.k[li], a.k[li], 2, is_bf16, D, a.n[li], a.bh, P);
    if (rc != PSA_OK) return rc;
    rc = encode_tmap_3d(&maps.v[li], a.v[li], 2, is_bf16, D, a.n[li], a.bh, P);
    if (rc != PSA_OK) return rc;
  }
  TcParams p;
  p.mask = a.mask; p.out = a.out; p.status = a.status; p.seq_q = a.seq_q;
  for (int i = 0; i < 4; ++i) p.n[i] = a.n[i];
  p.mq = (int)cdiv64(a.seq_q, 128); p.bn = a.bn; p.tn = a.tn; p.width = a.width; p.quirk = a.quirk;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.kimg = (const unsigned char*)a.kimg; p.vimg = (const unsigned char*)a.vimg;
  p.img = make_img_levels(a.bh, a.seq_k, D, IMG ? a.bn : 64);
  p.scatter = a.scatter;
  cudaError_t e = cudaFuncSetAttribute(psa_fwd_tc_kernel<D, FMT, IMG>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_fwd: shared-memory opt-in (%d B) failed: %s", C::SMEM_BYTES,
              cudaGetErrorString(e));
  dim3 grid(p.mq, (unsigned)a.bh);
  psa_fwd_tc_kernel<D, FMT, IMG><<<grid, kThreads, C::SMEM_BYTES, st>>>(maps, p);
  PSA_CHECK_LAUNCH("psa_fwd(tcgen05)");
  return PSA_OK;
}

int fwd_tc_launch(const FwdArgs& a, cudaStream_t st) {
  const int fmt = a.dtype == PSA_BF16 ? 1 : 0;
  const bool img = a.kimg != nullptr && a.vimg != nullptr;
  if (img) {
    PSA_REQUIRE(a.bn >= 64, PSA_ERR_UNSUPPORTED, "tile images need block_n >= 64 (blocks of at least 8 pooled rows)");
    PSA_REQUIRE((((uintptr_t)a.kimg | (uintptr_t)a.vimg) & 15) == 0, PSA_ERR_ARG, "tile images must be 16-byte aligned");
    if (a.D == 64) return fmt ? launch_tc<64, 1, true>(a, st) : launch_tc<64, 0, true>(a, st);
    return fmt ? launch_tc<128, 1, true>(a, st) : launch_tc<128, 0, true>(a, st);
  }
  if (a.D == 64) return fmt ? launch_tc<64, 1, false>(a, st) : launch_tc<64, 0, false>(a, st);
  return fmt ? launch_tc<128, 1, false>(a, st) : launch_tc<128, 0, false>(a, st);
}

}  // namespace psa

#ifdef PSA_FWD_PROFILE
extern "C" int psa_debug_read_prof(long long* host64) {
  return (int)cudaMemcpyFromSymbol(host64, psa::g_prof, sizeof(long long) * 64);
}
extern "C" int psa_debug_read_trace(long long* host512) {
  return (int)cudaMemcpyFromSymbol(host512, psa::g_trace, sizeof(long long) * 1024);
}
#endif
