// Multi-level block-sparse flash-attention forward on tcgen05 tensor cores (f16/bf16, block_m = 128).
//
// Persistent CTAs, one per SM (221 KB of shared memory and all 512 TMEM columns each), 12 warps.  A CTA starts with query
// row R = blockIdx.x (R = batch*head * Mq + query block) and claims further rows from a global counter; its roles run the
// rows as ONE continuous stream of 128-token tiles: ring stages, score buffers and barrier phases are indexed by the
// running tile count, so nothing is drained between rows.
//   warps 0-2   producers: decode a row's index list into a flat item table (double-buffered; the next row is decoded,
//               and the list after it prefetched with cp.async, while the rings of the current row are full), then gather
//               the selected K/V blocks of every pyramid level into 128-token tiles, PACKING blocks of different levels
//               into the same tile.  A block is P = block_n/level contiguous pooled rows.  From tile images it is ONE
//               linear bulk copy per operand; from row-major tensors one TMA box {64 ch, P rows} per 64-channel slab
//               (128-byte swizzle).  Never multicast.  A copy costs its issuing thread ~100 cycles whatever its size, an
//               mbarrier arrive ~250 and a wait ~170, so the blocks of a tile are spread over the lanes of ONE warp and the
//               three warps take turns (K tile t is job 2t, V tile t job 2t+1, job J belongs to warp J mod 3); every warp
//               still passes every tile's stage barrier, in order.  K tiles and V tiles live in separate rings (K is
//               released after S = Q K^T, V after O += P V) and every warp walks them with two cursors, whichever stage
//               is free first: a V stage is released late, a K stage early, and in one fixed order every K gather
//               queued behind the wait for a V stage.  The producers also write the logit bias of
//               the tile's columns (log2 of the level, -inf for columns that do not exist), per column and per group of
//               4 columns, publish every row (tile count) to the other roles and fetch its query tile as soon as the
//               previous row's last Q K^T has read the old one.
//   warp 3      MMA issuer (one thread): S = Q K^T (operands in shared memory) into one of the TMEM score buffers, and
//               O += P V with P read from TMEM and V read MN-major from its swizzled tile.  Descriptors are built once;
//               per MMA only an immediate is added.  It polls (non-blocking) for whichever product is ready and issues in
//               the fixed order QK0 QK1 PV0 QK2 PV1 ...; the tensor pipe runs in issue order, so "S of tile t ready" also
//               says that P V of tile t-2 is done with the buffer and with the accumulator (two score buffers; with three,
//               at head_dim 64, Q K^T runs up to two tiles ahead of P V and every P V is signalled instead).  The first
//               scores of the next row are computed while the softmax warps are still in the epilogue of the current one.
//   warps 4-11  softmax: two groups of four warps, ONE thread per query row.  Group g owns the tiles whose running index
//               is g (mod 2), with its own running maximum, running sum and output accumulator (a split-KV inside the
//               CTA), so no thread needs another thread's partial result and the two warps on a scheduler work on
//               different tiles.  Two passes over the score tile in TMEM, 32 columns at a time with the next chunk's load
//               in flight: maximum, then exp2 / sum / round to the element type, written back IN PLACE over the scores.
//               The running maximum is only raised when the new one exceeds it by more than 2^8 ("lazy" rescale of the
//               accumulator).  Epilogue of a row: the groups exchange (max, sum), every thread reads BOTH accumulators of
//               its row from TMEM, and after an 8x8 transpose by warp shuffles 8 lanes store one row's 128 contiguous bytes.
// TMEM (512 columns), head_dim 128: S0/P0 [0,128), S1/P1 [128,256), O of even tiles [256,384), O of odd tiles [384,512);
// head_dim 64: three score buffers [0,384), O of even tiles [384,448), O of odd tiles [448,512).
//
// bf16 without the causal rule runs the FIXED-REFERENCE variant of the same kernel: the exponent that the probabilities of
// a query row are taken relative to is the maximum of the row's FIRST tile (the group that owns that tile leaves it in
// shared memory for the other one) and is never raised.  A bf16 probability has the exponent range of fp32, so later scores
// may exceed the reference by dozens of octaves without losing a bit; the sum stays in fp32.  That removes the maximum
// pass from every tile but the first and the rescaling of the accumulator, so both groups add into ONE accumulator
// ([384, 384 + head_dim)), a third score buffer fits at head_dim 128 as well, and the row's end needs only the two sums.
// A row whose sum of probabilities exceeds 2^90 (or is NaN) sets a guard word; the exact kernel is launched right behind
// on the same stream and returns at once unless that word is set, in which case it redoes the call.  fp16 probabilities
// (range 2^-24 .. 2^15) and the causal variants always take the exact kernel.
//
// Every wait is bounded - mbarrier waits, the issuer's polling loop and the warp-group rendezvous (mbarriers, never
// bar.sync, inside the role loops); on expiry the CTA records PSA_ERR_TIMEOUT in the status word, lets copies in
// flight land, frees its TMEM and returns.
#include <cstddef>
#include <mutex>

#include "psa_common.cuh"
#include "fwd.h"
#include "tc_common.cuh"

namespace psa {

namespace {

constexpr int kMaxWidth = 1472;        // longest index list (entries) the kernel handles
constexpr int kMaxItems = 1504;        // item table capacity (entries + extra + padding blocks); two tables
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
  int total_rows;     // query blocks of all heads: mq * bh
  int* row_counter;   // device word, zero at launch: rows beyond the first one of every CTA are claimed from it
  float scale_log2;   // sm_scale * log2(e)
  // tile-image mode: K/V of all levels pre-laid-out as shared-memory images (one linear bulk copy per block)
  const unsigned char* kimg;
  const unsigned char* vimg;
  ImgLevels img;
  OutScatter scatter;   // n_peers > 0: rows go to the peer that owns the token (plain stores over NVLink)
  float* lse;           // optional log-sum-exp output
  int legacy;           // rows without a visible key give 0 / -inf instead of 0/0
  int causal;           // legacy causal rule on the diagonal block (index rows hold no block beyond the diagonal)
  int* guard;           // fixed-reference variant: set when a row's probabilities left the safe exponent range
  const int* only_if;   // run only if this word is non-zero (the exact kernel as the fixed-reference variant's fallback)
};

// FIXED (bf16, head_dim 128, no causal rule): the reference exponent of a query row is the maximum of its FIRST tile and
// is never raised - bf16 probabilities have the exponent range of fp32, so later scores may exceed it by dozens of
// octaves without harm (a guard word reports rows that came near the range; the exact kernel then redoes the call).
// No maximum pass after the first tile, no rescaling of the accumulator, hence ONE accumulator for both softmax groups
// and room for a third score buffer.
template <int D, bool FIXED = false> struct Cfg {
  static constexpr int SLABS = D / 64;
  static constexpr int NK = D == 64 ? 4 : 3;   // K-tile ring
  static constexpr int NV = D == 64 ? 4 : 2;   // V-tile ring
  // Score buffers in TMEM.  At D = 128 the two accumulators leave room for two; at D = 64 for three, and the third one
  // lets Q K^T run two tiles ahead of P V, so that a softmax group finds its next scores ready when it is done with a tile.
  static constexpr int NSB = (D == 64 || FIXED) ? 3 : 2;
  static constexpr int O_BASE = NSB * 128;          // first TMEM column of the accumulators
  static constexpr int O_STRIDE = FIXED ? 0 : (NSB == 3 ? 64 : 128);
  // head_dim 128: ONE tcgen05.commit per tile.  "Scores of tile t complete" (the barrier that frees t's K stage) is also what
  // the softmax waits for and what frees the V stage of tile t-NSB, whose product was issued before these scores - the
  // tensor pipe runs in issue order, and a commit costs the issuing thread more than an MMA.  At head_dim 64 the V ring is
  // deeper than the score buffers, the late release costs more than the commits save, and the three signals stay apart.
  static constexpr bool ONE_SIGNAL = D == 128;
  // The V stage of tile t is free when P V of tile t is complete.  With as many score buffers as V stages the scores of
  // tile t+NV say so; with more score buffers than V stages no later score does, and the product is signalled itself.
  static constexpr bool V_SIGNAL = !ONE_SIGNAL || NSB > NV;
  static constexpr int TILE_BYTES = SLABS * kSlabBytes;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + TILE_BYTES;
  static constexpr int OFF_V = OFF_K + NK * TILE_BYTES;
  static constexpr int OFF_BIAS = OFF_V + NV * TILE_BYTES;
  static constexpr int OFF_BIASG = OFF_BIAS + kBiasSlots * 128 * 4;   // one bias word per 4 columns + per-warp tile flags
  static constexpr int OFF_MINROW = OFF_BIASG + kBiasSlots * (32 + 4) * 4;   // causal: first query row that sees a column
  static constexpr int OFF_XCH = OFF_MINROW + kBiasSlots * 128;
  static constexpr int OFF_ROW = OFF_XCH + 2 * 2 * 2 * 128 * 4 + 4 * 128 * 4;   // (max, sum) of both groups, two rows in flight; reference exponents of four rows
  static constexpr int OFF_RAW = OFF_ROW + 2 * kMaxItems * 4;      // raw index list of the row being decoded
  static constexpr int OFF_CTRL = OFF_RAW + kMaxWidth * 4;
  static constexpr int SMEM_BYTES = OFF_CTRL + 1024 + 1024;   // control block + alignment slack
};

struct Ctrl {
  uint64_t k_full[4], v_full[4];
  // "stage may be refilled": two barriers per stage, used by alternate fills.  Only the warp that fills a tile arrives on
  // its full barrier, so a producer warp that was held up can find a stage two fills ahead of the one it is waiting
  // for - with one barrier per stage that looks exactly like "not yet" to a parity wait, and the warp (which owns one of
  // the next tiles) would block for good.  With two, a waiter may be up to three fills behind.
  uint64_t k_empty[8], v_empty[8];      // k_empty doubles as "scores ready" when there is one signal per tile
  uint64_t s_full[3], pv_done[2], q_full, mref_full[4];
  // probabilities of a tile written: two barriers per group, used by the group's alternate tiles.  With three score
  // buffers a group can finish its NEXT tile before the issuer has seen this one (P V also waits for the V tile), and a
  // parity wait must never fall two phases behind its barrier.
  uint64_t p_full[4];
  uint64_t row_ready[4], row_done[4], q_free, o_free;   // hand-over of query rows between the roles of a persistent CTA
  uint64_t prod_sync, xch_full;                         // bounded rendezvous of the producer warps / of the softmax warps
  int row_tiles[4], row_last_cols[4], row_index[4];   // row_index >= total_rows: no more rows
  int claimed[2];
  uint32_t tmem_base;
  int abort_flag;
  int n_sep;
  int sep[16];
  struct RowDec { int n_tiles, last_cols, n_items; float qbias2[4]; } dec[2];   // decoded rows (current / next)
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

// Rendezvous of a fixed set of warps on an mbarrier (count = number of warps): like a named barrier, but the wait is
// bounded, so a role that gave up can never leave the others parked in a hardware barrier.  `uses` counts the calls.
__device__ __forceinline__ bool warps_rendezvous(uint64_t* bar, int& uses, volatile int* abort_flag) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) tc::mbar_arrive(bar);
  const bool ok = tc::mbar_wait(bar, uses & 1, abort_flag);
  ++uses;
  return __all_sync(0xffffffffu, ok);
}

// Item table entry (one gathered block): bits 0-11 block index, 12-13 level index, 14 extra block of a narrow level
// (reference compatibility), 15 inert padding block, 16-31 first tile column of the block counted from the start
// of the row's token stream, in units of 4 tokens.
constexpr uint32_t kItemQuirk = 1u << 14, kItemPad = 1u << 15;


// IMG = true: K/V tiles use the image layout [8-row group][slab][8 rows][128 B] and are filled by linear bulk copies from
// the tile-image buffers; IMG = false: [slab][128 rows][128 B] filled by tensor-map TMA boxes from row-major tensors.
template <int D, int FMT, bool IMG, bool CAUSAL, bool FIXED>
__global__ void __launch_bounds__(kThreads, 1) psa_fwd_tc_kernel(const __grid_constant__ TmapPack maps, const TcParams p) {
  using C = Cfg<D, FIXED>;
  static_assert(!FIXED || (FMT == 1 && !CAUSAL), "the fixed reference needs bf16 probabilities and a first tile that every row sees");
  if (p.only_if && *p.only_if == 0) return;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = smem + C::OFF_Q;
  unsigned char* sK = smem + C::OFF_K;
  unsigned char* sV = smem + C::OFF_V;
  float* sBias = reinterpret_cast<float*>(smem + C::OFF_BIAS);
  float* sBiasG = reinterpret_cast<float*>(smem + C::OFF_BIASG);   // [slot][32 group words | 3 producer flags | pad]
  unsigned char* sMinRow = smem + C::OFF_MINROW;                   // [slot][128]
  float* sXch = reinterpret_cast<float*>(smem + C::OFF_XCH);      // [group][max | sum][row]
  uint32_t* sItems = reinterpret_cast<uint32_t*>(smem + C::OFF_ROW);
  Ctrl* ctl = reinterpret_cast<Ctrl*>(smem + C::OFF_CTRL);
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int32_t* sRaw = reinterpret_cast<int32_t*>(smem + C::OFF_RAW);

  // ---------------------------------------------------------------- setup (once per CTA)
  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) {
      tc::mbar_init(&ctl->k_full[i], 1);   // one producer warp fills a whole tile
      tc::mbar_init(&ctl->v_full[i], 1);
      tc::mbar_init(&ctl->k_empty[2 * i], 1); tc::mbar_init(&ctl->k_empty[2 * i + 1], 1);
      tc::mbar_init(&ctl->v_empty[2 * i], 1); tc::mbar_init(&ctl->v_empty[2 * i + 1], 1);
    }
    ctl->abort_flag = 0;
    tc::fence_mbar_init();
  } else if (threadIdx.x == 32) {
    tc::mbar_init(&ctl->s_full[2], 1);
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&ctl->s_full[i], 1);
      tc::mbar_init(&ctl->p_full[2 * i], 4);   // one arrival per softmax warp of the group
      tc::mbar_init(&ctl->p_full[2 * i + 1], 4);
      tc::mbar_init(&ctl->pv_done[i], 1);
    }
    tc::mbar_init(&ctl->q_full, 1);
    for (int i = 0; i < 4; ++i) tc::mbar_init(&ctl->mref_full[i], 4);   // the four warps of the group that owns a row's first tile
    tc::mbar_init(&ctl->q_free, 1);
    tc::mbar_init(&ctl->o_free, 8);        // one arrival per softmax warp
    tc::fence_mbar_init();
  } else if (threadIdx.x == 64) {
    for (int i = 0; i < 4; ++i) {
      tc::mbar_init(&ctl->row_ready[i], 1);
      tc::mbar_init(&ctl->row_done[i], 9);   // eight softmax warps and the MMA issuer
    }
    tc::mbar_init(&ctl->prod_sync, kProducerWarps);
    tc::mbar_init(&ctl->xch_full, 8);
    tc::fence_mbar_init();
  }
  if (warp == 3) {
    tc::tmem_alloc(&ctl->tmem_base, 512);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  volatile int* row_tiles = ctl->row_tiles;
  volatile int* row_last_cols = ctl->row_last_cols;
  volatile int* row_index = ctl->row_index;

  // A CTA is persistent: it starts with query row R = blockIdx.x (R = bh * mq + m) and claims further rows from a global
  // counter (SMs do not all run at the same speed, so a fixed split would leave the fast ones idle at the end); its three
  // roles run the rows as one continuous stream of tiles.  Ring stages, score buffers and barrier phases are indexed by
  // the running tile count g0 + t, so the producers decode and prefetch the next row while the MMAs and the softmax of
  // the current row are still in flight, and the first scores of the next row are computed under the epilogue.
  if (warp < kProducerWarps) {
    // ============================================================ producers
    const uint32_t ctl_a = tc::smem_u32(ctl);
    const uint32_t k_full_a = ctl_a + (uint32_t)offsetof(Ctrl, k_full), k_empty_a = ctl_a + (uint32_t)offsetof(Ctrl, k_empty);
    const uint32_t v_full_a = ctl_a + (uint32_t)offsetof(Ctrl, v_full), v_empty_a = ctl_a + (uint32_t)offsetof(Ctrl, v_empty);
    const uint32_t sK_a = tc::smem_u32(sK), sV_a = tc::smem_u32(sV);
    const uint64_t kmap0 = reinterpret_cast<uint64_t>(&maps.k[0]), vmap0 = reinterpret_cast<uint64_t>(&maps.v[0]);
    const int n0 = (int)p.n[0], n1 = (int)p.n[1], n2 = (int)p.n[2], n3 = (int)p.n[3];
    const int ptid = threadIdx.x;                     // 0..95
    int g0 = 0, q_rows = 0, syncs = 0;
    bool ok = true;
    // The raw index list of a row is fetched (cp.async, 4 bytes per entry) long before it is decoded.
    auto prefetch_raw = [&](int R_n) {
      if (R_n >= p.total_rows) return;
      const int32_t* mrow = p.mask + (int64_t)R_n * p.width;
      const uint32_t raw_a = tc::smem_u32(sRaw);
      for (int i = ptid; i < p.width; i += kProducerThreads)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(raw_a + 4u * (uint32_t)i), "l"(mrow + i) : "memory");
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // Decode row number rit_n (query row R_n) into item table rit_n & 1, publish it to the other roles, and start the
    // fetch of the row after it.  Called by all producer threads at the same point of their loops.
    auto decode_row = [&](int rit_n) -> bool {
      const int R_n = ctl->claimed[rit_n & 1];     // written before the rendezvous that ended the previous decode
      if (R_n >= p.total_rows) {
        // no more rows: tell the other roles through the same slot mechanism
        bool good = true;
        if (warp == 0) {
          const int rs = rit_n & 3;
          if (rit_n >= 4) {
            good = tc::mbar_wait(&ctl->row_done[rs], ((rit_n >> 2) - 1) & 1, abort_flag);
            good = __all_sync(0xffffffffu, good);
          }
          if (good && lane == 0) {
            row_index[rs] = R_n;
            __threadfence_block();
            tc::mbar_arrive(&ctl->row_ready[rs]);
          }
        }
        return good;
      }
      uint32_t* table = sItems + (rit_n & 1) * kMaxItems;
      asm volatile("cp.async.wait_all;" ::: "memory");
      if (!warps_rendezvous(&ctl->prod_sync, syncs, abort_flag)) return false;
      for (int i = ptid; i < p.width; i += kProducerThreads)
        if (sRaw[i] == -1) {
          int slot = atomicAdd(&ctl->n_sep, 1);
          if (slot < 16) ctl->sep[slot] = i;
        }
      if (!warps_rendezvous(&ctl->prod_sync, syncs, abort_flag)) return false;
      // every thread derives the level segments from the (at most 16) separator positions by itself: the four smallest
      const int ns = ctl->n_sep < 16 ? ctl->n_sep : 16;
      int sp[4];
      {
        int below = -1;
        for (int li = 0; li < 4; ++li) {
          int best = p.width;
          for (int a = 0; a < ns; ++a) {
            const int v = ctl->sep[a];
            if (v > below && v < best) best = v;
          }
          sp[li] = best;
          below = best < p.width ? best : p.width;
        }
      }
      int prev = -1, tokens = 0, n_items = 0, last_P = p.bn;
      float qb[4];
#pragma unroll
      for (int li = 0; li < 4; ++li) {
        const int end = sp[li];
        const int start = prev + 1;
        const int cnt = end > start ? end - start : 0;      // a row that ended early leaves later segments empty
        const int P = p.bn >> li;
        const bool quirk = p.quirk && P < p.tn && cnt >= 2;
        const int ib = n_items, tb = tokens;
        for (int e = ptid; e < cnt; e += kProducerThreads)
          table[ib + e] = ((uint32_t)sRaw[start + e] & 0xfffu) | (uint32_t)li << 12 | ((uint32_t)((tb + e * P) >> 2) << 16);
        if (quirk)
          for (int j = 2 + ptid; j < p.tn / P; j += kProducerThreads)
            table[ib + cnt + j - 2] = (uint32_t)j | (uint32_t)li << 12 | kItemQuirk | ((uint32_t)((tb + (cnt + j - 2) * P) >> 2) << 16);
        const int items = cnt + (quirk ? p.tn / P - 2 : 0);
        qb[li] = quirk ? (float)li + log2f((float)(cnt / 2)) : 0.f;
        if (items > 0) last_P = P;
        tokens += items * P;
        n_items += items;
        prev = end < p.width ? end : p.width;
      }
      // inert padding blocks (block 0 of the last used level, bias -inf) up to a multiple of 16 columns
      const int padded = (tokens + 15) & ~15;
      const int n_tiles = (padded + 127) / 128;
      if (ptid == 0) {
        const int last_li = 31 - __clz(p.bn / last_P);
        for (int t = tokens; t < padded; t += last_P)
          table[n_items++] = (uint32_t)last_li << 12 | kItemPad | ((uint32_t)(t >> 2) << 16);
        Ctrl::RowDec& d = ctl->dec[rit_n & 1];
        d.n_items = n_items;
        d.n_tiles = n_tiles;
        d.last_cols = padded - (n_tiles - 1) * 128;
        for (int li = 0; li < 4; ++li) d.qbias2[li] = qb[li];
      }
      // thread 0 also claims the row after this one
      if (ptid == 0) ctl->claimed[(rit_n + 1) & 1] = (int)gridDim.x + atomicAdd(p.row_counter, 1);
      if (!warps_rendezvous(&ctl->prod_sync, syncs, abort_flag)) return false;
      if (ptid == 0) ctl->n_sep = 0;
      // publish the row to the other roles.  The slot was last used four rows ago: wait until that row is finished.
      bool good = true;
      if (warp == 0) {
        const int rs = rit_n & 3;
        if (rit_n >= 4) {
          good = tc::mbar_wait(&ctl->row_done[rs], ((rit_n >> 2) - 1) & 1, abort_flag);
          good = __all_sync(0xffffffffu, good);
        }
        if (good && lane == 0) {
          row_tiles[rs] = n_tiles;
          row_last_cols[rs] = padded - (n_tiles - 1) * 128;
          row_index[rs] = R_n;
          __threadfence_block();
          tc::mbar_arrive(&ctl->row_ready[rs]);
        }
      }
      prefetch_raw(ctl->claimed[(rit_n + 1) & 1]);
      return good;
    };
    if (ptid == 0) ctl->n_sep = 0;
    if (ptid == 0) ctl->claimed[0] = (int)blockIdx.x;
    prefetch_raw(blockIdx.x);
    ok = warps_rendezvous(&ctl->prod_sync, syncs, abort_flag) && decode_row(0);
    for (int rit = 0; ok; ++rit) {
      const int R = ctl->claimed[rit & 1];         // fixed since the decode of this row
      if (R >= p.total_rows) break;
      const int m = R % p.mq, bh = R / p.mq;
      const uint32_t* sIt = sItems + (rit & 1) * kMaxItems;     // this row's item table
      // the decode (by every producer thread) ended with a rendezvous, so the row's figures are visible
      const int n_tiles = ctl->dec[rit & 1].n_tiles, last_cols = ctl->dec[rit & 1].last_cols, n_items = ctl->dec[rit & 1].n_items;
      const float qb0 = ctl->dec[rit & 1].qbias2[0], qb1 = ctl->dec[rit & 1].qbias2[1], qb2 = ctl->dec[rit & 1].qbias2[2],
                  qb3 = ctl->dec[rit & 1].qbias2[3];
      const int decode_step = n_tiles < C::NK ? n_tiles : C::NK;   // where the next row is decoded: the rings are full by then
      // The row's query tile replaces the previous one as soon as the last Q K^T of the previous non-empty row has read
      // it; warp 0 polls for that between its copies instead of holding the K/V stream back.
      bool q_pending = warp == 0 && n_tiles > 0;
      const int q_prev = q_rows;
      auto fetch_q = [&](bool block) {
        bool ready = q_prev == 0;
        if (!ready) {
          if (block) {
            ready = tc::mbar_wait(&ctl->q_free, (q_prev - 1) & 1, abort_flag);
            ready = __all_sync(0xffffffffu, ready);
            if (!ready) ok = false;
          } else {
            ready = __all_sync(0xffffffffu, tc::mbar_try_wait(&ctl->q_free, (q_prev - 1) & 1));
          }
        }
        if (ready) {
          if (lane == 0) {
            for (int s = 0; s < C::SLABS; ++s) tc::tma_load_3d(sQ + s * kSlabBytes, &maps.q, &ctl->q_full, s * 64, m * 128, bh);
            tc::mbar_arrive_expect_tx(&ctl->q_full, C::TILE_BYTES);
          }
          q_pending = false;
        }
      };
      if (q_pending) fetch_q(false);
      if (n_tiles > 0) ++q_rows;
      int ki = 0, vi = 0;              // first item of the next K tile / V tile
        // Two cursors per warp: the next V tile and the next K tile of the row.  A V stage is released late (by the completion
        // of a P V product), a K stage early (by the scores of the tile three before); walking them in one fixed order
        // made every K gather queue behind the wait for a V stage.  Every warp still passes every stage's barrier in
        // order (per cursor), the tile's owner gathers it; the row bookkeeping (query tile, decode of the next row) is
        // keyed to the K cursor.
        int kt = 0, vt = 0;
        bool decoded = false;
        uint32_t spins = 0;
        while (ok && (vt < n_tiles || !decoded)) {
          bool progressed = false;
          if (vt < kt) {
            const int t = vt, gt = g0 + t, stage = gt % C::NV;
            bool ready = true;
            if (gt >= C::NV) {
              if (!C::V_SIGNAL) {      // the scores of tile u were issued after P V of tile gt-NV, which held this stage
                const int u = gt - C::NV + C::NSB, fu = u / C::NK;
                ready = tc::mbar_test_wait_a(k_empty_a + ((u % C::NK) * 2 + (fu & 1)) * 8, (fu >> 1) & 1);
              } else {
                const int f = gt / C::NV - 1;
                ready = tc::mbar_test_wait_a(v_empty_a + (stage * 2 + (f & 1)) * 8, (f >> 1) & 1);
              }
            }
            ready = __all_sync(0xffffffffu, ready);
            if (ready) {
            const int probe = vi + lane;
            const int in_tile = __popc(__ballot_sync(0xffffffffu, probe < n_items && (int)(sIt[probe < n_items ? probe : 0] >> 21) == t));
            if ((2 * gt + 1) % kProducerWarps == warp) {
            const uint32_t tile_a = sV_a + stage * C::TILE_BYTES, bar_a = v_full_a + stage * 8;
            const int mine = vi + lane;
            uint32_t my_bytes = 0;
            if (lane < in_tile) {
              const uint32_t x = sIt[mine];
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
            const uint32_t bytes = __reduce_add_sync(0xffffffffu, my_bytes);
            if (lane == 0) tc::mbar_arrive_expect_tx_a(bar_a, bytes);
            }
            vi += in_tile;
              ++vt;
              progressed = true;
            }
          }
          if (kt < n_tiles || !decoded) {
            if (q_pending) fetch_q(kt >= C::NK - 1);   // latest before the copy that needs the previous row's last tile gone
            if (ok && !decoded && kt == decode_step) {
              ok = decode_row(rit + 1);
              decoded = true;
              progressed = true;
            }
            if (ok && kt < n_tiles) {
              const int t = kt, gt = g0 + t, stage = gt % C::NK, slot = gt % kBiasSlots;
              bool ready = true;
              if (gt >= C::NK) {      // fill number f of the stage waits for the scores of fill f-1
                const int f = gt / C::NK - 1;
                ready = tc::mbar_test_wait_a(k_empty_a + (stage * 2 + (f & 1)) * 8, (f >> 1) & 1);
              }
              ready = __all_sync(0xffffffffu, ready);
              if (ready) {
            const int probe = ki + lane;
            const int in_tile = __popc(__ballot_sync(0xffffffffu, probe < n_items && (int)(sIt[probe < n_items ? probe : 0] >> 21) == t));
            // Every producer warp waits for every tile's stage, in order (a parity wait is only valid for a waiter at most
            // one phase ahead of its barrier), but ONE warp gathers the whole tile and the warps take turns: an mbarrier
            // arrive costs its thread ~250 cycles and a wait ~170, so three warps that each handle a third of every tile
            // spend far longer per tile than one warp that handles all of it while the others work on the next ones.
            if ((2 * gt) % kProducerWarps == warp) {
            const uint32_t tile_a = sK_a + stage * C::TILE_BYTES, bar_a = k_full_a + stage * 8;
            float* bias_row = sBias + slot * 128;
            float* biasg_row = sBiasG + slot * 36;
            const bool active = lane < in_tile;
            const uint32_t x = active ? sIt[ki + lane] : 0u;
            const int li = (x >> 12) & 3, blk = x & 0xfff, P = p.bn >> li, col = ((int)(x >> 16) << 2) & 127, row0 = blk * P;
            // logit bias of the block's columns
            const int nl = li == 0 ? n0 : (li == 1 ? n1 : (li == 2 ? n2 : n3));
            const float qb = li == 0 ? qb0 : (li == 1 ? qb1 : (li == 2 ? qb2 : qb3));
            const float bias2 = (x & kItemPad) ? -INFINITY : ((x & kItemQuirk) ? qb : (float)li);
            const int nvalid = nl - row0;
            const bool diag = CAUSAL && active && blk == m && !(x & (kItemPad | kItemQuirk));
            unsigned char* minrow_row = sMinRow + slot * 128;
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
                  if (CAUSAL) {
                    const int l = 1 << li;
                    *reinterpret_cast<uchar4*>(minrow_row + col + c) =
                        diag ? make_uchar4((c + 1) * l - 1, (c + 2) * l - 1, (c + 3) * l - 1, (c + 4) * l - 1) : make_uchar4(0, 0, 0, 0);
                  }
                }
              }
            }
            // a block that ends inside a group of 4 columns, or the diagonal block of a causal row, makes the tile take the
            // per-column path of the softmax
            const bool odd_edge = active && ((nvalid > 0 && nvalid < P && (nvalid & 3) != 0) || diag);
            const bool any_odd = __any_sync(0xffffffffu, odd_edge);
            if (lane < 3) reinterpret_cast<int*>(biasg_row)[32 + lane] = (lane == 0 && any_odd) ? 1 : 0;
            // wide blocks (at most 4 per tile): the whole warp writes the bias, 4 columns per lane
            unsigned wide = __ballot_sync(0xffffffffu, active && P > 16);
            while (wide) {
              const int src_lane = __ffs(wide) - 1;
              wide &= wide - 1;
              const int w_col = __shfl_sync(0xffffffffu, col, src_lane), w_P = __shfl_sync(0xffffffffu, P, src_lane);
              const int w_nv = __shfl_sync(0xffffffffu, nvalid, src_lane);
              const float w_b = __shfl_sync(0xffffffffu, bias2, src_lane);
              const int w_diag = __shfl_sync(0xffffffffu, (int)diag, src_lane), w_li = __shfl_sync(0xffffffffu, li, src_lane);
              const int c = lane * 4;
              if (c < w_P) {
                *reinterpret_cast<float4*>(bias_row + w_col + c) =
                    make_float4(c < w_nv ? w_b : -INFINITY, c + 1 < w_nv ? w_b : -INFINITY, c + 2 < w_nv ? w_b : -INFINITY,
                                c + 3 < w_nv ? w_b : -INFINITY);
                biasg_row[(w_col + c) >> 2] = c < w_nv ? w_b : -INFINITY;
                if (CAUSAL) {
                  const int l = 1 << w_li;
                  *reinterpret_cast<uchar4*>(minrow_row + w_col + c) =
                      w_diag ? make_uchar4((c + 1) * l - 1, (c + 2) * l - 1, (c + 3) * l - 1, (c + 4) * l - 1) : make_uchar4(0, 0, 0, 0);
                }
              }
            }
            // the bias of this tile must be complete before the tile is announced: the softmax warps read it once the
            // scores are ready, and "scores ready" follows "K tile full" through the MMA issuer
            if (t == n_tiles - 1)
              for (int c = last_cols + lane; c < 128; c += 32) { bias_row[c] = -INFINITY; biasg_row[c >> 2] = -INFINITY; }
            const uint32_t bytes = __reduce_add_sync(0xffffffffu, my_bytes);
            if (lane == 0) tc::mbar_arrive_expect_tx_a(bar_a, bytes);
            }
            ki += in_tile;
                ++kt;
                progressed = true;
              }
            }
          }
          if (progressed) {
            spins = 0;
          } else if (++spins > (1u << 24) || ((spins & 255) == 255 && *abort_flag)) {
            *abort_flag = 1;
            ok = false;
          }
        }
      if (ok && q_pending) fetch_q(true);
      g0 += n_tiles;
      if (!ok) break;
    }
  } else if (warp == 3) {
    // ============================================================ MMA issuer
    if (lane == 0) {
      bool ok = true;
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
      const uint32_t q_free_a = ctl_a + (uint32_t)offsetof(Ctrl, q_free), o_free_a = ctl_a + (uint32_t)offsetof(Ctrl, o_free);
      uint32_t idle = 0;
      int g0 = 0, q_rows = 0;
      for (int rit = 0; ok; ++rit) {
        const int rslot = rit & 3;
        ok = tc::mbar_wait(&ctl->row_ready[rslot], (rit >> 2) & 1, abort_flag);
        if (!ok || row_index[rslot] >= p.total_rows) break;
        const int n_tiles = row_tiles[rslot], last_cols = row_last_cols[rslot];
        if (n_tiles == 0) {
          tc::mbar_arrive(&ctl->row_done[rslot]);
          continue;
        }
        ok = tc::mbar_wait(&ctl->q_full, q_rows & 1, abort_flag);
        if (!ok) break;
        // both accumulators are overwritten by this row's first P V products: the previous row's epilogue must have read
        // them by then (the first Q K^T products of the row do not wait for that)
        bool o_ok = q_rows == 0;
        tc::tc_fence_after();
        int qk_next = 0, pv_next = 0;
          while (ok && pv_next < n_tiles) {
            bool progressed = false;
            if (pv_next < qk_next) {
              const int t = pv_next, gt = g0 + t, b = gt & 1, stage = gt % C::NV;
              if (!o_ok) o_ok = tc::mbar_test_wait_a(o_free_a, (q_rows - 1) & 1);
            if (o_ok && tc::mbar_test_wait_a(p_full_a + (b * 2 + ((gt >> 1) & 1)) * 8, (gt >> 2) & 1) && tc::mbar_test_wait_a(v_full_a + stage * 8, (gt / C::NV) & 1)) {
                tc::tc_fence_after();
                const uint64_t vdesc = vdesc0 + (uint64_t)(stage * (C::TILE_BYTES >> 4));
                const uint32_t tP = tmem + (gt % C::NSB) * 128;              // probabilities overwrite the scores they came from
                const uint32_t tO = tmem + C::O_BASE + b * C::O_STRIDE;      // even and odd tiles accumulate separately
                if (t < n_tiles - 1 || last_cols == 128) {
                  tc::umma_ts(tO, tP, vdesc, idesc_pv, t > (FIXED ? 0 : 1) ? 1u : 0u);
#pragma unroll
                  for (int ks = 1; ks < 8; ++ks) tc::umma_ts(tO, tP + ks * 8, vdesc + (uint64_t)(ks * ((2 * kGroupStride) >> 4)), idesc_pv, 1u);
                } else {
                  for (int ks = 0; ks < last_cols / 16; ++ks)
                    tc::umma_ts(tO, tP + ks * 8, vdesc + (uint64_t)(ks * ((2 * kGroupStride) >> 4)), idesc_pv, (t > (FIXED ? 0 : 1) || ks > 0) ? 1u : 0u);
                }
                if (C::V_SIGNAL) tc::umma_commit_a(v_empty_a + (stage * 2 + ((gt / C::NV) & 1)) * 8);   // V tile may be refilled
                // a tcgen05.commit costs this thread 100-500 cycles: "accumulator b is final" is only signalled for its last
                // tile of the row (in between, the scores of tile t+2 - issued after this product - say the same)
                // With three score buffers the next scores of this group may be issued before this product, so every product
                // is signalled (the softmax waits for it before it rescales the accumulator).
                if (FIXED) {      // one accumulator, never touched between products: only the row's last product is signalled
                  if (t == n_tiles - 1) tc::umma_commit_a(pv_done_a);
                } else if (C::NSB == 3 || t >= n_tiles - 2) tc::umma_commit_a(pv_done_a + b * 8);
                ++pv_next;
                progressed = true;
              }
            }
            // S = Q K^T of tile t is only issued once P V of tile t-NSB has been (NSB score buffers): the tensor pipe runs in
            // issue order, so "S_t ready" then also means that P V of tile t-NSB has finished reading the probabilities that
            // were written over the scores of buffer t mod NSB
            if (qk_next < n_tiles && qk_next <= pv_next + C::NSB - 1) {
              const int t = qk_next, gt = g0 + t, stage = gt % C::NK;
              if (tc::mbar_test_wait_a(k_full_a + stage * 8, (gt / C::NK) & 1)) {
                tc::tc_fence_after();
                const uint64_t kdesc = kdesc0 + (uint64_t)(stage * (C::TILE_BYTES >> 4));
                const uint32_t idesc_qk = t == n_tiles - 1 ? tc::make_idesc(FMT, 128, last_cols, 0, 0) : idesc_qk_full;
                const uint32_t tSb = tmem + (gt % C::NSB) * 128;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                  const uint32_t qoff = (uint32_t)(((ks >> 2) * kSlabBytes + (ks & 3) * 32) >> 4);
                  const uint32_t koff = (uint32_t)(((ks >> 2) * kSlabStride + (ks & 3) * 32) >> 4);
                  tc::umma_ss(tSb, qdesc + qoff, kdesc + koff, idesc_qk, ks > 0 ? 1u : 0u);
                }
                tc::umma_commit_a(k_empty_a + (stage * 2 + ((gt / C::NK) & 1)) * 8);   // K tile may be refilled (ONE_SIGNAL: scores ready)
                if (!C::ONE_SIGNAL) tc::umma_commit_a(s_full_a + (gt % C::NSB) * 8);
              if (t == n_tiles - 1) tc::umma_commit_a(q_free_a);   // the query tile may be replaced
                ++qk_next;
                progressed = true;
              }
            }
            if (progressed) {
              idle = 0;
            } else if (++idle > (1u << 24) || ((idle & 255) == 255 && *abort_flag)) {
              *abort_flag = 1;
              ok = false;
            }
          }
        if (ok) tc::mbar_arrive(&ctl->row_done[rslot]);
        ++q_rows;
        g0 += n_tiles;
      }
    }
  } else {
    // ============================================================ softmax / epilogue
    // Two groups of four warps, one thread per query row.  Group g owns the tiles whose running index is g (mod 2),
    // with its own running maximum, running sum and output accumulator, so the two warps that share a scheduler are in
    // different phases of different tiles and no thread ever needs its neighbour's partial result.  At the end of a row
    // every thread reads BOTH accumulators of its row from TMEM (a warp may read any column of its own lanes) and writes
    // half of the channels.
    const int quarter = warp & 3;                 // TMEM lanes this warp may touch
    const int g = (warp - 4) >> 2;                // softmax group = tile parity = score buffer = accumulator
    const int r = quarter * 32 + lane;            // row inside the query block
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS_mine = tmem + g * 128 + lane_base;    // scores of my tiles (two score buffers); probabilities go back in place
    const uint32_t tO = tmem + C::O_BASE + g * C::O_STRIDE + lane_base;   // my accumulator
    const uint32_t tO_other = tmem + C::O_BASE + (g ^ 1) * C::O_STRIDE + lane_base;
    const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
    bool ok = true;
    int g0 = 0, q_rows = 0, pv_rows = 0;
    float* sMref = sXch + 1024;                   // fixed reference: [row & 3][128], behind the exchange area
    for (int rit = 0; ok; ++rit) {
      const int rslot = rit & 3;
      ok = tc::mbar_wait(&ctl->row_ready[rslot], (rit >> 2) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int R = row_index[rslot];
      if (R >= p.total_rows) break;
      const int m = R % p.mq, bh = R / p.mq;
      const int n_tiles = row_tiles[rslot], last_cols = row_last_cols[rslot];
      constexpr int HALF = D / 2;
      const int64_t qrow = (int64_t)m * 128 + r;
      uint16_t* orow;
      if (p.scatter.n_peers > 0 && qrow < p.seq_q) {
        const int64_t drow = p.scatter.row_perm ? (int64_t)p.scatter.row_perm[qrow] : qrow;
        const int64_t owner = drow / p.scatter.tokens_per_rank, local = drow - owner * p.scatter.tokens_per_rank;
        orow = reinterpret_cast<uint16_t*>(p.scatter.peer_out[owner]) +
               (local * p.scatter.heads_total + p.scatter.head0 + bh) * D + g * HALF;
      } else {
        const int64_t drow = (p.scatter.row_perm && qrow < p.seq_q) ? (int64_t)p.scatter.row_perm[qrow] : qrow;
        orow = reinterpret_cast<uint16_t*>(p.out) + ((int64_t)bh * p.seq_q + drow) * D + g * HALF;
      }
      if (n_tiles == 0) {
        // no block selected at all: the reference divides 0 by 0
        if (qrow < p.seq_q) {
          const uint32_t nan2 = p.legacy ? 0u : pack2<FMT>(__int_as_float(0x7fc00000), __int_as_float(0x7fc00000));
          for (int c = 0; c < HALF; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(nan2, nan2, nan2, nan2);
          if (p.lse && g == 0) p.lse[(int64_t)bh * p.seq_q + qrow] = p.legacy ? -INFINITY : __int_as_float(0x7fc00000);
        }
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&ctl->row_done[rslot]);
        continue;
      }
      float m_run = -INFINITY, l_run = 0.f;
      const int first = ((g0 & 1) == g) ? 0 : 1;    // my first tile of this row
      bool have_ref = false;                        // fixed reference: m_run holds the row's reference exponent
      const int ne = q_rows;                        // rows with tiles before this one
      const int ref_slot = ne & 3;
        for (int j = first; j < n_tiles; j += 2) {
          const int gj = g0 + j, slot = gj % kBiasSlots, it = gj >> 1;
          // scores ready (and the tile's bias words visible)
          if (C::ONE_SIGNAL)
            ok = tc::mbar_wait(&ctl->k_empty[(gj % C::NK) * 2 + ((gj / C::NK) & 1)], ((gj / C::NK) >> 1) & 1, abort_flag);
          else if (C::NSB == 2) ok = tc::mbar_wait(&ctl->s_full[g], it & 1, abort_flag);
          else ok = tc::mbar_wait(&ctl->s_full[gj % 3], (gj / 3) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          // Two score buffers: the scores of running tile gj were issued after P V of tile gj-2 (same group), so that product
          // is complete and the accumulator may be rescaled below.  Three: see the wait before the rescale.
          tc::tc_fence_after();
          const uint32_t tS = C::NSB == 2 ? tS_mine : tmem + (uint32_t)(gj % 3) * 128 + lane_base;
          const bool ragged = j == n_tiles - 1 && last_cols < 128;   // columns the MMA did not write hold stale bits
          const float4* bias4 = reinterpret_cast<const float4*>(sBias + slot * 128);
          const float4* bg4 = reinterpret_cast<const float4*>(sBiasG + slot * 36);     // one bias word per 4 columns
          const int* flagw = reinterpret_cast<const int*>(sBiasG + slot * 36) + 32;
          const uchar4* minrow4 = reinterpret_cast<const uchar4*>(sMinRow + slot * 128);
          // Fast path: the bias is uniform inside every aligned group of 4 columns (blocks are at least 4 wide), so the
          // maximum is taken on raw scores per group and the bias enters once per group.  A tile with a block that ends
          // inside a group, or with unwritten columns, takes the per-column path.
          const bool slow = ragged || (flagw[0] | flagw[1] | flagw[2]) != 0;
          uint32_t va[32], vb[32];      // two chunks of 32 score columns in flight
          float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
          const bool ref_tile = !FIXED || j == 0;      // fixed reference: only a row's first tile takes the maximum pass
          if (!ref_tile) {
            if (!slow) tc::tmem_ld32(tS, va);          // chunk 0 for pass 2
          } else if (!slow) {
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
                float4 ba = bias4[h * 8 + q4];
                if (CAUSAL) {
                  const uchar4 mr = minrow4[h * 8 + q4];
                  if (r < mr.x) ba.x = -INFINITY;
                  if (r < mr.y) ba.y = -INFINITY;
                  if (r < mr.z) ba.z = -INFINITY;
                  if (r < mr.w) ba.w = -INFINITY;
                }
                mx0 = fmaxf(mx0, fmaf(__uint_as_float(va[4 * q4 + 0]), p.scale_log2, ba.x));
                mx1 = fmaxf(mx1, fmaf(__uint_as_float(va[4 * q4 + 1]), p.scale_log2, ba.y));
                mx2 = fmaxf(mx2, fmaf(__uint_as_float(va[4 * q4 + 2]), p.scale_log2, ba.z));
                mx3 = fmaxf(mx3, fmaf(__uint_as_float(va[4 * q4 + 3]), p.scale_log2, ba.w));
              }
            }
          }
          const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
          // raise the running maximum only when it is far off (or still unset)
          float alpha = 1.f;
          bool raise = false;
          if (FIXED) {
            if (j == 0) {
              // the group that owns the row's first tile sets the reference for both groups
              m_run = mx == -INFINITY ? 0.f : mx;
              sMref[ref_slot * 128 + r] = m_run;
              __syncwarp();
              if (lane == 0) tc::mbar_arrive(&ctl->mref_full[ref_slot]);
              have_ref = true;
            } else if (!have_ref) {
              ok = tc::mbar_wait(&ctl->mref_full[ref_slot], (ne >> 2) & 1, abort_flag);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) break;
              m_run = sMref[ref_slot * 128 + r];
              have_ref = true;
            }
          } else {
            raise = mx > m_run + 8.f;
            if (raise) {
              alpha = m_run == -INFINITY ? 0.f : ex2(m_run - mx);
              m_run = mx;
              l_run *= alpha;
            }
          }
          if (!FIXED && C::NSB == 3 && j >= 2) {
            // Every product of this group is signalled; each signal is waited for exactly once and in order (here for the
            // product of tile j-2, in the epilogue for the last one), so the waiter is never more than one phase behind.
            // By now - a whole maximum pass after the scores were found ready - it has normally long completed.
            ok = tc::mbar_wait(&ctl->pv_done[g], pv_rows & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            ++pv_rows;
            tc::tc_fence_after();
          }
          if (!FIXED && j >= 2 && __any_sync(0xffffffffu, raise)) {
            // the accumulator may only be touched between two of its P V products: the one of tile j-2 is complete (see
            // above), the one of tile j waits for the probabilities written below
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
                float4 ba = bias4[h * 8 + q4];
                if (CAUSAL) {
                  const uchar4 mr = minrow4[h * 8 + q4];
                  if (r < mr.x) ba.x = -INFINITY;
                  if (r < mr.y) ba.y = -INFINITY;
                  if (r < mr.z) ba.z = -INFINITY;
                  if (r < mr.w) ba.w = -INFINITY;
                }
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
          if (lane == 0) tc::mbar_arrive(&ctl->p_full[g * 2 + (it & 1)]);   // one arrival per warp
        }
      // ---- epilogue: merge the two groups' partial results
      const int my_tiles = n_tiles > first ? (n_tiles - first + 1) >> 1 : 0;
      if (FIXED) {
        if (ok && !have_ref) {      // a group without tiles in this row still passes the phase (and needs the reference for lse)
          ok = tc::mbar_wait(&ctl->mref_full[ref_slot], (ne >> 2) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (ok) m_run = sMref[ref_slot * 128 + r];
        }
        if (ok) {                   // the row's last product: the one accumulator is final
          ok = tc::mbar_wait(&ctl->pv_done[0], ne & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
        }
      } else if (ok && my_tiles > 0) {
        // signalled once per row in which this group has tiles: after the last of them
        ok = tc::mbar_wait(&ctl->pv_done[g], pv_rows & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        ++pv_rows;
      }
      // group g publishes (maximum, sum); after the barrier both groups' last products are complete.  An aborting group
      // still joins the barrier so that the other one is not left waiting.
      float* xch = sXch + (rit & 1) * 512;
      xch[g * 256 + r] = m_run;
      xch[g * 256 + 128 + r] = l_run;
      if (ok) ok = warps_rendezvous(&ctl->xch_full, q_rows, abort_flag); else ++q_rows;
      if (ok) {
        const float m_o = xch[(g ^ 1) * 256 + r], l_o = xch[(g ^ 1) * 256 + 128 + r];
        const float m_all = FIXED ? m_run : fmaxf(m_run, m_o);      // fixed reference: both groups used the same exponent
        const float w_me = FIXED ? 1.f : (m_run == -INFINITY ? 0.f : ex2(m_run - m_all));
        const float w_ot = FIXED ? 1.f : (m_o == -INFINITY ? 0.f : ex2(m_o - m_all));
        const float l_all = l_run * w_me + l_o * w_ot;
        // legacy kernel: no visible key -> 0, lse -inf (fixed reference: every row sees its first tile, so "no key" = sum 0)
        const bool dead = p.legacy && (FIXED ? l_all == 0.f : m_all == -INFINITY);
        const float inv = dead ? 0.f : 1.0f / l_all;              // otherwise an empty row is 0/0 like the reference
        const float w = w_me * inv, wo = w_ot * inv;
        if (FIXED && p.guard && !(l_all < 1.2e27f) && qrow < p.seq_q) *p.guard = 1;   // 2^90: near the end of the exponent range (or NaN)
        if (p.lse && g == 0 && qrow < p.seq_q)
          p.lse[(int64_t)bh * p.seq_q + qrow] = dead ? -INFINITY : (m_all + log2f(l_all)) * 0.6931471805599453f;
        const bool other_has = !FIXED && n_tiles - my_tiles > 0;
        const bool mine_has = FIXED || my_tiles > 0;
        tc::tc_fence_after();
        float f[HALF];
#pragma unroll
        for (int c0 = 0; c0 < HALF; c0 += 32) {
          uint32_t va[32], vb[32];
          if (mine_has) tc::tmem_ld32(tO + g * HALF + c0, va);
          if (other_has) tc::tmem_ld32(tO_other + g * HALF + c0, vb);
          tc::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            f[c0 + i] = (mine_has ? __uint_as_float(va[i]) * w : 0.f) + (other_has ? __uint_as_float(vb[i]) * wo : 0.f);
        }
        // the accumulators may be overwritten by the next row from here on
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&ctl->o_free);
        // A thread holds HALF channels of its own row; stored as they are, every store instruction of a warp would touch 32
        // different 128-byte lines.  The 16-byte pieces are transposed inside groups of 8 lanes first (three butterfly
        // stages), so that 8 lanes write one row's contiguous 128 bytes.
        constexpr int NCH = HALF / 8;                 // 16-byte pieces per thread: 8 (D = 128) or 4 (D = 64)
        uint4 ch[NCH];
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          ch[c].x = pack2<FMT>(f[8 * c + 0], f[8 * c + 1]);
          ch[c].y = pack2<FMT>(f[8 * c + 2], f[8 * c + 3]);
          ch[c].z = pack2<FMT>(f[8 * c + 4], f[8 * c + 5]);
          ch[c].w = pack2<FMT>(f[8 * c + 6], f[8 * c + 7]);
        }
#pragma unroll
        for (int sft = 1; sft < NCH; sft <<= 1) {
          const bool upper = (lane & sft) != 0;
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            if ((c & sft) == 0) {
              // the lower lane keeps piece c and receives the partner's piece c; the upper lane keeps piece c|sft
              const uint4 send = upper ? ch[c] : ch[c | sft];
              uint4 recv;
              recv.x = __shfl_xor_sync(0xffffffffu, send.x, sft);
              recv.y = __shfl_xor_sync(0xffffffffu, send.y, sft);
              recv.z = __shfl_xor_sync(0xffffffffu, send.z, sft);
              recv.w = __shfl_xor_sync(0xffffffffu, send.w, sft);
              if (upper) ch[c] = recv; else ch[c | sft] = recv;
            }
          }
        }
        // now piece k of lane (base + i) is piece i of row (base + k), base = the first lane of the group of NCH lanes
        {
          const int sub = lane & (NCH - 1), base = lane & ~(NCH - 1);
          const unsigned long long my_ptr = reinterpret_cast<unsigned long long>(orow);
#pragma unroll
          for (int k = 0; k < NCH; ++k) {
            const unsigned long long dst = __shfl_sync(0xffffffffu, my_ptr, base + k);
            const int64_t row_k = (int64_t)m * 128 + quarter * 32 + base + k;
            if (row_k < p.seq_q) *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(dst) + sub * 8) = ch[k];
          }
        }
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&ctl->row_done[rslot]);
      }
      g0 += n_tiles;
    }
  }

  // ---------------------------------------------------------------- teardown
  tc::tc_fence_before();
  __syncthreads();
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

// Row counters of the persistent forward: a ring of device words; every launch takes the next one and zeroes it on its
// own stream right before the kernel, so launches in flight on different streams do not share a counter (unless more than
// kCounterRing launches of one device overlap in time).
constexpr int kCounterRing = 256;
__device__ int g_row_counters[kCounterRing];

static int next_row_counter(int** out, cudaStream_t st) {
  constexpr int kMaxDevices = 64;
  static int* base[kMaxDevices] = {nullptr};
  static unsigned next[kMaxDevices] = {0};
  static std::mutex mu;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  PSA_REQUIRE(e == cudaSuccess && dev >= 0 && dev < kMaxDevices, PSA_ERR_CUDA, "psa_fwd: cudaGetDevice failed: %s", cudaGetErrorString(e));
  std::lock_guard<std::mutex> lock(mu);
  if (!base[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_row_counters);
    PSA_REQUIRE(e == cudaSuccess && ptr, PSA_ERR_CUDA, "psa_fwd: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    base[dev] = (int*)ptr;
  }
  int* c = base[dev] + (next[dev]++ % kCounterRing);
  e = cudaMemsetAsync(c, 0, sizeof(int), st);
  PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_fwd: cudaMemsetAsync failed: %s", cudaGetErrorString(e));
  *out = c;
  return PSA_OK;
}

template <int D, int FMT, bool IMG, bool CAUSAL = false, bool FIXED = false>
static int launch_tc(const FwdArgs& a, cudaStream_t st, int* guard = nullptr, const int* only_if = nullptr) {
  using C = Cfg<D, FIXED>;
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
  p.total_rows = (int)((int64_t)p.mq * a.bh);
  p.kimg = (const unsigned char*)a.kimg; p.vimg = (const unsigned char*)a.vimg;
  p.img = make_img_levels(a.bh, a.seq_k, D, IMG ? a.bn : 64);
  p.scatter = a.scatter;
  p.lse = a.lse; p.legacy = a.legacy; p.causal = a.causal;
  p.guard = guard; p.only_if = only_if;
  cudaError_t e = cudaFuncSetAttribute(psa_fwd_tc_kernel<D, FMT, IMG, CAUSAL, FIXED>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_fwd: shared-memory opt-in (%d B) failed: %s", C::SMEM_BYTES,
              cudaGetErrorString(e));
  // persistent: one CTA per SM (221 KB of shared memory and all 512 TMEM columns each), rows dealt round-robin so that
  // the CTAs running at the same time work on neighbouring rows of the same head (K/V stay in L2)
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  PSA_REQUIRE(sms > 0, PSA_ERR_CUDA, "psa_fwd: cannot read the SM count");
  const unsigned grid = (unsigned)(p.total_rows < sms ? p.total_rows : sms);
  rc = next_row_counter(&p.row_counter, st);
  if (rc != PSA_OK) return rc;
  psa_fwd_tc_kernel<D, FMT, IMG, CAUSAL, FIXED><<<grid, kThreads, C::SMEM_BYTES, st>>>(maps, p);
  PSA_CHECK_LAUNCH("psa_fwd(tcgen05)");
  return PSA_OK;
}

// bf16 without the causal rule: the fixed-reference kernel, then the exact one, which returns at once unless the first one
// raised its guard word (a row whose probabilities came near the end of the exponent range) - no host round trip.
template <int D, bool IMG>
static int launch_fixed_then_exact(const FwdArgs& a, cudaStream_t st) {
  int* guard = nullptr;
  int rc = next_row_counter(&guard, st);      // a zeroed device word of this launch
  if (rc != PSA_OK) return rc;
  rc = launch_tc<D, 1, IMG, false, true>(a, st, guard, nullptr);
  if (rc != PSA_OK) return rc;
  return launch_tc<D, 1, IMG, false, false>(a, st, nullptr, guard);
}

int fwd_tc_launch(const FwdArgs& a, cudaStream_t st) {
  const int fmt = a.dtype == PSA_BF16 ? 1 : 0;
  const bool img = a.kimg != nullptr && a.vimg != nullptr;
  if (img) {
    PSA_REQUIRE(a.bn >= 64, PSA_ERR_UNSUPPORTED, "tile images need block_n >= 64 (blocks of at least 8 pooled rows)");
    PSA_REQUIRE((((uintptr_t)a.kimg | (uintptr_t)a.vimg) & 15) == 0, PSA_ERR_ARG, "tile images must be 16-byte aligned");
    if (a.causal) {   // only the legacy forward asks for it; a variant of its own keeps the common kernel lean
      if (a.D == 64) return fmt ? launch_tc<64, 1, true, true>(a, st) : launch_tc<64, 0, true, true>(a, st);
      return fmt ? launch_tc<128, 1, true, true>(a, st) : launch_tc<128, 0, true, true>(a, st);
    }
    if (a.D == 64) return fmt ? launch_fixed_then_exact<64, true>(a, st) : launch_tc<64, 0, true>(a, st);
    return fmt ? launch_fixed_then_exact<128, true>(a, st) : launch_tc<128, 0, true>(a, st);
  }
  PSA_REQUIRE(!a.causal, PSA_ERR_UNSUPPORTED, "the causal rule needs the tile-image path");
  if (a.D == 64) return fmt ? launch_fixed_then_exact<64, false>(a, st) : launch_tc<64, 0, false>(a, st);
  return fmt ? launch_fixed_then_exact<128, false>(a, st) : launch_tc<128, 0, false>(a, st);
}

}  // namespace psa
