// Multi-level block-sparse flash-attention forward on tcgen05 tensor cores (f16/bf16, block_m = 128).
//
// One CTA per (128-row query block, batch*head), 10 warps:
//   warp 0      producer: walks the block's index list and gathers the selected K/V blocks of every pyramid level
//               with TMA (128-byte swizzle, one {64 ch, P tokens} box per block and 64-channel slab, no multicast;
//               lanes 0..3 each issue one of the four copies of a block) into 128-token tiles, PACKING blocks of
//               different levels into the same tile; it also writes the per-column logit bias (log2 of the level,
//               -inf for columns that do not exist).
//   warp 1      MMA issuer: S = Q K^T (operands in shared memory) into one of two TMEM score buffers, then
//               O += P V with P read from TMEM and V read MN-major from the same swizzled tile; software-pipelined
//               so that the next tile's S is in flight while the softmax warps work on the current one.
//   warps 2-9   softmax: two threads per query row, 64 columns each.  One TMEM read of the row half into registers
//               (the score buffer is released at once), row maximum exchanged through shared memory, exp2, running
//               sum in fp32, probabilities rounded to the element type and stored to one of two TMEM P buffers.
//               The running maximum is only raised when the new maximum exceeds it by more than 2^8 ("lazy"
//               rescale); raising it rescales the O accumulator in TMEM.  Epilogue: O / sum -> global.
// TMEM (512 columns): S0 [0,128), S1 [128,256), O [256,256+D), P0 [384,448), P1 [448,512).
//
// Every mbarrier wait is bounded; on expiry the CTA records PSA_ERR_TIMEOUT in the status word, lets copies in
// flight land, frees its TMEM and returns.
#include "psa_common.cuh"
#include "fwd.h"
#include "tc_common.cuh"

namespace psa {

namespace {

constexpr int kMaxWidth = 4096;        // longest index list (entries) the kernel stages in shared memory
constexpr int kSlabBytes = 128 * 128;  // 128 rows x 128 B (64 16-bit channels)
constexpr int kThreads = 320;
constexpr int kSoftmaxThreads = 256;

struct TmapPack {
  CUtensorMap q;
  CUtensorMap k[4];
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
};

template <int D> struct Cfg {
  static constexpr int SLABS = D / 64;
  static constexpr int NST = D == 64 ? 4 : 2;
  static constexpr int Q_BYTES = SLABS * kSlabBytes;
  static constexpr int KV_BYTES = 2 * SLABS * kSlabBytes;   // K then V of one stage
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = OFF_Q + Q_BYTES;
  static constexpr int OFF_BIAS = OFF_KV + NST * KV_BYTES;
  static constexpr int OFF_XCH = OFF_BIAS + NST * 128 * 4;
  static constexpr int OFF_ROW = OFF_XCH + 2 * 2 * 128 * 4;
  static constexpr int OFF_CTRL = OFF_ROW + kMaxWidth * 4;
  static constexpr int SMEM_BYTES = OFF_CTRL + 512 + 1024;   // + alignment slack
};

struct Ctrl {
  uint64_t full[4], empty[4], s_full[2], s_empty[2], p_full[2], pv_done[2], q_full;
  uint32_t tmem_base;
  int abort_flag;
  int n_sep;
  int sep[16];
  int n_tiles, last_cols;
  int seg_start[4], seg_cnt[4];
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

template <int D, int FMT>
__global__ void __launch_bounds__(kThreads, 1) psa_fwd_tc_kernel(const __grid_constant__ TmapPack maps, const TcParams p) {
  using C = Cfg<D>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  unsigned char* sQ = smem + C::OFF_Q;
  unsigned char* sKV = smem + C::OFF_KV;
  float* sBias = reinterpret_cast<float*>(smem + C::OFF_BIAS);
  float* sXch = reinterpret_cast<float*>(smem + C::OFF_XCH);      // [tile parity][half][row]
  int32_t* sRow = reinterpret_cast<int32_t*>(smem + C::OFF_ROW);
  Ctrl* ctl = reinterpret_cast<Ctrl*>(smem + C::OFF_CTRL);
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x;
  const int bh = blockIdx.y;
  const int32_t* mrow = p.mask + ((int64_t)bh * p.mq + m) * p.width;

  // ---------------------------------------------------------------- setup
  if (threadIdx.x == 0) {
    for (int i = 0; i < C::NST; ++i) { tc::mbar_init(&ctl->full[i], 1); tc::mbar_init(&ctl->empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&ctl->s_full[i], 1);
      tc::mbar_init(&ctl->s_empty[i], kSoftmaxThreads);
      tc::mbar_init(&ctl->p_full[i], kSoftmaxThreads);
      tc::mbar_init(&ctl->pv_done[i], 1);
    }
    tc::mbar_init(&ctl->q_full, 1);
    ctl->abort_flag = 0;
    ctl->n_sep = 0;
    tc::fence_mbar_init();
  }
  for (int i = threadIdx.x; i < p.width; i += kThreads) sRow[i] = mrow[i];
  __syncthreads();
  if (warp == 1) {
    tc::tmem_alloc(&ctl->tmem_base, 512);
    tc::tmem_relinquish();
  }
  // separators of the index list (their order is recovered by a tiny sort)
  for (int i = threadIdx.x; i < p.width; i += kThreads)
    if (sRow[i] == -1) {
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
    int prev = -1, tokens = 0;
    for (int li = 0; li < 4; ++li) {
      int end = li < ns ? ctl->sep[li] : p.width;
      int start = prev + 1;
      int cnt = end > start ? end - start : 0;      // a row that ended early leaves later segments empty
      ctl->seg_start[li] = start;
      ctl->seg_cnt[li] = cnt;
      const int P = p.bn >> li;
      int items = cnt;
      if (p.quirk && P < p.tn && cnt >= 2) items += p.tn / P - 2;
      tokens += items * P;
      prev = end;
    }
    const int padded = (tokens + 15) & ~15;
    ctl->n_tiles = (padded + 127) / 128;
    ctl->last_cols = padded - (ctl->n_tiles - 1) * 128;
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const int n_tiles = ctl->n_tiles;
  const int last_cols = ctl->last_cols;
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t tO = tmem + 256;

  if (n_tiles > 0) {
    if (warp == 0) {
      // ============================================================ producer
      if (lane == 0) {
        tc::tma_prefetch_desc(&maps.q);
        for (int s = 0; s < C::SLABS; ++s) tc::tma_load_3d(sQ + s * kSlabBytes, &maps.q, &ctl->q_full, s * 64, m * 128, bh);
        tc::mbar_arrive_expect_tx(&ctl->q_full, C::Q_BYTES);
      }
      int tile = 0, fill = 0;
      uint32_t bytes = 0;
      bool ok = true;
      int last_li = 0;
      const int op_is_v = lane / C::SLABS, op_slab = lane % C::SLABS;   // lanes 0 .. 2*SLABS-1 each own one copy
      auto emit = [&](int li, int blk, float bias2) {
        if (!ok) return;
        const int stage = tile % C::NST;
        if (fill == 0) {
          ok = tc::mbar_wait(&ctl->empty[stage], ((tile / C::NST) & 1) ^ 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) return;
        }
        const int P = p.bn >> li;
        if (lane < 2 * C::SLABS) {
          unsigned char* dst = sKV + stage * C::KV_BYTES + (op_is_v * C::SLABS + op_slab) * kSlabBytes + fill * 128;
          tc::tma_load_3d(dst, op_is_v ? &maps.v[li] : &maps.k[li], &ctl->full[stage], op_slab * 64, blk * P, bh);
        }
        bytes += 2u * C::SLABS * P * 128u;
        const int64_t t0 = (int64_t)blk * P;
        for (int c = lane; c < P; c += 32) sBias[stage * 128 + fill + c] = (t0 + c < p.n[li]) ? bias2 : -INFINITY;
        fill += P;
        last_li = li;
        if (fill == 128) {
          __syncwarp();
          if (lane == 0) tc::mbar_arrive_expect_tx(&ctl->full[stage], bytes);
          ++tile; fill = 0; bytes = 0;
        }
      };
      for (int li = 0; li < 4; ++li) {
        const int P = p.bn >> li;
        const int cnt = ctl->seg_cnt[li], start = ctl->seg_start[li];
        const float bias2 = (float)li;   // log2(level)
        for (int e = 0; e < cnt; ++e) emit(li, sRow[start + e], bias2);
        if (p.quirk && P < p.tn && cnt >= 2) {
          const float qb = bias2 + log2f((float)(cnt / 2));
          for (int j = 2; j < p.tn / P; ++j) emit(li, j, qb);
        }
      }
      if (ok && fill > 0) {
        while (ok && (fill & 15)) emit(last_li, 0, -INFINITY);   // inert columns up to a multiple of 16
        if (ok && fill > 0) {
          const int stage = tile % C::NST;
          for (int c = fill + lane; c < 128; c += 32) sBias[stage * 128 + c] = -INFINITY;
          __syncwarp();
          if (lane == 0) tc::mbar_arrive_expect_tx(&ctl->full[stage], bytes);
        }
      }
    } else if (warp == 1) {
      // ============================================================ MMA issuer
      if (lane == 0) {
        bool ok = tc::mbar_wait(&ctl->q_full, 0, abort_flag);
        const uint32_t idesc_pv = tc::make_idesc(FMT, 128, D, 0, 1);
        const uint32_t q_addr = tc::smem_u32(sQ);
        for (int j = 0; ok && j <= n_tiles; ++j) {
          if (j < n_tiles) {
            const int stage = j % C::NST, b = j & 1;
            const int ncols = j == n_tiles - 1 ? last_cols : 128;
            ok = tc::mbar_wait(&ctl->full[stage], (j / C::NST) & 1, abort_flag);
            if (!ok) break;
            ok = tc::mbar_wait(&ctl->s_empty[b], ((j >> 1) & 1) ^ 1, abort_flag);
            if (!ok) break;
            tc::tc_fence_after();
            const uint32_t k_addr = tc::smem_u32(sKV + stage * C::KV_BYTES);
            const uint32_t idesc_qk = tc::make_idesc(FMT, 128, ncols, 0, 0);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              const uint32_t off = (ks >> 2) * kSlabBytes + (ks & 3) * 32;
              tc::umma_ss(tmem + b * 128, tc::make_smem_desc(q_addr + off, 16, 1024),
                          tc::make_smem_desc(k_addr + off, 16, 1024), idesc_qk, ks > 0);
            }
            tc::umma_commit(&ctl->s_full[b]);
          }
          if (j > 0) {
            const int t = j - 1;
            const int stage = t % C::NST, b = t & 1;
            const int ncols = t == n_tiles - 1 ? last_cols : 128;
            ok = tc::mbar_wait(&ctl->p_full[b], (t >> 1) & 1, abort_flag);
            if (!ok) break;
            tc::tc_fence_after();
            const uint32_t v_addr = tc::smem_u32(sKV + stage * C::KV_BYTES + C::SLABS * kSlabBytes);
            const uint32_t tP = tmem + 384 + b * 64;
            for (int ks = 0; ks < ncols / 16; ++ks)
              tc::umma_ts(tO, tP + ks * 8, tc::make_smem_desc(v_addr + ks * 2048, kSlabBytes, 1024), idesc_pv,
                          (t > 0 || ks > 0) ? 1u : 0u);
            tc::umma_commit(&ctl->empty[stage]);   // K/V stage may be refilled
            tc::umma_commit(&ctl->pv_done[b]);     // O is consistent again, P buffer b may be rewritten
          }
        }
      }
    } else {
      // ============================================================ softmax / epilogue (8 warps, 2 threads per row)
      const int quarter = warp & 3;                 // TMEM lanes this warp may touch
      const int half = (warp - 2) >> 2;             // which 64 score columns / which half of the O channels
      const int r = quarter * 32 + lane;            // row inside the query block
      const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
      float m_run = -INFINITY, l_run = 0.f;
      bool ok = true;
      for (int j = 0; j < n_tiles; ++j) {
        const int stage = j % C::NST, b = j & 1;
        ok = tc::mbar_wait(&ctl->full[stage], (j / C::NST) & 1, abort_flag);   // bias[] of this tile is visible
        ok = ok && tc::mbar_wait(&ctl->s_full[b], (j >> 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc::tc_fence_after();
        uint32_t v0[32], v1[32];
        tc::tmem_ld32(tmem + b * 128 + lane_base + half * 64, v0);
        tc::tmem_ld32(tmem + b * 128 + lane_base + half * 64 + 32, v1);
        tc::tmem_wait_ld();
        tc::tc_fence_before();
        tc::mbar_arrive(&ctl->s_empty[b]);          // the score buffer is free for tile j+2
        if (j == n_tiles - 1 && last_cols < 128) {  // columns the MMA did not write hold stale bits
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (half * 64 + i >= last_cols) v0[i] = 0u;
            if (half * 64 + 32 + i >= last_cols) v1[i] = 0u;
          }
        }
        // biased, scaled logits (log2 domain) in place, and their maximum
        const float4* bias4 = reinterpret_cast<const float4*>(sBias + stage * 128 + half * 64);
        float mx = -INFINITY;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 ba = bias4[g], bb = bias4[8 + g];
          float x;
          x = fmaf(__uint_as_float(v0[4 * g + 0]), p.scale_log2, ba.x); v0[4 * g + 0] = __float_as_uint(x); mx = fmaxf(mx, x);
          x = fmaf(__uint_as_float(v0[4 * g + 1]), p.scale_log2, ba.y); v0[4 * g + 1] = __float_as_uint(x); mx = fmaxf(mx, x);
          x = fmaf(__uint_as_float(v0[4 * g + 2]), p.scale_log2, ba.z); v0[4 * g + 2] = __float_as_uint(x); mx = fmaxf(mx, x);
          x = fmaf(__uint_as_float(v0[4 * g + 3]), p.scale_log2, ba.w); v0[4 * g + 3] = __float_as_uint(x); mx = fmaxf(mx, x);
          x = fmaf(__uint_as_float(v1[4 * g + 0]), p.scale_log2, bb.x); v1[4 * g + 0] = __float_as_uint(x); mx = fmaxf(mx, x);
          x = fmaf(__uint_as_float(v1[4 * g + 1]), p.scale_log2, bb.y); v1[4 * g + 1] = __float_as_uint(x); mx = fmaxf(mx, x);
          x = fmaf(__uint_as_float(v1[4 * g + 2]), p.scale_log2, bb.z); v1[4 * g + 2] = __float_as_uint(x); mx = fmaxf(mx, x);
          x = fmaf(__uint_as_float(v1[4 * g + 3]), p.scale_log2, bb.w); v1[4 * g + 3] = __float_as_uint(x); mx = fmaxf(mx, x);
        }
        // the two threads of a row exchange their partial maxima
        float* xch = sXch + (j & 1) * 256;
        xch[half * 128 + r] = mx;
        tc::named_bar_sync(1 + quarter, 64);
        mx = fmaxf(mx, xch[(half ^ 1) * 128 + r]);
        // raise the running maximum only when it is far off (or still unset); both threads of a row agree
        float alpha = 1.f;
        const bool raise = mx > m_run + 8.f;
        if (raise) {
          alpha = m_run == -INFINITY ? 0.f : ex2(m_run - mx);
          m_run = mx;
          l_run *= alpha;
        }
        // P buffer b was last read by the P V of tile j-2
        ok = tc::mbar_wait(&ctl->pv_done[b], ((j >> 1) & 1) ^ 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (j > 0 && __any_sync(0xffffffffu, raise)) {
          // O may only be touched between two P V products: wait for the one of tile j-1
          ok = tc::mbar_wait(&ctl->pv_done[b ^ 1], ((j - 1) >> 1) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc::tc_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < D / 2; c0 += 32) {
            uint32_t o[32];
            tc::tmem_ld32(tO + lane_base + half * (D / 2) + c0, o);
            tc::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tc::tmem_st32(tO + lane_base + half * (D / 2) + c0, o);
          }
          tc::tmem_wait_st();
        }
        // probabilities (rounded to the element type) -> TMEM, running sum
        const float m_use = m_run == -INFINITY ? 0.f : m_run;
        float lsum = 0.f;
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ex2(__uint_as_float(v0[i]) - m_use), p1 = ex2(__uint_as_float(v0[i + 1]) - m_use);
          const float p2 = ex2(__uint_as_float(v1[i]) - m_use), p3 = ex2(__uint_as_float(v1[i + 1]) - m_use);
          lsum += (p0 + p1) + (p2 + p3);
          pk[i >> 1] = pack2<FMT>(p0, p1);
          pk[16 + (i >> 1)] = pack2<FMT>(p2, p3);
        }
        l_run += lsum;
        tc::tmem_st32(tmem + 384 + b * 64 + lane_base + half * 32, pk);
        tc::tmem_wait_st();
        tc::tc_fence_before();
        tc::mbar_arrive(&ctl->p_full[b]);
      }
      // epilogue
      if (ok) {
        const int t = n_tiles - 1;
        ok = tc::mbar_wait(&ctl->pv_done[t & 1], (t >> 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc::tc_fence_after();
        float* xch = sXch + (n_tiles & 1) * 256;
        xch[half * 128 + r] = l_run;
        tc::named_bar_sync(1 + quarter, 64);
        const float l_tot = l_run + xch[(half ^ 1) * 128 + r];
        const int64_t qrow = (int64_t)m * 128 + r;
        const float inv = 1.0f / l_tot;     // empty row: 0/0 like the reference
        uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + ((int64_t)bh * p.seq_q + qrow) * D + half * (D / 2);
#pragma unroll 1
        for (int c0 = 0; c0 < D / 2; c0 += 32) {
          uint32_t v[32];
          tc::tmem_ld32(tO + lane_base + half * (D / 2) + c0, v);
          tc::tmem_wait_ld();
          if (qrow < p.seq_q) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 o;
              o.x = pack2<FMT>(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
              o.y = pack2<FMT>(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
              o.z = pack2<FMT>(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
              o.w = pack2<FMT>(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c0 + i) = o;
            }
          }
        }
      }
    }
  } else if (warp >= 2) {
    // no block selected at all: the reference divides 0 by 0
    const int half = (warp - 2) >> 2;
    const int64_t qrow = (int64_t)m * 128 + (warp & 3) * 32 + lane;
    if (qrow < p.seq_q) {
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + ((int64_t)bh * p.seq_q + qrow) * D + half * (D / 2);
      const uint32_t nan2 = pack2<FMT>(__int_as_float(0x7fc00000), __int_as_float(0x7fc00000));
      for (int c = 0; c < D / 2; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(nan2, nan2, nan2, nan2);
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
  if (warp == 1) {
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
  const void* ptrs[] = {a.q, a.out, a.k[0], a.k[1], a.k[2], a.k[3], a.v[0], a.v[1], a.v[2], a.v[3]};
  for (const void* ptr : ptrs)
    if ((uintptr_t)ptr & 15) return false;
  return true;
}

template <int D, int FMT>
static int launch_tc(const FwdArgs& a, cudaStream_t st) {
  using C = Cfg<D>;
  TmapPack maps;
  const int is_bf16 = FMT == 1;
  int rc = encode_tmap_3d(&maps.q, a.q, 2, is_bf16, D, a.seq_q, a.bh, 128);
  if (rc != PSA_OK) return rc;
  for (int li = 0; li < 4; ++li) {
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
  cudaError_t e = cudaFuncSetAttribute(psa_fwd_tc_kernel<D, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_fwd: shared-memory opt-in (%d B) failed: %s", C::SMEM_BYTES,
              cudaGetErrorString(e));
  dim3 grid(p.mq, (unsigned)a.bh);
  psa_fwd_tc_kernel<D, FMT><<<grid, kThreads, C::SMEM_BYTES, st>>>(maps, p);
  PSA_CHECK_LAUNCH("psa_fwd(tcgen05)");
  return PSA_OK;
}

int fwd_tc_launch(const FwdArgs& a, cudaStream_t st) {
  const int fmt = a.dtype == PSA_BF16 ? 1 : 0;
  if (a.D == 64) return fmt ? launch_tc<64, 1>(a, st) : launch_tc<64, 0>(a, st);
  return fmt ? launch_tc<128, 1>(a, st) : launch_tc<128, 0>(a, st);
}

}  // namespace psa
