// Antidiagonal block-importance estimate of the causal call site on tcgen05 tensor cores (f16/bf16, lengths that are a
// multiple of the stride).  Replaces flat_group_gemm_fuse_reshape and softmax_fuse_block_sum
// (qwen2.5-vl-example/src/attention/PSA_casual/kernels/block_importance_kernels.py:255-323, 6-192); the fp32 logits
// never reach HBM.
//
// logit(i, j) = sum_s q[i*stride + stride-1-s] . k[j*stride + s]: one GEMM of the two [n, stride*D] group matrices.
// Neither matrix is materialised: q and k are described to TMA as 4-D tensors {channel, token in group, group,
// batch*head}, so a K-chunk (64 channels of token s of every group) of 128 consecutive groups is ONE box
// {64, 1, 128, 1}, landing in shared memory as a 128-byte-swizzled [128 rows][128 B] operand tile; the query side
// simply asks for token stride-1-s.  Groups past the end are zero-filled by TMA.
//
// Persistent CTAs (one per SM) walk the 128x128 logit tiles (tiles above the diagonal are skipped when causal):
//   warp 0   producer: per K-chunk two boxes (A, B) into a 4-stage ring (32 KB per stage)
//   warp 1   MMA issuer: stride*D/16 tcgen05.mma (M = N = 128, K = 16) per tile into one of two TMEM accumulators
//   warps 2-5 epilogue (thread = group row): the 128 logits of the row go to registers (the accumulator is released at
//            once, so the issuer already works on the next tile), then the row's maximum over the tile's visible columns
//            and, per key block (block/stride columns), the sum of exp2(logit - maximum): a partial softmax.
// antidiag_combine_kernel then merges the partial results of a row (its maximum over all tiles, the normaliser, the
// rescaled block sums) and adds the rows of a query block: the softmax mass per (query block, key block).
// Per row the first kernel writes n/128 maxima and n/(block/stride) sums instead of n logits.
// Tensor-bound: 2*BH*n^2*stride*D flops (half when causal).  Every mbarrier wait is bounded; on expiry the CTA sets the
// abort flag, lets copies in flight land, frees its TMEM and returns PSA_ERR_TIMEOUT through the status word.
#include <cmath>

#include "psa_common.cuh"
#include "tc_common.cuh"

namespace psa {

namespace {

constexpr int kStages = 4;
constexpr int kOperandBytes = 128 * 128;           // 128 groups x 64 channels x 2 bytes
constexpr int kStageBytes = 2 * kOperandBytes;     // A and B
constexpr int kThreads = 192;

struct Ctrl {
  uint64_t full[kStages], empty[kStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct Params {
  float* tile_max;     // [bh][n][n / 128]: maximum of the row's visible logits inside a column tile
  float* block_sum;    // [bh][n][col_tiles * 128 / rb]: sum of exp2(logit - that maximum) over a key block's columns
  int n;               // groups of the padded length
  int n_valid;         // groups that hold a valid query token
  int rb;              // groups per block (power of two, 2..32)
  int row_tiles;       // tiles that hold a valid query group
  int col_tiles;       // non-causal: tiles per row
  int stride;
  int causal;
  int64_t bh;
  float scale_log2;
  int32_t* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
          tc::smem_u32(smem_dst)),
      "l"(map), "r"(tc::smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// tile number t of one head -> (row tile, column tile); causal heads enumerate the lower triangle row by row
__device__ __forceinline__ void tile_of(int t, const Params& p, int& it, int& jt) {
  if (!p.causal) {
    it = t / p.col_tiles;
    jt = t - it * p.col_tiles;
    return;
  }
  int r = (int)((sqrtf(8.0f * (float)t + 1.0f) - 1.0f) * 0.5f);
  while ((r + 1) * (r + 2) / 2 <= t) ++r;
  while (r * (r + 1) / 2 > t) --r;
  it = r;
  jt = t - r * (r + 1) / 2;
}

template <int D, int FMT>
__global__ void __launch_bounds__(kThreads, 1) antidiag_logits_tc_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                                        const __grid_constant__ CUtensorMap tm_k, const Params p) {
  constexpr int SLABS = D / 64;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  Ctrl* ctl = reinterpret_cast<Ctrl*>(smem + kStages * kStageBytes);
  volatile int* abort_flag = &ctl->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) { tc::mbar_init(&ctl->full[i], 1); tc::mbar_init(&ctl->empty[i], 1); }
    for (int i = 0; i < 2; ++i) { tc::mbar_init(&ctl->acc_full[i], 1); tc::mbar_init(&ctl->acc_empty[i], 128); }
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

  const int tiles_per_head = p.causal ? p.row_tiles * (p.row_tiles + 1) / 2 : p.row_tiles * p.col_tiles;
  const int64_t total = p.bh * tiles_per_head;
  const int chunks = p.stride * SLABS;            // K-chunks of 64 channels per tile

  if (warp == 0) {
    if (lane == 0) {
      int64_t c = 0;                              // running chunk count (ring position)
      bool ok = true;
      for (int64_t w = blockIdx.x; ok && w < total; w += gridDim.x) {
        const int bh = (int)(w / tiles_per_head);
        int it, jt;
        tile_of((int)(w - (int64_t)bh * tiles_per_head), p, it, jt);
        for (int kc = 0; kc < chunks; ++kc, ++c) {
          const int stage = (int)(c % kStages);
          ok = tc::mbar_wait(&ctl->empty[stage], (uint32_t)(((c / kStages) & 1) ^ 1), abort_flag);
          if (!ok) break;
          const int s = kc / SLABS, d0 = (kc - s * SLABS) * 64;
          unsigned char* dst = smem + stage * kStageBytes;
          tma_load_4d(dst, &tm_q, &ctl->full[stage], d0, p.stride - 1 - s, it * 128, bh);
          tma_load_4d(dst + kOperandBytes, &tm_k, &ctl->full[stage], d0, s, jt * 128, bh);
          tc::mbar_arrive_expect_tx(&ctl->full[stage], kStageBytes);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = tc::make_idesc(FMT, 128, 128, 0, 0);
      int64_t c = 0;
      int tile = 0;
      bool ok = true;
      for (int64_t w = blockIdx.x; ok && w < total; w += gridDim.x, ++tile) {
        const int b = tile & 1;
        ok = tc::mbar_wait(&ctl->acc_empty[b], (uint32_t)(((tile >> 1) & 1) ^ 1), abort_flag);
        if (!ok) break;
        tc::tc_fence_after();
        for (int kc = 0; kc < chunks; ++kc, ++c) {
          const int stage = (int)(c % kStages);
          ok = tc::mbar_wait(&ctl->full[stage], (uint32_t)((c / kStages) & 1), abort_flag);
          if (!ok) break;
          tc::tc_fence_after();
          const uint32_t a_addr = tc::smem_u32(smem + stage * kStageBytes), b_addr = a_addr + kOperandBytes;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            tc::umma_ss(tmem + b * 128, tc::make_smem_desc(a_addr + ks * 32, 16, 1024), tc::make_smem_desc(b_addr + ks * 32, 16, 1024),
                        idesc, (kc > 0 || ks > 0) ? 1u : 0u);
          tc::umma_commit(&ctl->empty[stage]);
        }
        if (ok) tc::umma_commit(&ctl->acc_full[b]);
      }
    }
  } else {
    const int quarter = warp & 3;                  // TMEM lanes this warp may touch
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    int tile = 0;
    bool ok = true;
    for (int64_t w = blockIdx.x; ok && w < total; w += gridDim.x, ++tile) {
      const int bh = (int)(w / tiles_per_head);
      int it, jt;
      tile_of((int)(w - (int64_t)bh * tiles_per_head), p, it, jt);
      const int b = tile & 1;
      ok = tc::mbar_wait(&ctl->acc_full[b], (uint32_t)((tile >> 1) & 1), abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc::tc_fence_after();
      const int row = it * 128 + r;
      uint32_t v[4][32];
      tc::tmem_ld32(tmem + b * 128 + lane_base, v[0]);
      tc::tmem_ld32(tmem + b * 128 + lane_base + 32, v[1]);
      tc::tmem_ld32(tmem + b * 128 + lane_base + 64, v[2]);
      tc::tmem_ld32(tmem + b * 128 + lane_base + 96, v[3]);
      tc::tmem_wait_ld();
      tc::tc_fence_before();
      tc::mbar_arrive(&ctl->acc_empty[b]);          // the accumulator may be overwritten: the row lives in registers now
      if (row >= p.n_valid) continue;               // group rows without a valid query token contribute nothing
      // visible columns: all of the tile, or (causal, diagonal tile) those up to the row's own group
      int last = (p.causal && jt == it) ? r : 127;
      if (jt * 128 + last >= p.n) last = p.n - 1 - jt * 128;      // columns past the padded length do not exist
      float m = -INFINITY;
#pragma unroll
      for (int c = 0; c < 128; ++c)
        if (c <= last) m = fmaxf(m, __uint_as_float(v[c >> 5][c & 31]));
      m *= p.scale_log2;                            // the scale is positive
      const int nbt = 128 / p.rb;                   // key blocks per tile: 4 .. 64
      const int64_t rowi = (int64_t)bh * p.n + row;
      p.tile_max[rowi * p.col_tiles + jt] = m;
      float* sums = p.block_sum + rowi * ((int64_t)p.col_tiles * nbt) + (int64_t)jt * nbt;
      // sums of groups of 2 columns first, then merged up to the block width (a power of two)
      float part[64];
#pragma unroll
      for (int c = 0; c < 128; c += 2) {
        const float e0 = c <= last ? ex2(fmaf(__uint_as_float(v[c >> 5][c & 31]), p.scale_log2, -m)) : 0.f;
        const float e1 = c + 1 <= last ? ex2(fmaf(__uint_as_float(v[(c + 1) >> 5][(c + 1) & 31]), p.scale_log2, -m)) : 0.f;
        part[c >> 1] = e0 + e1;
      }
      if (p.rb == 2) {
#pragma unroll
        for (int i = 0; i < 64; i += 4) *reinterpret_cast<float4*>(sums + i) = make_float4(part[i], part[i + 1], part[i + 2], part[i + 3]);
      } else if (p.rb == 4) {
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          *reinterpret_cast<float4*>(sums + i) = make_float4(part[2 * i] + part[2 * i + 1], part[2 * i + 2] + part[2 * i + 3],
                                                              part[2 * i + 4] + part[2 * i + 5], part[2 * i + 6] + part[2 * i + 7]);
      } else {
        float q4[16];                               // sums of 8 columns
#pragma unroll
        for (int i = 0; i < 16; ++i) q4[i] = (part[4 * i] + part[4 * i + 1]) + (part[4 * i + 2] + part[4 * i + 3]);
        if (p.rb == 8) {
#pragma unroll
          for (int i = 0; i < 16; i += 4) *reinterpret_cast<float4*>(sums + i) = make_float4(q4[i], q4[i + 1], q4[i + 2], q4[i + 3]);
        } else if (p.rb == 16) {
#pragma unroll
          for (int i = 0; i < 8; i += 4)
            *reinterpret_cast<float4*>(sums + i) = make_float4(q4[2 * i] + q4[2 * i + 1], q4[2 * i + 2] + q4[2 * i + 3],
                                                                q4[2 * i + 4] + q4[2 * i + 5], q4[2 * i + 6] + q4[2 * i + 7]);
        } else {
          *reinterpret_cast<float4*>(sums) = make_float4((q4[0] + q4[1]) + (q4[2] + q4[3]), (q4[4] + q4[5]) + (q4[6] + q4[7]),
                                                          (q4[8] + q4[9]) + (q4[10] + q4[11]), (q4[12] + q4[13]) + (q4[14] + q4[15]));
        }
      }
    }
  }

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
    tc::tmem_dealloc(tmem, 256);
  }
}

// One CTA per query block (rb group rows), a warp per row: the row's maximum over its column tiles, its normaliser,
// then the rescaled block sums, accumulated per warp in shared memory in a fixed order (deterministic) and added up.
// part: [8 warps][n / rb] floats.
template <int FMT>
__global__ void __launch_bounds__(256) antidiag_combine_kernel(const float* __restrict__ tile_max, const float* __restrict__ block_sum,
                                                              uint16_t* __restrict__ out, int n, int n_valid, int rb, int nb, int causal) {
  extern __shared__ float part[];
  const int qb = blockIdx.x;
  const int64_t bh = blockIdx.y;
  const int nkb = n / rb, tiles = (n + 127) / 128, nbt = 128 / rb;
  const int pitch = tiles * nbt;                       // row pitch of block_sum (whole tiles)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < 8 * nkb; e += blockDim.x) part[e] = 0.f;
  __syncthreads();
  float* mine = part + warp * nkb;
  for (int r = warp; r < rb; r += 8) {
    const int i = qb * rb + r;
    if (i >= n_valid) continue;
    const int nt = causal ? i / 128 + 1 : tiles;        // column tiles the row has
    const int nblk = causal ? i / rb + 1 : nkb;         // key blocks with a visible column
    const float* tm = tile_max + (bh * n + i) * (int64_t)tiles;
    const float* bs = block_sum + (bh * n + i) * (int64_t)pitch;
    float m = -INFINITY;
    for (int j = lane; j < nt; j += 32) m = fmaxf(m, tm[j]);
    for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    float l = 0.f;
    for (int b = lane; b < nblk; b += 32) l += bs[b] * ex2(tm[b / nbt] - m);
    for (int off = 16; off; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
    const float inv = 1.0f / l;
    for (int b = lane; b < nblk; b += 32) mine[b] += bs[b] * ex2(tm[b / nbt] - m) * inv;
    __syncwarp();
  }
  __syncthreads();
  uint16_t* dst = out + (bh * nb + qb) * (int64_t)nb;
  for (int c = threadIdx.x; c < nb; c += blockDim.x) {
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) sum += part[w * nkb + c];
    dst[c] = FMT ? __bfloat16_as_ushort(__float2bfloat16_rn(sum)) : __half_as_ushort(__float2half_rn(sum));
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// {channel, token in group, group, batch*head} over a [bh][seq][D] tensor whose length is a multiple of the stride
int encode_groups_4d(CUtensorMap* map, const void* base, int is_bf16, int D, int stride, int64_t seq, int64_t bh) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  PSA_REQUIRE(fn != nullptr, PSA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)stride, (cuuint64_t)(seq / stride), (cuuint64_t)bh};
  cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)stride * D * 2, (cuuint64_t)seq * D * 2};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PSA_REQUIRE(r == CUDA_SUCCESS, PSA_ERR_CUDA, "cuTensorMapEncodeTiled (4-D groups) failed with CUresult %d", (int)r);
  return PSA_OK;
}

template <int D, int FMT>
int launch(const void* q, const void* k, void* out, float* scratch, int64_t bh, int64_t seq, int stride, int n, int n_valid, int rb,
           int nb, int causal, float scale_log2, int32_t* status, cudaStream_t st) {
  CUtensorMap tq, tk;
  int rc = encode_groups_4d(&tq, q, FMT, D, stride, seq, bh);
  if (rc != PSA_OK) return rc;
  rc = encode_groups_4d(&tk, k, FMT, D, stride, seq, bh);
  if (rc != PSA_OK) return rc;
  Params p;
  p.tile_max = scratch;
  p.block_sum = scratch + (size_t)bh * n * ((n + 127) / 128);
  p.n = n; p.n_valid = n_valid; p.rb = rb; p.stride = stride; p.causal = causal; p.bh = bh; p.scale_log2 = scale_log2; p.status = status;
  p.row_tiles = (n_valid + 127) / 128;
  p.col_tiles = (n + 127) / 128;
  const int smem = kStages * kStageBytes + 256 + 1024;
  cudaError_t e = cudaFuncSetAttribute(antidiag_logits_tc_kernel<D, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_antidiag_scores: shared-memory opt-in failed: %s", cudaGetErrorString(e));
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  const int64_t tiles = bh * (causal ? (int64_t)p.row_tiles * (p.row_tiles + 1) / 2 : (int64_t)p.row_tiles * p.col_tiles);
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  antidiag_logits_tc_kernel<D, FMT><<<grid, kThreads, smem, st>>>(tq, tk, p);
  PSA_CHECK_LAUNCH("psa_antidiag_scores(tcgen05 logits)");
  dim3 grid2((unsigned)nb, (unsigned)bh);
  antidiag_combine_kernel<FMT><<<grid2, 256, (size_t)8 * (n / rb) * sizeof(float), st>>>(p.tile_max, p.block_sum, (uint16_t*)out, n, n_valid,
                                                                                         rb, nb, causal);
  PSA_CHECK_LAUNCH("psa_antidiag_scores(combine)");
  return PSA_OK;
}

}  // namespace

bool antidiag_tc_supported(int64_t seq, int head_dim, int stride, int n, int dtype) {
  (void)n;
  return (dtype == PSA_F16 || dtype == PSA_BF16) && (head_dim == 64 || head_dim == 128) && stride >= 1 && seq % stride == 0 &&
         seq / stride >= 1;
}

// Whole estimate: out [bh][nb][nb] in the element type.  scratch: bh * n * ceil(n/128) * (1 + 128/rb) floats (at most
// bh * n * n for rb >= 2 and n >= 256; the caller's buffer holds bh * n * n).
int launch_antidiag_tc(const void* q, const void* k, void* out, float* scratch, int64_t bh, int64_t seq, int head_dim, int stride, int n,
                       int n_valid, int rb, int nb, int causal, float scale_log2, int dtype, int32_t* status, cudaStream_t st) {
  const int fmt = dtype == PSA_BF16;
  if (head_dim == 64)
    return fmt ? launch<64, 1>(q, k, out, scratch, bh, seq, stride, n, n_valid, rb, nb, causal, scale_log2, status, st)
               : launch<64, 0>(q, k, out, scratch, bh, seq, stride, n, n_valid, rb, nb, causal, scale_log2, status, st);
  return fmt ? launch<128, 1>(q, k, out, scratch, bh, seq, stride, n, n_valid, rb, nb, causal, scale_log2, status, st)
             : launch<128, 0>(q, k, out, scratch, bh, seq, stride, n, n_valid, rb, nb, causal, scale_log2, status, st);
}

}  // namespace psa
