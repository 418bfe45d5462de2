// Level assignment: one CTA per score row sorts the row (descending, equal scores by ascending block
// index), derives each pyramid level's rank interval and emits the mask row in either format.
//
// HBM/latency-bound integer work.  Algorithmic bytes per row: nk*e read + width*4 written.
//
// Sort: 64-bit keys = (order-reversed float bits << 32) | index, bitonic network in shared memory; keys are
// unique, so any correct network yields the stable order.
// Cumulative-energy mode reproduces the host library's CPU arithmetic bit for bit: the running sum is
// SEQUENTIAL (double accumulator for fp32 scores, fp32 accumulator for f16/bf16) and rounded to the score
// type at every element; ratio = round(cs / cs[last]) in the score type; the comparison threshold arrives
// already rounded to the score type.
#include "psa_common.cuh"

namespace psa {

struct AssignParams {
  int nk, width, n_levels, threshold_mode, newtype, min_index, text_blocks, npow2;
  int level[PSA_MAX_LEVELS], start[PSA_MAX_LEVELS], end[PSA_MAX_LEVELS], align[PSA_MAX_LEVELS];
  float thr[PSA_MAX_LEVELS];
  // causal call site (variant 1): square score matrices, quotas that follow the row's causal length
  int variant, causal, special;
  float rs[PSA_MAX_LEVELS], re[PSA_MAX_LEVELS], lo[PSA_MAX_LEVELS];
};

__device__ __forceinline__ uint32_t desc_key(float v) {
  uint32_t u = __float_as_uint(v == 0.f ? 0.f : v);      // -0 -> +0
  uint32_t ord = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // ascending order of floats
  return ~ord;                                              // descending
}
__device__ __forceinline__ float key_value(uint32_t hi) {
  uint32_t ord = ~hi;
  uint32_t u = (ord & 0x80000000u) ? (ord & 0x7fffffffu) : ~ord;
  return __uint_as_float(u);
}

// Everything after the sort: keys[] holds the row in rank order (score key << 32 | block index); s_cnt is zeroed.
template <typename T>
__device__ __forceinline__ void emit_mask_row(const unsigned long long* keys, float* ratio, int* s_start, int* s_end, int* s_cnt,
                                              int32_t* __restrict__ mask, const AssignParams& p, int64_t row, int tid, int nt) {
  if (p.threshold_mode) {
    if (tid == 0) {
      if (sizeof(T) == 4) {
        double acc = 0.0;
        for (int i = 0; i < p.nk; ++i) { acc += (double)key_value((uint32_t)(keys[i] >> 32)); ratio[i] = (float)acc; }
      } else {
        float acc = 0.f;
        for (int i = 0; i < p.nk; ++i) { acc += key_value((uint32_t)(keys[i] >> 32)); ratio[i] = Elem<T>::round(acc); }
      }
    }
    __syncthreads();
    const float total = ratio[p.nk - 1];
    int cnt[PSA_MAX_LEVELS];
#pragma unroll
    for (int l = 0; l < PSA_MAX_LEVELS; ++l) cnt[l] = 0;
    for (int i = tid; i < p.nk; i += nt) {
      float r = Elem<T>::round(__fdiv_rn(ratio[i], total));
#pragma unroll
      for (int l = 0; l < PSA_MAX_LEVELS; ++l) cnt[l] += (l < p.n_levels && r <= p.thr[l]) ? 1 : 0;
    }
#pragma unroll
    for (int l = 0; l < PSA_MAX_LEVELS; ++l) {
      int c = cnt[l];
      for (int off = 16; off; off >>= 1) c += __shfl_xor_sync(0xffffffffu, c, off);
      if ((tid & 31) == 0 && c) atomicAdd(&s_cnt[l], c);
    }
    __syncthreads();
    if (tid == 0) {
      int last = 0;
      for (int l = 0; l < p.n_levels; ++l) {
        const int a = p.align[l], c = s_cnt[l];
        const int init_end = c > 0 ? c + 1 : last;
        const int start = last;
        int end;
        if (a > 1) {
          int len = init_end - start; len = len > 0 ? len : 0;
          int rem = len % a;
          int aligned = rem ? len + (a - rem) : len;
          end = start + aligned; end = end < p.nk ? end : p.nk;
          if (end == p.nk) end = start + ((end - start) / a) * a;
        } else {
          end = init_end > 0 ? init_end : 0; end = end < p.nk ? end : p.nk; end = end > start ? end : start;
          if (p.level[l] == 1) end = end > p.min_index ? end : p.min_index;
        }
        s_start[l] = start; s_end[l] = end; last = end;
      }
    }
    __syncthreads();
  } else {
    if (tid < p.n_levels) { s_start[tid] = p.start[tid]; s_end[tid] = p.end[tid]; }
    __syncthreads();
  }

  int32_t* dst = mask + row * p.width;
  if (p.newtype) {
    for (int pos = tid; pos < p.width; pos += nt) {
      int32_t val = 0;
      for (int l = 0; l < p.n_levels; ++l) {
        const int s = s_start[l], e = s_end[l];
        int sep = l + e; sep = sep < 0 ? 0 : (sep > p.width - 1 ? p.width - 1 : sep);
        const int rank = pos - l;
        if (rank >= s && rank < e) val = (int32_t)(keys[rank] & 0xffffffffu);
        if (pos == sep) val = -1;
      }
      dst[pos] = val;
    }
  } else {
    for (int pos = tid; pos < p.nk; pos += nt) dst[pos] = 0;
    __syncthreads();
    for (int l = 0; l < p.n_levels; ++l) {
      const int s = s_start[l], e = s_end[l];
      for (int rank = s + tid; rank < e; rank += nt) dst[(int)(keys[rank] & 0xffffffffu)] = p.level[l];
      __syncthreads();   // later levels overwrite earlier ones, in order
    }
    if (p.text_blocks > 0) {
      int tb = p.text_blocks < p.nk ? p.text_blocks : p.nk;
      for (int pos = p.nk - tb + tid; pos < p.nk; pos += nt) dst[pos] = 1;
    }
  }
}

// Mask row of the causal call site (dense format, square matrices): quotas are fractions of the row's causal length
// i+1 (fp32 product, truncated), or bands of the cumulative mass; then the fixed rules: special (text) blocks, nothing
// above the diagonal, diagonal and first column always at level 1.
template <typename T>
__device__ __forceinline__ void emit_causal_row(const unsigned long long* keys, float* ratio, const T* __restrict__ src,
                                                int32_t* __restrict__ mask, const AssignParams& p, int64_t row, int tid, int nt) {
  const int n = p.nk;
  const int i = (int)(row % n);
  int32_t* dst = mask + row * n;
  for (int pos = tid; pos < n; pos += nt) dst[pos] = 0;
  __syncthreads();
  if (!p.threshold_mode) {
    const float valid = p.causal ? (float)(i + 1) : (float)n;
    for (int l = 0; l < p.n_levels; ++l) {
      int s = (int)__fmul_rn(valid, p.rs[l]), e = (int)__fmul_rn(valid, p.re[l]);
      s = s < n ? s : n; e = e < n ? e : n;
      for (int rank = s + tid; rank < e; rank += nt) dst[(int)(keys[rank] & 0xffffffffu)] = p.level[l];
      __syncthreads();   // later levels overwrite earlier ones, in order
    }
  } else {
    __shared__ float s_total;
    if (tid == 0) {
      float total;
      if (sizeof(T) == 4) {
        double t = 0.0, acc = 0.0;
        for (int c = 0; c < n; ++c) t += (double)Elem<T>::to_f(src[c]);
        for (int r = 0; r < n; ++r) { acc += (double)key_value((uint32_t)(keys[r] >> 32)); ratio[r] = (float)acc; }
        total = (float)t;
      } else {
        float t = 0.f, acc = 0.f;
        for (int c = 0; c < n; ++c) t += Elem<T>::to_f(src[c]);
        for (int r = 0; r < n; ++r) { acc += key_value((uint32_t)(keys[r] >> 32)); ratio[r] = Elem<T>::round(acc); }
        total = Elem<T>::round(t);
      }
      s_total = fmaxf(total, Elem<T>::round(1e-10f));
    }
    __syncthreads();
    const float total = s_total;
    for (int r = tid; r < n; r += nt) {
      const float e = Elem<T>::round(__fdiv_rn(ratio[r], total));
      int32_t val = 0;
      for (int l = 0; l < p.n_levels; ++l)
        if (e > p.lo[l] && e <= p.thr[l]) val = p.level[l];
      dst[(int)(keys[r] & 0xffffffffu)] = val;
    }
    __syncthreads();
  }
  for (int j = tid; j < n; j += nt) {
    int32_t v = dst[j];
    if (p.special > 0 && (j >= n - p.special || i >= n - p.special)) v = 1;
    if (p.causal && j > i) v = 0;
    if (j == i || j == 0) v = 1;
    dst[j] = v;
  }
}

// General kernel (any score type, any row length up to 8192): bitonic network over 64-bit keys in shared memory.
template <typename T>
__global__ void __launch_bounds__(256) assign_levels_kernel(const T* __restrict__ po, int32_t* __restrict__ mask,
                                                           AssignParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(smem_raw);
  float* ratio = reinterpret_cast<float*>(keys + p.npow2);  // threshold mode only
  __shared__ int s_start[PSA_MAX_LEVELS], s_end[PSA_MAX_LEVELS];
  __shared__ int s_cnt[PSA_MAX_LEVELS];

  const int64_t row = blockIdx.x;
  const T* src = po + row * p.nk;
  const int tid = threadIdx.x, nt = blockDim.x;

  for (int i = tid; i < p.npow2; i += nt)
    keys[i] = i < p.nk ? (((unsigned long long)desc_key(Elem<T>::to_f(src[i])) << 32) | (unsigned)i) : ~0ull;
  if (tid < PSA_MAX_LEVELS) s_cnt[tid] = 0;
  __syncthreads();

  for (int k = 2; k <= p.npow2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = tid; i < p.npow2; i += nt) {
        int ixj = i ^ j;
        if (ixj > i) {
          unsigned long long a = keys[i], b = keys[ixj];
          bool asc = (i & k) == 0;
          if ((a > b) == asc) { keys[i] = b; keys[ixj] = a; }
        }
      }
      __syncthreads();
    }
  }
  if (p.variant == 1) emit_causal_row<T>(keys, ratio, src, mask, p, row, tid, nt);
  else emit_mask_row<T>(keys, ratio, s_start, s_end, s_cnt, mask, p, row, tid, nt);
}

// Fast kernel for 16-bit scores and rows of at most 4096 blocks: the key fits 32 bits (16 score bits, 16 index bits),
// every thread keeps E consecutive keys in registers, and the network's exchanges run in registers (distance < E),
// through warp shuffles (distance < 32 E) or through shared memory (only the last few stages).
template <typename T, int E>
__global__ void __launch_bounds__(256) assign_levels_reg_kernel(const T* __restrict__ po, int32_t* __restrict__ mask,
                                                               AssignParams p) {
  constexpr int N = E * 256;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(smem_raw);
  float* ratio = reinterpret_cast<float*>(keys + N);          // threshold mode; doubles as exchange buffer during the sort
  uint32_t* xch = reinterpret_cast<uint32_t*>(ratio);
  __shared__ int s_start[PSA_MAX_LEVELS], s_end[PSA_MAX_LEVELS];
  __shared__ int s_cnt[PSA_MAX_LEVELS];

  const int64_t row = blockIdx.x;
  const unsigned short* src = reinterpret_cast<const unsigned short*>(po + row * p.nk);
  const int tid = threadIdx.x;
  if (tid < PSA_MAX_LEVELS) s_cnt[tid] = 0;

  uint32_t a[E];
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const int i = tid * E + e;
    uint32_t key = 0xffffffffu;
    if (i < p.nk) {
      uint32_t b = src[i];
      if (b == 0x8000u) b = 0;                                             // -0 -> +0
      const uint32_t ord = (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);   // ascending order of the values
      key = ((~ord & 0xffffu) << 16) | (uint32_t)i;                        // descending value, then ascending index
    }
    a[e] = key;
  }
#pragma unroll
  for (int k = 2; k <= N; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      if (j >= 32 * E) {
        // partner lives in another warp: same lane, same e
#pragma unroll
        for (int e = 0; e < E; ++e) xch[e * 256 + tid] = a[e];
        __syncthreads();
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const int i = tid * E + e;
          const uint32_t pv = xch[e * 256 + (tid ^ (j / E))];
          const bool take_min = ((i & j) == 0) == ((i & k) == 0);
          a[e] = take_min ? min(a[e], pv) : max(a[e], pv);
        }
        __syncthreads();
      } else if (j >= E) {
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const int i = tid * E + e;
          const uint32_t pv = __shfl_xor_sync(0xffffffffu, a[e], j / E);
          const bool take_min = ((i & j) == 0) == ((i & k) == 0);
          a[e] = take_min ? min(a[e], pv) : max(a[e], pv);
        }
      } else {
#pragma unroll
        for (int e = 0; e < E; ++e) {
          if ((e & j) == 0) {
            const int i = tid * E + e;
            const uint32_t lo = min(a[e], a[e | j]), hi = max(a[e], a[e | j]);
            const bool asc = (i & k) == 0;
            a[e] = asc ? lo : hi;
            a[e | j] = asc ? hi : lo;
          }
        }
      }
    }
  }
  // back to the common key format, in rank order
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const uint32_t ord = ~(a[e] >> 16) & 0xffffu;
    const uint32_t b = (ord & 0x8000u) ? (ord & 0x7fffu) : (~ord & 0xffffu);
    const unsigned short raw = (unsigned short)b;
    const float v = Elem<T>::to_f(*reinterpret_cast<const T*>(&raw));
    keys[tid * E + e] = a[e] == 0xffffffffu ? ~0ull : (((unsigned long long)desc_key(v) << 32) | (a[e] & 0xffffu));
  }
  __syncthreads();
  if (p.variant == 1) emit_causal_row<T>(keys, ratio, po + row * p.nk, mask, p, row, tid, 256);
  else emit_mask_row<T>(keys, ratio, s_start, s_end, s_cnt, mask, p, row, tid, 256);
}

// ------------------------------------------------------------------------------ density -------------
// One CTA per (batch, head); a warp walks one mask row at a time.  Deterministic summation order.
__global__ void __launch_bounds__(256) density_kernel(const int32_t* __restrict__ mask, float* __restrict__ per_bh,
                                                     int mq, int width, int newtype) {
  __shared__ float s_part[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int32_t* base = mask + (int64_t)blockIdx.x * mq * width;
  float acc = 0.f;
  for (int r = warp; r < mq; r += 8) {
    const int32_t* row = base + (int64_t)r * width;
    if (newtype) {
      // segments 0..3 are levels 1,2,4,8; a segment ends at a -1 (or at the row end)
      int seg = 0, seg_start = 0;
      float dens = 0.f;
      for (int c0 = 0; c0 < width && seg < 4; c0 += 32) {
        int v = (c0 + lane < width) ? row[c0 + lane] : 0;
        unsigned bits = __ballot_sync(0xffffffffu, v == -1);
        while (bits && seg < 4) {
          int pos = c0 + __ffs(bits) - 1;
          bits &= bits - 1;
          dens += (float)(pos - seg_start) / (float)(1 << seg);
          ++seg; seg_start = pos + 1;
        }
      }
      if (seg < 4) dens += (float)(width - seg_start) / (float)(1 << seg);
      acc += dens / (float)(width - 5);
    } else {
      float dens = 0.f;
      for (int c = lane; c < width; c += 32) { int v = row[c]; dens += v > 0 ? 1.0f / (float)v : 0.f; }
      for (int off = 16; off; off >>= 1) dens += __shfl_xor_sync(0xffffffffu, dens, off);
      acc += dens / (float)width;
    }
  }
  if (lane == 0) s_part[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += s_part[w];
    per_bh[blockIdx.x] = t / (float)mq;
  }
}

}  // namespace psa

namespace psa {
// Launch of the sort + emit kernels for a filled parameter block (p.npow2 is set here).
static int launch_assign(const void* po, int32_t* mask, int64_t rows, AssignParams p, int dtype, cudaStream_t st) {
  const int nk = p.nk;
  const int threshold_mode = p.threshold_mode;
  int np2 = 2; while (np2 < nk) np2 <<= 1;
  p.npow2 = np2;
  if ((dtype == PSA_F16 || dtype == PSA_BF16) && nk <= 4096) {
    // register-resident sort: E keys per thread, 256 threads
    const int E = np2 <= 512 ? 2 : np2 / 256;
    p.npow2 = E * 256;
    const size_t smem_reg = (size_t)E * 256 * 12;
#define PSA_ASSIGN_REG(TT, EE)                                                                                              \
  do {                                                                                                                     \
    if (smem_reg > 40 * 1024) {                                                                                            \
      cudaError_t e = cudaFuncSetAttribute(assign_levels_reg_kernel<TT, EE>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem_reg);                                                                 \
      PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_assign_levels: smem opt-in failed: %s", cudaGetErrorString(e));     \
    }                                                                                                                      \
    assign_levels_reg_kernel<TT, EE><<<(unsigned)rows, 256, smem_reg, st>>>((const TT*)po, mask, p);                       \
  } while (0)
#define PSA_ASSIGN_REG_E(TT)                                                                  \
  do {                                                                                       \
    if (E == 2) PSA_ASSIGN_REG(TT, 2); else if (E == 4) PSA_ASSIGN_REG(TT, 4);               \
    else if (E == 8) PSA_ASSIGN_REG(TT, 8); else PSA_ASSIGN_REG(TT, 16);                     \
  } while (0)
    if (dtype == PSA_F16) PSA_ASSIGN_REG_E(__half); else PSA_ASSIGN_REG_E(__nv_bfloat16);
#undef PSA_ASSIGN_REG_E
#undef PSA_ASSIGN_REG
    PSA_CHECK_LAUNCH("psa_assign_levels");
    return PSA_OK;
  }
  size_t smem = (size_t)np2 * 8 + (threshold_mode ? (size_t)nk * 4 : 0);
  int threads = np2 / 2 < 256 ? (np2 / 2 < 32 ? 32 : np2 / 2) : 256;
  PSA_DISPATCH_DTYPE(dtype, T, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(assign_levels_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      PSA_REQUIRE(e == cudaSuccess, PSA_ERR_CUDA, "psa_assign_levels: smem opt-in failed: %s", cudaGetErrorString(e));
    }
    assign_levels_kernel<T><<<(unsigned)rows, threads, smem, st>>>((const T*)po, mask, p);
  });
  PSA_CHECK_LAUNCH("psa_assign_levels");
  return PSA_OK;
}
}  // namespace psa

extern "C" int psa_assign_levels(const void* po, int32_t* mask, int64_t rows, int nk, int dtype, int threshold_mode,
                                 int newtype, int n_levels, const int32_t* level_values, const int32_t* starts,
                                 const int32_t* ends, const float* thresholds, const int32_t* aligns, int min_index,
                                 int text_blocks, void* stream) {
  using namespace psa;
  PSA_REQUIRE(po && mask && level_values, PSA_ERR_ARG, "psa_assign_levels: null pointer");
  PSA_REQUIRE(rows > 0 && rows < (1ll << 31), PSA_ERR_ARG, "psa_assign_levels: rows=%lld out of range", (long long)rows);
  PSA_REQUIRE(nk > 0 && nk <= 8192, PSA_ERR_ARG, "psa_assign_levels: nk=%d out of range (1..8192)", nk);
  PSA_REQUIRE(n_levels > 0 && n_levels <= PSA_MAX_LEVELS, PSA_ERR_ARG, "psa_assign_levels: n_levels=%d", n_levels);
  if (threshold_mode) PSA_REQUIRE(thresholds && aligns, PSA_ERR_ARG, "psa_assign_levels: thresholds/aligns missing");
  else PSA_REQUIRE(starts && ends, PSA_ERR_ARG, "psa_assign_levels: starts/ends missing");
  AssignParams p = {};
  p.nk = nk; p.n_levels = n_levels; p.threshold_mode = threshold_mode; p.newtype = newtype;
  p.width = newtype ? nk + n_levels : nk;
  p.min_index = min_index; p.text_blocks = text_blocks;
  for (int i = 0; i < PSA_MAX_LEVELS; ++i) {
    p.level[i] = i < n_levels ? level_values[i] : 0;
    p.start[i] = (i < n_levels && !threshold_mode) ? starts[i] : 0;
    p.end[i] = (i < n_levels && !threshold_mode) ? ends[i] : 0;
    p.align[i] = (i < n_levels && threshold_mode) ? aligns[i] : 1;
    p.thr[i] = (i < n_levels && threshold_mode) ? thresholds[i] : 0.f;
    if (i < n_levels && !threshold_mode)
      PSA_REQUIRE(p.start[i] >= 0 && p.start[i] <= p.end[i] && p.end[i] <= nk, PSA_ERR_ARG,
                  "psa_assign_levels: interval %d = [%d,%d) outside [0,%d]", i, p.start[i], p.end[i], nk);
  }
  return launch_assign(po, mask, rows, p, dtype, (cudaStream_t)stream);
}

extern "C" int psa_assign_levels_causal(const void* attn, int32_t* mask, int64_t bh, int n, int dtype, int energy_mode, int causal,
                                        int n_levels, const int32_t* level_values, const float* start_ratios,
                                        const float* end_ratios, const float* lower_bounds, const float* upper_bounds,
                                        int special_blocks, void* stream) {
  using namespace psa;
  PSA_REQUIRE(attn && mask && level_values, PSA_ERR_ARG, "psa_assign_levels_causal: null pointer");
  PSA_REQUIRE(bh > 0 && n > 0 && n <= 8192 && bh * n < (1ll << 31), PSA_ERR_ARG, "psa_assign_levels_causal: bad shape");
  PSA_REQUIRE(n_levels > 0 && n_levels <= PSA_MAX_LEVELS, PSA_ERR_ARG, "psa_assign_levels_causal: n_levels=%d", n_levels);
  PSA_REQUIRE(special_blocks >= 0 && special_blocks <= n, PSA_ERR_ARG, "psa_assign_levels_causal: special_blocks=%d", special_blocks);
  if (energy_mode) PSA_REQUIRE(lower_bounds && upper_bounds, PSA_ERR_ARG, "psa_assign_levels_causal: bounds missing");
  else PSA_REQUIRE(start_ratios && end_ratios, PSA_ERR_ARG, "psa_assign_levels_causal: ratios missing");
  AssignParams p = {};
  p.nk = n; p.width = n; p.n_levels = n_levels; p.threshold_mode = energy_mode ? 1 : 0; p.newtype = 0;
  p.variant = 1; p.causal = causal ? 1 : 0; p.special = special_blocks;
  for (int i = 0; i < n_levels; ++i) {
    p.level[i] = level_values[i];
    if (energy_mode) { p.lo[i] = lower_bounds[i]; p.thr[i] = upper_bounds[i]; }
    else { p.rs[i] = start_ratios[i]; p.re[i] = end_ratios[i]; }
  }
  return launch_assign(attn, mask, bh * n, p, dtype, (cudaStream_t)stream);
}

extern "C" int psa_density(const int32_t* mask, float* per_bh, int64_t bh, int64_t mq, int width, int newtype,
                           void* stream) {
  using namespace psa;
  PSA_REQUIRE(mask && per_bh, PSA_ERR_ARG, "psa_density: null pointer");
  PSA_REQUIRE(bh > 0 && mq > 0 && width > (newtype ? 5 : 0), PSA_ERR_ARG, "psa_density: bad shape");
  density_kernel<<<(unsigned)bh, 256, 0, (cudaStream_t)stream>>>(mask, per_bh, (int)mq, width, newtype);
  PSA_CHECK_LAUNCH("psa_density");
  return PSA_OK;
}
