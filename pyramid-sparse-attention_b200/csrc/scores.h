// Shapes of one block-score call and the hooks between the scalar and the tcgen05 stage A.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <type_traits>

#include "fwd.h"

namespace psa {

struct ScoreDims {
  int64_t seq_q, seq_k;
  int D, bm, bn;
  int kq, kk;      // samples kept per query / key block (block/4)
  int Mq, Nk;      // query / key blocks
  int nq_s, nk_s;  // sampled rows before padding
  int nk_cols;     // sampled key rows padded to a multiple of 64
  int n_d;         // key cells including padded ones
  float qk_scale;  // D^-0.5 * log2(e), both factors rounded to fp32 first
};

int make_score_dims(ScoreDims& d, int64_t seq_q, int64_t seq_k, int D, int bm, int bn);

// tcgen05 stage A (scores_tc.cu)
bool scores_tc_supported(const ScoreDims& d);
// bytes of scratch the tcgen05 path needs beyond R and rowmax (compacted sample matrices)
size_t scores_tc_extra_scratch(const ScoreDims& d, int64_t bh);
int launch_scores_cellmax_tc(const RowSource& q, const RowSource& k, const int32_t* idx_q, const int32_t* idx_k, void* R,
                             float* rowmax, void* extra, const ScoreDims& d, int64_t bh, int dtype, cudaStream_t st,
                             const RopeTables& rope = RopeTables{});

// the same stage A on sample matrices that are already compacted: qs [bh][nq_s][D], ks [bh][nk_cols][D]
int launch_scores_cellmax_tc_samples(const void* qs, const void* ks, void* R, float* rowmax, const ScoreDims& d, int64_t bh,
                                     int dtype, cudaStream_t st);

}  // namespace psa
