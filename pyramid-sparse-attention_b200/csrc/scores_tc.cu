#include "psa_common.cuh"
#include "scores.h"
namespace psa {
bool scores_tc_supported(const ScoreDims&) { return false; }
int launch_scores_cellmax_tc(const void*, const void*, const int32_t*, const int32_t*, void*, float*, const ScoreDims&,
                             int64_t, int, cudaStream_t) { set_error("tcgen05 scores not built"); return PSA_ERR_UNSUPPORTED; }
}
