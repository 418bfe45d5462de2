#include "psa_common.cuh"
#include "fwd.h"
namespace psa {
bool fwd_tc_supported(const FwdArgs&) { return false; }
int fwd_tc_launch(const FwdArgs&, cudaStream_t) { set_error("tcgen05 forward not built"); return PSA_ERR_UNSUPPORTED; }
}
