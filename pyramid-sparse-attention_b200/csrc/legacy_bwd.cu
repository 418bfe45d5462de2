#include "psa_common.cuh"
extern "C" int psa_legacy_bwd(const void*, const void*, const void*, const void*, const void*, const void*, const void*,
                              const void*, const void*, const int32_t*, const void*, const float*, const void*, void*, void*,
                              void*, float*, int64_t, int64_t, int, int, float, int, int, void*) {
  psa::set_error("psa_legacy_bwd: not built yet");
  return PSA_ERR_UNSUPPORTED;
}
