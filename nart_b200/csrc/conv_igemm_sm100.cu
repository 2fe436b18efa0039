#include "common.cuh"
#include "kernels.h"
namespace b200 {
struct ConvIgemmPlan {};
int conv_igemm_supported(const ConvGeom &, char *why, size_t n) { snprintf(why, n, "stub"); return 0; }
int conv_igemm_create(const ConvGeom &, const std::vector<int8_t> &, const int32_t *, const uint32_t *, const int32_t *, ConvIgemmPlan **) { return B200_ERR_UNSUPPORTED; }
int conv_igemm_launch(ConvIgemmPlan *, const uint8_t *, int, uint8_t *, cudaStream_t) { return B200_ERR_UNSUPPORTED; }
void conv_igemm_destroy(ConvIgemmPlan *) {}
}
