// placeholder replaced below
#include "common.cuh"
namespace opsnn {
bool qmm_umma_eligible(const OpsnnQmmParams*) { return false; }
uint64_t qmm_umma_workspace_size(const OpsnnQmmParams*) { return 0; }
int32_t qmm_umma_launch(const OpsnnQmmParams*, cudaStream_t) { return (int32_t)cudaErrorNotSupported; }
}
