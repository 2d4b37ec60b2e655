/* aclnnWeightQuantBatchMatmulNz: aclnnWeightQuantBatchMatmulV2 for a weight stored in FRACTAL_NZ.
 * Prototypes of matmul/weight_quant_batch_matmul_v2/op_host/op_api/aclnn_weight_quant_batch_matmul_nz.h:38-54 of the reference.
 *
 * weight: view (k, n) (INT8, INT4, or INT32 words of eight INT4), format ACL_FORMAT_FRACTAL_NZ, storage dims
 * [ceil(n / n0), ceil(k / k0), k0, n0] in elements of the tensor's dtype (the layout of nz_to_nd in
 * matmul/common/tests/st/arch35/matmul_golden_util.py:76-114). The fractal layout serves the Ascend cube unit; here a pre-pass
 * rewrites the weight row-major into the workspace (k * n elements) and the V2 kernels run on it. A weight in any other
 * format is ACLNN_ERR_PARAM_INVALID, as in the reference (.cpp:1836-1839). */
#ifndef OPSNN_ACLNN_WEIGHT_QUANT_BATCH_MATMUL_NZ_H_
#define OPSNN_ACLNN_WEIGHT_QUANT_BATCH_MATMUL_NZ_H_

#include "aclnn_compat/acl_base.h"

#ifdef __cplusplus
extern "C" {
#endif

ACLNN_API aclnnStatus aclnnWeightQuantBatchMatmulNzGetWorkspaceSize(
    const aclTensor* x, const aclTensor* weight, const aclTensor* antiquantScale, const aclTensor* antiquantOffsetOptional,
    const aclTensor* quantScaleOptional, const aclTensor* quantOffsetOptional, const aclTensor* biasOptional,
    int antiquantGroupSize, const aclTensor* y, uint64_t* workspaceSize, aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnWeightQuantBatchMatmulNz(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                                    aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif
