/*
 * aclnnWeightQuantBatchMatmulV3 — same operator as V2 plus `innerPrecise` (0 = high precision, 1 = high
 * performance; any other value is ACLNN_ERR_PARAM_INVALID).
 *
 * Replaces the reference's
 *   matmul/weight_quant_batch_matmul_v2/op_host/op_api/aclnn_weight_quant_batch_matmul_v3.h:24-34
 * (implementation: aclnn_weight_quant_batch_matmul_v2.cpp:1772-1889; innerPrecise check :283-291).
 * On the reference's current NPU generation the flag is documented to have no effect
 * (docs/aclnnWeightQuantBatchMatmulV3.md:414); here it is accepted and the same bit-faithful kernel runs
 * for both values.
 */
#ifndef OPSNN_B200_ACLNN_WEIGHT_QUANT_BATCH_MATMUL_V3_H_
#define OPSNN_B200_ACLNN_WEIGHT_QUANT_BATCH_MATMUL_V3_H_

#include "aclnn_compat/acl_base.h"

#ifdef __cplusplus
extern "C" {
#endif

ACLNN_API aclnnStatus aclnnWeightQuantBatchMatmulV3GetWorkspaceSize(
    const aclTensor* x, const aclTensor* weight, const aclTensor* antiquantScale,
    const aclTensor* antiquantOffsetOptional, const aclTensor* quantScaleOptional,
    const aclTensor* quantOffsetOptional, const aclTensor* biasOptional, int antiquantGroupSize, int innerPrecise,
    const aclTensor* y, uint64_t* workspaceSize, aclOpExecutor** executor);

ACLNN_API aclnnStatus aclnnWeightQuantBatchMatmulV3(void* workspace, uint64_t workspaceSize,
                                                    aclOpExecutor* executor, aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif
