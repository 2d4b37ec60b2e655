/*
 * aclnnWeightQuantBatchMatmulV3 — same operator as V2 plus `innerPrecise` (0 = high precision, 1 = high
 * performance; any other value is ACLNN_ERR_PARAM_INVALID).
 *
 * Replaces the reference's
 *   matmul/weight_quant_batch_matmul_v2/op_host/op_api/aclnn_weight_quant_batch_matmul_v3.h:24-34
 * (implementation: aclnn_weight_quant_batch_matmul_v2.cpp:1772-1889; innerPrecise check :283-291).
 * The reference documents innerPrecise = 1 as the faster, slightly less faithful mode for A16W4 per-group with
 * m <= 16 (docs/aclnnWeightQuantBatchMatmulV3.md:28, :389) and as having no effect elsewhere (:414). Here:
 *   innerPrecise = 0  every dequantised weight is rounded twice in x's dtype, exactly as the reference's golden does;
 *   innerPrecise = 1  where the streaming decode kernel applies (INT4 weight stored (k,n), m <= 16, 32-column pieces)
 *                     scale and offset are applied per k-group to the fp32 accumulators instead: no weight is rounded,
 *                     the result is closer to the fp32 dequantised product but not bit-identical to innerPrecise = 0;
 *                     on every other shape the flag changes nothing.
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
