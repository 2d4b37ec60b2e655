/*
 * aclnnWeightQuantBatchMatmulV2 — weight-only quantized matmul (A16W4 / A16W8 ...): the weight is dequantised
 * ("antiquant") on the fly and multiplied with a bf16/fp16 activation.
 *
 * Replaces the reference's
 *   matmul/weight_quant_batch_matmul_v2/op_host/op_api/aclnn_weight_quant_batch_matmul_v2.h:38-54
 * (implementation: aclnn_weight_quant_batch_matmul_v2.cpp:1719-1767, 1870-1874).
 *
 *   W' = cast_x( cast_x( W + antiquantOffset ) * antiquantScale )     (two roundings in x's dtype, no FMA)
 *   y  = cast_x( x @ W' (fp32 accumulate) + bias )
 *
 *   x               (m,k) bf16|fp16, contiguous
 *   weight          (k,n) int8 | int4 | int32 (8 int4 per word along the inner axis, element j at bits 4j) |
 *                   a strided-transposed view of (n,k) storage
 *   antiquantScale  (1,) (n,) (1,n) per-tensor/-channel, or (ceil(k/g), n) per-group with antiquantGroupSize g
 *   antiquantOffset same shape as the scale, optional
 *   quantScale / quantOffset must be NULL on this target (they only exist for int8 outputs on older NPUs)
 *   bias            (n,) | (1,n), dtype of x (or fp32 when x is bf16)
 *   y               (m,n), dtype of x
 */
#ifndef OPSNN_B200_ACLNN_WEIGHT_QUANT_BATCH_MATMUL_V2_H_
#define OPSNN_B200_ACLNN_WEIGHT_QUANT_BATCH_MATMUL_V2_H_

#include "aclnn_compat/acl_base.h"

#ifdef __cplusplus
extern "C" {
#endif

ACLNN_API aclnnStatus aclnnWeightQuantBatchMatmulV2GetWorkspaceSize(
    const aclTensor* x, const aclTensor* weight, const aclTensor* antiquantScale,
    const aclTensor* antiquantOffsetOptional, const aclTensor* quantScaleOptional,
    const aclTensor* quantOffsetOptional, const aclTensor* biasOptional, int antiquantGroupSize,
    const aclTensor* y, uint64_t* workspaceSize, aclOpExecutor** executor);

ACLNN_API aclnnStatus aclnnWeightQuantBatchMatmulV2(void* workspace, uint64_t workspaceSize,
                                                    aclOpExecutor* executor, aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif
