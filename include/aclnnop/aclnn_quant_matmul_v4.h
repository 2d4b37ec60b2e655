/*
 * aclnnQuantMatmulV4 / aclnnQuantMatmulV3: the older entry points of the same operator family, with the argument order
 * (scale, offset, pertokenScale, bias) instead of V5's (x1Scale, x2Scale, ..., x2Offset, ..., bias, groupSize).
 *
 * Prototypes as in the reference:
 *   matmul/quant_batch_matmul_v3/op_api/aclnn_quant_matmul_v4.h:41-60
 *   matmul/quant_batch_matmul_v3/op_api/aclnn_quant_matmul_v3.h:40-58
 * Semantics: aclnnQuantMatmulV4(x1, x2, scale, offset, pertokenScale, bias, tX1, tX2, out) ==
 *            aclnnQuantMatmulV5(x1, x2, x1Scale = pertokenScale, x2Scale = scale, yScale = null, x1Offset = null,
 *                               x2Offset = offset, yOffset = null, bias, tX1, tX2, groupSize = 0, out);
 *            aclnnQuantMatmulV3 is V4 without pertokenScale. The quant modes reachable this way are K-C, T-C, T-T and
 *            their uint64-scale forms (no per-block / MX: those need V5's groupSize and scale shapes).
 */
#ifndef ACLNN_QUANT_MATMUL_V4_H_
#define ACLNN_QUANT_MATMUL_V4_H_

#include "aclnn_compat/acl_base.h"

#ifdef __cplusplus
extern "C" {
#endif

ACLNN_API aclnnStatus aclnnQuantMatmulV4GetWorkspaceSize(const aclTensor* x1, const aclTensor* x2, const aclTensor* scale,
                                                         const aclTensor* offset, const aclTensor* pertokenScaleOptional,
                                                         const aclTensor* bias, bool transposeX1, bool transposeX2,
                                                         const aclTensor* out, uint64_t* workspaceSize, aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnQuantMatmulV4(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor, aclrtStream stream);

ACLNN_API aclnnStatus aclnnQuantMatmulV3GetWorkspaceSize(const aclTensor* x1, const aclTensor* x2, const aclTensor* scale,
                                                         const aclTensor* offset, const aclTensor* bias, bool transposeX1,
                                                         bool transposeX2, const aclTensor* out, uint64_t* workspaceSize,
                                                         aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnQuantMatmulV3(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor, aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif /* ACLNN_QUANT_MATMUL_V4_H_ */
