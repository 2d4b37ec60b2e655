/*
 * aclnnQuantMatmulWeightNz - aclnnQuantMatmulV5 with x2 stored in the FRACTAL_NZ format.
 *
 * Replaces the reference's
 *   matmul/quant_batch_matmul_v3/op_api/aclnn_quant_matmul_weight_nz.h:41-55
 * (implementation: matmul/quant_batch_matmul_v3/op_api/aclnn_quant_matmul_v4.cpp; the format requirement at :855).
 * Same arguments, argument order and status codes as aclnnQuantMatmulV5. x2 must be a 2-D tensor whose storage format is
 * ACL_FORMAT_FRACTAL_NZ with storage dims [ceil(cols / c0), ceil(rows / r0), r0, c0] over the (rows, cols) matrix its view
 * describes (nz_to_nd of matmul/common/tests/st/arch35/matmul_golden_util.py:76-114). The fractal layout exists for the Ascend
 * cube unit; here phase 2 rewrites x2 row-major into the head of the workspace with one copy kernel and runs the same kernels
 * as aclnnQuantMatmulV5 on it, so results are those of the ND call bit for bit. The workspace size phase 1 reports includes the copy.
 */
#ifndef OPSNN_B200_ACLNN_QUANT_MATMUL_WEIGHT_NZ_H_
#define OPSNN_B200_ACLNN_QUANT_MATMUL_WEIGHT_NZ_H_

#include "aclnn_compat/acl_base.h"

#ifdef __cplusplus
extern "C" {
#endif

ACLNN_API aclnnStatus aclnnQuantMatmulWeightNzGetWorkspaceSize(const aclTensor* x1, const aclTensor* x2,
                                                               const aclTensor* x1Scale, const aclTensor* x2Scale,
                                                               const aclTensor* yScale, const aclTensor* x1Offset,
                                                               const aclTensor* x2Offset, const aclTensor* yOffset,
                                                               const aclTensor* bias, bool transposeX1,
                                                               bool transposeX2, int64_t groupSize, aclTensor* out,
                                                               uint64_t* workspaceSize, aclOpExecutor** executor);

ACLNN_API aclnnStatus aclnnQuantMatmulWeightNz(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                               aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif /* OPSNN_B200_ACLNN_QUANT_MATMUL_WEIGHT_NZ_H_ */
