/*
 * aclnnDynamicMxQuant — on-the-fly microscaling quantisation of a bf16/fp16 tensor: one e8m0 shared exponent per
 * `blocksize` (32) elements along `axis`, elements to fp8 (e4m3/e5m2) or fp4 (e2m1), round-to-nearest-even,
 * saturating. This is the "dynamic activation quant fused ahead" of the MXFP8 matmul.
 *
 * Replaces the reference's aclnnDynamicMxQuant (quant/dynamic_mx_quant/docs/aclnnDynamicMxQuant.md:76-95; arithmetic:
 * quant/dynamic_mx_quant/tests/assets/golden.py:141-154, 197-217, 272-336).
 *
 *   x          (..., k) bf16|fp16, contiguous
 *   axis       only the last axis (-1 or rank-1) is implemented here
 *   roundMode  "rint" (NULL means "rint")
 *   dstType    aclDataType of yOut: 36 e4m3fn, 35 e5m2, 40 e2m1 (packed two per byte, low nibble first)
 *   blocksize  32
 *   scaleAlg   0 (OCP: shared exponent = floor(log2(amax)) - emax_of_dst)
 *   yOut       same shape as x
 *   mxscaleOut e8m0 bytes, shape (..., ceil(ceil(k/32)/2), 2); the count is padded to even with 2^-127
 */
#ifndef OPSNN_B200_ACLNN_DYNAMIC_MX_QUANT_H_
#define OPSNN_B200_ACLNN_DYNAMIC_MX_QUANT_H_

#include "aclnn_compat/acl_base.h"

#ifdef __cplusplus
extern "C" {
#endif

ACLNN_API aclnnStatus aclnnDynamicMxQuantGetWorkspaceSize(const aclTensor* x, int64_t axis, char* roundModeOptional,
                                                          int64_t dstType, int64_t blocksize, int64_t scaleAlg,
                                                          const aclTensor* yOut, const aclTensor* mxscaleOut,
                                                          uint64_t* workspaceSize, aclOpExecutor** executor);

ACLNN_API aclnnStatus aclnnDynamicMxQuant(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                          aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif
