/*
 * aclnnQuantMatmulV5 — full-quantized (both operands low precision) batched matmul with fused dequantisation.
 *
 * Replaces, symbol for symbol, the reference's
 *   matmul/quant_batch_matmul_v4/op_host/op_api/aclnn_quant_matmul_v5.h:43-60
 * (implementation: aclnn_quant_matmul_v5.cpp:1189-1227). Argument order, meaning, the `groupSize` bit packing
 * (K | N<<16 | M<<32; a zero field is inferred from the scale shapes) and the returned status codes are the
 * reference's; everything underneath is CUDA for sm_100a.
 *
 *   out = dequant( x1 @ x2 ) [+ bias]
 *
 *   quant mode (derived from the scale tensors exactly as the reference's host code does,
 *   quant_batch_matmul_v3/op_host/op_tiling/quant_batch_matmul_v3_tiling_base.cpp:458-557):
 *     int8 x int8, x2Scale fp32/bf16 (n,)|(1,), optional x1Scale fp32 (m,)  : per-channel/-tensor (x per-token)
 *     int8 x int8, x2Scale uint64/int64 packed (n,)|(1,)                   : fixpipe-style packed scale
 *     fp8  x fp8,  x1Scale fp32 (m|m/128, k/128), x2Scale fp32 (k/128,n/128): per-block, groupSize [1|128,128,128]
 *     fp8|fp4,     x1Scale/x2Scale e8m0 (.., k/64, 2)                      : microscaling, groupSize [1,1,32]
 *
 * Phase 1 does no device work and may be called without a GPU present. Phase 2 enqueues kernels on `stream`
 * and returns without synchronising; it consumes `executor` (do not reuse or free it afterwards).
 */
#ifndef OPSNN_B200_ACLNN_QUANT_MATMUL_V5_H_
#define OPSNN_B200_ACLNN_QUANT_MATMUL_V5_H_

#include "aclnn_compat/acl_base.h"

#ifdef __cplusplus
extern "C" {
#endif

ACLNN_API aclnnStatus aclnnQuantMatmulV5GetWorkspaceSize(
    const aclTensor* x1, const aclTensor* x2, const aclTensor* x1Scale, const aclTensor* x2Scale,
    const aclTensor* yScale, const aclTensor* x1Offset, const aclTensor* x2Offset, const aclTensor* yOffset,
    const aclTensor* bias, bool transposeX1, bool transposeX2, int64_t groupSize, aclTensor* out,
    uint64_t* workspaceSize, aclOpExecutor** executor);

ACLNN_API aclnnStatus aclnnQuantMatmulV5(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                         aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif
