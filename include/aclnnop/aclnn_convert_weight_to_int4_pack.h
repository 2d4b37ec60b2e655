/* aclnnConvertWeightToINT4Pack: 4-bit weights carried one per 32-bit element -> tightly packed.
 * Prototypes of matmul/convert_weight_to_int4_pack/op_host/op_api/aclnn_convert_weight_to_int4_pack.h:30-45 of the reference.
 *
 * weight INT32 (k, n) or (g, k, n), one int4 value per element -> weightInt4Pack INT4 (same shape) or INT32 (.., n / 8);
 * weight FLOAT, one e2m1-representable value per element      -> weightInt4Pack FLOAT4_E2M1 (same shape) or FLOAT (.., n / 8).
 * Element 2i goes to the low nibble of byte i (op_api .cpp:87-121). Both tensors contiguous, ND. The reference also lays the
 * result out as FRACTAL_NZ on request; that Ascend cube-unit layout is not accepted here (ACLNN_ERR_PARAM_INVALID).
 * The reference packs on the host with two device<->host copies; here a kernel packs on the stream. */
#ifndef OPSNN_ACLNN_CONVERT_WEIGHT_TO_INT4_PACK_H_
#define OPSNN_ACLNN_CONVERT_WEIGHT_TO_INT4_PACK_H_

#include "aclnn_compat/acl_base.h"

#ifdef __cplusplus
extern "C" {
#endif

ACLNN_API aclnnStatus aclnnConvertWeightToINT4PackGetWorkspaceSize(const aclTensor* weight, aclTensor* weightInt4Pack,
                                                                   uint64_t* workspaceSize, aclOpExecutor** executor);
ACLNN_API aclnnStatus aclnnConvertWeightToINT4Pack(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor,
                                                   aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif
