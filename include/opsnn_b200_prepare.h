/*
 * Prepare-once weights for aclnnQuantMatmulV5 (the MX modes) and for the prefill path of aclnnWeightQuantBatchMatmulV2 / V3.
 *
 * A weight (x2) and its scale are static, yet part of every call's time goes into layout work on them that does not depend on
 * the activations: x2Scale is rewritten into the order the tensor core's scale copies want, an MXFP4 x2 stored (k,n) must be
 * rewritten k-contiguous before the tensor core can read it, and an MXFP8 x2 stored (k,n) runs ~20 % slower than one stored
 * (n,k). opsnnQuantMatmulPrepareX2 does that work one time, into memory the caller provides and keeps alive, and registers the
 * result under x2's device address. Every later aclnnQuantMatmulV5 / V4 / V3 call whose x2 and x2Scale are those same tensors
 * (address, shape, strides, dtype, transposeX2, groupSize) then skips it; any other call, and every call after
 * opsnnQuantMatmulReleaseX2, runs exactly as before. Results are bit-identical either way.
 *
 * No counterpart in the reference's aclnn API. Its precedent for offline weight re-layout is aclnnConvertWeightToINT4Pack
 * (matmul/convert_weight_to_int4_pack/op_host/op_api/aclnn_convert_weight_to_int4_pack.cpp:318-358: ND -> FRACTAL_NZ, once,
 * ahead of the matmuls), whose target layout is specific to the Ascend cube unit; this is the same idea for this hardware.
 *
 *   mHint         activation rows per batch of the calls to come: selects the tile width the scale atoms are laid out for. A
 *                 later call whose own m selects another width relays the scales itself and still uses the moved x2.
 *   storage       device memory of at least the size the first function reports; owned by the caller, must outlive the
 *                 registration; the library allocates nothing.
 *   The contents of x2 / x2Scale must not change while registered (the prepared copy would go stale).
 *   Modes with nothing to prepare (everything but MXFP8 x MXFP8 and MXFP4 x MXFP4 on the tensor-core path) report size 0 and
 *   register nothing.
 */
#ifndef OPSNN_B200_PREPARE_H_
#define OPSNN_B200_PREPARE_H_

#include "aclnn_compat/acl_base.h"

#ifdef __cplusplus
extern "C" {
#endif

ACLNN_API aclnnStatus opsnnQuantMatmulPrepareX2GetStorageSize(const aclTensor* x2, const aclTensor* x2Scale, bool transposeX2,
                                                              int64_t groupSize, int64_t mHint, uint64_t* storageSize);
ACLNN_API aclnnStatus opsnnQuantMatmulPrepareX2(const aclTensor* x2, const aclTensor* x2Scale, bool transposeX2, int64_t groupSize,
                                                int64_t mHint, void* storage, uint64_t storageSize, aclrtStream stream);
ACLNN_API aclnnStatus opsnnQuantMatmulReleaseX2(const aclTensor* x2);

/*
 * The same for aclnnWeightQuantBatchMatmulV2 / V3 beyond the decode range (m > 16). There a call first dequantises the whole
 * weight into 16-bit workspace (k x n x 2 bytes: 470 MB for the benchmark's decode weight) and then runs the tensor-core
 * matmul; the first step does not depend on the activations. opsnnWeightQuantPrepare runs it once into caller memory and
 * registers the image under the weight's device address; later calls with the same weight, antiquantScale, antiquantOffset,
 * antiquantGroupSize and x dtype and m > 16 skip the pre-pass and ask for no workspace (bit-identical results). Calls with
 * m <= 16 keep streaming the packed weight. The price is memory: the image is four (int4) or two (int8 / fp8) times the packed
 * weight, which is why this is the caller's choice. Weights with no prefill path report size 0 and register nothing.
 *
 *   xDtype   ACL_BF16 or ACL_FLOAT16: the dtype of the activations of the calls to come (the reference rounds the dequantised
 *            weight to it, so the image depends on it).
 */
ACLNN_API aclnnStatus opsnnWeightQuantPrepareGetStorageSize(const aclTensor* weight, const aclTensor* antiquantScale,
                                                            const aclTensor* antiquantOffset, int antiquantGroupSize, aclDataType xDtype,
                                                            uint64_t* storageSize);
ACLNN_API aclnnStatus opsnnWeightQuantPrepare(const aclTensor* weight, const aclTensor* antiquantScale, const aclTensor* antiquantOffset,
                                              int antiquantGroupSize, aclDataType xDtype, void* storage, uint64_t storageSize,
                                              aclrtStream stream);
ACLNN_API aclnnStatus opsnnWeightQuantRelease(const aclTensor* weight);

#ifdef __cplusplus
}
#endif
#endif /* OPSNN_B200_PREPARE_H_ */
