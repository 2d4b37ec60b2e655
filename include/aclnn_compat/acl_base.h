/*
 * Minimal ACL object model for the aclnn two-phase operator API, for hosts that have CUDA instead of
 * the CANN runtime.
 *
 * The reference library (hicann/ops-nn) compiles against CANN's `acl/acl.h` and `aclnn/aclnn_base.h`,
 * which are not part of its source tree. This header re-declares exactly the subset its quantized-matmul
 * entry points use, with the same names, argument order, enum values and status codes, so that caller code
 * written for the reference (see e.g. its examples/test_aclnn_quant_matmul_v5_perblock.cpp:64-86, 215-234)
 * compiles unchanged against this library:
 *
 *   - aclTensor      : opaque tensor *descriptor* (view shape, strides, offset, storage shape, format, dtype,
 *                      device pointer). The library never owns tensor memory.
 *   - aclOpExecutor  : opaque plan created by a `...GetWorkspaceSize` call (phase 1) and consumed by exactly one
 *                      execute call (phase 2). docs/zh/context/two_phase_api.md:14-24 of the reference.
 *   - aclrtStream    : a `cudaStream_t` passed as `void*`.
 *   - aclnnStatus    : docs/zh/context/aclnn_return_code.md of the reference.
 *
 * All functions are `extern "C"` with default visibility; no C++ or torch type crosses this boundary.
 */
#ifndef OPSNN_B200_ACL_BASE_H_
#define OPSNN_B200_ACL_BASE_H_

#include <stddef.h>
#include <stdint.h>
#ifndef __cplusplus
#include <stdbool.h>
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define ACLNN_API __attribute__((visibility("default")))

typedef int32_t aclnnStatus;

/* docs/zh/context/aclnn_return_code.md */
#define ACLNN_SUCCESS 0
#define ACLNN_ERR_PARAM_NULLPTR 161001
#define ACLNN_ERR_PARAM_INVALID 161002
#define ACLNN_ERR_RUNTIME_ERROR 361001
#define ACLNN_ERR_INNER 561000
#define ACLNN_ERR_INNER_INFERSHAPE_ERROR 561001
#define ACLNN_ERR_INNER_TILING_ERROR 561002
#define ACLNN_ERR_INNER_FIND_KERNEL_ERROR 561003
#define ACLNN_ERR_INNER_CREATE_EXECUTOR 561101
#define ACLNN_ERR_INNER_NOT_TRANS_EXECUTOR 561102
#define ACLNN_ERR_INNER_NULLPTR 561103

/* Numeric values follow CANN's aclDataType (the reference's goldens spell the same numbers out:
 * quant/dynamic_mx_quant/tests/assets/golden.py:22-58). */
typedef enum {
    ACL_DT_UNDEFINED = -1,
    ACL_FLOAT = 0,
    ACL_FLOAT16 = 1,
    ACL_INT8 = 2,
    ACL_INT32 = 3,
    ACL_UINT8 = 4,
    ACL_INT16 = 6,
    ACL_UINT16 = 7,
    ACL_UINT32 = 8,
    ACL_INT64 = 9,
    ACL_UINT64 = 10,
    ACL_DOUBLE = 11,
    ACL_BOOL = 12,
    ACL_BF16 = 27,
    ACL_INT4 = 29,
    ACL_HIFLOAT8 = 34,
    ACL_FLOAT8_E5M2 = 35,
    ACL_FLOAT8_E4M3FN = 36,
    ACL_FLOAT8_E8M0 = 37,
    ACL_FLOAT6_E3M2 = 38,
    ACL_FLOAT6_E2M3 = 39,
    ACL_FLOAT4_E2M1 = 40,
    ACL_FLOAT4_E1M2 = 41
} aclDataType;

typedef enum {
    ACL_FORMAT_UNDEFINED = -1,
    ACL_FORMAT_NCHW = 0,
    ACL_FORMAT_NHWC = 1,
    ACL_FORMAT_ND = 2,
    ACL_FORMAT_NC1HWC0 = 3,
    ACL_FORMAT_FRACTAL_Z = 4,
    ACL_FORMAT_FRACTAL_NZ = 29,
    ACL_FORMAT_FRACTAL_NZ_C0_32 = 52
} aclFormat;

typedef struct aclTensor aclTensor;
typedef struct aclOpExecutor aclOpExecutor;
typedef void* aclrtStream;

/*
 * Creates a tensor descriptor. `stride` may be NULL (dense row-major strides are derived from `viewDims`);
 * `offset` is in elements; `tensorData` is a device pointer (may be NULL for phase-1-only use, as the
 * reference's own op_api unit tests do). Returns NULL on invalid arguments (more than 8 dims, negative dim).
 */
ACLNN_API aclTensor* aclCreateTensor(const int64_t* viewDims, uint64_t viewDimsNum, aclDataType dataType,
                                     const int64_t* stride, int64_t offset, aclFormat format,
                                     const int64_t* storageDims, uint64_t storageDimsNum, void* tensorData);
ACLNN_API aclnnStatus aclDestroyTensor(const aclTensor* tensor);

/* Re-points an existing descriptor at other device memory (same shape/dtype); CANN spells this
 * aclSetRawTensorAddr / aclSetInputTensorAddr on an executor, which needs state this library does not keep. */
ACLNN_API aclnnStatus aclSetRawTensorAddr(aclTensor* tensor, void* tensorData);

/* Destroys an executor that will not be run (phase 2 frees it itself). */
ACLNN_API aclnnStatus aclDestroyAclOpExecutor(aclOpExecutor* executor);

/* Text of the most recent failure on the calling thread ("" if none). */
ACLNN_API const char* aclGetRecentErrMsg(void);

#ifdef __cplusplus
}
#endif
#endif /* OPSNN_B200_ACL_BASE_H_ */
