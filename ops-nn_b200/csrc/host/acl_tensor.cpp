// aclTensor / aclOpExecutor lifetime, thread-local error text, small view helpers.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "internal.h"

namespace opsnn {

static thread_local std::string g_last_err;

int log_level()
{
    static int lvl = [] {
        const char* e = std::getenv("OPSNN_LOG_LEVEL");
        return e ? std::atoi(e) : 0;
    }();
    return lvl;
}

void set_err(const char* fmt, ...)
{
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_err = buf;
    if (log_level() >= 1) fprintf(stderr, "[opsnn_b200][E] %s\n", buf);
}

void clear_err() { g_last_err.clear(); }

void log_info(const char* fmt, ...)
{
    if (log_level() < 2) return;
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    fprintf(stderr, "[opsnn_b200][I] %s\n", buf);
}

int dtype_bits(int dt)
{
    switch (dt) {
        case ACL_FLOAT: case ACL_INT32: case ACL_UINT32: return 32;
        case ACL_FLOAT16: case ACL_BF16: case ACL_INT16: case ACL_UINT16: return 16;
        case ACL_INT8: case ACL_UINT8: case ACL_BOOL: case ACL_HIFLOAT8: case ACL_FLOAT8_E5M2:
        case ACL_FLOAT8_E4M3FN: case ACL_FLOAT8_E8M0: return 8;
        case ACL_INT64: case ACL_UINT64: case ACL_DOUBLE: return 64;
        case ACL_INT4: case ACL_FLOAT4_E2M1: case ACL_FLOAT4_E1M2: return 4;
        default: return 0;
    }
}

const char* dtype_name(int dt)
{
    switch (dt) {
        case ACL_FLOAT: return "FLOAT";
        case ACL_FLOAT16: return "FLOAT16";
        case ACL_INT8: return "INT8";
        case ACL_INT32: return "INT32";
        case ACL_UINT8: return "UINT8";
        case ACL_INT64: return "INT64";
        case ACL_UINT64: return "UINT64";
        case ACL_BF16: return "BF16";
        case ACL_INT4: return "INT4";
        case ACL_HIFLOAT8: return "HIFLOAT8";
        case ACL_FLOAT8_E5M2: return "FLOAT8_E5M2";
        case ACL_FLOAT8_E4M3FN: return "FLOAT8_E4M3FN";
        case ACL_FLOAT8_E8M0: return "FLOAT8_E8M0";
        case ACL_FLOAT4_E2M1: return "FLOAT4_E2M1";
        case ACL_FLOAT4_E1M2: return "FLOAT4_E1M2";
        default: return "UNDEFINED";
    }
}

bool is_contiguous(const aclTensor* t)
{
    int64_t expect = 1;
    for (int64_t i = (int64_t)t->rank() - 1; i >= 0; --i) {
        if (t->shape[i] != 1 && t->strides[i] != expect) return false;
        expect *= t->shape[i];
    }
    return true;
}

bool is_transposed_last_two(const aclTensor* t)
{
    int64_t r = (int64_t)t->rank();
    if (r < 2 || r > 6) return false;
    int64_t d1 = t->shape[r - 1], d2 = t->shape[r - 2];
    if (t->strides[r - 2] != 1 || t->strides[r - 1] != d2) return false;
    if (d1 == 1 && d2 == 1) return false;
    int64_t expect = d1 * d2;
    for (int64_t i = r - 3; i >= 0; --i) {
        if (t->strides[i] != expect) return false;
        expect *= t->shape[i];
    }
    return true;
}

bool row_strided_view(const aclTensor* t, int64_t* ld, int64_t* batch_stride)
{
    int64_t r = (int64_t)t->rank();
    if (r < 2) return false;
    int64_t rows = t->shape[r - 2], cols = t->shape[r - 1];
    if (cols != 1 && t->strides[r - 1] != 1) return false;
    int64_t pitch = rows == 1 ? cols : t->strides[r - 2];
    if (pitch < cols) return false;
    *ld = pitch;
    // batch dims must collapse to a single index with one stride (or broadcast / absent)
    int64_t bs = 0;
    int64_t expect = -1;
    for (int64_t i = r - 3; i >= 0; --i) {
        if (t->shape[i] == 1) continue;
        if (expect < 0) {
            bs = t->strides[i];
            expect = t->strides[i] * t->shape[i];
        } else {
            if (t->strides[i] != expect) return false;
            expect *= t->shape[i];
        }
    }
    *batch_stride = bs;
    return true;
}

}  // namespace opsnn

extern "C" {

aclTensor* aclCreateTensor(const int64_t* viewDims, uint64_t viewDimsNum, aclDataType dataType, const int64_t* stride,
                           int64_t offset, aclFormat format, const int64_t* storageDims, uint64_t storageDimsNum,
                           void* tensorData)
{
    if (viewDimsNum > 8 || storageDimsNum > 8 || (viewDimsNum > 0 && viewDims == nullptr)) return nullptr;
    auto* t = new aclTensor();
    t->shape.assign(viewDims, viewDims + viewDimsNum);
    for (auto d : t->shape) {
        if (d < 0) {
            delete t;
            return nullptr;
        }
    }
    if (stride != nullptr) {
        t->strides.assign(stride, stride + viewDimsNum);
    } else {
        t->strides.resize(viewDimsNum);
        int64_t s = 1;
        for (int64_t i = (int64_t)viewDimsNum - 1; i >= 0; --i) {
            t->strides[i] = s;
            s *= t->shape[i];
        }
    }
    if (storageDims != nullptr) t->storage_shape.assign(storageDims, storageDims + storageDimsNum);
    else t->storage_shape = t->shape;
    t->offset = offset;
    t->dtype = dataType;
    t->format = format;
    t->data = tensorData;
    return t;
}

aclnnStatus aclDestroyTensor(const aclTensor* tensor)
{
    delete tensor;
    return ACLNN_SUCCESS;
}

aclnnStatus aclSetRawTensorAddr(aclTensor* tensor, void* tensorData)
{
    if (tensor == nullptr) return ACLNN_ERR_PARAM_NULLPTR;
    tensor->data = tensorData;
    return ACLNN_SUCCESS;
}

aclnnStatus aclDestroyAclOpExecutor(aclOpExecutor* executor)
{
    if (executor == nullptr) return ACLNN_ERR_PARAM_NULLPTR;
    if (executor->magic != 0x4F50534E) return ACLNN_ERR_PARAM_INVALID;
    executor->magic = 0;
    delete executor;
    return ACLNN_SUCCESS;
}

const char* aclGetRecentErrMsg(void) { return opsnn::g_last_err.c_str(); }

}  // extern "C"
