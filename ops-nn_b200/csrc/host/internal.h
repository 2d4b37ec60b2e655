// Host-side object model shared by the aclnn entry points: tensor descriptor, executor (plan), error text.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <string>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "aclnn_compat/acl_base.h"
#include "opsnn_b200_kernels.h"

// An NVTX range around each phase of every entry point (the reference brackets its entry points with L2_DFX_PHASE_1 / _2,
// aclnn_quant_matmul_v5.cpp:1196, :1225): shows up in a timeline tool when one is attached, costs a null check otherwise.
namespace opsnn {
struct DfxRange {
    explicit DfxRange(const char* name) { nvtxRangePushA(name); }
    ~DfxRange() { nvtxRangePop(); }
    DfxRange(const DfxRange&) = delete;
    DfxRange& operator=(const DfxRange&) = delete;
};
}  // namespace opsnn
#define OPSNN_DFX_RANGE(name) ::opsnn::DfxRange opsnn_dfx_range_(name)


// Tensor descriptor. Mirrors what the reference's aclTensor carries (docs/zh/context/non_contiguous_tensor.md of
// the reference): view shape, strides and offset in elements, storage shape, format, dtype, device address.
struct aclTensor {
    std::vector<int64_t> shape;
    std::vector<int64_t> strides;
    std::vector<int64_t> storage_shape;
    int64_t offset = 0;
    aclDataType dtype = ACL_FLOAT;
    aclFormat format = ACL_FORMAT_ND;
    void* data = nullptr;

    size_t rank() const { return shape.size(); }
    int64_t dim(int64_t i) const { return shape[i < 0 ? (int64_t)shape.size() + i : i]; }
    int64_t numel() const
    {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
    bool empty() const { return numel() == 0; }
};

enum class ExecKind : int { kNone = 0, kQmm = 1, kWqbmm = 2, kMxQuant = 3, kPackB4 = 4 };

// Plan produced by phase 1 and consumed by phase 2.
struct aclOpExecutor {
    uint32_t magic = 0x4F50534E;  // "OPSN"
    ExecKind kind = ExecKind::kNone;
    bool nothing_to_do = false;   // empty output: phase 2 returns success without launching
    bool unsupported = false;     // arguments are valid for the reference but no kernel exists here
    std::string unsupported_why;
    int32_t kernel_choice = 0;
    uint64_t workspace_size = 0;
    OpsnnQmmParams qmm{};
    OpsnnWqbmmParams wq{};
    OpsnnMxQuantParams mxq{};
    OpsnnPackB4Params pack{};
    // aclnnQuantMatmulWeightNz: x2 arrives FRACTAL_NZ and is rewritten row-major into the head of the workspace before the matmul
    const void* nz_src = nullptr;
    int64_t nz_rows = 0, nz_row_bytes = 0, nz_r0 = 0, nz_c0_bytes = 0;
    uint64_t nz_bytes = 0;
    // aclnnQuantMatmulV5 with a BF16 / FLOAT16 x1 and no x1Scale in the MX modes: x1 is quantised first (aclnnDynamicMxQuant's
    // arithmetic, `mxq`) into the head of the workspace: dq_q_bytes of payload, then dq_s_bytes of e8m0 scales
    bool dyn_quant = false;
    uint64_t dq_q_bytes = 0, dq_s_bytes = 0;
};

namespace opsnn {

// Records the text returned by aclGetRecentErrMsg() for the calling thread and, when OPSNN_LOG_LEVEL >= 1,
// prints it to stderr.
void set_err(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
void clear_err();
int log_level();
void log_info(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

// Bits per element of an aclDataType (4 for int4/fp4, 0 if unknown).
int dtype_bits(int dt);
const char* dtype_name(int dt);

// Dense row-major check over the view shape.
bool is_contiguous(const aclTensor* t);
// "Transposed view" rule of the reference (matmul/common/op_host/op_api/matmul_util.cpp:2040-2064): rank 2..6,
// stride[-2] == 1, stride[-1] == shape[-2], batch strides dense over that, and not the 1x1 case.
bool is_transposed_last_two(const aclTensor* t);
// Inner stride 1, any row pitch >= inner extent, batch dims dense over (rows * pitch) or broadcast... returns the
// row pitch and the batch stride (elements) of a view whose leading dims collapse to one batch index.
bool row_strided_view(const aclTensor* t, int64_t* ld, int64_t* batch_stride);

inline const uint8_t* data_ptr(const aclTensor* t)
{
    if (t == nullptr || t->data == nullptr) return nullptr;
    int bits = dtype_bits(t->dtype);
    return static_cast<const uint8_t*>(t->data) + (t->offset * bits) / 8;
}

inline int64_t ceil_div(int64_t a, int64_t b) { return b == 0 ? 0 : (a + b - 1) / b; }

}  // namespace opsnn
