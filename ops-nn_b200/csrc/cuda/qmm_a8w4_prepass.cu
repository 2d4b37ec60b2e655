// A8W4 (fp8 activations x fp4 weights) of aclnnQuantMatmulV5: the fp4 operand is rewritten as fp8 once per call, into the
// head of the workspace, and the fp8 tensor-core kernels run on the result.
//
//   WIDEN        mx mode (matmul/quant_batch_matmul_v4/tests/assets/qbmmv4_kernel_golden.py:119-186): x2 and its e8m0
//                scales are widened to fp32 and multiplied, so storing every e2m1 value as the same value in e4m3 (all
//                eight magnitudes are e4m3 numbers) changes nothing; the block-scaled MMA applies the scales.
//   GROUP_SCALE  T-CG mode (same file :189-255): w' = a_dtype( mid( mid(w) * mid(scale[n, k/32]) ) ), mid = the scale's
//                dtype (bf16 or fp16). mid(w) is exact, the product of two bf16/fp16 numbers is exact in fp32, so the
//                kernel rounds that fp32 product once to mid and once more to fp8 - the golden's two roundings. The fp8
//                cast does not saturate (a value beyond the largest finite number becomes NaN / inf, as in the golden).
//
// Purely HBM bound: 0.5 byte in, 1 byte out per weight. One thread expands 8 weights (4 bytes -> 8 bytes).
#include "common.cuh"

namespace opsnn {

namespace {

// four e2m1 codes (low 16 bits of `h`, low nibble first) -> four e4m3 bytes
__device__ __forceinline__ uint32_t widen4(uint32_t h)
{
    // e4m3 of the magnitudes 0, .5, 1, 1.5 | 2, 3, 4, 6
    const uint32_t codes = __byte_perm(0x3C383000u, 0x4C484440u, h & 0x7777u);
    uint32_t y = (h & 0x00FFu) | ((h & 0xFF00u) << 8);
    y = (y | (y << 4)) & 0x0F0F0F0Fu;  // one nibble per byte
    return codes | ((y & 0x08080808u) << 4);
}

__device__ __forceinline__ float e2m1_value(uint32_t code)
{
    const uint32_t mag = code & 7u;
    // 0, .5, 1, 1.5, 2, 3, 4, 6
    const float v = mag == 0 ? 0.f : (mag == 1 ? 0.5f : __uint_as_float((126u + (mag >> 1)) << 23 | (mag & 1u) << 22));
    return (code & 8u) ? -v : v;
}

__device__ __forceinline__ float round_mid(float p, int mid_dtype)
{
    if (mid_dtype == ACL_BF16) return __bfloat162float(__float2bfloat16_rn(p));
    return __half2float(__float2half_rn(p));
}

__device__ __forceinline__ uint8_t to_fp8_nosat(float v, int dtype)
{
    return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_NOSAT, dtype == ACL_FLOAT8_E5M2 ? __NV_E5M2 : __NV_E4M3);
}

// rows x inner elements; src rows are src_ld elements apart (two per byte), dst rows are packed (inner bytes)
__global__ void __launch_bounds__(256) a8w4_widen_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows,
                                                         int64_t inner, int64_t src_ld, int vec)
{
    if (vec) {
        const int64_t per_row = inner / 8, total = rows * per_row;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
            const int64_t r = i / per_row, c = i % per_row;
            const uint32_t w = __ldcs(reinterpret_cast<const uint32_t*>(src + (r * src_ld) / 2) + c);
            reinterpret_cast<uint2*>(dst + r * inner)[c] = make_uint2(widen4(w & 0xFFFFu), widen4(w >> 16));
        }
    } else {
        const int64_t per_row = inner / 2, total = rows * per_row;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
            const int64_t r = i / per_row, c = i % per_row;
            const uint32_t w = widen4(src[(r * src_ld) / 2 + c]);
            dst[r * inner + 2 * c] = (uint8_t)w;
            dst[r * inner + 2 * c + 1] = (uint8_t)(w >> 8);
        }
    }
}

// kInnerK: b stored (n,k), scale (n, k/group); otherwise b stored (k,n), scale (k/group, n)
template <bool kInnerK>
__global__ void __launch_bounds__(256) a8w4_group_scale_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows,
                                                               int64_t inner, int64_t src_ld, const uint16_t* __restrict__ scale,
                                                               int scale_dtype, int group, int out_dtype)
{
    const int64_t per_row = inner / 2, total = rows * per_row;
    const int64_t scale_row = kInnerK ? (inner + group - 1) / group : inner;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / per_row, c = i % per_row;
        const uint32_t byte = src[(r * src_ld) / 2 + c];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int64_t col = 2 * c + h;
            const int64_t si = kInnerK ? r * scale_row + col / group : (r / group) * scale_row + col;
            const uint16_t sb = scale[si];
            const float s = scale_dtype == ACL_BF16 ? __uint_as_float((uint32_t)sb << 16) : __half2float(__ushort_as_half(sb));
            const float mid = round_mid(e2m1_value((byte >> (4 * h)) & 15u) * s, scale_dtype);
            dst[r * inner + col] = to_fp8_nosat(mid, out_dtype);
        }
    }
}

// INT4 -> INT8, sign extended: rows x inner nibbles (two per byte, low first), src rows src_ld nibbles apart, dst packed
__global__ void __launch_bounds__(256) widen_int4_kernel(const uint8_t* __restrict__ src, int8_t* __restrict__ dst, int64_t rows,
                                                         int64_t inner, int64_t src_ld)
{
    const int64_t per_row = inner / 2, total = rows * per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / per_row, c = i % per_row;
        const int32_t byte = src[(r * src_ld) / 2 + c];
        *reinterpret_cast<char2*>(dst + r * inner + 2 * c) = make_char2((signed char)((byte << 28) >> 28), (signed char)((byte << 24) >> 28));
    }
}

}  // namespace

// ---- INT4 x INT4: both operands widened to INT8 -------------------------------------------------------------------------
static int64_t int4_rows(const OpsnnQmmParams* p, bool is_a) { return is_a ? (p->trans_a ? p->k : p->m) : (p->trans_b ? p->n : p->k); }
static int64_t int4_inner(const OpsnnQmmParams* p, bool is_a) { return is_a ? (p->trans_a ? p->m : p->k) : (p->trans_b ? p->k : p->n); }
static uint64_t int4_bytes_one(const OpsnnQmmParams* p, bool is_a)
{
    const int64_t nb = (is_a ? p->a_bs : p->b_bs) != 0 ? p->batch : 1;
    return ((uint64_t)(nb * int4_rows(p, is_a) * int4_inner(p, is_a)) + 255u) & ~(uint64_t)255u;
}

uint64_t qmm_int4_prepass_bytes(const OpsnnQmmParams* p)
{
    uint64_t n = 0;
    if (p->a_prepass == OPSNN_PREPASS_WIDEN_INT4) n += int4_bytes_one(p, true);
    if (p->b_prepass == OPSNN_PREPASS_WIDEN_INT4) n += int4_bytes_one(p, false);
    return n;
}

// Parameters of the INT8 problem the widening leaves behind (operands packed at `dst`).
void qmm_int4_view(const OpsnnQmmParams* p, OpsnnQmmParams* q, void* dst)
{
    *q = *p;
    uint8_t* at = static_cast<uint8_t*>(dst);
    uint64_t used = 0;
    if (p->a_prepass == OPSNN_PREPASS_WIDEN_INT4) {
        q->a = dst == nullptr ? nullptr : at;
        q->a_dtype = ACL_INT8;
        q->a_ld = int4_inner(p, true);
        q->a_bs = p->a_bs != 0 ? int4_rows(p, true) * int4_inner(p, true) : 0;
        used += int4_bytes_one(p, true);
        q->a_prepass = OPSNN_B_PREPASS_NONE;
    }
    if (p->b_prepass == OPSNN_PREPASS_WIDEN_INT4) {
        q->b = dst == nullptr ? nullptr : at + used;
        q->b_dtype = ACL_INT8;
        q->b_ld = int4_inner(p, false);
        q->b_bs = p->b_bs != 0 ? int4_rows(p, false) * int4_inner(p, false) : 0;
        used += int4_bytes_one(p, false);
        q->b_prepass = OPSNN_B_PREPASS_NONE;
    }
    q->workspace = dst == nullptr ? nullptr : at + used;
    q->workspace_size = p->workspace_size > used ? p->workspace_size - used : 0;
}

int32_t qmm_int4_prepass_launch(const OpsnnQmmParams* p, void* dst, cudaStream_t stream)
{
    uint8_t* at = static_cast<uint8_t*>(dst);
    for (int side = 0; side < 2; ++side) {
        const bool is_a = side == 0;
        if ((is_a ? p->a_prepass : p->b_prepass) != OPSNN_PREPASS_WIDEN_INT4) continue;
        const int64_t rows1 = int4_rows(p, is_a), inner = int4_inner(p, is_a);
        const int64_t ld = is_a ? p->a_ld : p->b_ld, bs = is_a ? p->a_bs : p->b_bs;
        const int64_t nb = bs != 0 ? p->batch : 1;
        if (inner % 2 != 0 || ld % 2 != 0 || bs % 2 != 0) return (int32_t)cudaErrorInvalidValue;
        const uint8_t* src = static_cast<const uint8_t*>(is_a ? p->a : p->b);
        for (int64_t b = 0; b < nb; ++b) {
            int64_t grid = (rows1 * inner / 2 + 255) / 256;
            if (grid > 148 * 16) grid = 148 * 16;
            if (grid < 1) grid = 1;
            widen_int4_kernel<<<(unsigned)grid, 256, 0, stream>>>(src + (b * bs) / 2, reinterpret_cast<int8_t*>(at) + b * rows1 * inner, rows1,
                                                                   inner, ld);
            note_launch("widen_int4");
            const cudaError_t e = cudaGetLastError();
            if (e != cudaSuccess) return (int32_t)e;
        }
        at += int4_bytes_one(p, is_a);
    }
    return 0;
}

uint64_t qmm_a8w4_prepass_bytes(const OpsnnQmmParams* p)
{
    if (p->b_prepass != OPSNN_B_PREPASS_WIDEN && p->b_prepass != OPSNN_B_PREPASS_GROUP_SCALE) return 0;
    const int64_t rows = p->trans_b ? p->n : p->k, inner = p->trans_b ? p->k : p->n;
    const int64_t nb = p->b_bs != 0 ? p->batch : 1;
    return ((uint64_t)(nb * rows * inner) + 255u) & ~(uint64_t)255u;
}

// Fills `q` with the parameters the matmul sees after the pre-pass: b is fp8 at `dst`, rows packed.
void qmm_a8w4_view(const OpsnnQmmParams* p, OpsnnQmmParams* q, void* dst)
{
    *q = *p;
    const int64_t rows = p->trans_b ? p->n : p->k, inner = p->trans_b ? p->k : p->n;
    q->b = dst;
    q->b_dtype = p->b_prepass == OPSNN_B_PREPASS_WIDEN ? (int32_t)ACL_FLOAT8_E4M3FN : p->a_dtype;
    q->b_ld = inner;
    q->b_bs = p->b_bs != 0 ? rows * inner : 0;
    q->b_prepass = OPSNN_B_PREPASS_NONE;
    q->pre_scale = nullptr;
    const uint64_t used = qmm_a8w4_prepass_bytes(p);
    q->workspace = dst == nullptr ? nullptr : static_cast<uint8_t*>(dst) + used;
    q->workspace_size = p->workspace_size > used ? p->workspace_size - used : 0;
}

int32_t qmm_a8w4_prepass_launch(const OpsnnQmmParams* p, void* dst, cudaStream_t stream)
{
    if (p->b_dtype != ACL_FLOAT4_E2M1) return (int32_t)cudaErrorInvalidValue;
    const int64_t rows1 = p->trans_b ? p->n : p->k, inner = p->trans_b ? p->k : p->n;
    if (inner % 2 != 0 || p->b_ld % 2 != 0) return (int32_t)cudaErrorInvalidValue;
    const int64_t nb = p->b_bs != 0 ? p->batch : 1;
    const uint8_t* src = static_cast<const uint8_t*>(p->b);
    uint8_t* out = static_cast<uint8_t*>(dst);
    // batches: contiguous ones are folded into the row count, anything else goes batch by batch
    const bool folded = nb == 1 || p->b_bs == rows1 * p->b_ld;
    const int64_t launches = folded ? 1 : nb, rows = folded ? nb * rows1 : rows1;
    for (int64_t b = 0; b < launches; ++b) {
        const uint8_t* s = src + (b * p->b_bs) / 2;
        uint8_t* d = out + b * rows1 * inner;
        const int64_t work = rows * inner / 8;
        int64_t grid = (work + 255) / 256;
        if (grid > 148 * 16) grid = 148 * 16;
        if (grid < 1) grid = 1;
        if (p->b_prepass == OPSNN_B_PREPASS_WIDEN) {
            const int vec = inner % 8 == 0 && p->b_ld % 8 == 0 && (reinterpret_cast<uintptr_t>(s) & 3) == 0 &&
                            (reinterpret_cast<uintptr_t>(d) & 7) == 0;
            a8w4_widen_kernel<<<(unsigned)grid, 256, 0, stream>>>(s, d, rows, inner, p->b_ld, vec);
        } else {
            if (p->pre_scale == nullptr || p->pre_group <= 0 || launches != 1 || nb != 1) return (int32_t)cudaErrorInvalidValue;
            const uint16_t* sc = static_cast<const uint16_t*>(p->pre_scale);
            if (p->trans_b)
                a8w4_group_scale_kernel<true><<<(unsigned)grid, 256, 0, stream>>>(s, d, rows, inner, p->b_ld, sc, p->pre_scale_dtype,
                                                                                 p->pre_group, p->a_dtype);
            else
                a8w4_group_scale_kernel<false><<<(unsigned)grid, 256, 0, stream>>>(s, d, rows, inner, p->b_ld, sc, p->pre_scale_dtype,
                                                                                  p->pre_group, p->a_dtype);
        }
        note_launch("qmm_a8w4_prepass");
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int32_t)e;
    }
    return 0;
}

}  // namespace opsnn
