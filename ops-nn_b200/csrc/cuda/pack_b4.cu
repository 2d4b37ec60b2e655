// 4-bit weight packing (aclnnConvertWeightToINT4Pack): one value per 32-bit element -> two per byte, low nibble first.
// Arithmetic of matmul/convert_weight_to_int4_pack/op_host/op_api/aclnn_convert_weight_to_int4_pack.cpp:43-121 of the
// reference: INT32 keeps the low 4 bits; FLOAT keeps sign, exponent and the top mantissa bit (mask 0xFFC00000) and maps the
// sixteen e2m1 values to their codes, anything else to code 0. HBM bound: 32 bytes in, 4 bytes out per thread.
#include "common.cuh"

namespace opsnn {

namespace {

__device__ __forceinline__ uint32_t fp32_to_e2m1_code(uint32_t bits)
{
    bits &= 0xFFC00000u;
    const uint32_t sign = (bits >> 31) << 3, mag = bits & 0x7FFFFFFFu;
    uint32_t code;
    switch (mag) {
        case 0x00000000u: code = 0; break;
        case 0x3F000000u: code = 1; break;  // 0.5
        case 0x3F800000u: code = 2; break;  // 1
        case 0x3FC00000u: code = 3; break;  // 1.5
        case 0x40000000u: code = 4; break;  // 2
        case 0x40400000u: code = 5; break;  // 3
        case 0x40800000u: code = 6; break;  // 4
        case 0x40C00000u: code = 7; break;  // 6
        default: return 0u;                 // not an e2m1 value: code 0, sign dropped, as the reference's table lookup does
    }
    return code | sign;
}

template <bool kFloat>
__global__ void __launch_bounds__(256) pack_b4_kernel(const uint32_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t count)
{
    const int64_t words = count / 8;  // full output words (8 elements each)
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += (int64_t)gridDim.x * blockDim.x) {
        const uint4 a = __ldcs(reinterpret_cast<const uint4*>(src) + 2 * i), b = __ldcs(reinterpret_cast<const uint4*>(src) + 2 * i + 1);
        const uint32_t v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        uint32_t out = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) out |= ((kFloat ? fp32_to_e2m1_code(v[j]) : v[j]) & 0xFu) << (4 * j);
        reinterpret_cast<uint32_t*>(dst)[i] = out;
    }
    // tail: count % 8 elements (count is even), one byte per thread of block 0
    if (blockIdx.x == 0) {
        for (int64_t e = words * 8 + 2 * threadIdx.x; e + 1 < count; e += 2 * blockDim.x) {
            const uint32_t lo = kFloat ? fp32_to_e2m1_code(src[e]) : src[e], hi = kFloat ? fp32_to_e2m1_code(src[e + 1]) : src[e + 1];
            dst[e / 2] = (uint8_t)((lo & 0xFu) | ((hi & 0xFu) << 4));
        }
    }
}

}  // namespace

int32_t pack_b4_launch(const OpsnnPackB4Params* p, cudaStream_t stream)
{
    if (p->count <= 0) return 0;
    if (p->count % 2 != 0 || (reinterpret_cast<uintptr_t>(p->src) & 15) != 0 || (reinterpret_cast<uintptr_t>(p->dst) & 3) != 0)
        return (int32_t)cudaErrorInvalidValue;
    int64_t grid = (p->count / 8 + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    if (grid < 1) grid = 1;
    if (p->src_dtype == ACL_FLOAT)
        pack_b4_kernel<true><<<(unsigned)grid, 256, 0, stream>>>(static_cast<const uint32_t*>(p->src), static_cast<uint8_t*>(p->dst), p->count);
    else
        pack_b4_kernel<false><<<(unsigned)grid, 256, 0, stream>>>(static_cast<const uint32_t*>(p->src), static_cast<uint8_t*>(p->dst), p->count);
    note_launch("pack_b4");
    return (int32_t)cudaGetLastError();
}

}  // namespace opsnn
