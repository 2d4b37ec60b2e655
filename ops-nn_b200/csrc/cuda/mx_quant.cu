// Dynamic microscaling quantisation (aclnnDynamicMxQuant): bf16/fp16 -> fp8 (e4m3/e5m2) or fp4 (e2m1) with one e8m0
// shared exponent per 32 elements of the last axis.
//
// Arithmetic of the reference's golden (quant/dynamic_mx_quant/tests/assets/golden.py:141-154 shared exponent,
// :197-217 element quantisation, :272-336 _mx_quantize, scale_alg 0 = OCP):
//   amax = max|x| over the block (a short tail block is zero padded)
//   e    = floor(log2(amax)) - emax(dst)            emax: e2m1 2, e4m3 8, e5m2 15;  amax == 0 -> e = -127
//   e    clamped to [-127, 127]; stored as e8m0 byte e + 127
//   q    = saturate( round_to_nearest_even( x / 2^e ) ) in the destination format
//   the scale row is padded to an even count with byte 0 (2^-127) and shaped (.., ceil(k/64), 2)
// One thread per 32-block: 64 bytes in, 32 (or 16) bytes + 1 scale byte out; purely HBM bound.
#include "common.cuh"

namespace opsnn {

namespace {

__device__ __forceinline__ uint8_t quant_fp4_e2m1(float r)
{
    // RNE onto {0, .5, 1, 1.5, 2, 3, 4, 6}, saturating; ties go to the even mantissa
    const float a = fabsf(r);
    uint8_t code;
    if (a <= 0.25f) code = 0;
    else if (a < 0.75f) code = 1;
    else if (a <= 1.25f) code = 2;
    else if (a < 1.75f) code = 3;
    else if (a <= 2.5f) code = 4;
    else if (a < 3.5f) code = 5;
    else if (a <= 5.0f) code = 6;
    else code = 7;
    if (a != a) code = 7;
    return (r < 0.f || (r == 0.f && signbit(r))) ? (code | 8) : code;
}

template <bool kBf16>
__global__ void __launch_bounds__(256) mx_quant_kernel(const OpsnnMxQuantParams p, int64_t blocks_per_row,
                                                       int64_t scale_row)
{
    const int64_t total = p.rows * scale_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / scale_row, blk = i % scale_row;
        uint8_t* sc = reinterpret_cast<uint8_t*>(p.scale) + row * scale_row + blk;
        if (blk >= blocks_per_row) {  // padding entry that makes the count even
            *sc = 0;
            continue;
        }
        const int64_t k0 = blk * 32;
        const int cnt = (int)min((int64_t)32, p.k - k0);
        float v[32];
        const uint16_t* src = reinterpret_cast<const uint16_t*>(p.x) + row * p.k + k0;
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            float f = 0.f;
            if (j < cnt) {
                if (kBf16) f = __uint_as_float((uint32_t)src[j] << 16);
                else f = __half2float(reinterpret_cast<const __half*>(src)[j]);
            }
            v[j] = f;
            amax = fmaxf(amax, fabsf(f));
        }
        const int emax = p.y_dtype == ACL_FLOAT4_E2M1 ? 2 : (p.y_dtype == ACL_FLOAT8_E4M3FN ? 8 : 15);
        int e;
        if (amax == 0.f || !(amax == amax)) {
            e = -127;
        } else {
            // floor(log2(amax)) from the exponent field (subnormal inputs handled through frexp)
            int ex;
            frexpf(amax, &ex);  // amax = f * 2^ex, f in [0.5, 1)
            e = (ex - 1) - emax;
        }
        if (isinf(amax)) e = 128;
        e = max(-127, e);
        const uint8_t byte = e > 127 ? 255 : (uint8_t)(e + 127);
        *sc = byte;
        const float inv = e > 127 ? __uint_as_float(0x7FC00000u) : ldexpf(1.f, -e);  // exact power of two
        if (p.y_dtype == ACL_FLOAT4_E2M1) {
            uint8_t* dst = reinterpret_cast<uint8_t*>(p.y) + (row * p.k + k0) / 2;
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                if (j < cnt) {
                    uint8_t lo = quant_fp4_e2m1(v[j] * inv);
                    uint8_t hi = (j + 1 < cnt) ? quant_fp4_e2m1(v[j + 1] * inv) : 0;
                    dst[j / 2] = lo | (hi << 4);
                }
            }
        } else {
            uint8_t* dst = reinterpret_cast<uint8_t*>(p.y) + row * p.k + k0;
            const __nv_fp8_interpretation_t kind = p.y_dtype == ACL_FLOAT8_E4M3FN ? __NV_E4M3 : __NV_E5M2;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < cnt) dst[j] = (uint8_t)__nv_cvt_float_to_fp8(v[j] * inv, __NV_SATFINITE, kind);
        }
    }
}

}  // namespace

int32_t mx_quant_launch(const OpsnnMxQuantParams* p, cudaStream_t stream)
{
    const int64_t blocks_per_row = (p->k + 31) / 32;
    const int64_t scale_row = ((blocks_per_row + 1) / 2) * 2;
    const int64_t total = p->rows * scale_row;
    if (total == 0) return 0;
    int64_t grid = (total + 255) / 256;
    if (grid > 148 * 32) grid = 148 * 32;
    if (p->x_dtype == ACL_BF16) mx_quant_kernel<true><<<(unsigned)grid, 256, 0, stream>>>(*p, blocks_per_row, scale_row);
    else mx_quant_kernel<false><<<(unsigned)grid, 256, 0, stream>>>(*p, blocks_per_row, scale_row);
    note_launch("mx_quant");
    return (int32_t)cudaGetLastError();
}

}  // namespace opsnn
