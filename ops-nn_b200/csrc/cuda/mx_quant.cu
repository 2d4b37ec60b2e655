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
// Purely HBM bound. Rows whose length is a multiple of 32 (16-byte aligned) take the streaming kernel: four lanes share a
// 32-block, each moving 16 bytes in and 8 (4) bytes out, the block maximum combined with two shuffles; anything ragged
// takes the one-thread-per-block kernel.
#include <cstdlib>

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

// scale_alg 1: exponent of amax / max_norm, one more unless that quotient is a power of two (golden.py:157-177)
__device__ __forceinline__ int mx_shared_exp_up(float amax, float max_norm)
{
    if (amax == 0.f || !(amax == amax)) return -127;
    if (isinf(amax)) return 128;
    const uint32_t bits = __float_as_uint(__fdiv_rn(amax, max_norm));
    int ex = (int)((bits >> 23) & 0xFFu);
    const uint32_t mant = bits & 0x7FFFFFu;
    if ((ex > 0 && ex < 254 && mant > 0u) || (ex == 0 && mant > (1u << 22))) ++ex;
    return max(-127, ex - 127);
}

__device__ __forceinline__ int mx_shared_exp(float amax, int emax)
{
    int e;
    if (amax == 0.f || !(amax == amax)) {
        e = -127;
    } else {
        const int field = (int)((__float_as_uint(amax) >> 23) & 0xFFu);
        if (field != 0) {
            e = field - 127 - emax;  // floor(log2(amax)) of a normal float is its exponent
        } else {
            int ex;
            frexpf(amax, &ex);
            e = (ex - 1) - emax;
        }
    }
    if (isinf(amax)) e = 128;
    return max(-127, e);
}

__device__ __forceinline__ int mx_block_exp(float amax, const OpsnnMxQuantParams& p, int emax)
{
    if (p.scale_alg == 1 && p.y_dtype != ACL_FLOAT4_E2M1) return mx_shared_exp_up(amax, p.y_dtype == ACL_FLOAT8_E4M3FN ? 448.f : 57344.f);
    return mx_shared_exp(amax, emax);
}

// e2m1 with the golden's other rounding modes (golden.py:180-217): the value is scaled to its mantissa grid (0.5 below 2, 1 below
// 4, 2 above), rounded there (1: half away from zero, 2: floor of the signed value), clipped to +-6; the result is an e2m1 value.
__device__ __forceinline__ uint8_t quant_fp4_e2m1_mode(float r, int mode)
{
    if (mode == 0) return quant_fp4_e2m1(r);
    const float a = fabsf(r);
    const float step = a < 2.f ? 0.5f : (a < 4.f ? 1.f : 2.f);
    float t = r / step;
    if (mode == 1) t = copysignf(floorf(fabsf(t) + 0.5f), t);
    else t = floorf(t);
    const float q = fminf(fmaxf(t * step, -6.f), 6.f);
    const uint8_t code = quant_fp4_e2m1(q);  // exact
    return (q == 0.f && signbit(r) && mode == 1) ? (uint8_t)(code | 8) : code;
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
        const int e = mx_block_exp(amax, p, emax);
        const uint8_t byte = e > 127 ? 255 : (uint8_t)(e + 127);
        *sc = byte;
        const float inv = e > 127 ? __uint_as_float(0x7FC00000u) : ldexpf(1.f, -e);  // exact power of two
        if (p.y_dtype == ACL_FLOAT4_E2M1) {
            uint8_t* dst = reinterpret_cast<uint8_t*>(p.y) + (row * p.k + k0) / 2;
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                if (j < cnt) {
                    uint8_t lo = quant_fp4_e2m1_mode(v[j] * inv, p.round_mode);
                    uint8_t hi = (j + 1 < cnt) ? quant_fp4_e2m1_mode(v[j + 1] * inv, p.round_mode) : 0;
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

// Streaming form: k % 32 == 0, x and y 16-byte aligned. One lane = 8 consecutive elements; lanes 4j..4j+3 = one block.
template <bool kBf16>
__global__ void __launch_bounds__(256) mx_quant_stream_kernel(const OpsnnMxQuantParams p, int64_t blocks_per_row, int64_t scale_row)
{
    const int64_t pieces = p.rows * blocks_per_row * 4;  // 8-element pieces
    const int emax = p.y_dtype == ACL_FLOAT4_E2M1 ? 2 : (p.y_dtype == ACL_FLOAT8_E4M3FN ? 8 : 15);
    const uint4* src = reinterpret_cast<const uint4*>(p.x);
    for (int64_t i0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) & ~(int64_t)31; i0 < pieces; i0 += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = i0 + (threadIdx.x & 31);
        const bool live = i < pieces;  // pieces is a multiple of 4, so a block's four lanes are live together
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (live) raw = __ldcs(src + i);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        float v[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (kBf16) {
                v[2 * j] = __uint_as_float(w[j] << 16);
                v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
            } else {
                const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                v[2 * j] = f2.x;
                v[2 * j + 1] = f2.y;
            }
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const int e = mx_block_exp(amax, p, emax);
        if (!live) continue;
        const int64_t blk_lin = i >> 2;
        if ((i & 3) == 0) {
            const int64_t row = blk_lin / blocks_per_row, blk = blk_lin % blocks_per_row;
            uint8_t* sc = reinterpret_cast<uint8_t*>(p.scale) + row * scale_row + blk;
            *sc = e > 127 ? 255 : (uint8_t)(e + 127);
            if (blk == blocks_per_row - 1 && scale_row != blocks_per_row) sc[1] = 0;  // padding entry that makes the count even
        }
        const float inv = e > 127 ? __uint_as_float(0x7FC00000u) : __uint_as_float((uint32_t)(127 - e) << 23 | 0u);  // 2^-e, e in [-127, 127]
        const float inv2 = (e == 127) ? 0.5f : 1.f;  // 2^-127 is subnormal: split the scale in two exact factors
        const float s0 = (e == 127) ? __uint_as_float(1u << 23) : inv;  // 2^-126 when e == 127
        if (p.y_dtype == ACL_FLOAT4_E2M1) {
            uint32_t out = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) out |= (uint32_t)quant_fp4_e2m1_mode(v[j] * s0 * inv2, p.round_mode) << (4 * j);
            reinterpret_cast<uint32_t*>(p.y)[i] = out;
        } else {
            const __nv_fp8_interpretation_t kind = p.y_dtype == ACL_FLOAT8_E4M3FN ? __NV_E4M3 : __NV_E5M2;
            uint32_t lo = 0, hi = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                lo |= (uint32_t)__nv_cvt_float_to_fp8(v[j] * s0 * inv2, __NV_SATFINITE, kind) << (8 * j);
                hi |= (uint32_t)__nv_cvt_float_to_fp8(v[4 + j] * s0 * inv2, __NV_SATFINITE, kind) << (8 * j);
            }
            reinterpret_cast<uint2*>(p.y)[i] = make_uint2(lo, hi);
        }
    }
}

// Blocks along a non-last axis: x is (rows, k, inner); a thread owns one column i (two adjacent columns for fp4, which packs
// along inner) of one 32-row block, so consecutive threads read consecutive addresses in every one of the 32 rows.
template <bool kBf16, int kCols>
__global__ void __launch_bounds__(256) mx_quant_axis_kernel(const OpsnnMxQuantParams p, int64_t nblk, int64_t pairs)
{
    const int64_t icols = p.inner / kCols, total = p.rows * pairs * 2 * icols;
    const int emax = p.y_dtype == ACL_FLOAT4_E2M1 ? 2 : (p.y_dtype == ACL_FLOAT8_E4M3FN ? 8 : 15);
    const uint16_t* x = reinterpret_cast<const uint16_t*>(p.x);
    uint8_t* sc = reinterpret_cast<uint8_t*>(p.scale);
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t ic = t % icols, rb = (t / icols) % (pairs * 2), o = t / (icols * pairs * 2);
        const int64_t i0 = ic * kCols;
#pragma unroll
        for (int c = 0; c < kCols; ++c) {
            uint8_t* sp = sc + ((o * pairs + (rb >> 1)) * p.inner + i0 + c) * 2 + (rb & 1);
            if (rb >= nblk) *sp = 0;  // the entry that pads the block count to an even number
        }
        if (rb >= nblk) continue;
        const int cnt = (int)min((int64_t)32, p.k - rb * 32);
        float v[kCols][32];
        float amax[kCols];
#pragma unroll
        for (int c = 0; c < kCols; ++c) amax[c] = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
#pragma unroll
            for (int c = 0; c < kCols; ++c) {
                float f = 0.f;
                if (j < cnt) {
                    const uint16_t raw = x[(o * p.k + rb * 32 + j) * p.inner + i0 + c];
                    f = kBf16 ? __uint_as_float((uint32_t)raw << 16) : __half2float(__ushort_as_half(raw));
                }
                v[c][j] = f;
                amax[c] = fmaxf(amax[c], fabsf(f));
            }
        }
        float s0[kCols], s1[kCols];
#pragma unroll
        for (int c = 0; c < kCols; ++c) {
            const int e = mx_block_exp(amax[c], p, emax);
            sc[((o * pairs + (rb >> 1)) * p.inner + i0 + c) * 2 + (rb & 1)] = e > 127 ? 255 : (uint8_t)(e + 127);
            // 2^-e as two exact factors (2^-127 is subnormal)
            s0[c] = e > 127 ? __uint_as_float(0x7FC00000u) : (e == 127 ? __uint_as_float(1u << 23) : __uint_as_float((uint32_t)(127 - e) << 23));
            s1[c] = e == 127 ? 0.5f : 1.f;
        }
        if (p.y_dtype == ACL_FLOAT4_E2M1) {
            uint8_t* y = reinterpret_cast<uint8_t*>(p.y);
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < cnt)
                    y[((o * p.k + rb * 32 + j) * p.inner + i0) / 2] =
                        quant_fp4_e2m1_mode(v[0][j] * s0[0] * s1[0], p.round_mode) |
                        (quant_fp4_e2m1_mode(v[kCols - 1][j] * s0[kCols - 1] * s1[kCols - 1], p.round_mode) << 4);
        } else {
            uint8_t* y = reinterpret_cast<uint8_t*>(p.y);
            const __nv_fp8_interpretation_t kind = p.y_dtype == ACL_FLOAT8_E4M3FN ? __NV_E4M3 : __NV_E5M2;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < cnt) y[(o * p.k + rb * 32 + j) * p.inner + i0] = (uint8_t)__nv_cvt_float_to_fp8(v[0][j] * s0[0] * s1[0], __NV_SATFINITE, kind);
        }
    }
}

}  // namespace

int32_t mx_quant_launch(const OpsnnMxQuantParams* p, cudaStream_t stream)
{
    if (p->inner > 1) {
        const int64_t nblk = (p->k + 31) / 32, pairs = (nblk + 1) / 2;
        const bool f4 = p->y_dtype == ACL_FLOAT4_E2M1;
        if (f4 && p->inner % 2 != 0) return (int32_t)cudaErrorInvalidValue;
        const int64_t total = p->rows * pairs * 2 * (p->inner / (f4 ? 2 : 1));
        if (total == 0) return 0;
        int64_t grid = (total + 255) / 256;
        if (grid > 148 * 32) grid = 148 * 32;
        const bool bf = p->x_dtype == ACL_BF16;
        if (bf && f4) mx_quant_axis_kernel<true, 2><<<(unsigned)grid, 256, 0, stream>>>(*p, nblk, pairs);
        else if (bf) mx_quant_axis_kernel<true, 1><<<(unsigned)grid, 256, 0, stream>>>(*p, nblk, pairs);
        else if (f4) mx_quant_axis_kernel<false, 2><<<(unsigned)grid, 256, 0, stream>>>(*p, nblk, pairs);
        else mx_quant_axis_kernel<false, 1><<<(unsigned)grid, 256, 0, stream>>>(*p, nblk, pairs);
        note_launch("mx_quant_axis");
        return (int32_t)cudaGetLastError();
    }
    const int64_t blocks_per_row = (p->k + 31) / 32;
    const int64_t scale_row = ((blocks_per_row + 1) / 2) * 2;
    const int64_t total = p->rows * scale_row;
    if (total == 0) return 0;
    const bool stream_ok = p->k % 32 == 0 && (reinterpret_cast<uintptr_t>(p->x) & 15) == 0 && (reinterpret_cast<uintptr_t>(p->y) & 7) == 0 &&
                           getenv("OPSNN_MXQ_GENERIC") == nullptr;
    if (stream_ok) {
        const int64_t pieces = p->rows * blocks_per_row * 4;
        int64_t g2 = (pieces + 255) / 256;
        if (g2 > 148 * 16) g2 = 148 * 16;
        if (p->x_dtype == ACL_BF16) mx_quant_stream_kernel<true><<<(unsigned)g2, 256, 0, stream>>>(*p, blocks_per_row, scale_row);
        else mx_quant_stream_kernel<false><<<(unsigned)g2, 256, 0, stream>>>(*p, blocks_per_row, scale_row);
        note_launch("mx_quant_stream");
        return (int32_t)cudaGetLastError();
    }
    int64_t grid = (total + 255) / 256;
    if (grid > 148 * 32) grid = 148 * 32;
    if (p->x_dtype == ACL_BF16) mx_quant_kernel<true><<<(unsigned)grid, 256, 0, stream>>>(*p, blocks_per_row, scale_row);
    else mx_quant_kernel<false><<<(unsigned)grid, 256, 0, stream>>>(*p, blocks_per_row, scale_row);
    note_launch("mx_quant");
    return (int32_t)cudaGetLastError();
}

}  // namespace opsnn
