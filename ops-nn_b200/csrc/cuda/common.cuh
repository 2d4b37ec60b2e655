// Device helpers shared by every kernel: element decoding, output casts, launch bookkeeping.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "aclnn_compat/acl_base.h"
#include "opsnn_b200_kernels.h"

namespace opsnn {

// Host: count a launch and remember which kernel family ran (read back through opsnn_launch_count /
// opsnn_last_kernel_name).
void note_launch(const char* name, uint64_t n = 1);
void note_decode_plan(int64_t strips, int64_t splits, int32_t cluster);

// A column shard of an output that every rank of a communicator holds in full, in memory the ranks mapped into one another
// (opsnn_comm_bind_columns): the decode kernels then also store the shard's elements straight into every rank's full output -
// plain peer stores over NVLink, the all-gather folded into the epilogue.
constexpr int kMaxPeers = 8;
struct PeerBinding {
    void* full[kMaxPeers];  // every rank's full output (this rank's own included), as mapped into this process
    int32_t count;          // ranks; 0: not bound
    int64_t ld;             // elements per row of the full output
    int64_t col0;           // first column of this rank's shard in it
};
bool lookup_peer_binding(const void* y_local, PeerBinding* out);  // what the last streaming decode launch of this thread used

// Host: set-up that is a property of the (function, device) pair - the dynamic shared-memory limit of a kernel, occupancy - done the
// first time a launcher runs with each device current. `done` holds one bit per device ordinal. Two threads racing on the same first
// call both run `f`, which is idempotent.
template <typename F>
inline cudaError_t once_per_device(std::atomic<uint64_t>& done, F&& f)
{
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
    const cudaError_t rc = f();
    if (rc == cudaSuccess) done.fetch_or(bit, std::memory_order_release);
    return rc;
}

// Host: SM count of the current device (cached per device ordinal).
inline int current_sm_count()
{
    static std::atomic<int> cache[64];
    int dev = 0;
    cudaGetDevice(&dev);
    int v = cache[dev & 63].load(std::memory_order_relaxed);
    if (v <= 0) {
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        if (v <= 0) v = 148;
        cache[dev & 63].store(v, std::memory_order_relaxed);
    }
    return v;
}

__device__ __forceinline__ float e8m0_to_float(uint8_t b)
{
    // 2^(b-127); b == 0 is 2^-127 (an fp32 subnormal), b == 255 is NaN
    if (b == 0) return __uint_as_float(0x00400000u);
    if (b == 255) return __uint_as_float(0x7FC00000u);
    return __uint_as_float((uint32_t)b << 23);
}

__device__ __forceinline__ float fp4_e2m1_to_float(uint32_t nib)
{
    // sign | 2-bit exponent | 1-bit mantissa: magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6
    const float lut[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    float v = lut[nib & 7];
    return (nib & 8) ? -v : v;
}

__device__ __forceinline__ float fp8_to_float(uint8_t v, int dtype)
{
    __half_raw h = __nv_cvt_fp8_to_halfraw(v, dtype == ACL_FLOAT8_E5M2 ? __NV_E5M2 : __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&h));
}

// Element `idx` (in elements) of a tensor of `dtype` as float; 4-bit types are packed two per byte, low nibble first.
__device__ __forceinline__ float load_as_float(const void* base, int64_t idx, int dtype)
{
    switch (dtype) {
        case ACL_INT8: return (float)reinterpret_cast<const int8_t*>(base)[idx];
        case ACL_FLOAT8_E4M3FN:
        case ACL_FLOAT8_E5M2: return fp8_to_float(reinterpret_cast<const uint8_t*>(base)[idx], dtype);
        case ACL_FLOAT4_E2M1: {
            uint8_t b = reinterpret_cast<const uint8_t*>(base)[idx >> 1];
            return fp4_e2m1_to_float((idx & 1) ? (b >> 4) : (b & 0xF));
        }
        case ACL_INT4: {
            uint8_t b = reinterpret_cast<const uint8_t*>(base)[idx >> 1];
            int v = (idx & 1) ? (b >> 4) : (b & 0xF);
            return (float)((v ^ 8) - 8);
        }
        case ACL_FLOAT: return reinterpret_cast<const float*>(base)[idx];
        case ACL_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
        case ACL_FLOAT16: return __half2float(reinterpret_cast<const __half*>(base)[idx]);
        case ACL_INT32: return (float)reinterpret_cast<const int32_t*>(base)[idx];
        default: return 0.f;
    }
}

// Antiquant scale of the weight-only matmul as a float: in x's dtype, or e8m0 (mx) widened and, for fp16 activations, passed
// through fp16 as the golden does (wqbmmv2_kernel_golden.py:323-326 of the reference: 2^e outside fp16's range becomes 0 / inf).
__device__ __forceinline__ float load_wq_scale(const void* base, int64_t idx, int scale_dtype, bool x_is_bf16)
{
    if (scale_dtype == ACL_FLOAT8_E8M0) {
        const uint32_t b = reinterpret_cast<const uint8_t*>(base)[idx];
        const float f = b == 255u ? __uint_as_float(0x7FC00000u) : (b == 0u ? __uint_as_float(0x00400000u) : __uint_as_float(b << 23));
        return x_is_bf16 ? f : __half2float(__float2half_rn(f));
    }
    const uint16_t raw = reinterpret_cast<const uint16_t*>(base)[idx];
    return x_is_bf16 ? __uint_as_float((uint32_t)raw << 16) : __half2float(__ushort_as_half(raw));
}

// Dequant scale element as the reference's golden decodes it: fp32 as is, bf16 widened, uint64 = low word with the low
// 13 bits cleared (matmul/common/tests/st/arch35/matmul_quant_util.py:129-134 of the reference).
__device__ __forceinline__ float load_deq_scale(const void* base, int64_t idx, int dtype)
{
    if (dtype == ACL_FLOAT) return reinterpret_cast<const float*>(base)[idx];
    if (dtype == ACL_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
    uint32_t lo = (uint32_t)(reinterpret_cast<const unsigned long long*>(base)[idx] & 0xFFFFFFFFull);
    return __uint_as_float(lo & 0xFFFFE000u);
}

__device__ __forceinline__ float trunc19(float f) { return __uint_as_float(__float_as_uint(f) & 0xFFFFE000u); }

__device__ __forceinline__ void store_out(void* base, int64_t idx, float v, int dtype)
{
    switch (dtype) {
        case ACL_BF16: reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v); break;
        case ACL_FLOAT16: reinterpret_cast<__half*>(base)[idx] = __float2half_rn(v); break;
        case ACL_FLOAT: reinterpret_cast<float*>(base)[idx] = v; break;
        case ACL_INT8: reinterpret_cast<int8_t*>(base)[idx] = (int8_t)(int)v; break;  // v is integral and already clipped
        default: break;
    }
}

// Requantisation to int8 (qbmmv3_kernel_golden.py:465-487, matmul_quant_util.py:57-59, 137-143): the scaled accumulator is
// rounded half-to-even and clipped to nine signed bits, the optional nine-bit offset (bits 37..45 of the packed scale) is
// added, and the sum is clipped to int8. `f` is float(acc + int32 bias).
__device__ __forceinline__ float requant_s9(float f, float sb, const void* scale_b, int64_t col, int flags)
{
    f = fminf(fmaxf(rintf(__fmul_rn(f, sb)), -256.f), 255.f);
    if (flags & OPSNN_DEQ_REQUANT_OFFSET) {
        const uint64_t w = __ldg(reinterpret_cast<const unsigned long long*>(scale_b) + col);
        int off = (int)((w >> 37) & 0x1FFu);
        if (off & 0x100) off -= 0x200;
        f = __fadd_rn(f, (float)off);
    }
    return fminf(fmaxf(f, -128.f), 127.f);
}

__device__ __forceinline__ int out_elem_bytes(int dtype)
{
    return (dtype == ACL_FLOAT || dtype == ACL_INT32) ? 4 : (dtype == ACL_INT8 ? 1 : 2);
}

// The dequantisation epilogue of the per-tensor / per-channel / per-token modes, with the reference's rounding
// points: int32 accumulate (+int32 bias) -> RNE to fp32 -> * x2Scale -> * x1Scale -> + float bias -> RNE to out dtype
// (qbmmv3_kernel_golden.py:361-462; kernel quant_batch_matmul_v3/op_kernel/arch35/qbmm_mix_online_dynamic.h:674-720).
// `f` is the accumulator already converted to fp32 (after the int32 bias add for integer inputs).
__device__ __forceinline__ float deq_epilogue(float f, float sb, float sa, bool has_sa, float fbias, bool has_fbias,
                                              int flags)
{
    if (has_fbias && (flags & OPSNN_DEQ_FBIAS_BEFORE_SCALE)) f = __fadd_rn(f, fbias);
    if (flags & OPSNN_DEQ_TRUNC_SCALE_B) sb = trunc19(sb);
    if (flags & OPSNN_DEQ_MERGE_TRUNC) {
        f = __fmul_rn(f, trunc19(__fmul_rn(sb, sa)));
    } else {
        f = __fmul_rn(f, sb);
        if (has_sa) f = __fmul_rn(f, sa);
    }
    if (has_fbias && !(flags & OPSNN_DEQ_FBIAS_BEFORE_SCALE)) f = __fadd_rn(f, fbias);
    return f;
}

}  // namespace opsnn
