// Weight-only quant matmul, general kernel: any m, any weight storage (k,n)/(n,k), int4 or int8 weights,
// per-tensor / per-channel / per-group antiquant with arbitrary scale strides, bf16 or fp16 activations.
//
// Coverage kernel of the aclnnWeightQuantBatchMatmulV2/V3 path: a 64x64 output tile per CTA, the weight tile is
// dequantised while it is staged into shared memory, products run on the CUDA cores in fp32 (both factors are 16-bit
// floats, so every product is exact and only the accumulation order differs from the reference's numpy golden).
// The streaming decode kernel (wqbmm_decode.cu) replaces it for small m with n-packed int4 weights.
//
// Arithmetic (weight_quant_batch_matmul_v2/tests/assets/wqbmmv2_kernel_golden.py:199-297 of the reference; kernel
// op_kernel/arch35/weight_quant_batch_matmul_v2_vf.h:345-442):
//   w' = cast_x( cast_x( float(w) + float(offset) ) * float(scale) )      two roundings in x's dtype
//   y  = cast_x( sum_k float(x) * float(w') + float(bias) )
#include "common.cuh"

namespace opsnn {

namespace {
constexpr int TM = 64, TN = 64, TK = 32, NT = 256;

template <bool kBf16>
__device__ __forceinline__ float round_x(float v)
{
    if (kBf16) return __bfloat162float(__float2bfloat16_rn(v));
    return __half2float(__float2half_rn(v));
}

template <bool kBf16>
__device__ __forceinline__ float load_x(const void* base, int64_t idx)
{
    if (kBf16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
    return __half2float(reinterpret_cast<const __half*>(base)[idx]);
}

template <bool kBf16>
__global__ void __launch_bounds__(NT) wqbmm_generic_kernel(const OpsnnWqbmmParams p)
{
    __shared__ float Xs[TK][TM + 1];
    __shared__ float Ws[TK][TN + 1];
    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const int64_t tiles_n = (p.n + TN - 1) / TN;
    const int64_t m0 = ((int64_t)blockIdx.x / tiles_n) * TM, n0 = ((int64_t)blockIdx.x % tiles_n) * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int64_t k0 = 0; k0 < p.k; k0 += TK) {
        for (int e = tid; e < TK * TM; e += NT) {
            int mm = e / TK, kk = e % TK;
            int64_t gm = m0 + mm, gk = k0 + kk;
            Xs[kk][mm] = (gm < p.m && gk < p.k) ? load_x<kBf16>(p.x, gm * p.x_ld + gk) : 0.f;
        }
        for (int e = tid; e < TK * TN; e += NT) {
            int kk, nn;
            if (p.trans_w) { nn = e / TK; kk = e % TK; } else { kk = e / TN; nn = e % TN; }
            int64_t gn = n0 + nn, gk = k0 + kk;
            float w = 0.f;
            if (gn < p.n && gk < p.k) {
                int64_t idx = p.trans_w ? gn * p.w_ld + gk : gk * p.w_ld + gn;
                w = load_as_float(p.w, idx, p.w_dtype);
                int64_t g = p.group_size > 0 ? gk / p.group_size : 0;
                int64_t sidx = g * p.scale_sg + gn * p.scale_sn;
                if (p.offset != nullptr) w = round_x<kBf16>(__fadd_rn(w, load_x<kBf16>(p.offset, sidx)));
                w = round_x<kBf16>(__fmul_rn(w, load_wq_scale(p.scale, sidx, p.scale_dtype, kBf16)));
            }
            Ws[kk][nn] = w;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < TK; ++kk) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = Xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int64_t gm = m0 + ty * 4 + i;
        if (gm >= p.m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int64_t gn = n0 + tx * 4 + j;
            if (gn >= p.n) continue;
            float f = acc[i][j];
            if (p.bias != nullptr) f = __fadd_rn(f, load_as_float(p.bias, gn, p.bias_dtype));
            store_out(p.y, gm * p.y_ld + gn, f, p.x_dtype);
        }
    }
}
}  // namespace

int32_t wqbmm_generic_launch(const OpsnnWqbmmParams* p, cudaStream_t stream)
{
    const int64_t tiles = ((p->n + TN - 1) / TN) * ((p->m + TM - 1) / TM);
    if (tiles > 0x7FFFFFFF) return (int32_t)cudaErrorInvalidConfiguration;
    if (p->x_dtype == ACL_BF16) wqbmm_generic_kernel<true><<<(unsigned)tiles, NT, 0, stream>>>(*p);
    else wqbmm_generic_kernel<false><<<(unsigned)tiles, NT, 0, stream>>>(*p);
    note_launch("wqbmm_generic");
    return (int32_t)cudaGetLastError();
}

}  // namespace opsnn
