// Full-quant matmul, general kernel: any shape, row pitch, transpose and batch broadcast, every quant mode.
//
// This is the coverage kernel of the aclnnQuantMatmulV5 path, not the fast one: 64x64 output tile per CTA on the CUDA
// cores (integer multiply-add for int8, fp32 FMA for fp8/fp4), plain global loads. The TMA + tcgen05 kernel
// (qmm_umma.cu) takes over whenever its alignment rules hold; unaligned pitches, odd transposes and tiny shapes land here.
//
// Arithmetic follows the reference's goldens (quant_batch_matmul_v3/tests/assets/qbmmv3_kernel_golden.py):
//   DEQ      :361-462   exact int32 accumulate; epilogue in common.cuh::deq_epilogue
//   PERBLOCK :237-358   y += (x1[:,kb] @ x2[kb,:]) * (s1[m/gm,kb] * s2[kb,n/gn]) per 128-k block, fp32
//   MX       :153-234   (x1 * 2^e1) @ (x2 * 2^e2) + bias, fp32
#include "common.cuh"

namespace opsnn {

constexpr int TM = 64, TN = 64, TK = 32, NT = 256;

struct MxScaleIdx {
    // x1Scale (m, kq, 2) or, with x1 stored (k,m), (kq, m, 2); x2Scale (kq, n, 2) or, with x2 stored (n,k), (n, kq, 2)
    // (qbmmv3_kernel_golden.py:171-197). Group g = 2*p + j lives at [.., p, .., j].
    __device__ static int64_t a(int64_t m_idx, int64_t g, int64_t m, int64_t kq, int trans)
    {
        return trans ? ((g >> 1) * m + m_idx) * 2 + (g & 1) : m_idx * (2 * kq) + g;
    }
    __device__ static int64_t b(int64_t n_idx, int64_t g, int64_t n, int64_t kq, int trans)
    {
        return trans ? n_idx * (2 * kq) + g : ((g >> 1) * n + n_idx) * 2 + (g & 1);
    }
};

template <bool kInt>
__global__ void __launch_bounds__(NT) qmm_generic_kernel(const OpsnnQmmParams p)
{
    using AccT = typename std::conditional<kInt, int, float>::type;
    __shared__ AccT As[TK][TM + 1];
    __shared__ AccT Bs[TK][TN + 1];

    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int64_t tiles_n = (p.n + TN - 1) / TN;
    const int64_t m0 = ((int64_t)blockIdx.x / tiles_n) * TM, n0 = ((int64_t)blockIdx.x % tiles_n) * TN;
    const int64_t bz = blockIdx.z;
    const uint8_t* a = reinterpret_cast<const uint8_t*>(p.a);
    const uint8_t* b = reinterpret_cast<const uint8_t*>(p.b);
    const int a_bits = (p.a_dtype == ACL_FLOAT4_E2M1 || p.a_dtype == ACL_INT4) ? 4 : 8;
    const int b_bits = (p.b_dtype == ACL_FLOAT4_E2M1 || p.b_dtype == ACL_INT4) ? 4 : 8;
    a += (bz * p.a_bs * a_bits) / 8;
    b += (bz * p.b_bs * b_bits) / 8;
    const int64_t kq = (p.k + 63) / 64;
    const uint8_t* sa8 = reinterpret_cast<const uint8_t*>(p.scale_a);
    const uint8_t* sb8 = reinterpret_cast<const uint8_t*>(p.scale_b);
    const float* saf = reinterpret_cast<const float*>(p.scale_a);
    const float* sbf = reinterpret_cast<const float*>(p.scale_b);
    if (p.mode == OPSNN_QMM_MX) {
        sa8 += bz * p.sa_bs;
        sb8 += bz * p.sb_bs;
    } else if (p.mode == OPSNN_QMM_PERBLOCK) {
        saf += bz * p.sa_bs;
        sbf += bz * p.sb_bs;
    }

    AccT acc[4][4];
    float tot[4][4];
    float rs[4] = {0.f, 0.f, 0.f, 0.f};  // PERGROUP_ASYM: sums of this thread's rows of a over the current k-group
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0;
            tot[i][j] = 0.f;
        }

    const int64_t n_kblk = (p.k + 127) / 128;  // PERBLOCK scale row length along k
    for (int64_t k0 = 0; k0 < p.k; k0 += TK) {
        // ---- stage a TK x TM slice of A and a TK x TN slice of B (decoded, MX-scaled) ----
        for (int e = tid; e < TK * TM; e += NT) {
            int kk, mm;
            if (p.trans_a) { kk = e / TM; mm = e % TM; } else { mm = e / TK; kk = e % TK; }
            int64_t gm = m0 + mm, gk = k0 + kk;
            AccT v = 0;
            if (gm < p.m && gk < p.k) {
                int64_t idx = p.trans_a ? gk * p.a_ld + gm : gm * p.a_ld + gk;
                if (kInt) {
                    v = (AccT) reinterpret_cast<const int8_t*>(a)[idx];
                } else {
                    float f = load_as_float(a, idx, p.a_dtype);
                    if (p.mode == OPSNN_QMM_MX) f *= e8m0_to_float(sa8[MxScaleIdx::a(gm, gk / 32, p.m, kq, p.trans_a)]);
                    v = (AccT)f;
                }
            }
            As[kk][mm] = v;
        }
        for (int e = tid; e < TK * TN; e += NT) {
            int kk, nn;
            if (p.trans_b) { nn = e / TK; kk = e % TK; } else { kk = e / TN; nn = e % TN; }
            int64_t gn = n0 + nn, gk = k0 + kk;
            AccT v = 0;
            if (gn < p.n && gk < p.k) {
                int64_t idx = p.trans_b ? gn * p.b_ld + gk : gk * p.b_ld + gn;
                if (kInt) {
                    v = (AccT) reinterpret_cast<const int8_t*>(b)[idx];
                } else {
                    float f = load_as_float(b, idx, p.b_dtype);
                    if (p.mode == OPSNN_QMM_MX) f *= e8m0_to_float(sb8[MxScaleIdx::b(gn, gk / 32, p.n, kq, p.trans_b)]);
                    v = (AccT)f;
                }
            }
            Bs[kk][nn] = v;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < TK; ++kk) {
            AccT av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
            if (!kInt && p.mode == OPSNN_QMM_PERGROUP_ASYM) {
#pragma unroll
                for (int i = 0; i < 4; ++i) rs[i] += (float)av[i];
            }
        }
        __syncthreads();
        if (p.mode == OPSNN_QMM_PERGROUP_ASYM && (((k0 + TK) % p.group_k == 0) || k0 + TK >= p.k)) {
            // close the k-group: tot += (part - rowsum * offset[g,n]) * scale[g,n], every step rounded like the golden
            const int64_t g = k0 / p.group_k;
            const __half* offp = reinterpret_cast<const __half*>(p.b_offset);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int64_t gn = n0 + tx * 4 + j;
                    if (gn < p.n) {
                        const float off = __half2float(offp[g * p.n + gn]), sc = sbf[g * p.n + gn];
                        tot[i][j] = __fadd_rn(tot[i][j], __fmul_rn(__fsub_rn((float)acc[i][j], __fmul_rn(rs[i], off)), sc));
                    }
                    acc[i][j] = 0;
                }
                rs[i] = 0.f;
            }
        }
        if (p.mode == OPSNN_QMM_PERBLOCK && (((k0 + TK) % 128 == 0) || k0 + TK >= p.k)) {
            // promote the finished 128-k block: tot += part * (s1 * s2), the two scales multiplied first
            int64_t kb = k0 / 128;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int64_t gm = m0 + ty * 4 + i;
                if (gm >= p.m) continue;
                int64_t mg = gm / p.group_m;
                // x1Scale is (m/gm, k/128), or (k/128, m/gm) when x1 is stored transposed
                float s1 = p.trans_a ? saf[kb * ((p.m + p.group_m - 1) / p.group_m) + mg] : saf[mg * n_kblk + kb];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int64_t gn = n0 + tx * 4 + j;
                    if (gn >= p.n) continue;
                    int64_t ng = gn / p.group_n;
                    float s2 = p.trans_b ? sbf[ng * n_kblk + kb] : sbf[kb * ((p.n + p.group_n - 1) / p.group_n) + ng];
                    tot[i][j] = __fadd_rn(tot[i][j], __fmul_rn((float)acc[i][j], __fmul_rn(s1, s2)));
                    acc[i][j] = 0;
                }
            }
        }
    }

    // ---- epilogue ----
    uint8_t* out = reinterpret_cast<uint8_t*>(p.out);
    const int out_bytes = out_elem_bytes(p.out_dtype);
    out += bz * p.out_bs * out_bytes;
    const uint8_t* bias = reinterpret_cast<const uint8_t*>(p.bias);
    if (bias != nullptr) bias += bz * p.bias_bs * (p.bias_dtype == ACL_FLOAT || p.bias_dtype == ACL_INT32 ? 4 : 2);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int64_t gm = m0 + ty * 4 + i;
        if (gm >= p.m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int64_t gn = n0 + tx * 4 + j;
            if (gn >= p.n) continue;
            int64_t oidx = gm * p.out_ld + gn;
            if (p.mode == OPSNN_QMM_DEQ) {
                float f;
                if (kInt) {
                    int v = (int)acc[i][j];
                    if (p.bias_dtype == ACL_INT32) v += reinterpret_cast<const int32_t*>(bias)[gn];
                    if (p.out_dtype == ACL_INT32) {
                        reinterpret_cast<int32_t*>(out)[oidx] = v;
                        continue;
                    }
                    f = (float)v;  // cvt.rn
                } else {
                    f = (float)acc[i][j];
                }
                const bool has_fbias = p.bias != nullptr && p.bias_dtype != ACL_INT32;
                float fb = has_fbias ? load_as_float(bias, gn, p.bias_dtype) : 0.f;
                float sb = load_deq_scale(p.scale_b, p.scale_b_len == 1 ? 0 : gn, p.scale_b_dtype);
                const bool has_sa = p.scale_a != nullptr;
                float sa = has_sa ? saf[p.scale_a_len == 1 ? 0 : gm] : 1.f;
                if (p.deq_flags & OPSNN_DEQ_REQUANT) f = requant_s9(f, sb, p.scale_b, p.scale_b_len == 1 ? 0 : gn, p.deq_flags);
                else f = deq_epilogue(f, sb, sa, has_sa, fb, has_fbias, p.deq_flags);
                store_out(out, oidx, f, p.out_dtype);
            } else if (p.mode == OPSNN_QMM_PERGROUP_ASYM) {
                store_out(out, oidx, __fmul_rn(tot[i][j], saf[gm]), p.out_dtype);
            } else {
                float f = p.mode == OPSNN_QMM_PERBLOCK ? tot[i][j] : (float)acc[i][j];
                if (p.bias != nullptr) f = __fadd_rn(f, load_as_float(bias, gn, p.bias_dtype));
                store_out(out, oidx, f, p.out_dtype);
            }
        }
    }
}

int32_t qmm_generic_launch(const OpsnnQmmParams* p, cudaStream_t stream)
{
    const int64_t tiles = ((p->n + TN - 1) / TN) * ((p->m + TM - 1) / TM);
    if (tiles > 0x7FFFFFFF || p->batch > 65535) return (int32_t)cudaErrorInvalidConfiguration;
    dim3 grid((unsigned)tiles, 1, (unsigned)p->batch);
    const bool is_int = p->a_dtype == ACL_INT8 && p->b_dtype == ACL_INT8 && p->mode == OPSNN_QMM_DEQ;
    if (is_int) qmm_generic_kernel<true><<<grid, NT, 0, stream>>>(*p);
    else qmm_generic_kernel<false><<<grid, NT, 0, stream>>>(*p);
    note_launch("qmm_generic");
    return (int32_t)cudaGetLastError();
}

}  // namespace opsnn
