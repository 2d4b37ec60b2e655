// Weight-only quant matmul for m beyond the decode range ("prefill"): the weight is dequantised once into the workspace as
// a k-contiguous (n, k) matrix in x's dtype, then the tcgen05 kind::f16 matmul of qmm_umma.cu runs on x and that matrix.
//
// Reference: weight_quant_batch_matmul_v2/op_kernel/arch35/weight_quant_batch_matmul_v2_reg_base_common.h:164-286 (vector
// cores dequantise the weight tile by tile into L1, the cube unit multiplies in bf16/fp16); arithmetic of the golden
// weight_quant_batch_matmul_v2/tests/assets/wqbmmv2_kernel_golden.py:199-297:
//   w' = cast_x( cast_x( float(w) + float(offset) ) * float(scale) )     two roundings in x's dtype, as the decode kernel
//   y  = cast_x( sum_k x * w' (fp32) + bias )
// The dequantised weight is what the reference's cube unit sees too, so the result differs from the golden only by fp32
// summation order.
//
// HBM cost of the pre-pass: n*k/2 (int4) read + 2*n*k written, then 2*n*k read once by the matmul (x stays in L2):
// worthwhile once the matmul's 2*m*n*k flops dominate; below m = 17 the fused streaming decode kernels are used.
#include <cstdlib>

#include "common.cuh"
#include "wqbmm_decode_common.cuh"

namespace opsnn {

bool qmm_umma_eligible(const OpsnnQmmParams* p);
int32_t qmm_umma_launch(const OpsnnQmmParams* p, cudaStream_t stream);

namespace {

constexpr int TK = 64, TN = 64, NT = 256;

template <bool kBf16>
__device__ __forceinline__ float round_x(float v)
{
    if (kBf16) return __bfloat162float(__float2bfloat16_rn(v));
    return __half2float(__float2half_rn(v));
}
template <bool kBf16>
__device__ __forceinline__ float load_x(const void* base, int64_t idx)
{
    if (kBf16) return __uint_as_float((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(base) + idx) << 16);
    return __half2float(__ushort_as_half(__ldg(reinterpret_cast<const uint16_t*>(base) + idx)));
}
template <bool kBf16>
__device__ __forceinline__ uint16_t bits_x(float v)
{
    if (kBf16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    return __half_as_ushort(__float2half_rn(v));
}

// One CTA: a TK x TN tile of the weight -> dst[n][k] (row pitch kp elements). Any storage, one element at a time.
template <bool kBf16>
__global__ void __launch_bounds__(NT) wq_dequant_nk_kernel(const OpsnnWqbmmParams p, uint16_t* __restrict__ dst, int64_t kp,
                                                           float* __restrict__ one)
{
    __shared__ __align__(16) uint16_t tile[TN][TK + 8];  // row pitch 144 bytes: 16-byte aligned rows, skewed banks
    const int tid = threadIdx.x;
    const int64_t tiles_n = (p.n + TN - 1) / TN;
    const int64_t k0 = ((int64_t)blockIdx.x / tiles_n) * TK, n0 = ((int64_t)blockIdx.x % tiles_n) * TN;
    if (blockIdx.x == 0 && tid == 0) *one = 1.0f;  // the unit dequant scale the matmul's epilogue multiplies by
    for (int e = tid; e < TK * TN; e += NT) {
        int kk, nn;
        if (p.trans_w) { nn = e / TK; kk = e % TK; } else { kk = e / TN; nn = e % TN; }
        const int64_t gn = n0 + nn, gk = k0 + kk;
        float w = 0.f;
        if (gn < p.n && gk < p.k) {
            const int64_t idx = p.trans_w ? gn * p.w_ld + gk : gk * p.w_ld + gn;
            w = load_as_float(p.w, idx, p.w_dtype);
            const int64_t g = p.group_size > 0 ? gk / p.group_size : 0;
            const int64_t sidx = g * p.scale_sg + gn * p.scale_sn;
            if (p.offset != nullptr) w = round_x<kBf16>(__fadd_rn(w, load_x<kBf16>(p.offset, sidx)));
            w = round_x<kBf16>(__fmul_rn(w, load_wq_scale(p.scale, sidx, p.scale_dtype, kBf16)));
        }
        tile[nn][kk] = bits_x<kBf16>(w);
    }
    __syncthreads();
    // 64 rows (n) x 128 bytes (64 k): 16-byte pieces, 8 per row; kp % 8 == 0 and k0 % 64 == 0 keep them aligned
    for (int e = tid; e < TN * (TK / 8); e += NT) {
        const int nn = e / (TK / 8), c = e % (TK / 8);
        const int64_t gn = n0 + nn, gk = k0 + c * 8;
        if (gn < p.n && gk < kp)
            *reinterpret_cast<uint4*>(dst + gn * kp + gk) = *reinterpret_cast<const uint4*>(&tile[nn][c * 8]);
    }
}

// two fp32 -> packed pair in x's dtype (lo in the low half), and back
template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi)
{
    if (kBf16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
template <bool kBf16>
__device__ __forceinline__ float2 unpack2(uint32_t v)
{
    if (kBf16) return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xFFFF0000u));
    return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

// The common layout: int4 stored (k,n) as 32-bit words of 8 columns, n % 8 == 0, word-aligned rows, scale/offset
// contiguous along n and constant over a 64-row tile (per-channel, or groups of a multiple of 64 rows).
// Thread = one word column (8 n) x two adjacent k rows: the two rows of a column leave as one packed pair, so the tile
// is written with 32-bit stores; 16-byte pieces of a tile row are XOR-swizzled by the word column (conflict-free both ways).
template <bool kBf16>
__global__ void __launch_bounds__(NT) wq_dequant_nk_words_kernel(const OpsnnWqbmmParams p, uint16_t* __restrict__ dst, int64_t kp,
                                                                 float* __restrict__ one)
{
    __shared__ __align__(16) uint32_t tile[TN][TK / 2];  // [n][k pair], 128 bytes per row
    const int tid = threadIdx.x;
    const int64_t tiles_n = (p.n + TN - 1) / TN;
    const int64_t k0 = ((int64_t)blockIdx.x / tiles_n) * TK, n0 = ((int64_t)blockIdx.x % tiles_n) * TN;
    if (blockIdx.x == 0 && tid == 0) *one = 1.0f;
    const int wj = tid & 7, kr = tid >> 3;  // word column 0..7, row pair 0..31
    const int64_t gn = n0 + wj * 8, gk = k0 + 2 * kr;
    const bool col_live = gn < p.n;
    uint32_t w0 = 0u, w1 = 0u;
    if (col_live && gk < p.k) w0 = __ldcs(reinterpret_cast<const uint32_t*>(p.w) + (gk * p.w_ld + gn) / 8);
    if (col_live && gk + 1 < p.k) w1 = __ldcs(reinterpret_cast<const uint32_t*>(p.w) + ((gk + 1) * p.w_ld + gn) / 8);
    float sc[8], of[8];
    {
        const int64_t g = p.group_size > 0 ? min(k0, p.k - 1) / p.group_size : 0;
        const int64_t sidx = g * p.scale_sg + (col_live ? gn : 0) * p.scale_sn;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            sc[j] = load_x<kBf16>(p.scale, sidx + j * p.scale_sn);
            of[j] = p.offset != nullptr ? load_x<kBf16>(p.offset, sidx + j * p.scale_sn) : 0.f;
        }
    }
    const bool has_off = p.offset != nullptr;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float a = (float)(((int32_t)(w0 << (28 - 4 * j))) >> 28);  // sign-extended nibble j of each row
        float b = (float)(((int32_t)(w1 << (28 - 4 * j))) >> 28);
        if (has_off) {
            const float2 r = unpack2<kBf16>(pack2<kBf16>(__fadd_rn(a, of[j]), __fadd_rn(b, of[j])));  // first rounding
            a = r.x;
            b = r.y;
        }
        uint32_t v = pack2<kBf16>(__fmul_rn(a, sc[j]), __fmul_rn(b, sc[j]));  // second rounding
        if (gk >= p.k) v = 0u;
        else if (gk + 1 >= p.k) v &= 0xFFFFu;
        tile[wj * 8 + j][(((kr >> 2) ^ wj) << 2) | (kr & 3)] = v;
    }
    __syncthreads();
#pragma unroll
    for (int e = tid; e < TN * 8; e += NT) {
        const int nn = e >> 3, c = e & 7;  // row, 16-byte piece (8 k)
        const int64_t on = n0 + nn, ok = k0 + c * 8;
        if (on < p.n && ok < kp)
            *reinterpret_cast<uint4*>(dst + on * kp + ok) = *reinterpret_cast<const uint4*>(&tile[nn][(c ^ (nn >> 3)) << 2]);
    }
}

// The streaming form of the same layout: a thread owns one word column (8 n) over 8 consecutive k rows and does the
// arithmetic on packed pairs exactly as the decode kernels do (nibble -> 136 + w by one lop3, then sub / add / mul .rn on
// bf16x2 or f16x2: the reference's two roundings). A lop3 pairs columns j and j + 4 of one row; two rows' results are
// re-paired into (k, k + 1) words of one column with byte permutes and stored into a 64 x 256 tile whose word index is
// XOR-swizzled by the word column (bank = column + index, 129-word rows: conflict-free writes and reads).
// Needs group_size % 8 == 0 (a thread's 8 rows share their scales).
constexpr int PK = 256, PN = 64, PP = PK / 2 + 1;

template <bool kBf16>
__global__ void __launch_bounds__(NT) wq_dequant_nk_pairs_kernel(const OpsnnWqbmmParams p, uint16_t* __restrict__ dst, int64_t kp,
                                                                 float* __restrict__ one, int vec_scale)
{
    using N = Num<kBf16>;
    extern __shared__ uint32_t ptile[];  // [PN][PP]
    const int tid = threadIdx.x;
    const int64_t tiles_n = (p.n + PN - 1) / PN;
    const int64_t k0 = ((int64_t)blockIdx.x / tiles_n) * PK, n0 = ((int64_t)blockIdx.x % tiles_n) * PN;
    if (blockIdx.x == 0 && tid == 0) *one = 1.0f;
    const int wj = tid & 7, kr = tid >> 3;
    const int64_t gn = n0 + wj * 8, gk = k0 + 8 * kr;
    const bool col_live = gn < p.n;
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
        w[i] = (col_live && gk + i < p.k) ? __ldcs(reinterpret_cast<const uint32_t*>(p.w) + ((gk + i) * p.w_ld + gn) / 8) : 0u;
    // scale / offset of columns (j, j + 4), j = 0..3, as packed pairs
    uint32_t sp[4], op[4];
    const bool has_off = p.offset != nullptr;
    {
        const int64_t g = p.group_size > 0 ? min(gk, p.k - 1) / p.group_size : 0;
        const int64_t sidx = g * p.scale_sg + (col_live ? gn : 0) * p.scale_sn;
        if (vec_scale) {
            const uint4 sv = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.scale) + sidx));
            sp[0] = __byte_perm(sv.x, sv.z, 0x5410); sp[1] = __byte_perm(sv.x, sv.z, 0x7632);
            sp[2] = __byte_perm(sv.y, sv.w, 0x5410); sp[3] = __byte_perm(sv.y, sv.w, 0x7632);
            if (has_off) {
                const uint4 ov = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.offset) + sidx));
                op[0] = __byte_perm(ov.x, ov.z, 0x5410); op[1] = __byte_perm(ov.x, ov.z, 0x7632);
                op[2] = __byte_perm(ov.y, ov.w, 0x5410); op[3] = __byte_perm(ov.y, ov.w, 0x7632);
            }
        } else {
            const uint16_t* sc = reinterpret_cast<const uint16_t*>(p.scale);
            const uint16_t* of = reinterpret_cast<const uint16_t*>(p.offset);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                sp[j] = (uint32_t)__ldg(sc + sidx + j * p.scale_sn) | ((uint32_t)__ldg(sc + sidx + (j + 4) * p.scale_sn) << 16);
                if (has_off) op[j] = (uint32_t)__ldg(of + sidx + j * p.scale_sn) | ((uint32_t)__ldg(of + sidx + (j + 4) * p.scale_sn) << 16);
            }
        }
    }
    const int swz = (wj & 3) | ((wj >> 2) << 4);
#pragma unroll
    for (int rp = 0; rp < 4; ++rp) {
        const int col = (4 * kr + rp) ^ swz;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t t0, t1;
            asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(t0) : "r"(w[2 * rp] >> (4 * j)), "n"(0x000F000F), "r"(N::kMagic));
            asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(t1) : "r"(w[2 * rp + 1] >> (4 * j)), "n"(0x000F000F), "r"(N::kMagic));
            t0 = N::sub(t0, N::kBias);
            t1 = N::sub(t1, N::kBias);
            if (has_off) {
                t0 = N::add(t0, op[j]);
                t1 = N::add(t1, op[j]);
            }
            t0 = N::mul(t0, sp[j]);
            t1 = N::mul(t1, sp[j]);
            ptile[(wj * 8 + j) * PP + col] = __byte_perm(t0, t1, 0x5410);      // column j: rows (2rp, 2rp + 1)
            ptile[(wj * 8 + j + 4) * PP + col] = __byte_perm(t0, t1, 0x7632);  // column j + 4
        }
    }
    __syncthreads();
    uint32_t* out = reinterpret_cast<uint32_t*>(dst);
    for (int e = tid; e < PN * (PK / 2); e += NT) {
        const int nn = e >> 7, c = e & 127;
        const int64_t on = n0 + nn, ok = k0 + 2 * c;
        if (on < p.n && ok < kp) out[(on * kp + ok) >> 1] = ptile[nn * PP + (c ^ (((nn >> 3) & 3) | (((nn >> 5) & 1) << 4)))];
    }
}

// 8-bit weights (int8 / fp8) stored (k,n): a thread owns one 32-bit word (4 columns) over 4 consecutive k rows, the two row
// pairs of a column leave as packed words; 64 x 64 tile with 33-word rows. Needs n % 4 == 0, word-aligned rows,
// group_size % 4 == 0 and scales in x's dtype.
template <bool kBf16>
__global__ void __launch_bounds__(NT) wq_dequant_nk_bytes_kernel(const OpsnnWqbmmParams p, uint16_t* __restrict__ dst, int64_t kp,
                                                                 float* __restrict__ one)
{
    __shared__ uint32_t tile[TN][TK / 2 + 1];
    const int tid = threadIdx.x;
    const int64_t tiles_n = (p.n + TN - 1) / TN;
    const int64_t k0 = ((int64_t)blockIdx.x / tiles_n) * TK, n0 = ((int64_t)blockIdx.x % tiles_n) * TN;
    if (blockIdx.x == 0 && tid == 0) *one = 1.0f;
    const int wj = tid & 15, kq = tid >> 4;
    const int64_t gn = n0 + wj * 4, gk = k0 + 4 * kq;
    const bool col_live = gn < p.n;
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        w[i] = (col_live && gk + i < p.k) ? __ldcs(reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(p.w) + (gk + i) * p.w_ld + gn)) : 0u;
    float sc[4], of[4];
    const bool has_off = p.offset != nullptr;
    {
        const int64_t g = p.group_size > 0 ? min(gk, p.k - 1) / p.group_size : 0;
        const int64_t sidx = g * p.scale_sg + (col_live ? gn : 0) * p.scale_sn;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            sc[j] = load_x<kBf16>(p.scale, sidx + j * p.scale_sn);
            of[j] = has_off ? load_x<kBf16>(p.offset, sidx + j * p.scale_sn) : 0.f;
        }
    }
    const bool is_int = p.w_dtype == ACL_INT8;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t byte = (w[i] >> (8 * j)) & 0xFFu;
            v[i] = is_int ? (float)(int8_t)byte : fp8_to_float((uint8_t)byte, p.w_dtype);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float a = v[2 * h], b = v[2 * h + 1];
            if (has_off) {
                const float2 r = unpack2<kBf16>(pack2<kBf16>(__fadd_rn(a, of[j]), __fadd_rn(b, of[j])));
                a = r.x;
                b = r.y;
            }
            tile[wj * 4 + j][2 * kq + h] = pack2<kBf16>(__fmul_rn(a, sc[j]), __fmul_rn(b, sc[j]));
        }
    }
    __syncthreads();
    uint32_t* out = reinterpret_cast<uint32_t*>(dst);
    for (int e = tid; e < TN * (TK / 2); e += NT) {
        const int nn = e >> 5, c = e & 31;
        const int64_t on = n0 + nn, ok = k0 + 2 * c;
        if (on < p.n && ok < kp) out[(on * kp + ok) >> 1] = tile[nn][c];
    }
}

// Weight stored (n,k) (the transposed-view case, e.g. a torch Linear weight): the destination has the same orientation, so a
// thread dequantises one 32-bit word - kPer consecutive k of one column (8 for 4-bit, 4 for 8-bit weights) - and stores it as
// one 16- / 8-byte piece. One scale / offset per word (groups are multiples of kPer, or per-channel).
template <bool kBf16, int kPer>
__global__ void __launch_bounds__(NT) wq_dequant_nk_rows_kernel(const OpsnnWqbmmParams p, uint16_t* __restrict__ dst, int64_t kp,
                                                                float* __restrict__ one)
{
    if (blockIdx.x == 0 && threadIdx.x == 0) *one = 1.0f;
    const int64_t wpr = p.k / kPer, total = p.n * wpr;  // words per row
    const bool has_off = p.offset != nullptr;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t nn = i / wpr, kw = i % wpr, kk = kw * kPer;
        const uint32_t word = __ldcs(reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(p.w) + (nn * p.w_ld + kk) * (32 / kPer) / 8));
        const int64_t g = p.group_size > 0 ? kk / p.group_size : 0;
        const int64_t sidx = g * p.scale_sg + nn * p.scale_sn;
        const float sc = load_x<kBf16>(p.scale, sidx), of = has_off ? load_x<kBf16>(p.offset, sidx) : 0.f;
        uint32_t outw[kPer / 2];
#pragma unroll
        for (int h = 0; h < kPer / 2; ++h) {
            float a, b;
            if (kPer == 8) {
                const uint32_t n0 = (word >> (8 * h)) & 0xFu, n1 = (word >> (8 * h + 4)) & 0xFu;
                if (p.w_dtype == ACL_INT4) {
                    a = (float)((int)(n0 ^ 8u) - 8);
                    b = (float)((int)(n1 ^ 8u) - 8);
                } else {
                    a = fp4_e2m1_to_float((uint8_t)n0);
                    b = fp4_e2m1_to_float((uint8_t)n1);
                }
            } else {
                const uint32_t b0 = (word >> (16 * h)) & 0xFFu, b1 = (word >> (16 * h + 8)) & 0xFFu;
                a = p.w_dtype == ACL_INT8 ? (float)(int8_t)b0 : fp8_to_float((uint8_t)b0, p.w_dtype);
                b = p.w_dtype == ACL_INT8 ? (float)(int8_t)b1 : fp8_to_float((uint8_t)b1, p.w_dtype);
            }
            if (has_off) {
                const float2 r = unpack2<kBf16>(pack2<kBf16>(__fadd_rn(a, of), __fadd_rn(b, of)));
                a = r.x;
                b = r.y;
            }
            outw[h] = pack2<kBf16>(__fmul_rn(a, sc), __fmul_rn(b, sc));
        }
        uint16_t* o = dst + nn * kp + kk;
        if (kPer == 8) *reinterpret_cast<uint4*>(o) = make_uint4(outw[0], outw[1], outw[kPer / 2 - 2], outw[kPer / 2 - 1]);
        else *reinterpret_cast<uint2*>(o) = make_uint2(outw[0], outw[1]);
    }
}

int64_t padded_k(const OpsnnWqbmmParams* p) { return (p->k + 7) / 8 * 8; }

// The matmul the pre-pass leaves behind, as parameters of the quantised-matmul launcher.
void gemm_view(const OpsnnWqbmmParams* p, OpsnnQmmParams* q, void* wdeq, const void* one)
{
    *q = OpsnnQmmParams{};
    q->mode = OPSNN_QMM_DEQ;
    q->a_dtype = q->b_dtype = q->out_dtype = p->x_dtype;
    q->bias_dtype = p->bias != nullptr ? p->bias_dtype : -1;
    q->scale_b_dtype = ACL_FLOAT;
    q->trans_a = 0;
    q->trans_b = 1;
    q->batch = 1; q->m = p->m; q->n = p->n; q->k = p->k;
    q->a = p->x; q->a_ld = p->x_ld;
    q->b = wdeq; q->b_ld = padded_k(p);
    q->scale_b = one; q->scale_b_len = 1;
    q->group_m = q->group_n = q->group_k = 1;
    q->bias = p->bias;
    q->out = p->y; q->out_ld = p->y_ld; q->out_bs = p->m * p->y_ld;
}

}  // namespace

uint64_t wqbmm_prefill_image_size(const OpsnnWqbmmParams* p)
{
    return (uint64_t)p->n * (uint64_t)padded_k(p) * 2u + 512u;  // dequantised weight, alignment slack, the unit scale
}

uint64_t wqbmm_prefill_workspace_size(const OpsnnWqbmmParams* p) { return p->prep_w != nullptr ? 0 : wqbmm_prefill_image_size(p); }

bool wqbmm_prefill_eligible(const OpsnnWqbmmParams* p)
{
    if (getenv("OPSNN_WQ_NO_PREFILL")) return false;
    if (p->x_dtype != ACL_BF16 && p->x_dtype != ACL_FLOAT16) return false;
    if (p->w_dtype != ACL_INT4 && p->w_dtype != ACL_INT8 && p->w_dtype != ACL_FLOAT8_E4M3FN && p->w_dtype != ACL_FLOAT8_E5M2 &&
        p->w_dtype != ACL_FLOAT4_E2M1)
        return false;
    if (p->m < 1 || p->n < 1 || p->k < 1) return false;
    if (p->x_ld % 8 != 0 || (p->x != nullptr && (reinterpret_cast<uintptr_t>(p->x) & 15) != 0)) return false;
    OpsnnQmmParams q;
    gemm_view(p, &q, reinterpret_cast<void*>(uintptr_t(256)), reinterpret_cast<const void*>(uintptr_t(256)));
    q.a = nullptr;  // alignment of x was checked above; the stand-in addresses only serve the shape rules
    return qmm_umma_eligible(&q);
}

// The dequantisation pre-pass alone: the (n, padded k) 16-bit weight and the unit scale behind it, at `ws` (256-byte aligned).
int32_t wqbmm_prefill_prepass(const OpsnnWqbmmParams* p, uint8_t* ws, cudaStream_t stream)
{
    const int64_t kp = padded_k(p);
    uint16_t* wdeq = reinterpret_cast<uint16_t*>(ws);
    float* one = reinterpret_cast<float*>(ws + (((uint64_t)p->n * kp * 2u + 15u) & ~(uint64_t)15u));
    const int64_t tiles = ((p->n + TN - 1) / TN) * ((p->k + TK - 1) / TK);
    if (tiles > 0x7FFFFFFF) return (int32_t)cudaErrorInvalidConfiguration;
    const bool tile_const_scale = p->group_size == 0 || p->group_size % TK == 0;
    const bool fast = p->w_dtype == ACL_INT4 && !p->trans_w && p->w_ld % 8 == 0 && p->n % 8 == 0 &&
                      (reinterpret_cast<uintptr_t>(p->w) & 3) == 0 && tile_const_scale && p->scale_dtype != ACL_FLOAT8_E8M0;
    const bool bf = p->x_dtype == ACL_BF16;
    const bool pairs = p->w_dtype == ACL_INT4 && !p->trans_w && p->w_ld % 8 == 0 && p->n % 8 == 0 &&
                       (reinterpret_cast<uintptr_t>(p->w) & 3) == 0 && (p->group_size == 0 || p->group_size % 8 == 0) &&
                       p->scale_dtype != ACL_FLOAT8_E8M0 &&
                       getenv("OPSNN_WQ_PREFILL_SIMPLE") == nullptr;
    const bool four = p->w_dtype == ACL_INT4 || p->w_dtype == ACL_FLOAT4_E2M1;
    const int per = four ? 8 : 4;
    const bool rows_path = p->trans_w && p->k % per == 0 && p->w_ld % per == 0 && (p->group_size == 0 || p->group_size % per == 0) &&
                           p->scale_dtype != ACL_FLOAT8_E8M0 && (reinterpret_cast<uintptr_t>(p->w) & 3) == 0 &&
                           getenv("OPSNN_WQ_PREFILL_SIMPLE") == nullptr;
    if (rows_path) {
        const int64_t work = p->n * (p->k / per);
        int64_t grid = (work + NT - 1) / NT;
        if (grid > 148 * 32) grid = 148 * 32;
        if (grid < 1) grid = 1;
        if (bf && four) wq_dequant_nk_rows_kernel<true, 8><<<(unsigned)grid, NT, 0, stream>>>(*p, wdeq, kp, one);
        else if (bf) wq_dequant_nk_rows_kernel<true, 4><<<(unsigned)grid, NT, 0, stream>>>(*p, wdeq, kp, one);
        else if (four) wq_dequant_nk_rows_kernel<false, 8><<<(unsigned)grid, NT, 0, stream>>>(*p, wdeq, kp, one);
        else wq_dequant_nk_rows_kernel<false, 4><<<(unsigned)grid, NT, 0, stream>>>(*p, wdeq, kp, one);
    } else if (pairs) {
        const int64_t ptiles = ((p->n + PN - 1) / PN) * ((p->k + PK - 1) / PK);
        if (ptiles > 0x7FFFFFFF) return (int32_t)cudaErrorInvalidConfiguration;
        const int vec = p->scale_sn == 1 && p->scale_sg % 8 == 0 && (reinterpret_cast<uintptr_t>(p->scale) & 15) == 0 &&
                        (p->offset == nullptr || (reinterpret_cast<uintptr_t>(p->offset) & 15) == 0);
        const size_t sm = (size_t)PN * PP * 4;
        static std::atomic<uint64_t> configured{0};
        once_per_device(configured, [&] {
            cudaFuncSetAttribute(wq_dequant_nk_pairs_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
            return cudaFuncSetAttribute(wq_dequant_nk_pairs_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
        });
        if (bf) wq_dequant_nk_pairs_kernel<true><<<(unsigned)ptiles, NT, sm, stream>>>(*p, wdeq, kp, one, vec);
        else wq_dequant_nk_pairs_kernel<false><<<(unsigned)ptiles, NT, sm, stream>>>(*p, wdeq, kp, one, vec);
    } else if ((p->w_dtype == ACL_INT8 || p->w_dtype == ACL_FLOAT8_E4M3FN || p->w_dtype == ACL_FLOAT8_E5M2) && !p->trans_w &&
               p->n % 4 == 0 && p->w_ld % 4 == 0 && (reinterpret_cast<uintptr_t>(p->w) & 3) == 0 &&
               (p->group_size == 0 || p->group_size % 4 == 0) && p->scale_dtype != ACL_FLOAT8_E8M0 &&
               getenv("OPSNN_WQ_PREFILL_SIMPLE") == nullptr) {
        if (bf) wq_dequant_nk_bytes_kernel<true><<<(unsigned)tiles, NT, 0, stream>>>(*p, wdeq, kp, one);
        else wq_dequant_nk_bytes_kernel<false><<<(unsigned)tiles, NT, 0, stream>>>(*p, wdeq, kp, one);
    } else if (bf && fast) wq_dequant_nk_words_kernel<true><<<(unsigned)tiles, NT, 0, stream>>>(*p, wdeq, kp, one);
    else if (bf) wq_dequant_nk_kernel<true><<<(unsigned)tiles, NT, 0, stream>>>(*p, wdeq, kp, one);
    else if (fast) wq_dequant_nk_words_kernel<false><<<(unsigned)tiles, NT, 0, stream>>>(*p, wdeq, kp, one);
    else wq_dequant_nk_kernel<false><<<(unsigned)tiles, NT, 0, stream>>>(*p, wdeq, kp, one);
    note_launch("wq_dequant_nk");
    return (int32_t)cudaGetLastError();
}

int32_t wqbmm_prefill_launch(const OpsnnWqbmmParams* p, cudaStream_t stream)
{
    uint8_t* ws;
    if (p->prep_w != nullptr) {
        if ((reinterpret_cast<uintptr_t>(p->prep_w) & 255) != 0) return (int32_t)cudaErrorInvalidValue;
        ws = const_cast<uint8_t*>(static_cast<const uint8_t*>(p->prep_w));  // prepared once: nothing to do per call
    } else {
        if (p->workspace == nullptr || p->workspace_size < wqbmm_prefill_workspace_size(p)) return (int32_t)cudaErrorInvalidValue;
        ws = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p->workspace) + 255) & ~(uintptr_t)255);
        const int32_t rc = wqbmm_prefill_prepass(p, ws, stream);
        if (rc != 0) return rc;
    }
    const int64_t kp = padded_k(p);
    uint16_t* wdeq = reinterpret_cast<uint16_t*>(ws);
    float* one = reinterpret_cast<float*>(ws + (((uint64_t)p->n * kp * 2u + 15u) & ~(uint64_t)15u));
    OpsnnQmmParams q;
    gemm_view(p, &q, wdeq, one);
    if (!qmm_umma_eligible(&q)) return (int32_t)cudaErrorInvalidValue;
    return qmm_umma_launch(&q, stream);
}

}  // namespace opsnn
