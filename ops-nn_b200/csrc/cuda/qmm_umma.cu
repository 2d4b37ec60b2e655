// Full-quant matmul on the 5th-generation tensor cores: TMA -> 128B-swizzled shared memory -> tcgen05.mma -> TMEM ->
// fused dequantisation epilogue. Hand-written for sm_100a; no CUTLASS.
//
// Replaces the reference's arch35 kernels for the V3-routed modes of aclnnQuantMatmulV5:
//   int8 per-tensor/-channel(/-token)   quant_batch_matmul_v3/op_kernel/arch35/qbmm_mix_online_dynamic.h:56-147, 646-736
//   fp8 per-block (G-B / B-B)           matmul/common/cmct/kernel/kernel_qbmm_pertile.h:171-443,
//                                        block/block_mmad_pertile.h:262-447, epilogue/block_epilogue_pertile.h:501-883
// and their host tiling (op_host/op_tiling/arch35/adaptive_sliding_window_tiling.cpp:151-327, 563-781): what is left of it
// is the choice of the N tile and the persistent tile order below.
//
// CTA = one 128 x BN output tile at a time, persistent over tiles (tile index = blockIdx.x + i * gridDim.x; consecutive
// CTAs take consecutive M blocks of the same N block, so a wave shares one weight panel through L2).
//   warp EW     : TMA producer. One stage = 128 k-bytes of A (16 KB) and of B (BN x 128 B), 128-byte swizzle.
//   warp EW + 1 : MMA issuer (one elected lane): 4 x tcgen05.mma (K = 32 bytes each) per stage into a TMEM accumulator,
//                 tcgen05.commit releases the stage back to the producer and hands finished accumulators to the epilogue.
//   warps 0..EW-1 : epilogue. Warp w reads TMEM lanes 32*(w%4).. (its output rows) with tcgen05.ld.
// Modes:
//   DEQ       the accumulator (int32 for kind::i8, fp32 for kind::f8f6f4) covers the whole k range; two TMEM buffers let
//             the epilogue of tile i overlap the MMAs of tile i+1. Epilogue = common.cuh::deq_epilogue (exact rounding order).
//   PERBLOCK  every 128-k stage is its own accumulation group: the MMA warp alternates between two TMEM buffers and the
//             epilogue warps (8 of them for BN = 256, each thread owning one row x 128 columns) promote each partial with
//             acc += part * (s1[m, kb] * s2[kb, n/128]) in registers while the next group is being multiplied.
// Operand majorness follows the storage: x1 (m,k) / x2 (n,k) are K-major; x1 (k,m) / x2 (k,n) are MN-major, which
// tcgen05 reads directly for 8-bit types, so no operand is ever transposed in memory.
// Every mbarrier wait is bounded; a wait that gives up raises a CTA-wide abort flag, records the failure in a device
// status word (opsnn_qmm_umma_status) and the CTA tears down normally (TMEM freed).
#include <cstdio>
#include <algorithm>
#include <atomic>
#include <cstdlib>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace opsnn {

namespace {

constexpr int BM = 128;
constexpr int BK = 128;  // bytes of k per stage
constexpr int kATile = BM * BK;

struct UmmaArgs {
    int32_t mode, is_int;
    int32_t a_mn_major, b_mn_major;
    uint32_t idesc;
    int64_t batch, m, n, k;
    int32_t tiles_m, tiles_n, kblocks, stages;
    int64_t num_tiles;
    int32_t a_batched, b_batched;
    int32_t out_dtype, bias_dtype, scale_b_dtype, deq_flags;
    const void* scale_a;
    const void* scale_b;
    int64_t scale_a_len, scale_b_len, sa_bs, sb_bs;
    int32_t group_m, trans_a, trans_b;
    const void* bias;
    int64_t bias_bs;
    void* out;
    int64_t out_ld, out_bs;
    // block-scaled (MX) kernel only: scale-factor atoms in workspace (see qmm_mx_umma.cuh)
    const uint8_t* sfa;
    const uint8_t* sfb;
    int64_t sfa_bs, sfb_bs;  // bytes between batches; 0 broadcasts
    // split-k (dequant kernel, few tiles): work item = (tile, split); every split writes its raw accumulator tile to
    // ks_part, the split that arrives last at the tile's counter sums them in split order and runs the epilogue
    int32_t ksplit;                    // 1: off
    uint32_t* ks_part;                 // [tile][split][128][BN] raw 32-bit accumulators
    unsigned long long* ks_count;      // [tile] (nonce << 8) | arrivals; any other nonce counts as zero arrivals
    unsigned long long ks_nonce;
    // INT4 x INT4 asymmetric per-group on the pair kernel: two 128-deep k-blocks form one accumulation group of 256
    const float* row_sums;      // [m][groups]: sum of x1's row over each k-group (row_sums_kernel)
    const void* b_offset;       // x2Offset [groups][n], FLOAT16
    int32_t groups;
    int32_t test_stall_kblock;  // tests of the give-up path only: >= 0 makes the producer stop issuing copies from this k-block of each
                                // work item on (nothing is in flight then), so the MMA warp's wait for it runs out; 0 / negative: off
};

// Order of the tiles of one batch. m runs fastest inside bands of kBand tile rows; a band is finished over all of n before
// the next one starts. The tiles in flight at one time then span about as many rows as columns, so both operands are
// fetched from L2; with m simply fastest, a matrix of tens of thousands of rows would stream the whole of A from DRAM once
// per tile column. Up to kBand tile rows the order is plain m-fastest.
template <uint32_t kBand>
__device__ __forceinline__ void tile_of(uint32_t r, uint32_t tiles_m, uint32_t tiles_n, uint32_t& tm, uint32_t& tn)
{
    const uint32_t band_tiles = kBand * tiles_n;
    const uint32_t band = r / band_tiles, rr = r - band * band_tiles;
    const uint32_t rows = min(kBand, tiles_m - band * kBand);
    tn = rr / rows;
    tm = band * kBand + (rr - tn * rows);
}

__device__ unsigned int g_umma_status = 0;  // 0 ok; otherwise (role << 8) | reason of the first failed wait
// The same word in pinned host memory (set once per device by arm_status_mirror): the host reads it before the next launch
// without synchronising anything, which is how a give-up turns into an error code of the following call.
__device__ volatile unsigned int* g_umma_status_host = nullptr;

template <int BN>
struct Smem {
    static constexpr int kBTile = BN * BK;
    static constexpr int kStage = kATile + kBTile;
};

__device__ __forceinline__ void report(volatile uint32_t* abort_flag, unsigned int code)
{
    *abort_flag = 1u;
    if (atomicCAS(&g_umma_status, 0u, code) == 0u && g_umma_status_host != nullptr) {
        *g_umma_status_host = code;
        __threadfence_system();
    }
}

// Converts 32 accumulator columns of one output row and stores them. `col` is the first column (global), valid = number
// of columns inside n. Register arrays are only ever indexed with compile-time constants (a run-time index would move
// them to local memory).
__device__ __forceinline__ void store_row32(const UmmaArgs& a, uint8_t* out, int64_t row, int64_t col, const float (&f)[32],
                                            int valid)
{
    if (a.out_dtype == ACL_FLOAT) {
        float* o = reinterpret_cast<float*>(out) + row * a.out_ld + col;
        if (valid == 32 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(o + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (i < valid) o[i] = f[i];
        }
        return;
    }
    if (a.out_dtype == ACL_INT8) {  // requantised: f holds integers in [-128, 127]
        uint32_t q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            q[i] = ((uint32_t)(int)f[4 * i] & 0xFFu) | (((uint32_t)(int)f[4 * i + 1] & 0xFFu) << 8) |
                   (((uint32_t)(int)f[4 * i + 2] & 0xFFu) << 16) | (((uint32_t)(int)f[4 * i + 3] & 0xFFu) << 24);
        }
        uint8_t* o = out + row * a.out_ld + col;
        if (valid == 32 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
            *reinterpret_cast<uint4*>(o) = make_uint4(q[0], q[1], q[2], q[3]);
            *reinterpret_cast<uint4*>(o + 16) = make_uint4(q[4], q[5], q[6], q[7]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (i < valid) o[i] = (uint8_t)(q[i >> 2] >> (8 * (i & 3)));
        }
        return;
    }
    uint32_t pk[16];
    if (a.out_dtype == ACL_BF16) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            pk[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            pk[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
    uint16_t* o = reinterpret_cast<uint16_t*>(out) + row * a.out_ld + col;
    if (valid == 32 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 16; i += 4) *reinterpret_cast<uint4*>(o + 2 * i) = make_uint4(pk[i], pk[i + 1], pk[i + 2], pk[i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (2 * i < valid) o[2 * i] = (uint16_t)(pk[i] & 0xFFFFu);
            if (2 * i + 1 < valid) o[2 * i + 1] = (uint16_t)(pk[i] >> 16);
        }
    }
}

// 32 accumulator columns of one row -> dequantised values, for the common rounding order (no truncation flags):
// f = float(acc + int_bias) * x2Scale [* x1Scale] [+ float_bias]. The flag combinations are template parameters so that
// the per-element code is a handful of instructions; it runs on one warp per scheduler and is latency bound.
template <bool kInt, bool kHasSa, bool kHasFb>
__device__ __forceinline__ void deq_chunk(const uint32_t (&v)[32], const float* sc, const uint32_t* bi, float sav, float (&f)[32])
{
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        const float4 s4 = *reinterpret_cast<const float4*>(sc + i);
        const uint4 b4 = *reinterpret_cast<const uint4*>(bi + i);
        const float ss[4] = {s4.x, s4.y, s4.z, s4.w};
        const uint32_t bb[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float x = kInt ? (float)((int32_t)v[i + j] + (kHasFb ? 0 : (int32_t)bb[j])) : __uint_as_float(v[i + j]);
            x = __fmul_rn(x, ss[j]);
            if (kHasSa) x = __fmul_rn(x, sav);
            if (kHasFb) x = __fadd_rn(x, __uint_as_float(bb[j]));
            f[i + j] = x;
        }
    }
}

// Column scales and bias of an n tile, decoded to 32 bit, into shared memory (128 epilogue threads).
template <int BN>
__device__ __forceinline__ void deq_stage_cols(const UmmaArgs& a, const uint8_t* bias, bool has_ibias, bool has_fbias, int64_t n0,
                                               float* s_scale, uint32_t* s_bias)
{
    for (int c = threadIdx.x; c < BN; c += 128) {
        const int64_t cc = min(n0 + c, a.n - 1);
        float sb = load_deq_scale(a.scale_b, a.scale_b_len == 1 ? 0 : cc, a.scale_b_dtype);
        if (a.deq_flags & OPSNN_DEQ_TRUNC_SCALE_B) sb = trunc19(sb);
        s_scale[c] = sb;
        uint32_t bv = 0u;
        if (has_ibias) bv = (uint32_t)__ldg(reinterpret_cast<const int32_t*>(bias) + cc);
        else if (has_fbias) bv = __float_as_uint(load_as_float(bias, cc, a.bias_dtype));
        s_bias[c] = bv;
    }
}

// One thread's row of NCOLS accumulator columns starting at TMEM address tmem_addr / output column col0: dequantise in the
// reference's order (qbmm_mix_online_dynamic.h:646-736) and store. s_scale / s_bias point at the tile's staged columns,
// offset so that index 0 is col0's entry.
template <int NCOLS>
__device__ __forceinline__ void deq_store_cols(const UmmaArgs& a, uint32_t tmem_addr, uint8_t* out, int64_t row, bool row_ok,
                                               int64_t col0, const float* s_scale, const uint32_t* s_bias, float sav, bool has_sa,
                                               bool has_fbias, bool has_ibias, const uint32_t* ks_row = nullptr, int ks_n = 0,
                                               int64_t ks_stride = 0)
{
                    const int flags = a.deq_flags & ~OPSNN_DEQ_TRUNC_SCALE_B;  // already applied while staging
                    const bool simple = flags == 0 && a.out_dtype != ACL_INT32;
                    const int variant = simple ? ((a.is_int ? 4 : 0) | (has_sa ? 2 : 0) | (has_fbias ? 1 : 0)) : -1;
    #pragma unroll 1
                    for (int c = 0; c < NCOLS; c += 32) {
                        uint32_t v[32];
                        if (ks_row == nullptr) {
                            ptx::tmem_ld32(tmem_addr + c, v);
                            ptx::tmem_ld_wait();
                        } else {
                            // split-k: the accumulator is the sum of the splits' partial tiles, in split order (deterministic)
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = 0u;
                            for (int sp = 0; sp < ks_n; ++sp) {
                                const uint4* src = reinterpret_cast<const uint4*>(ks_row + sp * ks_stride + c);
#pragma unroll
                                for (int q = 0; q < 8; ++q) {
                                    const uint4 t = __ldcg(src + q);
                                    if (a.is_int) {
                                        v[4 * q] += t.x; v[4 * q + 1] += t.y; v[4 * q + 2] += t.z; v[4 * q + 3] += t.w;
                                    } else {
                                        v[4 * q] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * q]), __uint_as_float(t.x)));
                                        v[4 * q + 1] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * q + 1]), __uint_as_float(t.y)));
                                        v[4 * q + 2] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * q + 2]), __uint_as_float(t.z)));
                                        v[4 * q + 3] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * q + 3]), __uint_as_float(t.w)));
                                    }
                                }
                            }
                        }
                        const int64_t col = col0 + c;
                        const int valid = (int)max((int64_t)0, min((int64_t)32, a.n - col));
                        if (row_ok && valid > 0) {
                            if (a.out_dtype == ACL_INT32) {
                                int32_t* o = reinterpret_cast<int32_t*>(out) + row * a.out_ld + col;
    #pragma unroll
                                for (int i = 0; i < 32; ++i)
                                    if (i < valid) o[i] = (int32_t)v[i] + (has_ibias ? (int32_t)s_bias[c + i] : 0);
                            } else {
                                float f[32];
                                switch (variant) {
                                    case 0: deq_chunk<false, false, false>(v, s_scale + c, s_bias + c, sav, f); break;
                                    case 1: deq_chunk<false, false, true>(v, s_scale + c, s_bias + c, sav, f); break;
                                    case 2: deq_chunk<false, true, false>(v, s_scale + c, s_bias + c, sav, f); break;
                                    case 3: deq_chunk<false, true, true>(v, s_scale + c, s_bias + c, sav, f); break;
                                    case 4: deq_chunk<true, false, false>(v, s_scale + c, s_bias + c, sav, f); break;
                                    case 5: deq_chunk<true, false, true>(v, s_scale + c, s_bias + c, sav, f); break;
                                    case 6: deq_chunk<true, true, false>(v, s_scale + c, s_bias + c, sav, f); break;
                                    case 7: deq_chunk<true, true, true>(v, s_scale + c, s_bias + c, sav, f); break;
                                    default:
    #pragma unroll
                                        for (int i = 0; i < 32; ++i) {
                                            float x;
                                            if (a.is_int) x = (float)((int32_t)v[i] + (has_ibias ? (int32_t)s_bias[c + i] : 0));
                                            else x = __uint_as_float(v[i]);
                                            if (flags & OPSNN_DEQ_REQUANT)
                                                f[i] = requant_s9(x, s_scale[c + i], a.scale_b, a.scale_b_len == 1 ? 0 : min(col + i, a.n - 1), flags);
                                            else f[i] = deq_epilogue(x, s_scale[c + i], sav, has_sa, __uint_as_float(s_bias[c + i]), has_fbias, flags);
                                        }
                                        break;
                                }
                                store_row32(a, out, row, col, f, valid);
                            }
                        }
                    }
}

// Per-block promotion of one accumulator value into the running fp32 sum. fp8: one fused multiply-add. int8: the
// reference rounds the product and the sum separately (float32(int32 partial) * (s1 * s2), then +=), and the int8 mode is
// tested bit for bit, so it is a multiply and an add here too; |partial| <= 128 * 127 * 127 < 2^22, so the conversion is
// the exact add-a-constant form (integer add + float subtract) rather than the slower convert instruction.
template <ptx::MmaKind kKind>
__device__ __forceinline__ float promote(uint32_t v, float sc, float acc)
{
    if (kKind == ptx::MmaKind::kI8) {
        const float f = __fsub_rn(__uint_as_float(v + 0x4B400000u), 12582912.f);
        return __fadd_rn(acc, __fmul_rn(f, sc));
    }
    return fmaf(__uint_as_float(v), sc, acc);
}

template <int BN, bool kPerBlock, ptx::MmaKind kKind, int EW = 4>
__global__ void __launch_bounds__((EW + 2) * 32, 1)
qmm_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const UmmaArgs a)
{
    // EW epilogue warps: warp w reads TMEM lane quarter w % 4 (a hardware rule) and the column slice w / 4
    static_assert(EW % 4 == 0 && (kPerBlock || EW == 4), "dequant epilogue is written for four warps");
    constexpr int kCols = BN * 4 / EW;  // accumulator columns one epilogue thread handles
    static_assert(kCols >= 32, "one epilogue thread handles at least 32 columns");
    constexpr int kStage = Smem<BN>::kStage;
    constexpr uint32_t kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;  // two accumulator buffers

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)a.stages * kStage);
    uint64_t* full = bars;                    // [stages]
    uint64_t* empty = bars + a.stages;        // [stages]
    uint64_t* tfull = bars + 2 * a.stages;    // [2]
    uint64_t* tempty = tfull + 2;             // [2]
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile uint32_t* abort_flag = tmem_ptr + 1;
    float* s_scale = reinterpret_cast<float*>(tmem_ptr + 4);  // [BN] x2Scale of the tile's columns, decoded to fp32
    uint32_t* s_bias = reinterpret_cast<uint32_t*>(s_scale + BN);  // [BN] bias of the tile's columns: int32 bits or fp32 bits

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&tfull[b], 1);
            ptx::mbar_init(&tempty[b], EW);  // one arrival per epilogue warp
        }
        *abort_flag = 0u;
        ptx::fence_mbar_init();
    }
    if (warp == EW + 1) ptx::tmem_alloc(tmem_ptr, kTmemCols);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;

    const uint32_t tiles_per_batch = (uint32_t)a.tiles_m * (uint32_t)a.tiles_n;
    const uint32_t ntiles = (uint32_t)a.num_tiles;
    const uint32_t ks = kPerBlock ? 1u : (uint32_t)a.ksplit;  // split-k factor; work item = tile * ks + split
    const uint32_t nwork = ntiles * ks;

    if (warp == EW) {
        // ======================= TMA producer =======================
        // The whole warp runs the loop (uniform control flow: waits, ring counters and coordinates stay cheap); one
        // elected lane issues the copies. Ring position is kept as (stage, parity) counters, parameters in registers.
        if (lane == 0) {
            ptx::tma_prefetch_desc(&map_a);
            ptx::tma_prefetch_desc(&map_b);
        }
        __syncwarp();
        uint32_t s = 0, par = 0;
        bool ok = true;
        const uint32_t stages = (uint32_t)a.stages;
        const int kblocks = a.kblocks;
        const bool a_mn = a.a_mn_major != 0, b_mn = a.b_mn_major != 0;
        const uint32_t smem0 = ptx::smem_u32(smem), full0 = ptx::smem_u32(full), empty0 = ptx::smem_u32(empty);
        for (uint32_t work = blockIdx.x; work < nwork && ok; work += gridDim.x) {
            const uint32_t tile = work / ks, split = work - tile * ks;
            const uint32_t b = tile / tiles_per_batch, r = tile % tiles_per_batch;
            uint32_t tm, tn;
            tile_of<16>(r, (uint32_t)a.tiles_m, (uint32_t)a.tiles_n, tm, tn);
            const int32_t m0 = (int32_t)tm * BM, n0 = (int32_t)tn * BN;
            const int32_t ba = a.a_batched ? (int32_t)b : 0, bb = a.b_batched ? (int32_t)b : 0;
            const int kb_begin = (int)((int64_t)split * kblocks / (int)ks), kb_end = (int)((int64_t)(split + 1) * kblocks / (int)ks);
            int32_t kk = kb_begin * BK;
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (a.test_stall_kblock > 0 && kb >= a.test_stall_kblock) {  // test switch: the producer simply stops
                    ok = false;
                    break;
                }
                if (!ptx::mbar_wait_a(empty0 + 8u * s, par ^ 1u, abort_flag)) {
                    report(abort_flag, (1u << 8) | 1u);
                    ok = false;
                    break;
                }
                if (ptx::elect_one()) {
                    const uint32_t fb = full0 + 8u * s, sa = smem0 + s * (uint32_t)kStage, sb = sa + (uint32_t)kATile;
                    ptx::mbar_expect_tx_a(fb, (uint32_t)kStage);
                    ptx::tma_load_3d_a(sa, &map_a, fb, a_mn ? m0 : kk, a_mn ? kk : m0, ba);
                    ptx::tma_load_3d_a(sb, &map_b, fb, b_mn ? n0 : kk, b_mn ? kk : n0, bb);
                    if (BN > 128 && b_mn) ptx::tma_load_3d_a(sb + 128u * BK, &map_b, fb, n0 + 128, kk, bb);
                }
                __syncwarp();
                kk += BK;
                if (++s == stages) {
                    s = 0;
                    par ^= 1u;
                }
            }
        }
    } else if (warp == EW + 1) {
        // ======================= MMA issuer =======================
        // Same shape: whole warp, one elected lane issues the four MMAs of a stage and the commits. A stage of BN = 256
        // is 512 tensor-core cycles; the loop below has to cost this warp less than that per stage.
        uint32_t s = 0, par = 0, grp = 0;
        bool ok = true;
        const uint32_t smem0 = ptx::smem_u32(smem), full0 = ptx::smem_u32(full), empty0 = ptx::smem_u32(empty);
        const uint32_t tfull0 = ptx::smem_u32(tfull), tempty0 = ptx::smem_u32(tempty);
        // descriptors: only the 14-bit start-address field (low word) changes: stage base, then the k step inside the
        // stage. K-major operand: a k step is 32 bytes along the swizzled row; MN-major: 32 k-rows = 4 KB (units of 16 B)
        const uint64_t da0 = a.a_mn_major ? ptx::make_smem_desc(smem0, 128 * BK, 1024, 2) : ptx::make_smem_desc(smem0, 0, 1024, 2);
        // n-major B narrower than a 128-byte swizzle row (BN 64 / 32): rows of BN bytes in the 64- / 32-byte swizzle
        // (layout type 4 / 6), 8 rows = 8 * BN bytes, one MMA = 32 rows
        const uint64_t db0 = !a.b_mn_major ? ptx::make_smem_desc(smem0 + kATile, 0, 1024, 2)
                             : BN >= 128   ? ptx::make_smem_desc(smem0 + kATile, 128 * BK, 1024, 2)
                                           : ptx::make_smem_desc(smem0 + kATile, BN * BK, 8 * BN, BN == 64 ? 4 : 6);
        const uint32_t a_lo = (uint32_t)da0, b_lo = (uint32_t)db0;
        const uint64_t a_hi = da0 & 0xFFFFFFFF00000000ull, b_hi = db0 & 0xFFFFFFFF00000000ull;
        const uint32_t a_k1 = a.a_mn_major ? 256u : 2u, b_k1 = !a.b_mn_major ? 2u : (BN >= 128 ? 256u : 2u * BN);
        const uint32_t stages = (uint32_t)a.stages, idesc = a.idesc;
        const int kblocks = a.kblocks;
        for (uint32_t work = blockIdx.x; work < nwork && ok; work += gridDim.x) {
            const uint32_t split = work % ks;
            const int kb_begin = (int)((int64_t)split * kblocks / (int)ks), kb_end = (int)((int64_t)(split + 1) * kblocks / (int)ks);
            uint32_t acc = 0u;
            if (!kPerBlock) {
                if (!ptx::mbar_wait_a(tempty0 + 8u * (grp & 1u), ((grp >> 1) & 1u) ^ 1u, abort_flag)) {
                    report(abort_flag, (2u << 8) | 1u);
                    ok = false;
                    break;
                }
            }
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (kPerBlock) {
                    if (!ptx::mbar_wait_a(tempty0 + 8u * (grp & 1u), ((grp >> 1) & 1u) ^ 1u, abort_flag)) {
                        report(abort_flag, (2u << 8) | 1u);
                        ok = false;
                        break;
                    }
                }
                if (!ptx::mbar_wait_a(full0 + 8u * s, par, abort_flag)) {
                    report(abort_flag, (2u << 8) | 2u);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                if (ptx::elect_one()) {
                    const uint32_t stage_off = (s * (uint32_t)kStage) >> 4;
                    const uint32_t d = tmem_base + (grp & 1u) * BN;
                    const uint32_t al = a_lo + stage_off, bl = b_lo + stage_off;
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        ptx::umma<kKind>(d, a_hi | (uint64_t)(al + k * a_k1), b_hi | (uint64_t)(bl + k * b_k1), idesc,
                                         k == 0 ? acc : 1u);
                    ptx::umma_commit_a(empty0 + 8u * s);
                    if (kPerBlock) ptx::umma_commit_a(tfull0 + 8u * (grp & 1u));
                }
                __syncwarp();
                if (kPerBlock) ++grp;
                else acc = 1u;
                if (++s == stages) {
                    s = 0;
                    par ^= 1u;
                }
            }
            if (!kPerBlock && ok) {
                if (ptx::elect_one()) ptx::umma_commit_a(tfull0 + 8u * (grp & 1u));
                __syncwarp();
                ++grp;
            }
        }
    } else {
        // ======================= epilogue warps =======================
        const int quad = warp & 3, half = warp >> 2;
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        uint32_t grp = 0;
        bool ok = true;
        for (uint32_t work = blockIdx.x; work < nwork && ok; work += gridDim.x) {
            const uint32_t tile = work / ks, split = work - tile * ks;
            const uint32_t b = tile / tiles_per_batch, r = tile % tiles_per_batch;
            uint32_t tm, tn;
            tile_of<16>(r, (uint32_t)a.tiles_m, (uint32_t)a.tiles_n, tm, tn);
            const int64_t m0 = (int64_t)tm * BM, n0 = (int64_t)tn * BN;
            const int64_t row = m0 + quad * 32 + lane;
            const bool row_ok = row < a.m;
            const int out_bytes = out_elem_bytes(a.out_dtype);
            uint8_t* out = reinterpret_cast<uint8_t*>(a.out) + b * a.out_bs * out_bytes;
            const int64_t colbase = n0 + half * kCols;
            if (!kPerBlock) {
                const uint32_t buf = grp & 1, gpar = (grp >> 1) & 1;
                const uint8_t* bias = reinterpret_cast<const uint8_t*>(a.bias);
                if (bias != nullptr) bias += b * a.bias_bs * ((a.bias_dtype == ACL_FLOAT || a.bias_dtype == ACL_INT32) ? 4 : 2);
                const bool has_sa = a.scale_a != nullptr;
                const float sav = (has_sa && row_ok) ? reinterpret_cast<const float*>(a.scale_a)[a.scale_a_len == 1 ? 0 : row] : 1.f;
                const bool has_fbias = bias != nullptr && a.bias_dtype != ACL_INT32;
                const bool has_ibias = bias != nullptr && a.bias_dtype == ACL_INT32;
                // Stage the tile's column scales and bias (decoded to 32 bit) while the main loop is still running.
                // 128 epilogue threads, named barrier 1; every epilogue warp executes every barrier of every tile.
                asm volatile("bar.sync 1, 128;" ::: "memory");  // the previous tile's readers are done
                deq_stage_cols<BN>(a, bias, has_ibias, has_fbias, n0, s_scale, s_bias);
                if (!ptx::mbar_wait_relaxed(&tfull[buf], gpar, abort_flag)) report(abort_flag, (3u << 8) | 1u);
                // the four epilogue warps leave together: a named barrier is only safe if nobody has left the loop
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (*abort_flag != 0u) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                if (ks == 1u) {
                    deq_store_cols<kCols>(a, tmem_base + lane_addr + buf * BN, out, row, row_ok, colbase, s_scale, s_bias, sav, has_sa,
                                          has_fbias, has_ibias);
                } else {
                    // split-k: park this split's raw accumulator rows in the workspace; whoever completes the tile's count reduces
                    uint32_t* my_row = a.ks_part + (((int64_t)tile * ks + split) * BM + (quad * 32 + lane)) * BN;
#pragma unroll 1
                    for (int c = 0; c < kCols; c += 32) {
                        uint32_t v[32];
                        ptx::tmem_ld32(tmem_base + lane_addr + buf * BN + c, v);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            __stcg(reinterpret_cast<uint4*>(my_row + c) + q, make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
                    }
                    __threadfence();
                    asm volatile("bar.sync 1, 128;" ::: "memory");  // all four warps' rows are written and fenced
                    if (threadIdx.x == 0) {
                        unsigned long long* cnt = a.ks_count + tile;
                        unsigned long long cur = *reinterpret_cast<volatile unsigned long long*>(cnt), want = 0ull;
                        bool done = false;
                        for (int it = 0; it < 64 && !done; ++it) {  // at most ks - 1 other splits can get in between
                            want = ((cur >> 8) == a.ks_nonce) ? cur + 1ull : ((a.ks_nonce << 8) | 1ull);
                            const unsigned long long prev = atomicCAS(cnt, cur, want);
                            done = prev == cur;
                            cur = prev;
                        }
                        if (!done) report(abort_flag, (3u << 8) | 3u);
                        tmem_ptr[2] = (done && (uint32_t)(want & 0xFFull) == ks) ? 1u : 0u;
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (tmem_ptr[2] != 0u) {
                        __threadfence();
                        const uint32_t* tile_row = a.ks_part + ((int64_t)tile * ks * BM + (quad * 32 + lane)) * BN;
                        deq_store_cols<kCols>(a, 0u, out, row, row_ok, colbase, s_scale, s_bias, sav, has_sa, has_fbias, has_ibias, tile_row,
                                              (int)ks, (int64_t)BM * BN);
                    }
                }
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&tempty[buf]);
                ++grp;
            } else {
                float acc[kCols];
#pragma unroll
                for (int i = 0; i < kCols; ++i) acc[i] = 0.f;
                const float* s1 = reinterpret_cast<const float*>(a.scale_a) + b * a.sa_bs;
                const float* s2 = reinterpret_cast<const float*>(a.scale_b) + b * a.sb_bs;
                const int64_t mg = (row_ok ? row : 0) / a.group_m;
                const int64_t n_mg = (a.m + a.group_m - 1) / a.group_m, n_ng = (a.n + 127) / 128;
                const int64_t ng = min(colbase / 128, n_ng - 1);
                // scale of a (row, k-block, n-block): x1Scale is (m/gm, kblocks) or, transposed, (kblocks, m/gm); x2Scale is
                // (kblocks, n/128) or, transposed, (n/128, kblocks). Four k-blocks' products are fetched while the previous
                // four are consumed: an L2 round trip in front of every k-block would otherwise bound the whole kernel.
                auto load_s1 = [&](int kb) {
                    kb = min(kb, a.kblocks - 1);
                    return a.trans_a ? __ldg(s1 + kb * n_mg + mg) : __ldg(s1 + mg * a.kblocks + kb);
                };
                auto load_s2 = [&](int kb) {
                    kb = min(kb, a.kblocks - 1);
                    return a.trans_b ? __ldg(s2 + ng * a.kblocks + kb) : __ldg(s2 + kb * n_ng + ng);
                };
                // the raw values wait in registers; multiplying them here would stall on the loads just issued
                float s1_next[4], s2_next[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    s1_next[j] = load_s1(j);
                    s2_next[j] = load_s2(j);
                }
                for (int kb0 = 0; kb0 < a.kblocks && ok; kb0 += 4) {
                    float sc_cur[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) sc_cur[j] = __fmul_rn(s1_next[j], s2_next[j]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        s1_next[j] = load_s1(kb0 + 4 + j);
                        s2_next[j] = load_s2(kb0 + 4 + j);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (kb0 + j >= a.kblocks) break;
                        const uint32_t buf = grp & 1, gpar = (grp >> 1) & 1;
                        const float sc = sc_cur[j];
                        if (!ptx::mbar_wait(&tfull[buf], gpar, abort_flag)) {
                            report(abort_flag, (3u << 8) | 2u);
                            ok = false;
                            break;
                        }
                        ptx::tc_fence_after();
                        // TMEM -> registers in chunks of 16 columns, one chunk in flight while the previous one is folded into
                        // acc; the buffer goes back to the MMA warp as soon as the last chunk has arrived
                        constexpr int W = 16;
                        const uint32_t t0 = tmem_base + lane_addr + buf * BN + half * kCols;
                        uint32_t va[W], vb[W];
                        ptx::tmem_ld16(t0, va);
#pragma unroll
                        for (int c = 0; c < kCols; c += 2 * W) {
                            ptx::tmem_ld_wait();
                            ptx::tmem_ld16(t0 + c + W, vb);
#pragma unroll
                            for (int i = 0; i < W; ++i) acc[c + i] = promote<kKind>(va[i], sc, acc[c + i]);
                            ptx::tmem_ld_wait();
                            if (c + 2 * W < kCols) {
                                ptx::tmem_ld16(t0 + c + 2 * W, va);
                            } else {
                                ptx::tc_fence_before();
                                __syncwarp();
                                if (lane == 0) ptx::mbar_arrive(&tempty[buf]);
                            }
#pragma unroll
                            for (int i = 0; i < W; ++i) acc[c + W + i] = promote<kKind>(vb[i], sc, acc[c + W + i]);
                        }
                        ++grp;
                    }
                }
                if (ok && row_ok) {
#pragma unroll
                    for (int c = 0; c < kCols; c += 32) {
                        const int64_t col = colbase + c;
                        const int valid = (int)max((int64_t)0, min((int64_t)32, a.n - col));
                        if (valid > 0) {
                            float f[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i) f[i] = acc[c + i];
                            if (a.bias != nullptr) {
                                const uint8_t* bias = reinterpret_cast<const uint8_t*>(a.bias) +
                                                      b * a.bias_bs * ((a.bias_dtype == ACL_FLOAT || a.bias_dtype == ACL_INT32) ? 4 : 2);
#pragma unroll
                                for (int i = 0; i < 32; ++i)
                                    if (i < valid) f[i] = __fadd_rn(f[i], load_as_float(bias, col + i, a.bias_dtype));
                            }
                            store_row32(a, out, row, col, f, valid);
                        }
                    }
                }
            }
        }
    }
    // ---- teardown: everyone meets here, also after an aborted wait; then the allocating warp frees TMEM ----
    if (*abort_flag != 0u) __nanosleep(200000);  // lets bulk copies that are still in flight land before the CTA leaves
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == EW + 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace

// =================================================== host side ===================================================
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode()
{
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

// 3-D byte tensor (inner bytes, rows, batch) with a (128, box_rows, 1) box and 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows, uint64_t batch, uint64_t row_pitch,
              uint64_t batch_pitch, uint32_t box_rows, uint32_t box_inner = 128)
{
    EncodeFn enc = get_encode();
    if (enc == nullptr) return false;
    cuuint64_t dims[3] = {inner, rows, batch};
    cuuint64_t strides[2] = {row_pitch, batch_pitch ? batch_pitch : row_pitch * rows};
    if (strides[1] % 16 != 0) strides[1] = ((strides[1] + 15) / 16) * 16;  // only reached when batch == 1
    cuuint32_t box[3] = {box_inner, box_rows, 1};  // rows of 128 bytes in the 128-byte swizzle, or of 64 bytes in the 64-byte one
    cuuint32_t estr[3] = {1, 1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE,
               box_inner == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : (box_inner == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_128B),
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() { return current_sm_count(); }

bool is_fp8(int dt) { return dt == ACL_FLOAT8_E4M3FN || dt == ACL_FLOAT8_E5M2; }

// Host tile selection: the widest N tile that still yields about one tile per SM.
int pick_bn(const OpsnnQmmParams* p)
{
    if (const char* e = getenv("OPSNN_QMM_BN")) {
        int v = atoi(e);
        if (v == 32 || v == 64 || v == 128 || v == 256) return v;
    }
    // per-block: the promotion epilogue (registers: 128 accumulators per thread) keeps up with 128-column tiles only
    if (p->mode == OPSNN_QMM_PERBLOCK) return 128;
    const int64_t tiles_m = (p->m + BM - 1) / BM;
    const int sms = 148;
    const int lo = p->mode == OPSNN_QMM_PERBLOCK ? 128 : 32;
    for (int bn = 256; bn > lo; bn /= 2) {
        if (bn / 2 >= p->n) continue;  // half the width still covers n
        const int64_t tiles = p->batch * tiles_m * ((p->n + bn - 1) / bn);
        if (tiles >= sms) return bn;
    }
    return lo;
}

// Split-k for problems with few output tiles (a decode-sized m against a square weight). Opt-in (OPSNN_QMM_KSPLIT=2..8):
// on m128 k4096 n4096 the partial tiles' round trip through L2 and the reduction cost more than the shorter main loop
// saves (44 us against 17 us), so the host never picks it by itself; 1 = off.
int pick_ksplit(const OpsnnQmmParams* p, int bn, int kblocks)
{
    (void)bn;
    if (p->mode != OPSNN_QMM_DEQ) return 1;
    if (const char* e = getenv("OPSNN_QMM_KSPLIT")) {
        const int v = atoi(e);
        return (v >= 1 && v <= 8 && v * 2 <= kblocks) ? v : 1;
    }
    return 1;
}

uint64_t ksplit_workspace(const OpsnnQmmParams* p)
{
    if (p->mode != OPSNN_QMM_DEQ) return 0;
    const bool f16 = p->a_dtype == ACL_BF16 || p->a_dtype == ACL_FLOAT16;
    const int kblocks = (int)((p->k * (f16 ? 2 : 1) + BK - 1) / BK);
    const int bn = pick_bn(p);
    const int ks = pick_ksplit(p, bn, kblocks);
    if (ks == 1) return 0;
    const uint64_t tiles = (uint64_t)(p->batch * ((p->m + BM - 1) / BM) * ((p->n + bn - 1) / bn));
    return tiles * (uint64_t)ks * BM * (uint64_t)bn * 4u + tiles * 8u + 512u;
}

unsigned long long next_ks_nonce()
{
    static std::atomic<unsigned long long> seq{0x5EED0000ull};
    return seq.fetch_add(1, std::memory_order_relaxed) + 1;
}

template <int BN, bool PB, ptx::MmaKind KIND, int EW = 4>
int32_t launch_one(const CUtensorMap& ma, const CUtensorMap& mb, UmmaArgs& a, cudaStream_t stream)
{
    constexpr int kStage = Smem<BN>::kStage;
    int stages = (227 * 1024 - 2048) / kStage;
    if (stages > 8) stages = 8;
    if (stages > a.kblocks + 1) stages = a.kblocks + 1 > 2 ? a.kblocks + 1 : 2;
    a.stages = stages;
    const size_t smem = (size_t)stages * kStage + 1024 + 256 + 2 * BN * 4;
    static std::atomic<uint64_t> configured{0};
    auto kern = qmm_umma_kernel<BN, PB, KIND, EW>;
    if (once_per_device(configured, [&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); }) != cudaSuccess)
        return (int32_t)cudaGetLastError();
    const int64_t work = a.num_tiles * (PB ? 1 : a.ksplit);
    int64_t grid = work < sm_count() ? work : sm_count();
    kern<<<(unsigned)grid, (EW + 2) * 32, smem, stream>>>(ma, mb, a);
    note_launch(PB ? "qmm_umma_perblock" : (a.ksplit > 1 ? "qmm_umma_deq_splitk" : "qmm_umma_deq"));
    return (int32_t)cudaGetLastError();
}

// Per-block epilogue width. The promotion is bound by instruction issue (one warp instruction per clock and SM
// sub-partition): fp8 needs one fused multiply-add per element and four warps keep up; int8 needs four instructions
// per element (exact conversion, multiply, add) and a second warp per sub-partition hides the TMEM load waits.
template <ptx::MmaKind KIND>
int32_t launch_pb(int bn, const CUtensorMap& ma, const CUtensorMap& mb, UmmaArgs& a, cudaStream_t stream)
{
    if (bn == 256) return launch_one<256, true, KIND, 8>(ma, mb, a, stream);
    int ew = KIND == ptx::MmaKind::kI8 ? 8 : 4;
    if (const char* e = getenv("OPSNN_QMM_PB_EW")) ew = atoi(e);
    if (ew == 8) return launch_one<128, true, KIND, 8>(ma, mb, a, stream);
    return launch_one<128, true, KIND, 4>(ma, mb, a, stream);
}

template <bool PB, ptx::MmaKind KIND>
int32_t launch_bn(int bn, const CUtensorMap& ma, const CUtensorMap& mb, UmmaArgs& a, cudaStream_t stream)
{
    if (PB) return launch_pb<KIND>(bn, ma, mb, a, stream);
    switch (bn) {
        case 256: return launch_one<256, false, KIND>(ma, mb, a, stream);
        case 128: return launch_one<128, false, KIND>(ma, mb, a, stream);
        case 64: if (!PB) return launch_one<64, false, KIND>(ma, mb, a, stream); break;
        case 32: if (!PB) return launch_one<32, false, KIND>(ma, mb, a, stream); break;
        default: break;
    }
    return (int32_t)cudaErrorInvalidValue;
}

}  // namespace

#include "qmm_mx_umma.cuh"
#include "qmm_umma_pair.cuh"
#include "qmm_umma_pair_pb.cuh"
#include "qmm_mx_umma_pair.cuh"

bool qmm_umma_eligible(const OpsnnQmmParams* p)
{
    if (getenv("OPSNN_QMM_NO_UMMA")) return false;
    if (p->mode == OPSNN_QMM_MX) return qmm_mx_umma_eligible(p);
    const bool i8 = p->a_dtype == ACL_INT8 && p->b_dtype == ACL_INT8;
    const bool f8 = is_fp8(p->a_dtype) && is_fp8(p->b_dtype);
    // bf16 x bf16 / fp16 x fp16 (the weight-only quant prefill path hands over a dequantised weight): both operands
    // k-contiguous; seen as bytes they are the 8-bit k-major case with twice the k extent
    const bool f16 = p->a_dtype == p->b_dtype && (p->a_dtype == ACL_BF16 || p->a_dtype == ACL_FLOAT16);
    const int es = f16 ? 2 : 1;
    if (p->mode == OPSNN_QMM_DEQ) {
        if (!i8 && !f8 && !f16) return false;
        if (f16 && (p->trans_a || !p->trans_b)) return false;
    } else if (p->mode == OPSNN_QMM_PERBLOCK) {
        if ((!f8 && !i8) || p->group_k != 128 || p->group_n != 128 || (p->group_m != 1 && p->group_m != 128)) return false;
    } else if (p->mode == OPSNN_QMM_PERGROUP_ASYM) {
        // INT4 x INT4 asymmetric per-group, operands already widened to INT8: groups of two 128-deep k-blocks on the pair kernel
        if (!i8 || p->group_k != 256 || p->batch != 1 || p->b_offset == nullptr || p->scale_a == nullptr || p->bias != nullptr) return false;
        if (getenv("OPSNN_QMM_ASYM_GENERIC")) return false;
    } else {
        return false;
    }
    if (p->out_dtype != ACL_BF16 && p->out_dtype != ACL_FLOAT16 && p->out_dtype != ACL_FLOAT &&
        !((p->out_dtype == ACL_INT32 || (p->out_dtype == ACL_INT8 && (p->deq_flags & OPSNN_DEQ_REQUANT))) && i8 &&
          p->mode == OPSNN_QMM_DEQ))
        return false;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (p->a != nullptr && (!al16(p->a) || !al16(p->b))) return false;
    if ((p->a_ld * es) % 16 != 0 || (p->b_ld * es) % 16 != 0 || (p->a_bs * es) % 16 != 0 || (p->b_bs * es) % 16 != 0) return false;
    if (p->m < 1 || p->n < 1 || p->k < 1 || p->batch < 1 || p->batch > 0x7FFFFFFF) return false;
    if (p->batch * ((p->m + 127) / 128) * ((p->n + 31) / 32) > 0x7FFFFFFF) return false;  // tile index is 32 bit
    if (p->m > 0x7FFFFF00 || p->n > 0x7FFFFF00 || p->k > 0x7FFFFF00) return false;
    return true;
}

uint64_t qmm_umma_workspace_size(const OpsnnQmmParams* p)
{
    if (p->mode == OPSNN_QMM_MX) return qmm_mx_umma_workspace_size(p);
    if (p->mode == OPSNN_QMM_PERGROUP_ASYM) return (uint64_t)p->m * (uint64_t)((p->k + 255) / 256) * 4u + 256u;  // row sums per k-group
    return p->mode == OPSNN_QMM_PERBLOCK ? 0 : ksplit_workspace(p);
}

namespace {

std::atomic<unsigned int*> g_status_host_word{nullptr};
std::atomic<uint64_t> g_status_armed{0};

// Once per process: one pinned, device-visible word. Once per device: its address into g_umma_status_host.
cudaError_t arm_status_mirror()
{
    return once_per_device(g_status_armed, [] {
        unsigned int* w = g_status_host_word.load(std::memory_order_acquire);
        if (w == nullptr) {
            unsigned int* fresh = nullptr;
            cudaError_t rc = cudaHostAlloc(reinterpret_cast<void**>(&fresh), 64, cudaHostAllocPortable | cudaHostAllocMapped);
            if (rc != cudaSuccess) return rc;
            *fresh = 0u;
            if (g_status_host_word.compare_exchange_strong(w, fresh)) w = fresh;
            else cudaFreeHost(fresh);
        }
        unsigned int* dptr = nullptr;
        cudaError_t rc = cudaHostGetDevicePointer(reinterpret_cast<void**>(&dptr), w, 0);
        if (rc != cudaSuccess) return rc;
        return cudaMemcpyToSymbol(g_umma_status_host, &dptr, sizeof(dptr));
    });
}

}  // namespace

void set_err(const char* fmt, ...);  // thread-local text behind aclGetRecentErrMsg (host library)

// Called by every tensor-core launcher before it enqueues anything: non-zero when an earlier tensor-core kernel of this process
// gave up a bounded wait (its output is undefined). The condition is sticky until opsnn_qmm_umma_status(1) clears it.
int32_t umma_prelaunch_check()
{
    if (arm_status_mirror() != cudaSuccess) {
        cudaGetLastError();
        return 0;  // no mirror (host allocation refused): the device word is still there for opsnn_qmm_umma_status
    }
    const unsigned int* w = g_status_host_word.load(std::memory_order_acquire);
    const unsigned int code = w ? *reinterpret_cast<const volatile unsigned int*>(w) : 0u;
    if (code == 0u) return 0;
    set_err("an earlier tensor-core kernel gave up a bounded wait (role %u, reason %u): its output is undefined; "
            "opsnn_qmm_umma_status(1) clears the condition",
            code >> 8, code & 0xFFu);
    return (int32_t)cudaErrorLaunchFailure;
}

int32_t qmm_umma_launch(const OpsnnQmmParams* p, cudaStream_t stream)
{
    if (const int32_t bad = umma_prelaunch_check()) return bad;
    if (p->mode == OPSNN_QMM_MX) return qmm_mx_umma_launch(p, stream);
    const bool pair = pair_worthwhile(p) && p->mode == OPSNN_QMM_DEQ && p->out_dtype != ACL_INT32 && p->out_dtype != ACL_INT8;
    // per-block on CTA pairs: 256 x 128 tiles
    const bool asym = p->mode == OPSNN_QMM_PERGROUP_ASYM;
    const bool pair_pb = asym || pair_pb_worthwhile(p);
    const uint8_t* b_ptr = static_cast<const uint8_t*>(p->b);
    int64_t b_ld = p->b_ld, b_bs = p->b_bs;
    int b_trans = p->trans_b;
    const int pb_bn = asym ? 128 : (pair_pb ? pair_pb_bn(p) : 0);
    const int bn = pair ? 256 : (pair_pb ? pb_bn : pick_bn(p));
    const int bm = (pair || pair_pb) ? 256 : BM;
    UmmaArgs a{};
    a.mode = p->mode;
    a.is_int = p->a_dtype == ACL_INT8;
    a.a_mn_major = p->trans_a ? 1 : 0;   // stored (k,m): m contiguous
    a.b_mn_major = b_trans ? 0 : 1;      // stored (k,n): n contiguous
    a.batch = p->batch; a.m = p->m; a.n = p->n; a.k = p->k;
    a.tiles_m = (int32_t)((p->m + bm - 1) / bm);
    a.tiles_n = (int32_t)((p->n + bn - 1) / bn);
    const bool f16 = p->a_dtype == ACL_BF16 || p->a_dtype == ACL_FLOAT16;
    const uint64_t es = f16 ? 2 : 1;  // bytes per operand element: extents and pitches below are in bytes
    a.kblocks = (int32_t)((p->k * (int64_t)es + BK - 1) / BK);
    a.num_tiles = p->batch * a.tiles_m * a.tiles_n;
    a.ksplit = 1;
    if (!pair && !pair_pb && p->mode == OPSNN_QMM_DEQ) {
        const int ks = pick_ksplit(p, bn, a.kblocks);
        const uint64_t need = ksplit_workspace(p);
        if (ks > 1 && p->workspace != nullptr && p->workspace_size >= need && a.num_tiles * ks < 0x7FFFFFFF) {
            uint8_t* ws = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p->workspace) + 255) & ~(uintptr_t)255);
            a.ksplit = ks;
            a.ks_count = reinterpret_cast<unsigned long long*>(ws);
            a.ks_part = reinterpret_cast<uint32_t*>(ws + (((uint64_t)a.num_tiles * 8u + 255u) & ~(uint64_t)255u));
            a.ks_nonce = next_ks_nonce();
        }
    }
    if (const char* e = getenv("OPSNN_TEST_UMMA_STALL_KBLOCK")) {  // tests of the give-up path only (single-CTA kernels)
        a.test_stall_kblock = atoi(e);
        const char* pl = getenv("OPSNN_TEST_UMMA_POLL_LIMIT");
        const uint32_t limit = pl != nullptr ? (uint32_t)atoi(pl) : 20000u;
        cudaMemcpyToSymbolAsync(ptx::g_spin_limit, &limit, sizeof(limit), 0, cudaMemcpyHostToDevice, stream);
    }
    a.a_batched = p->a_bs != 0;
    a.b_batched = b_bs != 0;
    a.out_dtype = p->out_dtype; a.bias_dtype = p->bias_dtype; a.scale_b_dtype = p->scale_b_dtype; a.deq_flags = p->deq_flags;
    a.scale_a = p->scale_a; a.scale_b = p->scale_b; a.scale_a_len = p->scale_a_len; a.scale_b_len = p->scale_b_len;
    a.sa_bs = p->sa_bs; a.sb_bs = p->sb_bs; a.group_m = p->group_m > 0 ? p->group_m : 1;
    a.trans_a = p->trans_a; a.trans_b = p->trans_b;
    a.bias = p->bias; a.bias_bs = p->bias_bs; a.out = p->out; a.out_ld = p->out_ld; a.out_bs = p->out_bs;
    const uint32_t fa = a.is_int ? 1u : (p->a_dtype == ACL_FLOAT8_E5M2 ? 1u : 0u);
    const uint32_t fb = a.is_int ? 1u : (p->b_dtype == ACL_FLOAT8_E5M2 ? 1u : 0u);
    a.idesc = make_idesc(a.is_int ? 2u : 1u, fa, fb, (uint32_t)a.a_mn_major, (uint32_t)a.b_mn_major, (uint32_t)bm, (uint32_t)bn);
    if (f16) {  // kind::f16 operand formats: 0 = fp16, 1 = bf16; fp32 accumulate
        const uint32_t ff = p->a_dtype == ACL_BF16 ? 1u : 0u;
        a.idesc = make_idesc(1u, ff, ff, 0u, 0u, (uint32_t)bm, (uint32_t)bn);
    }

    CUtensorMap ma, mb;
    const uint64_t nb_a = a.a_batched ? (uint64_t)p->batch : 1, nb_b = a.b_batched ? (uint64_t)p->batch : 1;
    bool ok;
    if (a.a_mn_major) ok = make_map(&ma, p->a, (uint64_t)p->m, (uint64_t)p->k, nb_a, (uint64_t)p->a_ld, (uint64_t)p->a_bs, 128);
    else ok = make_map(&ma, p->a, (uint64_t)p->k * es, (uint64_t)p->m, nb_a, (uint64_t)p->a_ld * es, (uint64_t)p->a_bs * es, 128);
    if (a.b_mn_major && pair_pb && pb_bn == 128) ok = ok && make_map(&mb, b_ptr, (uint64_t)p->n, (uint64_t)p->k, nb_b, (uint64_t)b_ld, (uint64_t)b_bs, 128, 64);
    else if (a.b_mn_major) ok = ok && make_map(&mb, b_ptr, (uint64_t)p->n, (uint64_t)p->k, nb_b, (uint64_t)b_ld, (uint64_t)b_bs, 128,
                                               bn < 128 ? (uint32_t)bn : 128u);
    else ok = ok && make_map(&mb, b_ptr, (uint64_t)p->k * es, (uint64_t)p->n, nb_b, (uint64_t)b_ld * es, (uint64_t)b_bs * es,
                             pair ? 128u : (pair_pb ? (uint32_t)(pb_bn / 2) : (uint32_t)bn));
    if (!ok) return (int32_t)cudaErrorInvalidValue;
    if (asym) {
        if (p->workspace == nullptr || p->workspace_size < qmm_umma_workspace_size(p)) return (int32_t)cudaErrorInvalidValue;
        float* rs = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(p->workspace) + 255) & ~(uintptr_t)255);
        a.groups = (int32_t)((p->k + 255) / 256);
        a.row_sums = rs;
        a.b_offset = p->b_offset;
        const int64_t total = p->m * a.groups;
        int64_t grid = (total + 255) / 256;
        if (grid > 148 * 8) grid = 148 * 8;
        row_sums_kernel<<<(unsigned)(grid < 1 ? 1 : grid), 256, 0, stream>>>(static_cast<const int8_t*>(p->a), p->a_ld, p->trans_a ? 1 : 0, p->m, p->k,
                                                                           a.groups, 256, rs);
        note_launch("row_sums");
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int32_t)e;
        return launch_pair_pb<ptx::MmaKind::kI8, 4, 128, true>(ma, mb, a, stream);
    }
    if (pair_pb) {
        if (pb_bn == 256)
            return a.is_int ? launch_pair_pb<ptx::MmaKind::kI8, 8, 256>(ma, mb, a, stream)
                            : launch_pair_pb<ptx::MmaKind::kF8F6F4, 8, 256>(ma, mb, a, stream);
        if (a.is_int) return launch_pair_pb<ptx::MmaKind::kI8, 8>(ma, mb, a, stream);
        return launch_pair_pb<ptx::MmaKind::kF8F6F4, 4>(ma, mb, a, stream);
    }
    if (pair && f16) return launch_pair<ptx::MmaKind::kF16>(ma, mb, a, stream);
    if (pair) return a.is_int ? launch_pair<ptx::MmaKind::kI8>(ma, mb, a, stream) : launch_pair<ptx::MmaKind::kF8F6F4>(ma, mb, a, stream);
    if (f16) return launch_bn<false, ptx::MmaKind::kF16>(bn, ma, mb, a, stream);

    if (p->mode == OPSNN_QMM_PERBLOCK)
        return a.is_int ? launch_bn<true, ptx::MmaKind::kI8>(bn, ma, mb, a, stream)
                        : launch_bn<true, ptx::MmaKind::kF8F6F4>(bn, ma, mb, a, stream);
    if (a.is_int) return launch_bn<false, ptx::MmaKind::kI8>(bn, ma, mb, a, stream);
    return launch_bn<false, ptx::MmaKind::kF8F6F4>(bn, ma, mb, a, stream);
}

}  // namespace opsnn

extern "C" __attribute__((visibility("default"))) uint32_t opsnn_qmm_umma_status(int32_t reset)
{
    unsigned int v = 0;
    cudaMemcpyFromSymbol(&v, opsnn::g_umma_status, sizeof(v));
    if (reset) {
        unsigned int z = 0;
        cudaMemcpyToSymbol(opsnn::g_umma_status, &z, sizeof(z));
        const uint32_t limit = opsnn::ptx::kSpinLimit;  // a test may have shortened the waits: back to the normal limit
        cudaMemcpyToSymbol(opsnn::ptx::g_spin_limit, &limit, sizeof(limit));
        if (unsigned int* w = opsnn::g_status_host_word.load(std::memory_order_acquire)) *reinterpret_cast<volatile unsigned int*>(w) = 0u;
    }
    return v;
}

#ifdef OPSNN_PB_DIAG
extern "C" __attribute__((visibility("default"))) int32_t opsnn_pb_diag(unsigned long long* host_out, int32_t ctas)
{
    return (int32_t)cudaMemcpyFromSymbol(host_out, opsnn::g_pb_diag, (size_t)ctas * 5 * sizeof(unsigned long long));
}
#endif
