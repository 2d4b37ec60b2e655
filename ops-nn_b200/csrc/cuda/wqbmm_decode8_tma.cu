// Weight-only quant matmul, streaming decode kernel for 8-bit weights (W8A16 / A16F8, m <= 16, INT8 or FLOAT8_E4M3FN weight stored
// (k,n)).
//
// The reference runs this regime on its n-first kernels (weight_quant_batch_matmul_v2/op_kernel/arch35/n_first/*); the arithmetic
// is the golden's: w' = rn(rn(w + offset) * scale) in x's dtype, y = x @ w' in fp32 (wqbmmv2_kernel_golden.py:199-297).
// Same structure as the int4 kernel of wqbmm_decode_tma.cu: a CTA of 8 warps owns 512 columns and a k range of whole 64-row stages,
// a stage is four TMA boxes of 128 bytes x 64 rows of weights + one of x in the 128-byte swizzle, the warp whose turn it is
// refills the buffer it left one stage ago, k-splits are combined through workspace by the last arriver in CTA order.
//
// Fragments. A warp's 64 columns are four 16-byte chunks of every k row. ldmatrix.trans works on 16-bit elements, i.e. on PAIRS of
// adjacent byte columns: lane (g, q) receives, per 8 x 16-byte matrix, the bytes of columns 2g and 2g+1 of rows 2q and 2q+1. The
// even column feeds one MMA tile, the odd one another (the column permutation is undone when y is written). A byte b = w mod 256
// becomes bf16(w) exactly with two logic ops and one subtraction: (b & 0x7f) | 0x4300 is 128 + (b & 0x7f), (b & 0x80) | 0x4300 is
// 128 or 256, their difference is w (fp16: 0x6400, 1024 + ..., same idea with ten mantissa bits).
//
// FLOAT8_E4M3FN weights (no offset: the API refuses one for fp8 weights, so w' = rn(w * scale), wqbmmv2_kernel_golden.py:199-297):
// the seven magnitude bits are moved under the 16-bit type's sign so that the e4m3 exponent sits in the low four bits of the wider
// exponent field and the three mantissa bits at the top of the wider mantissa; that reads as w * 2^-120 (bf16) / w * 2^-8 (fp16),
// subnormals and zero included, and one exact multiplication by 2^120 / 2^8 gives w. The two NaN encodings (magnitude 0x7f) would
// read as +-480: every weight register is also tested for a byte with all seven magnitude bits set, the hits are ORed per column,
// and a column that met one is written as NaN, as the golden's x @ w' does.
#include "common.cuh"
#include "sm100_ptx.cuh"
#include "wqbmm_decode_common.cuh"

namespace opsnn {

namespace {

constexpr int k8StageSteps = 4;
constexpr int k8StageRows = k8StageSteps * 16;          // 64 k rows
constexpr int k8WBox = 128 * k8StageRows;               // 8192: 128 columns x 64 rows
constexpr int k8XBox = 128 * 16;                        // x: 64 k x 16 rows
constexpr int k8Stage = 4 * k8WBox + k8XBox;            // 34816
constexpr int k8Stages = 3;
constexpr int k8Smem = k8Stages * k8Stage + 1024 + 256;
constexpr uint32_t k8Polls = 4u * 1000u * 1000u;

template <bool kBf16>
struct Num8;
template <>
struct Num8<true> {
    static constexpr uint32_t kLowMask = 0x007F007Fu, kHighMask = 0x00800080u, kMagic = 0x43004300u;  // bf16 128.0
    // e4m3: magnitude to bits 10..4 of each half (shift left 4 from the low byte, right 4 from the high byte), then * 2^120
    static constexpr int kF8Up = 4, kF8Down = 4;
    static constexpr uint32_t kF8Mag = 0x07F007F0u, kF8Rebias = 0x7B807B80u;
};
template <>
struct Num8<false> {
    // fp16 has ten mantissa bits: the whole byte fits under 0x6400 (1024.0): (b ^ 0x80) | 0x6400 = 1024 + 128 + w
    static constexpr uint32_t kLowMask = 0x00FF00FFu, kHighMask = 0x00800080u, kMagic = 0x64006400u;
    // e4m3: magnitude to bits 13..7 of each half, then * 2^8
    static constexpr int kF8Up = 7, kF8Down = 1;
    static constexpr uint32_t kF8Mag = 0x3F803F80u, kF8Rebias = 0x5C005C00u;
};

__device__ __forceinline__ void d8_ldsm4(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <int kOff>
__device__ __forceinline__ void d8_ldsm4_trans(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4+%5];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr), "n"(kOff));
}
__device__ __forceinline__ void d8_tma_2d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar_addr, int32_t c0, int32_t c1)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_addr), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void d8_arrive(uint32_t bar_addr) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_addr) : "memory"); }

__device__ unsigned int g_wq8_status = 0;  // 0, or 1 (a stage never arrived) / 2 (a stage buffer was never released)

static __device__ __noinline__ bool d8_wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, unsigned int code)
{
    for (uint32_t i = 0; i < k8Polls; ++i) {
        if (ptx::mbar_try_wait_a(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag != 0u) return false;
    }
    *abort_flag = 1u;
    atomicCAS(&g_wq8_status, 0u, code);
    return false;
}
__device__ __forceinline__ bool d8_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, unsigned int code)
{
    if (ptx::mbar_try_wait_a(bar, parity)) return true;
    return d8_wait_slow(bar, parity, abort_flag, code);
}

struct D8Args {
    DecodeArgs d;
    int32_t total_stages;      // ceil(k / 64)
    int32_t stages_per_group;  // group_size / 64, or "never" for a single group
};

template <bool kBf16, bool kHasOffset, bool kFp8>
__global__ void __launch_bounds__(kThreads, 2)
wqbmm_decode8_tma_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const D8Args ta)
{
    using N = Num<kBf16>;
    using N8 = Num8<kBf16>;
    const DecodeArgs& a = ta.d;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    __shared__ int s_reduce;
    __shared__ volatile uint32_t s_abort;
    __shared__ int s_issued[k8Stages];
    extern __shared__ uint8_t dyn_raw[];
    const uint32_t smem0 = (ptx::smem_u32(dyn_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = smem0 + k8Stages * k8Stage;  // full[i] at bar0 + 8 i, empty[i] at bar0 + 64 + 8 i

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int64_t c = blockIdx.x;
    const int64_t strip = a.cluster ? c / a.splits : c % a.strips;
    const int64_t chunk = a.cluster ? c % a.splits : c / a.strips;
    const int st_a = (int)((chunk * ta.total_stages) / a.splits);
    const int st_b = (int)(((chunk + 1) * ta.total_stages) / a.splits);
    const int nst = st_b - st_a;
    const int64_t warp_col = strip * kStripCols + warp * kWarpCols;
    const int32_t wcol_bytes = (int32_t)(strip * kStripCols);

    if (tid == 0) {
        s_abort = 0u;
        for (int i = 0; i < k8Stages; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar0 + 8u * i), "r"(1u) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar0 + 64u + 8u * i), "r"((uint32_t)kWarps) : "memory");
            s_issued[i] = -1;
        }
        ptx::fence_mbar_init();
        ptx::fence_proxy_async();
        ptx::tma_prefetch_desc(&map_w);
        ptx::tma_prefetch_desc(&map_x);
    }
    __syncthreads();
    asm volatile("griddepcontrol.wait;" ::: "memory");
    volatile uint32_t* abort_flag = &s_abort;

    auto issue_stage = [&](int t, int buf) {  // one lane: stage t of this CTA's range into buffer buf
        const uint32_t fb = bar0 + 8u * buf;
        const uint32_t dst = smem0 + (uint32_t)buf * k8Stage;
        const int32_t krow = (st_a + t) * k8StageRows;
        s_issued[buf] = t;
        ptx::mbar_expect_tx_a(fb, (uint32_t)k8Stage);
#pragma unroll
        for (int b = 0; b < 4; ++b) d8_tma_2d(dst + b * k8WBox, &map_w, fb, wcol_bytes + 128 * b, krow);
        d8_tma_2d(dst + 4 * k8WBox, &map_x, fb, krow * 2, 0);
    };
    if (tid == 0 && nst > 0) issue_stage(0, 0);  // the first stage alone, the rest of the ring once it has landed

    float total[kTiles][4];
#pragma unroll
    for (int t = 0; t < kTiles; ++t) total[t][0] = total[t][1] = total[t][2] = total[t][3] = 0.f;

    // ---- scale / offset of the current k-group: tile t = (chunk t / 2, column parity t & 1) is column 16 (t / 2) + 2 g + (t & 1)
    // for this lane, so one 32-bit load per chunk holds the two columns of its two tiles ----
    const int spg = (int)min(a.steps_per_group, (int64_t)0x7FFFFFFF);
    const int64_t n_groups = (a.ksteps + spg - 1) / spg;
    int64_t ecol[4];
#pragma unroll
    for (int cidx = 0; cidx < 4; ++cidx) ecol[cidx] = (warp_col + 16 * cidx + 2 * g < a.n) ? warp_col + 16 * cidx + 2 * g : 0;
    uint32_t sc[kTiles], of[kHasOffset ? kTiles : 1], rs_next[4], ro_next[kHasOffset ? 4 : 1];
    auto fetch = [&](int64_t group) {
        if (a.scale_sn != 0) {
            const uint16_t* sp = reinterpret_cast<const uint16_t*>(a.scale) + group * a.scale_sg;
#pragma unroll
            for (int cidx = 0; cidx < 4; ++cidx) rs_next[cidx] = __ldg(reinterpret_cast<const uint32_t*>(sp + ecol[cidx]));
            if (kHasOffset) {
                const uint16_t* op = reinterpret_cast<const uint16_t*>(a.offset) + group * a.scale_sg;
#pragma unroll
                for (int cidx = 0; cidx < 4; ++cidx) ro_next[kHasOffset ? cidx : 0] = __ldg(reinterpret_cast<const uint32_t*>(op + ecol[cidx]));
            }
        } else {
            const uint32_t sv = reinterpret_cast<const uint16_t*>(a.scale)[group * a.scale_sg];
#pragma unroll
            for (int cidx = 0; cidx < 4; ++cidx) rs_next[cidx] = sv | (sv << 16);
            if (kHasOffset) {
                const uint32_t ov = reinterpret_cast<const uint16_t*>(a.offset)[group * a.scale_sg];
#pragma unroll
                for (int cidx = 0; cidx < 4; ++cidx) ro_next[kHasOffset ? cidx : 0] = ov | (ov << 16);
            }
        }
    };
    auto load_group = [&](int64_t group) {
        if (group >= n_groups) group = n_groups - 1;
#pragma unroll
        for (int t = 0; t < kTiles; ++t) {  // each value in both halves of a register: the halves are two k rows of one column
            const uint32_t sel = (t & 1) ? 0x3232u : 0x1010u;
            sc[t] = prmt(rs_next[t >> 1], rs_next[t >> 1], sel);
            if (kHasOffset) of[kHasOffset ? t : 0] = prmt(ro_next[kHasOffset ? t >> 1 : 0], ro_next[kHasOffset ? t >> 1 : 0], sel);
        }
        fetch(min(group + 1, n_groups - 1));
    };
    // two bytes (rows 2q, 2q+1 of one column, in the low byte of each half) -> two dequantised weights
    auto deq = [&](uint32_t x, int t) {
        uint32_t lo, v;
        if (kBf16) {
            uint32_t hi;
            asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(lo) : "r"(x), "n"(N8::kLowMask), "n"(N8::kMagic));   // (x & mask) | magic
            asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(hi) : "r"(x), "n"(N8::kHighMask), "n"(N8::kMagic));
            v = N::sub(lo, hi);  // (128 + (b & 0x7f)) - (128 or 256) = w, exact
        } else {
            asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(lo) : "r"(x), "n"(N8::kLowMask), "n"(0x64806480));  // ((x & 0xff) ^ 0x80) | 0x6400
            v = N::sub(lo, 0x64806480u);  // (1024 + 128 + w) - 1152 = w, exact
        }
        if (kHasOffset) v = N::add(v, of[kHasOffset ? t : 0]);
        return N::mul(v, sc[t]);
    };
    // the same for two e4m3 bytes: `mag` holds them shifted so that the magnitude bits lie under kF8Mag, `sgn` so that the sign bits
    // are bits 15 and 31
    auto deq_f8 = [&](uint32_t mag, uint32_t sgn, int t) {
        uint32_t v;
        mag &= N8::kF8Mag;
        asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v) : "r"(sgn), "n"(0x80008000), "r"(mag));  // (sgn & 0x8000) | mag
        return N::mul(N::mul(v, N8::kF8Rebias), sc[t]);
    };
    // bit 7 of a byte of nan_seen[chunk]: that byte position (even column: bytes 0 and 2, odd column: bytes 1 and 3) held 0x7f / 0xff
    uint32_t nan_seen[kFp8 ? 4 : 1];
    if (kFp8) nan_seen[0] = nan_seen[kFp8 ? 1 : 0] = nan_seen[kFp8 ? 2 : 0] = nan_seen[kFp8 ? 3 : 0] = 0u;
    auto note_nan = [&](uint32_t x, int chunk) {
        const uint32_t carry = (x & 0x7F7F7F7Fu) + 0x01010101u;  // 0x7f + 1 reaches bit 7, nothing crosses into the next byte
        asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(nan_seen[kFp8 ? chunk : 0]) : "r"(carry), "n"(0x80808080), "r"(nan_seen[kFp8 ? chunk : 0]));
    };
    // the four B-fragment registers of one 16-byte chunk (r0: rows 0-7, r1: rows 8-15): even column -> tile 2 chunk, odd -> + 1
    auto chunk_mmas = [&](uint32_t r0, uint32_t r1, int chunk, const uint32_t(&af)[4]) {
        uint32_t e0, e1, o0, o1;
        if (kFp8) {
            note_nan(r0, chunk);
            note_nan(r1, chunk);
            e0 = deq_f8(r0 << N8::kF8Up, r0 << 8, 2 * chunk);
            e1 = deq_f8(r1 << N8::kF8Up, r1 << 8, 2 * chunk);
            o0 = deq_f8(r0 >> N8::kF8Down, r0, 2 * chunk + 1);
            o1 = deq_f8(r1 >> N8::kF8Down, r1, 2 * chunk + 1);
        } else {
            e0 = deq(r0, 2 * chunk);
            e1 = deq(r1, 2 * chunk);
            o0 = deq(r0 >> 8, 2 * chunk + 1);
            o1 = deq(r1 >> 8, 2 * chunk + 1);
        }
        N::mma_free(total[2 * chunk], af, e0, e1);
        N::mma_free(total[2 * chunk + 1], af, o0, o1);
    };
    // one k-step: 8 registers (two ldmatrix.x4.trans) -> 16 B-fragment registers -> 8 MMAs
    auto compute = [&](const uint32_t(&wa)[4], const uint32_t(&wb)[4], const uint32_t(&af)[4]) {
        // wa: chunks 0, 1 as (rows 0-7, rows 8-15) pairs; wb: chunks 2, 3
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) chunk_mmas(wa[2 * cc], wa[2 * cc + 1], cc, af);
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) chunk_mmas(wb[2 * cc], wb[2 * cc + 1], 2 + cc, af);
    };

    // ---- per-lane ldmatrix addresses inside a stage (128-byte swizzle: 16-byte chunk index ^ (row & 7)) ----
    // weights: the warp's 64 columns are chunks 4 (warp & 1) .. + 3 of box warp / 2; matrix j = lane / 8 is
    // (rows 0-7 | 8-15)[j & 1] x (chunk pair's first | second chunk)[j >> 1]; the second ldmatrix takes the next two chunks
    const int li = lane & 7, lj = lane >> 3;
    const uint32_t row_off = (uint32_t)(li + 8 * (lj & 1)) * 128u;
    const uint32_t cbase = 4u * (uint32_t)(warp & 1);
    const uint32_t wlane_a = (uint32_t)(warp >> 1) * k8WBox + row_off + (((cbase + (uint32_t)(lj >> 1)) ^ (uint32_t)li) << 4);
    const uint32_t wlane_b = (uint32_t)(warp >> 1) * k8WBox + row_off + (((cbase + 2u + (uint32_t)(lj >> 1)) ^ (uint32_t)li) << 4);
    const uint32_t xlane = 4u * k8WBox + row_off + ((((uint32_t)lj >> 1) ^ (uint32_t)li) << 4);

    int64_t group = ((int64_t)st_a * k8StageSteps) / spg;
    fetch(min(group, n_groups - 1));
    load_group(group);
    int until_change = ta.stages_per_group - (st_a % ta.stages_per_group);

    uint32_t wa0[4], wb0[4], a0[4], wa1[4], wb1[4], a1[4];
    int buf = 0;
    uint32_t par = 0;
    bool ok = nst > 0;
    if (ok) {
        ok = d8_wait(bar0, 0u, abort_flag, 1u);
        if (tid == 0 && ok) {
            const int pro = nst < k8Stages ? nst : k8Stages;
            for (int t = 1; t < pro; ++t) issue_stage(t, t);
        }
        d8_ldsm4_trans<0>(smem0 + wlane_a, wa0);
        d8_ldsm4_trans<0>(smem0 + wlane_b, wb0);
        d8_ldsm4(smem0 + xlane, a0);
    }
    const int duty = (warp + 8 * 8 - (k8Stages - 1)) & 7;  // this warp refills when (stage index & 7) == duty
    for (int j = 0; j < nst && ok; ++j) {
        const uint32_t sbase = smem0 + (uint32_t)buf * k8Stage;
        const uint32_t wba = sbase + wlane_a, wbb = sbase + wlane_b, xb = sbase + xlane;
        if (j >= 1 && (j & 7) == duty && j + k8Stages - 1 < nst) {
            if (lane == 0) {
                const int pbuf = buf == 0 ? k8Stages - 1 : buf - 1;
                const uint32_t ppar = buf == 0 ? par ^ 1u : par;
                if (d8_wait(bar0 + 64u + 8u * pbuf, ppar, abort_flag, 2u)) issue_stage(j + k8Stages - 1, pbuf);
            }
            __syncwarp();
        }
        if (j > 0 && until_change == 0) {
            load_group(++group);
            until_change = ta.stages_per_group;
        }
        // step 0
        d8_ldsm4_trans<2048>(wba, wa1);
        d8_ldsm4_trans<2048>(wbb, wb1);
        d8_ldsm4(xb ^ 32u, a1);
        compute(wa0, wb0, a0);
        // step 1
        d8_ldsm4_trans<4096>(wba, wa0);
        d8_ldsm4_trans<4096>(wbb, wb0);
        d8_ldsm4(xb ^ 64u, a0);
        compute(wa1, wb1, a1);
        // step 2
        d8_ldsm4_trans<6144>(wba, wa1);
        d8_ldsm4_trans<6144>(wbb, wb1);
        d8_ldsm4(xb ^ 96u, a1);
        compute(wa0, wb0, a0);
        // step 3, after the first fragments of the next stage have been requested
        int nbuf = buf + 1;
        uint32_t npar = par;
        if (nbuf == k8Stages) { nbuf = 0; npar ^= 1u; }
        if (j + 1 < nst) {
            ok = d8_wait(bar0 + 8u * nbuf, npar, abort_flag, 1u);
            const uint32_t nb = smem0 + (uint32_t)nbuf * k8Stage;
            d8_ldsm4_trans<0>(nb + wlane_a, wa0);
            d8_ldsm4_trans<0>(nb + wlane_b, wb0);
            d8_ldsm4(nb + xlane, a0);
        }
        compute(wa1, wb1, a1);
        --until_change;
        __syncwarp();
        if (lane == 0) d8_arrive(bar0 + 64u + 8u * buf);
        buf = nbuf;
        par = npar;
    }

    const bool aborted = __syncthreads_or(s_abort != 0u) != 0;
    if (aborted) {
        // A wait gave up. Nothing is written; the copies already issued get a bounded time to land before the CTA leaves.
        if (tid == 0) {
            for (int i = 0; i < k8Stages; ++i) {
                const int t = s_issued[i];
                if (t < 0) continue;
                const uint32_t p = (uint32_t)(t / k8Stages) & 1u;
                for (uint32_t it = 0; it < k8Polls; ++it)
                    if (ptx::mbar_try_wait_a(bar0 + 8u * i, p)) break;
            }
        }
        __syncthreads();
        if (!a.cluster) return;
    }
    if (kFp8) {
        // A column whose weights held a NaN encoding becomes NaN. The lanes 4 c .. 4 c + 3 hold column c of a tile's B fragments,
        // lane (g, q) holds columns 2 q and 2 q + 1 of its accumulators (rows g and g + 8).
        const float nan = __int_as_float(0x7FC00000);
#pragma unroll
        for (int t = 0; t < kTiles; ++t) {
            const uint32_t mine = nan_seen[kFp8 ? t >> 1 : 0] & ((t & 1) ? 0x80008000u : 0x00800080u);
            const uint32_t cols = __ballot_sync(0xffffffffu, mine != 0u);
            const uint32_t pair = (cols >> (8 * (lane & 3))) & 0xFFu;
            if (pair & 0x0Fu) total[t][0] = total[t][2] = nan;
            if (pair & 0xF0u) total[t][1] = total[t][3] = nan;
        }
    }
    // every warp is past its last stage (barrier above): the stage buffers are free to hold the fragments
    if (a.cluster) cluster_combine_and_store<kBf16, 2>(a, total, strip, warp, lane, tid, smem0, !aborted);
    else combine_and_store<kBf16, 2>(a, total, c, strip, warp, lane, tid, &s_reduce);
}

// ---------------------------------------------------------------------------------------------------------------------------------
// The same regime with the weight stored (n,k), k contiguous - the transposed view of the API (weight.t() of an (n,k) tensor).
//
// Same grid, ring, refill duty, bounded waits and combine; what changes is the shape of a stage and the fragments. A stage is still
// 64 k rows of the strip's 512 columns + x, 34 KB: 64 bytes of k x 512 weight rows (two boxes of 256; warp w's 64 rows are 4 KB
// number w) in the 64-byte swizzle (16-byte chunk index ^ ((row >> 1) & 3)). A row of a box is the 64 k values of one column, so plain ldmatrix (no
// transposition) hands lane (g, q) the bytes k = 16 j + 4 q .. + 3 of column 8 t + g: four matrices per instruction = four tiles of
// one 16-row k-step j. The two byte pairs the conversion works on are (4q, 4q+2) and (4q+1, 4q+3); they become the two B registers
// of one MMA, and the A fragment is permuted to match: x[row][4q .. 4q+3] is one 8-byte shared load, its even elements feed the
// first half of the MMA's k, its odd elements the second (a sum over k does not care in which order the MMA sees k). Tile t is
// columns 8 t .. 8 t + 7 of the warp's 64: no column permutation to undo when y is written.
constexpr int k8TBox = 64 * 64;  // one warp's 64 columns x 64 k

template <bool kBf16, bool kHasOffset, bool kFp8>
__global__ void __launch_bounds__(kThreads, 2)
wqbmm_decode8t_tma_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const D8Args ta)
{
    using N = Num<kBf16>;
    using N8 = Num8<kBf16>;
    const DecodeArgs& a = ta.d;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, q = lane & 3;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    __shared__ int s_reduce;
    __shared__ volatile uint32_t s_abort;
    __shared__ int s_issued[k8Stages];
    extern __shared__ uint8_t dyn_raw[];
    const uint32_t smem0 = (ptx::smem_u32(dyn_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = smem0 + k8Stages * k8Stage;  // full[i] at bar0 + 8 i, empty[i] at bar0 + 64 + 8 i

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int64_t c = blockIdx.x;
    const int64_t strip = a.cluster ? c / a.splits : c % a.strips;
    const int64_t chunk = a.cluster ? c % a.splits : c / a.strips;
    const int st_a = (int)((chunk * ta.total_stages) / a.splits);
    const int st_b = (int)(((chunk + 1) * ta.total_stages) / a.splits);
    const int nst = st_b - st_a;
    const int64_t warp_col = strip * kStripCols + warp * kWarpCols;
    const int32_t strip_row = (int32_t)(strip * kStripCols);

    if (tid == 0) {
        s_abort = 0u;
        for (int i = 0; i < k8Stages; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar0 + 8u * i), "r"(1u) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar0 + 64u + 8u * i), "r"((uint32_t)kWarps) : "memory");
            s_issued[i] = -1;
        }
        ptx::fence_mbar_init();
        ptx::fence_proxy_async();
        ptx::tma_prefetch_desc(&map_w);
        ptx::tma_prefetch_desc(&map_x);
    }
    __syncthreads();
    asm volatile("griddepcontrol.wait;" ::: "memory");
    volatile uint32_t* abort_flag = &s_abort;

    auto issue_stage = [&](int t, int buf) {  // one lane: stage t of this CTA's range into buffer buf
        const uint32_t fb = bar0 + 8u * buf;
        const uint32_t dst = smem0 + (uint32_t)buf * k8Stage;
        const int32_t krow = (st_a + t) * k8StageRows;
        s_issued[buf] = t;
        ptx::mbar_expect_tx_a(fb, (uint32_t)k8Stage);
        // two boxes of 256 weight rows: rows are contiguous in shared memory, so warp w's 64 rows start at w * k8TBox all the same
#pragma unroll
        for (int b = 0; b < 2; ++b) d8_tma_2d(dst + b * 4 * k8TBox, &map_w, fb, krow, strip_row + 256 * b);
        d8_tma_2d(dst + kWarps * k8TBox, &map_x, fb, krow * 2, 0);
    };
    if (tid == 0 && nst > 0) issue_stage(0, 0);  // the first stage alone, the rest of the ring once it has landed

    float total[kTiles][4];
#pragma unroll
    for (int t = 0; t < kTiles; ++t) total[t][0] = total[t][1] = total[t][2] = total[t][3] = 0.f;

    // ---- scale / offset of the current k-group. Tile t is column 8 t + g for this lane. The warp reads its 64 columns once - lane l
    // the columns l and 32 + l, scale and offset packed in one register each - a group ahead of use, and the lanes pick their eight
    // columns out of those registers by shuffle when the group becomes current (any element strides: a scale stored (n, groups) is
    // read in place) ----
    const int spg = (int)min(a.steps_per_group, (int64_t)0x7FFFFFFF);
    const int64_t n_groups = (a.ksteps + spg - 1) / spg;
    uint32_t sc[kTiles], of[kHasOffset ? kTiles : 1], raw_s0 = 0u, raw_s1 = 0u, raw_o0 = 0u, raw_o1 = 0u;
    const int64_t el_lo = (warp_col + lane < a.n ? warp_col + lane : 0) * (int64_t)a.scale_sn;
    const int64_t el_hi = (warp_col + 32 + lane < a.n ? warp_col + 32 + lane : 0) * (int64_t)a.scale_sn;
    auto fetch = [&](int64_t group) {
        const uint16_t* sp = reinterpret_cast<const uint16_t*>(a.scale) + group * a.scale_sg;
        // the loaded values stay untouched until the group becomes current: nothing here waits for the loads
        raw_s0 = __ldg(sp + el_lo);
        raw_s1 = __ldg(sp + el_hi);
        if (kHasOffset) {
            const uint16_t* op = reinterpret_cast<const uint16_t*>(a.offset) + group * a.scale_sg;
            raw_o0 = __ldg(op + el_lo);
            raw_o1 = __ldg(op + el_hi);
        }
    };
    auto load_group = [&](int64_t group) {
        if (group >= n_groups) group = n_groups - 1;
        const uint32_t next_lo = raw_s0 | (raw_o0 << 16), next_hi = raw_s1 | (raw_o1 << 16);
#pragma unroll
        for (int t = 0; t < kTiles; ++t) {  // each value in both halves of a register: the halves are two k rows of one column
            const uint32_t v = __shfl_sync(0xffffffffu, t < 4 ? next_lo : next_hi, (8 * t + g) & 31);
            sc[t] = prmt(v, v, 0x1010u);
            if (kHasOffset) of[kHasOffset ? t : 0] = prmt(v, v, 0x3232u);
        }
        fetch(min(group + 1, n_groups - 1));
    };
    // two bytes (in the low byte of each half) -> two dequantised weights
    auto deq = [&](uint32_t x, int t) {
        uint32_t lo, v;
        if (kBf16) {
            uint32_t hi;
            asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(lo) : "r"(x), "n"(N8::kLowMask), "n"(N8::kMagic));   // (x & mask) | magic
            asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(hi) : "r"(x), "n"(N8::kHighMask), "n"(N8::kMagic));
            v = N::sub(lo, hi);
        } else {
            asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(lo) : "r"(x), "n"(N8::kLowMask), "n"(0x64806480));
            v = N::sub(lo, 0x64806480u);
        }
        if (kHasOffset) v = N::add(v, of[kHasOffset ? t : 0]);
        return N::mul(v, sc[t]);
    };
    auto deq_f8 = [&](uint32_t mag, uint32_t sgn, int t) {
        uint32_t v;
        mag &= N8::kF8Mag;
        asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v) : "r"(sgn), "n"(0x80008000), "r"(mag));  // (sgn & 0x8000) | mag
        return N::mul(N::mul(v, N8::kF8Rebias), sc[t]);
    };
    // e4m3 NaN encodings: all four bytes of a register belong to the tile's one column of this lane
    uint32_t nan_seen[kFp8 ? kTiles : 1];
    if (kFp8) {
#pragma unroll
        for (int t = 0; t < kTiles; ++t) nan_seen[kFp8 ? t : 0] = 0u;
    }
    auto tile_mma = [&](uint32_t r, int t, const uint32_t(&af)[4]) {
        uint32_t b0, b1;
        if (kFp8) {
            const uint32_t carry = (r & 0x7F7F7F7Fu) + 0x01010101u;
            asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(nan_seen[kFp8 ? t : 0]) : "r"(carry), "n"(0x80808080), "r"(nan_seen[kFp8 ? t : 0]));
            b0 = deq_f8(r << N8::kF8Up, r << 8, t);
            b1 = deq_f8(r >> N8::kF8Down, r, t);
        } else {
            b0 = deq(r, t);
            b1 = deq(r >> 8, t);
        }
        N::mma_free(total[t], af, b0, b1);  // b0: k = 4q, 4q+2; b1: k = 4q+1, 4q+3 of this 16-row step
    };
    auto compute = [&](const uint32_t(&wa)[4], const uint32_t(&wb)[4], const uint32_t(&af)[4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) tile_mma(wa[i], i, af);
#pragma unroll
        for (int i = 0; i < 4; ++i) tile_mma(wb[i], 4 + i, af);
    };
    // A fragment of one k-step, permuted like the B registers: rows g and g + 8, x[row][4q .. 4q+3]
    auto load_a = [&](uint32_t addr, uint32_t(&af)[4]) {
        uint32_t l0, h0, l1, h1;
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(l0), "=r"(h0) : "r"(addr));
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+1024];" : "=r"(l1), "=r"(h1) : "r"(addr));
        af[0] = prmt(l0, h0, 0x5410u);
        af[1] = prmt(l1, h1, 0x5410u);
        af[2] = prmt(l0, h0, 0x7632u);
        af[3] = prmt(l1, h1, 0x7632u);
    };

    // ---- per-lane addresses inside a stage; k-step j is the 16-byte chunk j of a weight row (address ^ 16 j: the swizzle only
    // touches those two bits) and the chunk pair j of an x row (address ^ 32 j) ----
    const int li = lane & 7, lj = lane >> 3;
    const uint32_t wlane_a = (uint32_t)warp * k8TBox + (uint32_t)(8 * lj + li) * 64u + ((uint32_t)((li >> 1) & 3) << 4);  // tiles 0-3
    const uint32_t wlane_b = wlane_a + 32u * 64u;                                                                        // tiles 4-7
    const uint32_t xlane = (uint32_t)kWarps * k8TBox + (uint32_t)g * 128u + ((uint32_t)(((q >> 1) ^ g) & 7) << 4) + 8u * (uint32_t)(q & 1);

    int64_t group = ((int64_t)st_a * k8StageSteps) / spg;
    fetch(min(group, n_groups - 1));
    load_group(group);
    int until_change = ta.stages_per_group - (st_a % ta.stages_per_group);

    uint32_t wa0[4], wb0[4], a0[4], wa1[4], wb1[4], a1[4];
    int buf = 0;
    uint32_t par = 0;
    bool ok = nst > 0;
    if (ok) {
        ok = d8_wait(bar0, 0u, abort_flag, 1u);
        if (tid == 0 && ok) {
            const int pro = nst < k8Stages ? nst : k8Stages;
            for (int t = 1; t < pro; ++t) issue_stage(t, t);
        }
        d8_ldsm4(smem0 + wlane_a, wa0);
        d8_ldsm4(smem0 + wlane_b, wb0);
        load_a(smem0 + xlane, a0);
    }
    const int duty = (warp + 8 * 8 - (k8Stages - 1)) & 7;  // this warp refills when (stage index & 7) == duty
    for (int j = 0; j < nst && ok; ++j) {
        const uint32_t sbase = smem0 + (uint32_t)buf * k8Stage;
        const uint32_t wba = sbase + wlane_a, wbb = sbase + wlane_b, xb = sbase + xlane;
        if (j >= 1 && (j & 7) == duty && j + k8Stages - 1 < nst) {
            if (lane == 0) {
                const int pbuf = buf == 0 ? k8Stages - 1 : buf - 1;
                const uint32_t ppar = buf == 0 ? par ^ 1u : par;
                if (d8_wait(bar0 + 64u + 8u * pbuf, ppar, abort_flag, 2u)) issue_stage(j + k8Stages - 1, pbuf);
            }
            __syncwarp();
        }
        if (j > 0 && until_change == 0) {
            load_group(++group);
            until_change = ta.stages_per_group;
        }
        // step 0
        d8_ldsm4(wba ^ 16u, wa1);
        d8_ldsm4(wbb ^ 16u, wb1);
        load_a(xb ^ 32u, a1);
        compute(wa0, wb0, a0);
        // step 1
        d8_ldsm4(wba ^ 32u, wa0);
        d8_ldsm4(wbb ^ 32u, wb0);
        load_a(xb ^ 64u, a0);
        compute(wa1, wb1, a1);
        // step 2
        d8_ldsm4(wba ^ 48u, wa1);
        d8_ldsm4(wbb ^ 48u, wb1);
        load_a(xb ^ 96u, a1);
        compute(wa0, wb0, a0);
        // step 3, after the first fragments of the next stage have been requested
        int nbuf = buf + 1;
        uint32_t npar = par;
        if (nbuf == k8Stages) { nbuf = 0; npar ^= 1u; }
        if (j + 1 < nst) {
            ok = d8_wait(bar0 + 8u * nbuf, npar, abort_flag, 1u);
            const uint32_t nb = smem0 + (uint32_t)nbuf * k8Stage;
            d8_ldsm4(nb + wlane_a, wa0);
            d8_ldsm4(nb + wlane_b, wb0);
            load_a(nb + xlane, a0);
        }
        compute(wa1, wb1, a1);
        --until_change;
        __syncwarp();
        if (lane == 0) d8_arrive(bar0 + 64u + 8u * buf);
        buf = nbuf;
        par = npar;
    }

    const bool aborted = __syncthreads_or(s_abort != 0u) != 0;
    if (aborted) {
        // A wait gave up. Nothing is written; the copies already issued get a bounded time to land before the CTA leaves.
        if (tid == 0) {
            for (int i = 0; i < k8Stages; ++i) {
                const int t = s_issued[i];
                if (t < 0) continue;
                const uint32_t p = (uint32_t)(t / k8Stages) & 1u;
                for (uint32_t it = 0; it < k8Polls; ++it)
                    if (ptx::mbar_try_wait_a(bar0 + 8u * i, p)) break;
            }
        }
        __syncthreads();
        if (!a.cluster) return;
    }
    if (kFp8) {
        // lanes 4 c .. 4 c + 3 hold column c of a tile's weights; lane (g, q) holds columns 2 q, 2 q + 1 of its accumulators
        const float nan = __int_as_float(0x7FC00000);
#pragma unroll
        for (int t = 0; t < kTiles; ++t) {
            const uint32_t cols = __ballot_sync(0xffffffffu, nan_seen[kFp8 ? t : 0] != 0u);
            const uint32_t pair = (cols >> (8 * q)) & 0xFFu;
            if (pair & 0x0Fu) total[t][0] = total[t][2] = nan;
            if (pair & 0xF0u) total[t][1] = total[t][3] = nan;
        }
    }
    if (a.cluster) cluster_combine_and_store<kBf16, 3>(a, total, strip, warp, lane, tid, smem0, !aborted);
    else combine_and_store<kBf16, 3>(a, total, c, strip, warp, lane, tid, &s_reduce);
}

using D8EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

D8EncodeFn d8_encoder()
{
    static D8EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return reinterpret_cast<D8EncodeFn>(p);
    }();
    return fn;
}

bool d8_map_2d(CUtensorMap* map, const void* base, uint64_t inner_bytes, uint64_t rows, uint64_t pitch_bytes, uint32_t box_rows,
               uint32_t box_inner = 128, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B)
{
    D8EncodeFn enc = d8_encoder();
    if (enc == nullptr) return false;
    cuuint64_t dims[2] = {inner_bytes, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

std::atomic<uint64_t> g_d8_configured[12];

// variant = 2 bf16 + has_offset for INT8 weights, 4 + bf16 for FLOAT8_E4M3FN weights; + 6 for a weight stored (n,k)
const void* d8_kernel(int variant)
{
    switch (variant) {
        case 6: return reinterpret_cast<const void*>(&wqbmm_decode8t_tma_kernel<false, false, false>);
        case 7: return reinterpret_cast<const void*>(&wqbmm_decode8t_tma_kernel<false, true, false>);
        case 8: return reinterpret_cast<const void*>(&wqbmm_decode8t_tma_kernel<true, false, false>);
        case 9: return reinterpret_cast<const void*>(&wqbmm_decode8t_tma_kernel<true, true, false>);
        case 10: return reinterpret_cast<const void*>(&wqbmm_decode8t_tma_kernel<false, false, true>);
        case 11: return reinterpret_cast<const void*>(&wqbmm_decode8t_tma_kernel<true, false, true>);
        case 0: return reinterpret_cast<const void*>(&wqbmm_decode8_tma_kernel<false, false, false>);
        case 1: return reinterpret_cast<const void*>(&wqbmm_decode8_tma_kernel<false, true, false>);
        case 2: return reinterpret_cast<const void*>(&wqbmm_decode8_tma_kernel<true, false, false>);
        case 3: return reinterpret_cast<const void*>(&wqbmm_decode8_tma_kernel<true, true, false>);
        case 4: return reinterpret_cast<const void*>(&wqbmm_decode8_tma_kernel<false, false, true>);
        case 5: return reinterpret_cast<const void*>(&wqbmm_decode8_tma_kernel<true, false, true>);
        default: return nullptr;
    }
}

cudaError_t d8_configure_variant(int variant)
{
    const void* kern = d8_kernel(variant);
    return once_per_device(g_d8_configured[variant], [&] {
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);  // clusters of up to 16 k-splits
        return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, k8Smem);
    });
}

cudaError_t d8_launch_variant(int variant, int grid, int cluster_policy, const CUtensorMap& mw, const CUtensorMap& mx, const D8Args& ta, cudaStream_t stream)
{
    const char* pe = getenv("OPSNN_WQ_PDL");
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = k8Smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[3]{};
    unsigned na = 0;
    if (pe == nullptr || pe[0] != '0') {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (ta.d.cluster) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned)ta.d.splits;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
        if (cluster_policy == 1 || cluster_policy == 2) {
            attr[na].id = cudaLaunchAttributeClusterSchedulingPolicyPreference;
            attr[na].val.clusterSchedulingPolicyPreference = static_cast<cudaClusterSchedulingPolicy>(cluster_policy);
            ++na;
        }
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    void* args[3] = {const_cast<CUtensorMap*>(&mw), const_cast<CUtensorMap*>(&mx), const_cast<D8Args*>(&ta)};
    return cudaLaunchKernelExC(&cfg, d8_kernel(variant), args);
}

constexpr int k8ClusterMaxStrips = 28;
constexpr int k8MaxGrid = 148 * 4 * 2;

}  // namespace

uint64_t wqbmm_decode_workspace_size(const OpsnnWqbmmParams* p);

// INT8 or FLOAT8_E4M3FN (no offset) weight stored (k,n) or (n,k), m <= 16, scale (and offset) in x's dtype per channel / per tensor /
// per k-group of whole 64-row stages.
bool wqbmm_decode8_eligible(const OpsnnWqbmmParams* p)
{
    if ((p->w_dtype != ACL_INT8 && p->w_dtype != ACL_FLOAT8_E4M3FN) || p->nz_k0 != 0) return false;
    if (p->w_dtype == ACL_FLOAT8_E4M3FN && p->offset != nullptr) return false;
    if (p->scale_dtype == ACL_FLOAT8_E8M0) return false;
    if (p->m < 1 || p->m > 16 || p->k < 16 || p->k % 16 != 0) return false;
    if (p->n % 16 != 0 || p->w_ld % 16 != 0 || p->x_ld % 8 != 0) return false;  // 16-byte tensor-map pitches; column pairs for the scale loads
    if (p->group_size != 0 && p->group_size % 64 != 0) return false;           // group changes at stage boundaries only
    auto aligned = [](const void* q, uintptr_t al) { return (reinterpret_cast<uintptr_t>(q) % al) == 0; };
    if (!aligned(p->w, 16) || !aligned(p->x, 16)) return false;
    if (p->trans_w != 0) {  // scales are read one 16-bit element at a time, at any strides
        if (p->scale_sn < 0 || p->scale_sn >= ((int64_t)1 << 31) || p->scale_sg < 0) return false;
    } else {                // two adjacent columns per 32-bit load
        if (p->scale_sn != 0 && p->scale_sn != 1) return false;
        if (p->scale_sn == 1 && p->group_size != 0 && p->scale_sg % 2 != 0) return false;
        if (p->scale_sn == 1 && (!aligned(p->scale, 4) || (p->offset && !aligned(p->offset, 4)))) return false;
    }
    if (p->n >= ((int64_t)1 << 31) || p->k >= ((int64_t)1 << 30)) return false;
    return true;
}

int32_t wqbmm_decode8_launch(const OpsnnWqbmmParams* p, cudaStream_t stream)
{
    D8Args ta{};
    DecodeArgs& a = ta.d;
    a.scale = p->scale;
    a.offset = p->offset;
    a.scale_sg = p->group_size > 0 ? p->scale_sg : 0;
    a.scale_sn = (int32_t)p->scale_sn;
    a.bias = p->bias;
    a.bias_dtype = p->bias_dtype;
    a.y = p->y;
    a.y_ld = p->y_ld;
    if (!lookup_peer_binding(p->y, &a.peers)) a.peers.count = 0;
    a.m = (int32_t)p->m;
    a.n = p->n;
    a.k = p->k;
    a.strips = (p->n + kStripCols - 1) / kStripCols;
    a.ksteps = p->k / 16;
    a.steps_per_group = p->group_size > 0 ? p->group_size / 16 : a.ksteps;
    ta.total_stages = (int32_t)((a.ksteps + k8StageSteps - 1) / k8StageSteps);
    const bool single_group = a.steps_per_group >= a.ksteps;
    ta.stages_per_group = single_group ? 0x7FFFFFFF : (int32_t)(a.steps_per_group / k8StageSteps);
    const bool bf16 = p->x_dtype == ACL_BF16, has_off = p->offset != nullptr;

    const int variant = (p->w_dtype == ACL_FLOAT8_E4M3FN ? 4 + (bf16 ? 1 : 0) : (bf16 ? 2 : 0) + (has_off ? 1 : 0)) + (p->trans_w != 0 ? 6 : 0);
    cudaError_t crc = d8_configure_variant(variant);
    if (crc != cudaSuccess) return (int32_t)crc;
    int64_t splits = (2 * (int64_t)current_sm_count()) / a.strips;
    const char* se = getenv("OPSNN_WQ_DECODE_SPLITS");
    const char* ce = getenv("OPSNN_WQ_DECODE_CLUSTER");
    if (se != nullptr && atoi(se) > 0) splits = atoi(se);
    if (splits > ta.total_stages) splits = ta.total_stages;
    if (splits * a.strips > k8MaxGrid) splits = k8MaxGrid / a.strips;
    if (splits < 1) splits = 1;
    // narrow outputs: the k-splits of a strip as one cluster, summed over distributed shared memory; same rules as the int4 kernel
    a.cluster = 0;
    int cluster_policy = 0;
    if (ce == nullptr || ce[0] != '0') {
        if (se != nullptr || (ce != nullptr && splits <= 16)) {
            a.cluster = (splits >= 2 && splits <= 16 && (ce != nullptr || a.strips <= k8ClusterMaxStrips)) ? 1 : 0;
        } else if (a.strips <= k8ClusterMaxStrips && splits >= 2) {
            const int s_pick = pick_cluster_size(d8_kernel(variant), kThreads, k8Smem, a.strips, (int)(splits < 16 ? splits : 16));
            if (s_pick >= 2) {
                splits = s_pick;
                a.cluster = 1;
            }
        } else if (a.strips > k8ClusterMaxStrips && splits >= 2 && splits <= 16) {
            // wide outputs: clusters under the load-balancing policy when every strip's cluster is resident at once (see the int4 kernel)
            if ((int64_t)max_active_clusters(d8_kernel(variant), kThreads, k8Smem, (int)splits, (int)cudaClusterSchedulingPolicyLoadBalancing) >=
                a.strips) {
                a.cluster = 1;
                cluster_policy = (int)cudaClusterSchedulingPolicyLoadBalancing;
            }
        }
    }
    if (!a.cluster && se == nullptr && splits > 16) splits = 16;
    a.splits = splits;
    const int64_t grid64 = a.strips * splits;
    if (grid64 > 0x7FFFFFFF) return (int32_t)cudaErrorInvalidConfiguration;
    const uint64_t tag_bytes = (((uint64_t)k8MaxGrid * 8 + 255) / 256) * 256;
    if (splits > 1 && !a.cluster && (p->workspace == nullptr || p->workspace_size < wqbmm_decode_workspace_size(p))) return (int32_t)cudaErrorInvalidValue;
    a.tags = reinterpret_cast<unsigned long long*>(p->workspace);
    a.partials = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(p->workspace) + tag_bytes);
    a.nonce = next_nonce();

    CUtensorMap mw, mx;
    const bool w_ok = p->trans_w != 0 ? d8_map_2d(&mw, p->w, (uint64_t)p->k, (uint64_t)p->n, (uint64_t)p->w_ld, 256, 64, CU_TENSOR_MAP_SWIZZLE_64B)
                                      : d8_map_2d(&mw, p->w, (uint64_t)p->n, (uint64_t)p->k, (uint64_t)p->w_ld, k8StageRows);
    if (!w_ok ||
        !d8_map_2d(&mx, p->x, (uint64_t)p->k * 2, (uint64_t)p->m, (uint64_t)p->x_ld * 2, 16))
        return (int32_t)cudaErrorInvalidValue;
    const cudaError_t rc = d8_launch_variant(variant, (int)grid64, cluster_policy, mw, mx, ta, stream);
    note_launch("wqbmm_decode8");
    note_decode_plan(a.strips, a.splits, a.cluster);
    return (int32_t)rc;
}

uint32_t wqbmm_decode8_status(int reset)
{
    unsigned int v = 0;
    cudaMemcpyFromSymbol(&v, g_wq8_status, sizeof(v));
    if (reset) {
        unsigned int z = 0;
        cudaMemcpyToSymbol(g_wq8_status, &z, sizeof(z));
    }
    return v;
}

}  // namespace opsnn
