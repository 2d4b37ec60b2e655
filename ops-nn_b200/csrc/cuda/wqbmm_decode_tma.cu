// Weight-only quant matmul, streaming decode kernel (m <= 16, INT4 weight stored (k,n)), bulk-tensor-copy data path.
//
// Same arithmetic as the two ring kernels of wqbmm_decode_fast.cu - kExact: the reference's two roundings per weight
// (weight_quant_batch_matmul_v2/op_kernel/arch35/weight_quant_batch_matmul_v2_reg_base_common_vf.h:345-442, golden
// wqbmmv2_kernel_golden.py:242-297); group-wise: scale and offset applied per k-group to fp32 partial sums
// (innerPrecise = 1, docs/aclnnWeightQuantBatchMatmulV3.md:28, :389) - but the operands reach shared memory differently:
//
//   * A CTA (8 warps) owns a strip of 512 weight columns and a k range made of whole stages of 64 k rows. One stage is
//     three TMA boxes: two of 128 bytes x 64 rows of packed weights (columns 0-255 and 256-511 of the strip) and one
//     of 128 bytes x 16 rows of x (the same 64 k), all in the 128-byte swizzle, 18 KB together. Columns past n, rows of
//     x past m and k rows past the end arrive as zeros, so ragged strips and k tails need no special code.
//   * Six stages per CTA, two CTAs per SM: up to 192 KB of weights in flight per SM with one instruction per box. The
//     warp whose turn it is (stage index mod 8) refills the buffer it left one stage ago once all eight warps have
//     released it (an mbarrier with one arrival per warp); nobody else ever waits for another warp.
//   * Per k-step (16 k rows) a warp issues one ldmatrix.x4.trans on its 64 columns (four nibbles of two k rows per
//     register, already paired the way the MMA B fragment wants them) and one ldmatrix.x4 for the x fragment, with
//     immediate offsets inside the stage; there is no per-step address arithmetic, no copy instruction and no barrier.
//
// The integer pipe (logic and shifts: 28 instructions per k-step), the 16-bit-pair arithmetic (kExact: 48 per k-step) and
// mma.sync (8 or 9 per k-step) each run at one warp instruction per two clocks per SM sub-partition on this part, so the
// main loop is written to add as little as possible to any of them.
#include <cstdio>
#include "common.cuh"
#include "sm100_ptx.cuh"
#include "wqbmm_decode_common.cuh"

namespace opsnn {

namespace {

constexpr int kStageSteps = 4;                      // k-steps (16 rows each) per stage
constexpr int kStageRows = kStageSteps * 16;        // 64 k rows
constexpr int kWBoxBytes = 128 * kStageRows;        // one weight box: 256 columns x 64 rows
constexpr int kXBoxBytes = 128 * 16;                // x: 64 k x 16 rows
constexpr int kStageBytes = 2 * kWBoxBytes + kXBoxBytes;  // 18432
constexpr int kNumStages = 6;
constexpr int kTmaSmem = kNumStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr uint32_t kWaitPolls = 4u * 1000u * 1000u;  // polls before a wait is declared dead

template <bool kBf16>
struct GwNum;
template <>
struct GwNum<true> {
    static constexpr uint32_t kOnes = 0x3F803F80u;  // bf16x2 {1, 1}
    static constexpr float kB = 136.f;
    __device__ __forceinline__ static float lo(uint32_t r) { return __uint_as_float(r << 16); }
    __device__ __forceinline__ static float hi(uint32_t r) { return __uint_as_float(r & 0xFFFF0000u); }
};
template <>
struct GwNum<false> {
    static constexpr uint32_t kOnes = 0x3C003C00u;  // half2 {1, 1}
    static constexpr float kB = 1032.f;
    __device__ __forceinline__ static float lo(uint32_t r) { return __half2float(__ushort_as_half((unsigned short)(r & 0xFFFFu))); }
    __device__ __forceinline__ static float hi(uint32_t r) { return __half2float(__ushort_as_half((unsigned short)(r >> 16))); }
};

__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
template <int kOff>
__device__ __forceinline__ void ldsm4_trans(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4+%5];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr), "n"(kOff));
}
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar_addr, int32_t c0, int32_t c1)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_addr), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive_a(uint32_t bar_addr)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_addr) : "memory");
}

// 0 when every wait of every launch completed; otherwise 1 (a stage never arrived) or 2 (a stage was never released).
__device__ unsigned int g_wq_tma_status = 0;

// Poll limit of the waits: kWaitPolls, or what a test set to make a wait run out quickly (see TmaArgs::test_*).
__device__ uint32_t g_wq_tma_poll_limit = kWaitPolls;

__device__ __noinline__ bool wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, unsigned int code)
{
    const uint32_t limit = g_wq_tma_poll_limit;
    for (uint32_t i = 0; i < limit; ++i) {
        if (ptx::mbar_try_wait_a(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag != 0u) return false;
    }
    *abort_flag = 1u;
    atomicCAS(&g_wq_tma_status, 0u, code);
    return false;
}
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, unsigned int code)
{
    if (ptx::mbar_try_wait_a(bar, parity)) return true;
    return wait_slow(bar, parity, abort_flag, code);
}

#ifdef OPSNN_DECODE_TIMELINE
// Diagnostic builds only: per CTA {entry, dependency wait over, first stage landed, main loop over, exit, SM id} in globaltimer ns.
__device__ unsigned long long g_wq_tma_timeline[148 * 4 * 2 * 6];
__device__ __forceinline__ unsigned long long gtimer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define OPSNN_TL(slot) do { if (tid == 0) g_wq_tma_timeline[blockIdx.x * 6 + (slot)] = gtimer(); } while (0)
#else
#define OPSNN_TL(slot) do { } while (0)
#endif

struct TmaArgs {
    DecodeArgs d;
    int32_t total_stages;      // ceil(k / 64)
    int32_t stages_per_group;  // kAligned kernels: steps_per_group / 4
    int32_t test_stall_stage;  // tests only: >= 0 makes every CTA stop issuing copies from this stage of its range on, so that the
                               // consumers' wait for it runs out (nothing is in flight then) and the give-up path executes; -1 otherwise
};

// kAligned: every k-group is a whole number of stages (or there is a single group), so group changes happen at stage
// boundaries only. Otherwise groups are whole step pairs and the change is looked for before steps 0 and 2 of a stage.
template <bool kBf16, bool kExact, bool kAligned>
__global__ void __launch_bounds__(kThreads, 2)
wqbmm_decode_tma_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const TmaArgs ta)
{
    using N = Num<kBf16>;
    using F = GwNum<kBf16>;
    constexpr int kFirstStages = kExact ? 1 : kNumStages;  // stages requested before the first one has landed
    const DecodeArgs& a = ta.d;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, q = lane & 3;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    __shared__ int s_reduce;
    __shared__ volatile uint32_t s_abort;
    __shared__ int s_issued[kNumStages];
    extern __shared__ uint8_t dyn_raw[];
    const uint32_t smem0 = (ptx::smem_u32(dyn_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = smem0 + kNumStages * kStageBytes;  // full[i] at bar0 + 8 i, empty[i] at bar0 + 64 + 8 i

    // Programmatic dependent launch: the next kernel of the stream may be placed as soon as every CTA of this one has got here
    // (its CTAs take the SM slots this kernel's early finishers leave), and this kernel reads nothing another kernel may have
    // written before griddepcontrol.wait below has returned. Both are no-ops for an ordinary launch.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    OPSNN_TL(0);

    const int64_t c = blockIdx.x;
    const int64_t strip = a.cluster ? c / a.splits : c % a.strips;
    const int64_t chunk = a.cluster ? c % a.splits : c / a.strips;
    // this CTA's k range in stages
    const int st_a = (int)((chunk * ta.total_stages) / a.splits);
    const int st_b = (int)(((chunk + 1) * ta.total_stages) / a.splits);
    const int nst = st_b - st_a;
    const int64_t warp_col = strip * kStripCols + warp * kWarpCols;
    const int32_t wcol_bytes = (int32_t)(strip * (kStripCols / 2));

    if (tid == 0) {
        s_abort = 0u;
        for (int i = 0; i < kNumStages; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar0 + 8u * i), "r"(1u) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar0 + 64u + 8u * i), "r"((uint32_t)kWarps) : "memory");
            s_issued[i] = -1;
        }
        ptx::fence_mbar_init();
        ptx::fence_proxy_async();
    }
    __syncthreads();
    asm volatile("griddepcontrol.wait;" ::: "memory");
    OPSNN_TL(1);
    volatile uint32_t* abort_flag = &s_abort;

    auto issue_stage = [&](int t, int buf) {  // one lane: stage t of this CTA's range into buffer buf
        if (ta.test_stall_stage >= 0 && t >= ta.test_stall_stage) return;
        const uint32_t fb = bar0 + 8u * buf;
        const uint32_t dst = smem0 + (uint32_t)buf * kStageBytes;
        const int32_t krow = (st_a + t) * kStageRows;
        s_issued[buf] = t;
        ptx::mbar_expect_tx_a(fb, (uint32_t)kStageBytes);
        tma_load_2d(dst, &map_w, fb, wcol_bytes, krow);
        tma_load_2d(dst + kWBoxBytes, &map_w, fb, wcol_bytes + 128, krow);
        tma_load_2d(dst + 2 * kWBoxBytes, &map_x, fb, krow * 2, 0);
    };
    if (tid == 0) {
        ptx::tma_prefetch_desc(&map_w);
        ptx::tma_prefetch_desc(&map_x);
        // Default arithmetic: only the first stage is requested now, the rest of the ring once it has landed. With every CTA of
        // the grid asking for its whole ring at once (30 MB on the benchmark shape) the copies complete interleaved and the
        // first stage arrives with the last, 4.4 us after the request. Worth 1 us of 56 per launch there; the group-wise
        // arithmetic, which consumes a stage faster, measured no better with it and keeps the whole ring up front.
        const int pro = nst < kFirstStages ? nst : kFirstStages;
        for (int t = 0; t < pro; ++t) issue_stage(t, t);
    }

    float total[kTiles][4], part[kExact ? 1 : kTiles][4], xsum[4];
#pragma unroll
    for (int t = 0; t < kTiles; ++t) total[t][0] = total[t][1] = total[t][2] = total[t][3] = 0.f;
#pragma unroll
    for (int t = 0; t < (kExact ? 1 : kTiles); ++t) part[t][0] = part[t][1] = part[t][2] = part[t][3] = 0.f;
    xsum[0] = xsum[1] = xsum[2] = xsum[3] = 0.f;

    // ---- scale / offset of the current k-group ----
    const int spg = (int)min(a.steps_per_group, (int64_t)0x7FFFFFFF);
    const int64_t n_groups = (a.ksteps + spg - 1) / spg;
    // exact mode: the lane's B-fragment columns (tile t < 4: column 4g + t, else 32 + 4g + t - 4), each value in both halves
    const int64_t ecol0 = (warp_col + 4 * g < a.n) ? warp_col + 4 * g : 0;
    const int64_t ecol1 = (warp_col + 32 + 4 * g < a.n) ? warp_col + 32 + 4 * g : 0;
    // group-wise mode: the lane's 16 output columns, 8q..8q+7 of each 32-column half
    const int64_t scol0 = (warp_col + 8 * q < a.n) ? warp_col + 8 * q : 0;
    const int64_t scol1 = (warp_col + 32 + 8 * q < a.n) ? warp_col + 32 + 8 * q : 0;
    const bool has_off = a.offset != nullptr;
    uint32_t sc[kExact ? kTiles : 1], of[kExact ? kTiles : 1], rs_next[4], ro_next[4] = {0u, 0u, 0u, 0u};
    uint32_t raw_s[kExact ? 1 : 8], raw_o[kExact ? 1 : 8];

    auto fetch_exact = [&](int64_t group) {
        if (a.scale_sn != 0) {
            const uint16_t* sp = reinterpret_cast<const uint16_t*>(a.scale) + group * a.scale_sg;
            const uint2 s0 = __ldg(reinterpret_cast<const uint2*>(sp + ecol0)), s1 = __ldg(reinterpret_cast<const uint2*>(sp + ecol1));
            rs_next[0] = s0.x; rs_next[1] = s0.y; rs_next[2] = s1.x; rs_next[3] = s1.y;
            if (has_off) {
                const uint16_t* op = reinterpret_cast<const uint16_t*>(a.offset) + group * a.scale_sg;
                const uint2 o0 = __ldg(reinterpret_cast<const uint2*>(op + ecol0)), o1 = __ldg(reinterpret_cast<const uint2*>(op + ecol1));
                ro_next[0] = o0.x; ro_next[1] = o0.y; ro_next[2] = o1.x; ro_next[3] = o1.y;
            }
        } else {
            const uint32_t sv = reinterpret_cast<const uint16_t*>(a.scale)[group * a.scale_sg];
            const uint32_t ov = has_off ? reinterpret_cast<const uint16_t*>(a.offset)[group * a.scale_sg] : 0u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                rs_next[i] = sv | (sv << 16);
                ro_next[i] = ov | (ov << 16);
            }
        }
    };
    auto load_group = [&](int64_t group) {
        if (group >= n_groups) group = n_groups - 1;  // zero-filled stages past the end of k: any finite scale will do
        if (kExact) {
            // the values requested one group ago become this group's registers; the next group's are requested now
#pragma unroll
            for (int t = 0; t < kTiles; ++t) {
                const uint32_t sel = (t & 1) ? 0x3232u : 0x1010u;
                sc[t] = prmt(rs_next[t >> 1], rs_next[t >> 1], sel);
                of[t] = prmt(ro_next[t >> 1], ro_next[t >> 1], sel);
            }
            fetch_exact(min(group + 1, n_groups - 1));
            return;
        }
        if (a.scale_sn != 0) {
            const uint16_t* sp = reinterpret_cast<const uint16_t*>(a.scale) + group * a.scale_sg;
            const uint4 s0 = __ldg(reinterpret_cast<const uint4*>(sp + scol0)), s1 = __ldg(reinterpret_cast<const uint4*>(sp + scol1));
            raw_s[0] = s0.x; raw_s[1] = s0.y; raw_s[2] = s0.z; raw_s[3] = s0.w;
            raw_s[4] = s1.x; raw_s[5] = s1.y; raw_s[6] = s1.z; raw_s[7] = s1.w;
            if (has_off) {
                const uint16_t* op = reinterpret_cast<const uint16_t*>(a.offset) + group * a.scale_sg;
                const uint4 o0 = __ldg(reinterpret_cast<const uint4*>(op + scol0)), o1 = __ldg(reinterpret_cast<const uint4*>(op + scol1));
                raw_o[0] = o0.x; raw_o[1] = o0.y; raw_o[2] = o0.z; raw_o[3] = o0.w;
                raw_o[4] = o1.x; raw_o[5] = o1.y; raw_o[6] = o1.z; raw_o[7] = o1.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) raw_o[i] = 0u;
            }
        } else {
            const uint32_t sv = reinterpret_cast<const uint16_t*>(a.scale)[group * a.scale_sg];
            const uint32_t ov = has_off ? reinterpret_cast<const uint16_t*>(a.offset)[group * a.scale_sg] : 0u;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                raw_s[i] = sv | (sv << 16);
                raw_o[i] = ov | (ov << 16);
            }
        }
    };
    // group-wise mode: fold the finished group into the totals, total += scale * (part + (offset - B) * rowsum(x))
    auto finish_group = [&]() {
        if (kExact) return;
#pragma unroll
        for (int idx = 0; idx < 16; ++idx) {  // idx = 8*half + 4*(e&1) + (t&3): position among the lane's 16 columns
            const uint32_t rs = raw_s[idx >> 1], ro = raw_o[idx >> 1];
            const float sf = (idx & 1) ? F::hi(rs) : F::lo(rs);
            const float ofs = ((idx & 1) ? F::hi(ro) : F::lo(ro)) - F::kB;
            const int t = (idx >> 3) * 4 + (idx & 3), e0 = (idx >> 2) & 1;  // fragment entries e0 (row g) and e0 + 2 (row g + 8)
            total[t][e0] = fmaf(sf, fmaf(ofs, xsum[0], part[t][e0]), total[t][e0]);
            total[t][e0 + 2] = fmaf(sf, fmaf(ofs, xsum[2], part[t][e0 + 2]), total[t][e0 + 2]);
        }
#pragma unroll
        for (int t = 0; t < (kExact ? 1 : kTiles); ++t) part[t][0] = part[t][1] = part[t][2] = part[t][3] = 0.f;
        xsum[0] = xsum[1] = xsum[2] = xsum[3] = 0.f;
    };
    // one k-step: 4 registers of paired nibbles -> 16 B-fragment registers -> 8 MMAs (+ the row-sum MMA)
    auto compute = [&](const uint32_t(&w4)[4], const uint32_t(&af)[4]) {
        uint32_t b0[kTiles], b1[kTiles];
        if (kExact) {
            // (nibble ^ 8) | magic == B + w exactly; then the reference's rounding points: w' = mul(add(sub(v, B), offset), scale)
            auto deq = [&](uint32_t tw, int t) {
                uint32_t v;
                asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(v) : "r"(tw), "n"(0x000F000F), "n"(N::kMagic));
                v = N::sub(v, a.c_bias);
                v = N::add(v, of[kExact ? t : 0]);
                return N::mul(v, sc[kExact ? t : 0]);
            };
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                b0[t] = deq(w4[0] >> (4 * t), t);
                b1[t] = deq(w4[1] >> (4 * t), t);
                b0[4 + t] = deq(w4[2] >> (4 * t), 4 + t);
                b1[4 + t] = deq(w4[3] >> (4 * t), 4 + t);
            }
#pragma unroll
            for (int t = 0; t < kTiles; ++t) N::mma_free(total[t], af, b0[t], b1[t]);
            return;
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(b0[t]) : "r"(w4[0] >> (4 * t)), "n"(0x000F000F), "n"(N::kMagic));
            asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(b1[t]) : "r"(w4[1] >> (4 * t)), "n"(0x000F000F), "n"(N::kMagic));
            asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(b0[4 + t]) : "r"(w4[2] >> (4 * t)), "n"(0x000F000F), "n"(N::kMagic));
            asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(b1[4 + t]) : "r"(w4[3] >> (4 * t)), "n"(0x000F000F), "n"(N::kMagic));
        }
#pragma unroll
        for (int t = 0; t < kTiles; ++t) N::mma_free(part[kExact ? 0 : t], af, b0[t], b1[t]);
        N::mma_free(xsum, af, F::kOnes, F::kOnes);
    };

    // ---- per-lane ldmatrix addresses inside a stage (128-byte swizzle: 16-byte chunk index ^ (row & 7)) ----
    // weights: matrix j = lane / 8 is (rows 0-7 | 8-15)[j & 1] x (columns 0-31 | 32-63)[j >> 1] of the warp's 64 columns, lane % 8
    // its row; a k-step further down is + 2048 bytes (16 rows), which leaves row & 7 alone.
    const int li = lane & 7, lj = lane >> 3;
    const uint32_t wlane = (uint32_t)(warp >> 2) * kWBoxBytes + (uint32_t)(li + 8 * (lj & 1)) * 128u +
                           (uint32_t)(((2 * (warp & 3) + (lj >> 1)) ^ li) << 4);
    // x: rows (l % 8) + 8 ((l / 8) & 1), k half l / 16 of step s: chunk 2 s + (l / 16), i.e. the lane's address ^ (s << 5)
    const uint32_t xrow = (uint32_t)(li + 8 * (lj & 1));
    const uint32_t xlane = 2u * kWBoxBytes + xrow * 128u + ((((uint32_t)lj >> 1) ^ (uint32_t)li) << 4);

    // first group
    const int first_step = st_a * kStageSteps;
    int64_t group = first_step / spg;
    if (kExact) fetch_exact(min(group, n_groups - 1));
    load_group(group);
    int until_change;  // kAligned: stages left in the current group (counting the next one); else steps left
    if (kAligned) until_change = ta.stages_per_group - (st_a % ta.stages_per_group);
    else until_change = (int)((group + 1) * (int64_t)spg - first_step);

    uint32_t w0[4], a0[4], w1[4], a1[4];
    int buf = 0;
    uint32_t par = 0;
    bool ok = nst > 0;
    if (ok) {
        ok = wait_bar(bar0, 0u, abort_flag, 1u);
        OPSNN_TL(2);
        if (tid == 0 && ok) {
            const int pro = nst < kNumStages ? nst : kNumStages;
            for (int t = kFirstStages; t < pro; ++t) issue_stage(t, t);
        }
        ldsm4_trans<0>(smem0 + wlane, w0);
        ldsm4(smem0 + xlane, a0);
    }
    int duty = (warp + 8 * 8 - (kNumStages - 1)) & 7;  // this warp refills when (stage index & 7) == duty
    for (int j = 0; j < nst && ok; ++j) {
        const uint32_t sbase = smem0 + (uint32_t)buf * kStageBytes;
        const uint32_t wb = sbase + wlane, xb = sbase + xlane;
        // refill duty: stage j + kNumStages - 1 goes into the buffer this warp finished one stage ago
        if (j >= 1 && (j & 7) == duty && j + kNumStages - 1 < nst) {
            if (lane == 0) {
                const int pbuf = buf == 0 ? kNumStages - 1 : buf - 1;
                const uint32_t ppar = buf == 0 ? par ^ 1u : par;
                if (wait_bar(bar0 + 64u + 8u * pbuf, ppar, abort_flag, 2u)) issue_stage(j + kNumStages - 1, pbuf);
            }
            __syncwarp();
        }
        if (!kAligned) {
            if (until_change == 0) { finish_group(); load_group(++group); until_change = spg; }
        } else if (j > 0 && until_change == 0) {
            finish_group();
            load_group(++group);
            until_change = ta.stages_per_group;
        }
        // step 0
        ldsm4_trans<2048>(wb, w1);
        ldsm4(xb ^ 32u, a1);
        compute(w0, a0);
        // step 1
        ldsm4_trans<4096>(wb, w0);
        ldsm4(xb ^ 64u, a0);
        compute(w1, a1);
        if (!kAligned) {
            until_change -= 2;
            if (until_change == 0) { finish_group(); load_group(++group); until_change = spg; }
        }
        // step 2
        ldsm4_trans<6144>(wb, w1);
        ldsm4(xb ^ 96u, a1);
        compute(w0, a0);
        // step 3, after the first fragments of the next stage have been requested
        int nbuf = buf + 1;
        uint32_t npar = par;
        if (nbuf == kNumStages) { nbuf = 0; npar ^= 1u; }
        if (j + 1 < nst) {
            ok = wait_bar(bar0 + 8u * nbuf, npar, abort_flag, 1u);
            const uint32_t nb = smem0 + (uint32_t)nbuf * kStageBytes;
            ldsm4_trans<0>(nb + wlane, w0);
            ldsm4(nb + xlane, a0);
        }
        compute(w1, a1);
        if (!kAligned) until_change -= 2;
        else --until_change;
        // every lane has read the stage: release the buffer
        __syncwarp();
        if (lane == 0) mbar_arrive_a(bar0 + 64u + 8u * buf);
        buf = nbuf;
        par = npar;
    }
    finish_group();

    const bool aborted = __syncthreads_or(s_abort != 0u) != 0;
    OPSNN_TL(3);
    if (aborted) {
        // A wait gave up. Nothing is written; before the CTA leaves, the copies already issued get a bounded time to land
        // (shared memory must not be handed to another CTA while a bulk copy still targets it).
        if (tid == 0) {
            for (int i = 0; i < kNumStages; ++i) {
                const int t = s_issued[i];
                if (t < 0) continue;
                const uint32_t p = (uint32_t)(t / kNumStages) & 1u;
                for (uint32_t it = 0; it < kWaitPolls; ++it)
                    if (ptx::mbar_try_wait_a(bar0 + 8u * i, p)) break;
            }
        }
        __syncthreads();
        if (!a.cluster) return;
    }
    // every warp is past its last stage (barrier above): the stage buffers are free to hold the fragments
    if (a.cluster) cluster_combine_and_store<kBf16, 1>(a, total, strip, warp, lane, tid, smem0, !aborted);
    else combine_and_store<kBf16, 1>(a, total, c, strip, warp, lane, tid, &s_reduce);
#ifdef OPSNN_DECODE_TIMELINE
    if (tid == 0) {
        unsigned int smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        g_wq_tma_timeline[blockIdx.x * 6 + 4] = gtimer();
        g_wq_tma_timeline[blockIdx.x * 6 + 5] = smid;
    }
#endif
}

// ---------------------------------------------------------------------------------------------------------------------------------
// The default arithmetic for a weight stored (n,k): k contiguous, two nibbles per byte, the transposed view of the API.
//
// Same grid, ring size, refill duty, bounded waits and combine. A stage is 128 k rows of the strip's 512 columns: 64 bytes of k x
// 512 weight rows (two boxes of 256; warp w's 64 rows are 4 KB number w) in the 64-byte swizzle (16-byte chunk index ^ ((row >> 1) & 3)),
// and two boxes of x.
// A box row is 128 k values of one column, so plain ldmatrix (no transposition) hands lane (g, q) the eight nibbles
// k = 32 j + 8 q .. + 7 of column 8 t + g, four tiles per instruction. The nibble mask takes nibbles i and i + 4 of a register
// together, so the register feeds two MMAs whose B registers are the k pairs (0,4), (1,5) and (2,6), (3,7); the A fragments are
// permuted to match - x[row][32 j + 8 q .. + 7] is one 16-byte shared load, four byte permutes per row make the pairs (a sum over k
// does not care in which order the MMA sees k). Tile t is columns 8 t .. 8 t + 7: no column permutation to undo at the store. Scales
// and offsets are read one 16-bit element at a time at the tensor's own strides ((n, groups) storage is used in place); k-groups
// are whole stages (multiples of 128) or a single group.
#ifndef OPSNN_NK_STAGE_ROWS
#define OPSNN_NK_STAGE_ROWS 128
#endif
// 128 (64-byte rows, 64-byte swizzle, three stages) or 64 (32-byte rows and swizzle, six stages; measured slower: 69.6 against
// 64.2 us on k = 8192, n = 28672 - the narrower the rows of a box, the slower the copies deliver)
constexpr int kNkStageRows = OPSNN_NK_STAGE_ROWS;
constexpr int kNkRowBytes = kNkStageRows / 2;
constexpr int kNkChunks = kNkStageRows / 32;                       // 16-byte chunks per weight row
constexpr int kNkXBoxes = kNkStageRows / 64;
constexpr int kNkWBox = 64 * kNkRowBytes;                          // one warp's 64 columns
constexpr int kNkStageBytes = kWarps * kNkWBox + kNkXBoxes * kXBoxBytes;   // 36864 / 18432
constexpr int kNkStages = kNkStageRows == 128 ? 3 : 6;
static_assert(kNkStages * kNkStageBytes == kNumStages * kStageBytes, "both layouts use the same ring size");

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 2)
wqbmm_decode_tma_nk_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const TmaArgs ta)
{
    using N = Num<kBf16>;
    const DecodeArgs& a = ta.d;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, q = lane & 3;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    __shared__ int s_reduce;
    __shared__ volatile uint32_t s_abort;
    __shared__ int s_issued[kNkStages];
    extern __shared__ uint8_t dyn_raw[];
    const uint32_t smem0 = (ptx::smem_u32(dyn_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = smem0 + kNkStages * kNkStageBytes;  // full[i] at bar0 + 8 i, empty[i] at bar0 + 64 + 8 i

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
        for (int i = 0; i < kNkStages; ++i) {
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
        if (ta.test_stall_stage >= 0 && t >= ta.test_stall_stage) return;
        const uint32_t fb = bar0 + 8u * buf;
        const uint32_t dst = smem0 + (uint32_t)buf * kNkStageBytes;
        const int32_t krow = (st_a + t) * kNkStageRows;
        s_issued[buf] = t;
        ptx::mbar_expect_tx_a(fb, (uint32_t)kNkStageBytes);
        // two boxes of 256 weight rows: rows are contiguous in shared memory, so warp w's 64 rows start at w * kNkWBox all the same
#pragma unroll
        for (int b = 0; b < 2; ++b) tma_load_2d(dst + b * 4 * kNkWBox, &map_w, fb, krow / 2, strip_row + 256 * b);
        tma_load_2d(dst + kWarps * kNkWBox, &map_x, fb, krow * 2, 0);
        if (kNkXBoxes == 2) tma_load_2d(dst + kWarps * kNkWBox + kXBoxBytes, &map_x, fb, krow * 2 + 128, 0);
    };
    if (tid == 0 && nst > 0) issue_stage(0, 0);  // the first stage alone, the rest of the ring once it has landed (see the (k,n) kernel)

    float total[kTiles][4];
#pragma unroll
    for (int t = 0; t < kTiles; ++t) total[t][0] = total[t][1] = total[t][2] = total[t][3] = 0.f;

    // ---- scale / offset of the current k-group. Tile t is column 8 t + g for this lane. The warp reads its 64 columns once - lane l
    // the columns l and 32 + l, scale and offset packed in one register each - a group ahead of use, and the lanes pick their eight
    // columns out of those registers by shuffle when the group becomes current (any element strides: (n, groups) storage is read
    // in place) ----
    const int spg = (int)min(a.steps_per_group, (int64_t)0x7FFFFFFF);
    const int64_t n_groups = (a.ksteps + spg - 1) / spg;
    const bool has_off = a.offset != nullptr;
    uint32_t sc[kTiles], of[kTiles], raw_s0 = 0u, raw_s1 = 0u, raw_o0 = 0u, raw_o1 = 0u;
    const int64_t el_lo = (warp_col + lane < a.n ? warp_col + lane : 0) * (int64_t)a.scale_sn;
    const int64_t el_hi = (warp_col + 32 + lane < a.n ? warp_col + 32 + lane : 0) * (int64_t)a.scale_sn;
    auto fetch = [&](int64_t group) {
        const uint16_t* sp = reinterpret_cast<const uint16_t*>(a.scale) + group * a.scale_sg;
        // the loaded values stay untouched until the group becomes current: nothing here waits for the loads
        raw_s0 = __ldg(sp + el_lo);
        raw_s1 = __ldg(sp + el_hi);
        if (has_off) {
            const uint16_t* op = reinterpret_cast<const uint16_t*>(a.offset) + group * a.scale_sg;
            raw_o0 = __ldg(op + el_lo);
            raw_o1 = __ldg(op + el_hi);
        }
    };
    auto load_group = [&](int64_t group) {
        if (group >= n_groups) group = n_groups - 1;  // zero-filled stages past the end of k: any finite scale will do
        const uint32_t next_lo = raw_s0 | (raw_o0 << 16), next_hi = raw_s1 | (raw_o1 << 16);
#pragma unroll
        for (int t = 0; t < kTiles; ++t) {  // each value in both halves of a register: the halves are two k rows of one column
            const uint32_t v = __shfl_sync(0xffffffffu, t < 4 ? next_lo : next_hi, (8 * t + g) & 31);
            sc[t] = prmt(v, v, 0x1010u);
            of[t] = prmt(v, v, 0x3232u);
        }
        fetch(min(group + 1, n_groups - 1));
    };
    // (nibble ^ 8) | magic == B + w exactly; then the reference's rounding points: w' = mul(add(sub(v, B), offset), scale)
    auto deq = [&](uint32_t tw, int t) {
        uint32_t v;
        asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(v) : "r"(tw), "n"(0x000F000F), "n"(N::kMagic));
        v = N::sub(v, a.c_bias);
        v = N::add(v, of[t]);
        return N::mul(v, sc[t]);
    };
    // four tiles, the k pairs (0,4), (1,5) of a register / the pairs (2,6), (3,7)
    auto mma_lo = [&](const uint32_t(&w4)[4], int t0, const uint32_t(&af)[4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) N::mma_free(total[t0 + i], af, deq(w4[i], t0 + i), deq(w4[i] >> 4, t0 + i));
    };
    auto mma_hi = [&](const uint32_t(&w4)[4], int t0, const uint32_t(&af)[4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) N::mma_free(total[t0 + i], af, deq(w4[i] >> 8, t0 + i), deq(w4[i] >> 12, t0 + i));
    };
    auto load_x = [&](uint32_t addr, uint32_t(&X)[8]) {  // x[g][8 k], x[g + 8][8 k]
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(X[0]), "=r"(X[1]), "=r"(X[2]), "=r"(X[3]) : "r"(addr));
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+1024];" : "=r"(X[4]), "=r"(X[5]), "=r"(X[6]), "=r"(X[7]) : "r"(addr));
    };
    auto make_a = [&](const uint32_t(&X)[8], uint32_t(&lo)[4], uint32_t(&hi)[4]) {
        lo[0] = prmt(X[0], X[2], 0x5410u);  // row g:     (x0, x4)
        lo[1] = prmt(X[4], X[6], 0x5410u);  // row g + 8
        lo[2] = prmt(X[0], X[2], 0x7632u);  //            (x1, x5)
        lo[3] = prmt(X[4], X[6], 0x7632u);
        hi[0] = prmt(X[1], X[3], 0x5410u);  //            (x2, x6)
        hi[1] = prmt(X[5], X[7], 0x5410u);
        hi[2] = prmt(X[1], X[3], 0x7632u);  //            (x3, x7)
        hi[3] = prmt(X[5], X[7], 0x7632u);
    };

    // ---- per-lane addresses inside a stage. Weights: chunk j (32 k) of a row is address ^ 16 j (the swizzle only touches those two
    // bits). x: chunk j is box j / 2, 16-byte pieces 4 (j & 1) + q of a row in the 128-byte swizzle: address ^ 64 (j & 1) ----
    const int li = lane & 7, lj = lane >> 3;
    const uint32_t wswz = kNkRowBytes == 64 ? (uint32_t)((li >> 1) & 3) : (uint32_t)((li >> 2) & 1);  // 64- / 32-byte swizzle
    const uint32_t wlane_a = (uint32_t)warp * kNkWBox + (uint32_t)(8 * lj + li) * (uint32_t)kNkRowBytes + (wswz << 4);  // tiles 0-3
    const uint32_t wlane_b = wlane_a + 32u * (uint32_t)kNkRowBytes;                                                     // tiles 4-7
    const uint32_t xlane = (uint32_t)kWarps * kNkWBox + (uint32_t)g * 128u + ((uint32_t)((q ^ g) & 7) << 4);

    int64_t group = ((int64_t)st_a * (kNkStageRows / 16)) / spg;
    fetch(min(group, n_groups - 1));
    load_group(group);
    int until_change = ta.stages_per_group - (st_a % ta.stages_per_group);

    uint32_t wa[4], wb[4], X[8], alo[4], ahi[4];
    int buf = 0;
    uint32_t par = 0;
    bool ok = nst > 0;
    if (ok) {
        ok = wait_bar(bar0, 0u, abort_flag, 1u);
        if (tid == 0 && ok) {
            const int pro = nst < kNkStages ? nst : kNkStages;
            for (int t = 1; t < pro; ++t) issue_stage(t, t);
        }
        ldsm4(smem0 + wlane_a, wa);
        ldsm4(smem0 + wlane_b, wb);
        load_x(smem0 + xlane, X);
    }
    const int duty = (warp + 8 * 8 - (kNkStages - 1)) & 7;  // this warp refills when (stage index & 7) == duty
    for (int j = 0; j < nst && ok; ++j) {
        const uint32_t sbase = smem0 + (uint32_t)buf * kNkStageBytes;
        const uint32_t wba = sbase + wlane_a, wbb = sbase + wlane_b, xb = sbase + xlane;
        if (j >= 1 && (j & 7) == duty && j + kNkStages - 1 < nst) {
            if (lane == 0) {
                const int pbuf = buf == 0 ? kNkStages - 1 : buf - 1;
                const uint32_t ppar = buf == 0 ? par ^ 1u : par;
                if (wait_bar(bar0 + 64u + 8u * pbuf, ppar, abort_flag, 2u)) issue_stage(j + kNkStages - 1, pbuf);
            }
            __syncwarp();
        }
        if (j > 0 && until_change == 0) {
            load_group(++group);
            until_change = ta.stages_per_group;
        }
        int nbuf = buf + 1;
        uint32_t npar = par;
        if (nbuf == kNkStages) { nbuf = 0; npar ^= 1u; }
        const uint32_t nb = smem0 + (uint32_t)nbuf * kNkStageBytes;
#pragma unroll
        for (int cj = 0; cj < kNkChunks; ++cj) {
            // this chunk's A fragments; then the next chunk's operands are requested as this one's registers fall free
            make_a(X, alo, ahi);
            bool more = true;
            if (cj == kNkChunks - 1) {
                more = j + 1 < nst;
                if (more) ok = wait_bar(bar0 + 8u * nbuf, npar, abort_flag, 1u);
            }
            const uint32_t nwa = cj == kNkChunks - 1 ? nb + wlane_a : wba ^ (16u * (cj + 1));
            const uint32_t nwb = cj == kNkChunks - 1 ? nb + wlane_b : wbb ^ (16u * (cj + 1));
            const uint32_t nx = cj == kNkChunks - 1 ? nb + xlane : (xb + 2048u * ((cj + 1) >> 1)) ^ (64u * ((cj + 1) & 1));
            if (more) load_x(nx, X);
            mma_lo(wa, 0, alo);
            mma_lo(wb, 4, alo);
            mma_hi(wa, 0, ahi);
            if (more) ldsm4(nwa, wa);
            mma_hi(wb, 4, ahi);
            if (more) ldsm4(nwb, wb);
        }
        --until_change;
        __syncwarp();
        if (lane == 0) mbar_arrive_a(bar0 + 64u + 8u * buf);
        buf = nbuf;
        par = npar;
    }

    const bool aborted = __syncthreads_or(s_abort != 0u) != 0;
    if (aborted) {
        // A wait gave up. Nothing is written; the copies already issued get a bounded time to land before the CTA leaves.
        if (tid == 0) {
            for (int i = 0; i < kNkStages; ++i) {
                const int t = s_issued[i];
                if (t < 0) continue;
                const uint32_t p = (uint32_t)(t / kNkStages) & 1u;
                for (uint32_t it = 0; it < kWaitPolls; ++it)
                    if (ptx::mbar_try_wait_a(bar0 + 8u * i, p)) break;
            }
        }
        __syncthreads();
        if (!a.cluster) return;
    }
    if (a.cluster) cluster_combine_and_store<kBf16, 3>(a, total, strip, warp, lane, tid, smem0, !aborted);
    else combine_and_store<kBf16, 3>(a, total, c, strip, warp, lane, tid, &s_reduce);
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn tma_encoder()
{
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

// 2-D byte tensor (inner bytes, rows) with a (128, box_rows) box in the 128-byte swizzle (or the box width and swizzle given);
// out-of-range bytes read as zero.
bool make_map_2d(CUtensorMap* map, const void* base, uint64_t inner_bytes, uint64_t rows, uint64_t pitch_bytes, uint32_t box_rows,
                 uint32_t box_inner = 128, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B)
{
    EncodeFn enc = tma_encoder();
    if (enc == nullptr) return false;
    cuuint64_t dims[2] = {inner_bytes, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

std::atomic<uint64_t> g_tma_configured[10];

// variant = 4 exact + 2 bf16 + aligned; 8 + bf16: weight stored (n,k)
const void* tma_kernel(int variant)
{
    switch (variant) {
        case 8: return reinterpret_cast<const void*>(&wqbmm_decode_tma_nk_kernel<false>);
        case 9: return reinterpret_cast<const void*>(&wqbmm_decode_tma_nk_kernel<true>);
        case 0: return reinterpret_cast<const void*>(&wqbmm_decode_tma_kernel<false, false, false>);
        case 1: return reinterpret_cast<const void*>(&wqbmm_decode_tma_kernel<false, false, true>);
        case 2: return reinterpret_cast<const void*>(&wqbmm_decode_tma_kernel<true, false, false>);
        case 3: return reinterpret_cast<const void*>(&wqbmm_decode_tma_kernel<true, false, true>);
        case 4: return reinterpret_cast<const void*>(&wqbmm_decode_tma_kernel<false, true, false>);
        case 5: return reinterpret_cast<const void*>(&wqbmm_decode_tma_kernel<false, true, true>);
        case 6: return reinterpret_cast<const void*>(&wqbmm_decode_tma_kernel<true, true, false>);
        default: return reinterpret_cast<const void*>(&wqbmm_decode_tma_kernel<true, true, true>);
    }
}

cudaError_t configure_variant(int variant)
{
    const void* kern = tma_kernel(variant);
    return once_per_device(g_tma_configured[variant], [&] {
        cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);  // clusters of up to 16 k-splits
        return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kTmaSmem);
    });
}

cudaError_t launch_variant(int variant, int grid, int cluster_policy, const CUtensorMap& mw, const CUtensorMap& mx, const TmaArgs& ta, cudaStream_t stream)
{
    // launched as a programmatic dependent of whatever precedes it in the stream (OPSNN_WQ_PDL=0: an ordinary launch)
    const char* pe = getenv("OPSNN_WQ_PDL");
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kTmaSmem;
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
        if (const char* pol = getenv("OPSNN_WQ_CLUSTER_POLICY")) cluster_policy = atoi(pol);  // experiments: 1 spread, 2 load balancing
        if (cluster_policy == 1 || cluster_policy == 2) {
            attr[na].id = cudaLaunchAttributeClusterSchedulingPolicyPreference;
            attr[na].val.clusterSchedulingPolicyPreference = static_cast<cudaClusterSchedulingPolicy>(cluster_policy);
            ++na;
        }
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    void* args[3] = {const_cast<CUtensorMap*>(&mw), const_cast<CUtensorMap*>(&mx), const_cast<TmaArgs*>(&ta)};
    return cudaLaunchKernelExC(&cfg, tma_kernel(variant), args);
}

constexpr int kClusterMaxStrips = 28;  // wider outputs keep the workspace combination (measured equal or better there)
constexpr int kTmaMaxGrid = 148 * 4 * 2;  // same workspace layout and bound as the other decode kernels

}  // namespace

bool wqbmm_decode_eligible(const OpsnnWqbmmParams* p);
uint64_t wqbmm_decode_workspace_size(const OpsnnWqbmmParams* p);
bool wqbmm_decode_fast_eligible(const OpsnnWqbmmParams* p);

// What the bulk-copy data path needs beyond the ring kernels' conditions: 16-byte aligned x rows (tensor-map pitches) and a
// device that can encode tensor maps.
bool wqbmm_decode_tma_eligible(const OpsnnWqbmmParams* p)
{
    if (!wqbmm_decode_fast_eligible(p)) return false;
    if (p->x_ld % 8 != 0 || (reinterpret_cast<uintptr_t>(p->x) % 16) != 0) return false;
    if (p->n >= ((int64_t)1 << 31) || p->k >= ((int64_t)1 << 30)) return false;  // 32-bit tensor coordinates
    return true;
}

// The (n,k) kernel's conditions: INT4 weight stored k-contiguous with 16-byte aligned rows, m <= 16, k-groups of whole 128-row stages
// (or one group), scale / offset in x's dtype at any non-negative strides.
bool wqbmm_decode_tma_nk_eligible(const OpsnnWqbmmParams* p)
{
    if (p->w_dtype != ACL_INT4 || p->trans_w == 0 || p->nz_k0 != 0) return false;
    if (p->scale_dtype == ACL_FLOAT8_E8M0) return false;
    if (p->m < 1 || p->m > 16 || p->k < 32 || p->k % 32 != 0 || p->n % 8 != 0) return false;
    if (p->w_ld % 32 != 0 || p->x_ld % 8 != 0) return false;
    if (p->group_size != 0 && p->group_size % kNkStageRows != 0) return false;
    if (p->scale_sn < 0 || p->scale_sn >= ((int64_t)1 << 31) || p->scale_sg < 0) return false;
    if ((reinterpret_cast<uintptr_t>(p->w) % 16) != 0 || (reinterpret_cast<uintptr_t>(p->x) % 16) != 0) return false;
    if (p->n >= ((int64_t)1 << 31) || p->k >= ((int64_t)1 << 30)) return false;
    return tma_encoder() != nullptr;
}

// exact = true: the reference's default arithmetic; false: the group-wise form of innerPrecise = 1. A weight stored (n,k) always
// runs the default arithmetic.
int32_t wqbmm_decode_tma_launch(const OpsnnWqbmmParams* p, cudaStream_t stream, bool exact)
{
    const bool nk = p->trans_w != 0;
    if (nk) exact = true;
    TmaArgs ta{};
    DecodeArgs& a = ta.d;
    a.w = reinterpret_cast<const uint32_t*>(p->w);
    a.w_ld32 = p->w_ld / 8;
    a.x = p->x;
    a.x_ld = p->x_ld;
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
    const int stage_steps = nk ? kNkStageRows / 16 : kStageSteps;
    ta.total_stages = (int32_t)((a.ksteps + stage_steps - 1) / stage_steps);
    ta.test_stall_stage = -1;
    if (const char* e = getenv("OPSNN_TEST_DECODE_STALL_STAGE")) {  // tests of the give-up path only
        ta.test_stall_stage = atoi(e);
        const char* pl = getenv("OPSNN_TEST_DECODE_POLL_LIMIT");
        const uint32_t limit = pl != nullptr ? (uint32_t)atoi(pl) : 4096u;
        cudaMemcpyToSymbolAsync(g_wq_tma_poll_limit, &limit, sizeof(limit), 0, cudaMemcpyHostToDevice, stream);
    }
    const bool single_group = a.steps_per_group >= a.ksteps;
    const bool aligned = single_group || a.steps_per_group % stage_steps == 0;
    ta.stages_per_group = single_group ? 0x7FFFFFFF : (int32_t)(a.steps_per_group / stage_steps);
    const bool bf16 = p->x_dtype == ACL_BF16;
    const int variant = nk ? 8 + (bf16 ? 1 : 0) : (exact ? 4 : 0) + (bf16 ? 2 : 0) + (aligned ? 1 : 0);

    cudaError_t crc = configure_variant(variant);
    if (crc != cudaSuccess) return (int32_t)crc;
    const int resident = 2 * current_sm_count();
    int64_t splits = resident / a.strips;
    const char* se = getenv("OPSNN_WQ_DECODE_SPLITS");
    const char* ce = getenv("OPSNN_WQ_DECODE_CLUSTER");
    if (se != nullptr && atoi(se) > 0) splits = atoi(se);
    if (splits > ta.total_stages) splits = ta.total_stages;
    if (splits * a.strips > kTmaMaxGrid) splits = kTmaMaxGrid / a.strips;
    if (splits < 1) splits = 1;
    // Narrow outputs (a column shard of a wider problem, a small layer): the k-splits of a strip are launched as one thread-block
    // cluster and summed over distributed shared memory, every CTA of the cluster a slice of the strip - with many splits per
    // strip, one CTA summing all fragments out of global memory is a visible part of the launch (3584 columns of k = 8192:
    // 40.6 us with 42 splits through the workspace, 26.4 us with 16, 14.7 us with a cluster of 16). The split count is the largest
    // that lets every strip's cluster be resident at once (the occupancy query knows how clusters pack into the device's GPCs).
    // Wide outputs keep the workspace combination (measured equal or better there). OPSNN_WQ_DECODE_CLUSTER=0 / 1 forbids /
    // forces the cluster form; OPSNN_WQ_DECODE_SPLITS fixes the split count.
    a.cluster = 0;
    int cluster_policy = 0;
    if (ce == nullptr || ce[0] != '0') {
        if (se != nullptr || (ce != nullptr && splits <= 16)) {
            a.cluster = (splits >= 2 && splits <= 16 && (ce != nullptr || a.strips <= kClusterMaxStrips)) ? 1 : 0;
        } else if (a.strips <= kClusterMaxStrips && splits >= 2) {
            // (asking for one CTA per SM on top was measured: equal up to 7 strips, slower beyond)
            const int s_pick = pick_cluster_size(tma_kernel(variant), kThreads, kTmaSmem, a.strips, (int)(splits < 16 ? splits : 16));
            if (s_pick >= 2) {
                splits = s_pick;
                a.cluster = 1;
            }
        } else if (a.strips > kClusterMaxStrips && splits >= 2 && splits <= 16 && getenv("OPSNN_WQ_CLUSTER_POLICY") == nullptr) {
            // Wide outputs, two CTAs per SM: a cluster per strip pays when the hardware may pack the clusters' CTAs two to an SM
            // (the load-balancing scheduling policy; with the default, spreading one, a second wave forms: 74 us on the
            // benchmark shape) and every strip's cluster is resident at once. 56 strips x 5: 53.5 -> 49.8 us; 64 x 4: 61.7 -> 58.9;
            // cluster sizes that do not pack (6, 7, 9 CTAs: 47.6 -> 67 us) are what the occupancy question filters out.
            const int act = max_active_clusters(tma_kernel(variant), kThreads, kTmaSmem, (int)splits, (int)cudaClusterSchedulingPolicyLoadBalancing);
            if (getenv("OPSNN_DEBUG_PLAN")) fprintf(stderr, "[opsnn] decode plan: strips %lld splits %lld active clusters (load balancing) %d\n", (long long)a.strips, (long long)splits, act);
            if ((int64_t)act >= a.strips) {
                a.cluster = 1;
                cluster_policy = (int)cudaClusterSchedulingPolicyLoadBalancing;
            }
        }
    }
    if (!a.cluster && se == nullptr && splits > 16) splits = 16;  // workspace combination: beyond 16 fragments per strip the summing CTA costs more than the parallelism gives
    a.splits = splits;
    const int64_t grid64 = a.strips * splits;
    if (grid64 > 0x7FFFFFFF) return (int32_t)cudaErrorInvalidConfiguration;
    const uint64_t tag_bytes = (((uint64_t)kTmaMaxGrid * 8 + 255) / 256) * 256;
    if (splits > 1 && !a.cluster && (p->workspace == nullptr || p->workspace_size < wqbmm_decode_workspace_size(p))) return (int32_t)cudaErrorInvalidValue;
    a.tags = reinterpret_cast<unsigned long long*>(p->workspace);
    a.partials = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(p->workspace) + tag_bytes);
    a.nonce = next_nonce();
    a.c_mask = 0x000F000Fu;
    a.c_magic = bf16 ? Num<true>::kMagic : Num<false>::kMagic;
    a.c_bias = bf16 ? Num<true>::kBias : Num<false>::kBias;

    CUtensorMap mw, mx;
    const bool w_ok = nk ? make_map_2d(&mw, p->w, (uint64_t)p->k / 2, (uint64_t)p->n, (uint64_t)p->w_ld / 2, 256, kNkRowBytes,
                                      kNkRowBytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B)
                         : make_map_2d(&mw, p->w, (uint64_t)p->n / 2, (uint64_t)p->k, (uint64_t)p->w_ld / 2, kStageRows);
    if (!w_ok ||
        !make_map_2d(&mx, p->x, (uint64_t)p->k * 2, (uint64_t)p->m, (uint64_t)p->x_ld * 2, 16))
        return (int32_t)cudaErrorInvalidValue;

    const cudaError_t rc = launch_variant(variant, (int)grid64, cluster_policy, mw, mx, ta, stream);
    note_launch(exact ? "wqbmm_decode" : "wqbmm_decode_fast");
    note_decode_plan(a.strips, a.splits, a.cluster);
    return (int32_t)rc;
}

}  // namespace opsnn

#ifdef OPSNN_DECODE_TIMELINE
extern "C" __attribute__((visibility("default"))) int32_t opsnn_wqbmm_decode_timeline(unsigned long long* host_out, int32_t ctas)
{
    return (int32_t)cudaMemcpyFromSymbol(host_out, opsnn::g_wq_tma_timeline, (size_t)ctas * 6 * sizeof(unsigned long long));
}
#endif

// Error word of the bulk-copy decode kernels on the current device: 0 when every bounded wait inside them completed. Synchronises the
// device; reset != 0 clears the word after reading it.
extern "C" __attribute__((visibility("default"))) uint32_t opsnn_wqbmm_decode_status(int32_t reset)
{
    unsigned int v = 0;
    cudaMemcpyFromSymbol(&v, opsnn::g_wq_tma_status, sizeof(v));
    if (reset) {
        unsigned int z = 0;
        cudaMemcpyToSymbol(opsnn::g_wq_tma_status, &z, sizeof(z));
        const uint32_t limit = opsnn::kWaitPolls;  // a test may have shortened the waits: back to the normal limit
        cudaMemcpyToSymbol(opsnn::g_wq_tma_poll_limit, &limit, sizeof(limit));
    }
    return v;
}
