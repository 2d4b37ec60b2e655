// Weight-only quant matmul, decode kernel for the "high performance" precision mode (innerPrecise = 1 of
// aclnnWeightQuantBatchMatmulV3: weight_quant_batch_matmul_v2/docs/aclnnWeightQuantBatchMatmulV3.md:28, :389 -
// "A16W4 per-group with batch size <= 16 may set innerPrecise to 1 for speed, at some cost in accuracy").
//
// The reference's default arithmetic rounds every dequantised weight twice in the activation dtype,
// w' = rn(rn(w + offset) * scale), which costs two half-rate 16-bit-pair instructions per weight pair and makes the
// decode regime instruction bound. This kernel uses the algebraically equal group-wise form instead:
//
//     y[m,n] = sum over groups g of  scale[g,n] * ( P_g[m,n] + (offset[g,n] - B) * X_g[m] )
//     P_g[m,n] = sum_{k in g} x[m,k] * (B + w[k,n])      (tensor core; B + w is an exact bf16/fp16 made by one logic op)
//     X_g[m]   = sum_{k in g} x[m,k]                      (one more MMA per k-step against a tile of ones)
//
// with B = 136 (bf16) or 1032 (fp16), everything after the MMA in fp32. No weight is rounded at all, so the result is
// closer to the fp32 dequantised product than the default mode's (whose own double rounding is the larger error);
// it is not bit-identical to the default mode.
//
// Data movement. Same work split as the default decode kernel (strips of 512 columns x equal k ranges, cross-CTA
// combination through workspace), but the weight words go global -> shared with cp.async (16 bytes per lane: one
// instruction per warp moves one whole k-step of the warp's 64 columns, 16 rows x 32 bytes) into a per-warp ring of
// 16 k-steps, so up to 8 KB per warp (128 KB per SM) is in flight without holding registers, and no thread ever waits
// on another warp. A ring slot holds the step as four 8 x 16-byte matrices (rows 0-7 | 8-15) x (columns 0-31 | 32-63);
// one ldmatrix.x4.trans then gives lane (g, q) the 16-bit column g of rows 2q and 2q+1 (and 2q+8, 2q+9) in one register
// each: four nibbles of two k rows, already paired the way the MMA B fragment wants them, so a shift and one logic op
// per tile finish the job. A 16-bit column is four packed weight columns; nibble j is MMA tile j of its 32-column half,
// and the column permutation this implies is undone when y is written. x fragments come from ldmatrix.x4 as well.
#include "common.cuh"
#include "wqbmm_decode_common.cuh"

namespace opsnn {

namespace {

constexpr int kDepth = 12;                       // k-steps in a warp's ring (even)
constexpr int kStepBytes = 512;                  // 16 rows x 32 bytes
constexpr int kFChunk = 112;                     // k-steps of x staged at a time (one buffer: a CTA's whole k range when it fits,
                                                 // so that the warps of a CTA never meet at a barrier inside the main loop)
constexpr int kFXPitch = kFChunk * 16 + 8;       // elements; +8 skews rows over the banks
constexpr int kRingBytes = kWarps * kDepth * kStepBytes;
constexpr int kFastSmem = kRingBytes + 16 * kFXPitch * 2;

template <bool kBf16>
struct FastNum;
template <>
struct FastNum<true> {
    static constexpr uint32_t kOnes = 0x3F803F80u;  // bf16x2 {1, 1}
    static constexpr float kB = 136.f;
    __device__ __forceinline__ static float lo(uint32_t r) { return __uint_as_float(r << 16); }
    __device__ __forceinline__ static float hi(uint32_t r) { return __uint_as_float(r & 0xFFFF0000u); }
};
template <>
struct FastNum<false> {
    static constexpr uint32_t kOnes = 0x3C003C00u;  // half2 {1, 1}
    static constexpr float kB = 1032.f;
    __device__ __forceinline__ static float lo(uint32_t r) { return __half2float(__ushort_as_half((unsigned short)(r & 0xFFFFu))); }
    __device__ __forceinline__ static float hi(uint32_t r) { return __half2float(__ushort_as_half((unsigned short)(r >> 16))); }
};

// Four 8x8 b16 matrices from shared memory, one register each. Non-transposed: lane (g,q) gets elements (2q, 2q+1) of row g.
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
// Transposed: lane (g,q) gets column g of rows 2q (low half) and 2q+1 (high half).
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// kExact = false: the group-wise form described above. kExact = true: the same data path (cp.async ring, ldmatrix
// fragments, barrier-free main loop) with the reference's default arithmetic instead: every weight pair goes through
// sub / add / mul in the activation dtype (two roundings, no FMA) before the MMA, exactly as in wqbmm_decode.cu.
template <bool kBf16, bool kHasOffset, bool kExact>
__global__ void __launch_bounds__(kThreads, 2) wqbmm_decode_fast_kernel(const DecodeArgs a)
{
    using N = Num<kBf16>;
    using F = FastNum<kBf16>;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, q = lane & 3;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    __shared__ int s_reduce;
    extern __shared__ __align__(128) uint8_t dyn[];
    uint16_t(*xs)[kFXPitch] = reinterpret_cast<uint16_t(*)[kFXPitch]>(dyn + kRingBytes);

    const int64_t c = blockIdx.x;
    const int64_t strip = a.cluster ? c / a.splits : c % a.strips;
    const int64_t chunk = a.cluster ? c % a.splits : c / a.strips;
    const uint16_t* x16 = reinterpret_cast<const uint16_t*>(a.x);
    // this CTA's k range, in k-steps; both ends are multiples of k_align (a whole number of k-groups when there are enough
    // groups to go round, else of step pairs), so a pair of steps never straddles a group
    const int64_t units = a.ksteps / a.k_align;
    const int64_t sa = ((chunk * units) / a.splits) * a.k_align;
    const int64_t sb = (((chunk + 1) * units) / a.splits) * a.k_align;
    const int nsteps = (int)(sb - sa);
    const int64_t warp_col = strip * kStripCols + warp * kWarpCols;

    float total[kTiles][4], part[kTiles][4], xsum[4];
#pragma unroll
    for (int t = 0; t < kTiles; ++t) {
        total[t][0] = total[t][1] = total[t][2] = total[t][3] = 0.f;
        part[t][0] = part[t][1] = part[t][2] = part[t][3] = 0.f;
    }
    xsum[0] = xsum[1] = xsum[2] = xsum[3] = 0.f;

    // ---- weight copies: lane L moves the 16-byte piece (row L/2, half L%2) of every k-step of this warp's 64 columns.
    // Ring slot layout (512 B): piece (half, row) at ((half*2 + row/8)*8 + row%8)*16, i.e. four 8x16-byte matrices
    // (rows 0-7 | 8-15) x (columns 0-31 | 32-63), each 128 contiguous bytes: what one ldmatrix.x4 wants. ----
    const int64_t pitch_b = a.w_ld32 * 4;
    const int crow = lane >> 1, chalf = lane & 1;
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(dyn) + (uint32_t)warp * (kDepth * kStepBytes);
    const uint32_t cdst = ring + (uint32_t)(((chalf * 2 + (crow >> 3)) * 8 + (crow & 7)) * 16);
    const bool c_ok = warp_col + chalf * 32 < a.n;
    const char* cptr = reinterpret_cast<const char*>(a.w) + (sa * 16 + crow) * pitch_b + (c_ok ? (warp_col + chalf * 32) / 2 : 0);
    const int64_t step_b = 16 * pitch_b;
    if (!c_ok) {  // columns past n (last strip only): this lane's pieces of every ring slot are zero and never copied into
#pragma unroll
        for (int sidx = 0; sidx < kDepth; ++sidx)
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(cdst + (uint32_t)sidx * kStepBytes), "r"(0u) : "memory");
    }
    const int my_steps = c_ok ? nsteps : 0;
    auto issue_pair = [&](int first_step, uint32_t dst) {  // steps first_step, first_step + 1 into ring bytes dst, dst + 512
        if (first_step < my_steps) {  // ranges hold an even number of steps
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(cptr) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + kStepBytes), "l"(cptr + step_b) : "memory");
        }
        cptr += 2 * step_b;
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // ---- x[:, this run's k range] through shared memory, kFChunk steps at a time ----
    auto stage_x = [&](int chunk_idx) {
        const int64_t k_first = (sa + (int64_t)chunk_idx * kFChunk) * 16;
        const int64_t k_end = sb * 16;
        uint16_t(*dst)[kFXPitch] = xs;
        for (int e = tid; e < 16 * (kFChunk * 2); e += kThreads) {  // 16-byte pieces: 16 rows x (kFChunk*16/8)
            const int row = e / (kFChunk * 2), piece = e % (kFChunk * 2);
            const int64_t kk = k_first + piece * 8;
            uint16_t* d = &dst[row][piece * 8];
            if (row < a.m && kk < k_end) {
                const uint32_t saddr = (uint32_t)__cvta_generic_to_shared(d);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(x16 + (int64_t)row * a.x_ld + kk) : "memory");
            } else {
                *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage_x(0);
#pragma unroll
    for (int i = 0; i < kDepth; i += 2) issue_pair(i, cdst + (uint32_t)i * kStepBytes);

    // ---- scale/offset of the lane's 16 output columns: 8q..8q+7 of each 32-column half ----
    const int64_t scol0 = (warp_col + 8 * q < a.n) ? warp_col + 8 * q : 0;
    const int64_t scol1 = (warp_col + 32 + 8 * q < a.n) ? warp_col + 32 + 8 * q : 0;
    uint32_t raw_s[8], raw_o[8];
    const int spg = (int)min(a.steps_per_group, (int64_t)0x7FFFFFFF);
    // exact mode: scale/offset of the lane's B-fragment columns (tile t < 4: column 4g + t, else 32 + 4g + t - 4), each
    // duplicated into both halves of a register (the halves are two k rows of the same column)
    const int64_t ecol0 = (warp_col + 4 * g < a.n) ? warp_col + 4 * g : 0;
    const int64_t ecol1 = (warp_col + 32 + 4 * g < a.n) ? warp_col + 32 + 4 * g : 0;
    uint32_t sc[kTiles], of[kTiles];

    auto finish_group = [&]() {
        if (kExact) return;
#pragma unroll
        for (int idx = 0; idx < 16; ++idx) {  // idx = 8*half + 4*(e&1) + (t&3): position among the lane's 16 columns
            const uint32_t rs = raw_s[idx >> 1];
            const float sf = (idx & 1) ? F::hi(rs) : F::lo(rs);
            float of = -F::kB;
            if (kHasOffset) {
                const uint32_t ro = raw_o[idx >> 1];
                of += (idx & 1) ? F::hi(ro) : F::lo(ro);
            }
            const int t = (idx >> 3) * 4 + (idx & 3), e0 = (idx >> 2) & 1;  // fragment entries e0 (row g) and e0 + 2 (row g + 8)
            total[t][e0] = fmaf(sf, fmaf(of, xsum[0], part[t][e0]), total[t][e0]);
            total[t][e0 + 2] = fmaf(sf, fmaf(of, xsum[2], part[t][e0 + 2]), total[t][e0 + 2]);
        }
#pragma unroll
        for (int t = 0; t < kTiles; ++t) part[t][0] = part[t][1] = part[t][2] = part[t][3] = 0.f;
        xsum[0] = xsum[1] = xsum[2] = xsum[3] = 0.f;
    };
    uint32_t rs_next[4], ro_next[4] = {0u, 0u, 0u, 0u};
    const int64_t n_groups = (a.ksteps + spg - 1) / spg;
    auto fetch_exact = [&](int64_t group) {
        if (a.scale_sn != 0) {
            const uint16_t* sp = reinterpret_cast<const uint16_t*>(a.scale) + group * a.scale_sg;
            const uint2 s0 = __ldg(reinterpret_cast<const uint2*>(sp + ecol0)), s1 = __ldg(reinterpret_cast<const uint2*>(sp + ecol1));
            rs_next[0] = s0.x; rs_next[1] = s0.y; rs_next[2] = s1.x; rs_next[3] = s1.y;
            if (kHasOffset) {
                const uint16_t* op = reinterpret_cast<const uint16_t*>(a.offset) + group * a.scale_sg;
                const uint2 o0 = __ldg(reinterpret_cast<const uint2*>(op + ecol0)), o1 = __ldg(reinterpret_cast<const uint2*>(op + ecol1));
                ro_next[0] = o0.x; ro_next[1] = o0.y; ro_next[2] = o1.x; ro_next[3] = o1.y;
            }
        } else {
            const uint32_t sv = reinterpret_cast<const uint16_t*>(a.scale)[group * a.scale_sg];
            const uint32_t ov = kHasOffset ? reinterpret_cast<const uint16_t*>(a.offset)[group * a.scale_sg] : 0u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                rs_next[i] = sv | (sv << 16);
                ro_next[i] = ov | (ov << 16);
            }
        }
    };
    if (kExact) fetch_exact(sa / spg);
    auto load_group = [&](int64_t group) {
        if (kExact) {
            // the values fetched one group ago become this group's registers; the next group's are requested now, so that
            // their L2 round trip is not in front of the group's first dequantisation
#pragma unroll
            for (int t = 0; t < kTiles; ++t) {
                const uint32_t sel = (t & 1) ? 0x3232u : 0x1010u;
                sc[t] = prmt(rs_next[t >> 1], rs_next[t >> 1], sel);
                if (kHasOffset) of[t] = prmt(ro_next[t >> 1], ro_next[t >> 1], sel);
            }
            fetch_exact(min(group + 1, n_groups - 1));
            return;
        }
        if (a.scale_sn != 0) {
            const uint16_t* sp = reinterpret_cast<const uint16_t*>(a.scale) + group * a.scale_sg;
            const uint4 s0 = __ldg(reinterpret_cast<const uint4*>(sp + scol0)), s1 = __ldg(reinterpret_cast<const uint4*>(sp + scol1));
            raw_s[0] = s0.x; raw_s[1] = s0.y; raw_s[2] = s0.z; raw_s[3] = s0.w;
            raw_s[4] = s1.x; raw_s[5] = s1.y; raw_s[6] = s1.z; raw_s[7] = s1.w;
            if (kHasOffset) {
                const uint16_t* op = reinterpret_cast<const uint16_t*>(a.offset) + group * a.scale_sg;
                const uint4 o0 = __ldg(reinterpret_cast<const uint4*>(op + scol0)), o1 = __ldg(reinterpret_cast<const uint4*>(op + scol1));
                raw_o[0] = o0.x; raw_o[1] = o0.y; raw_o[2] = o0.z; raw_o[3] = o0.w;
                raw_o[4] = o1.x; raw_o[5] = o1.y; raw_o[6] = o1.z; raw_o[7] = o1.w;
            }
        } else {
            const uint32_t sv = reinterpret_cast<const uint16_t*>(a.scale)[group * a.scale_sg];
            const uint32_t ov = kHasOffset ? reinterpret_cast<const uint16_t*>(a.offset)[group * a.scale_sg] : 0u;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                raw_s[i] = sv | (sv << 16);
                raw_o[i] = ov | (ov << 16);
            }
        }
    };
    // one k-step: 4 registers of paired nibbles -> 16 B fragments (a shift and a logic op each) -> 8 MMAs + the row-sum MMA
    auto compute = [&](const uint32_t(&w4)[4], const uint32_t(&af)[4]) {
        uint32_t b0[kTiles], b1[kTiles];
        if (kExact) {
            // (nibble ^ 8) | magic == B + w exactly; then the reference's rounding points: w' = mul(add(sub(v, B), offset), scale)
            auto deq = [&](uint32_t tw, int t) {
                uint32_t v;
                asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(v) : "r"(tw), "n"(0x000F000F), "n"(N::kMagic));
                v = N::sub(v, a.c_bias);
                if (kHasOffset) v = N::add(v, of[t]);
                return N::mul(v, sc[t]);
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
        for (int t = 0; t < kTiles; ++t) N::mma_free(part[t], af, b0[t], b1[t]);
        N::mma_free(xsum, af, F::kOnes, F::kOnes);
    };

    // per-lane ldmatrix row addresses: weights: matrix l/8, row l%8 = byte l*16 of the slot; x: rows (l%8) + 8*((l/8)&1),
    // k offset 8*(l/16)
    const uint32_t wlane = ring + (uint32_t)lane * 16;
    const uint32_t xlane = (uint32_t)__cvta_generic_to_shared(&xs[(lane & 7) + 8 * ((lane >> 3) & 1)][8 * (lane >> 4)]);

    // Commit groups so far, oldest first: X0, G0..G(kDepth/2-1); from here on every pair p adds G(p + kDepth/2). A wait
    // for pair p's copies may therefore leave the kDepth/2 - 1 groups behind it in flight.
    asm volatile("cp.async.wait_group %0;" ::"n"(kDepth / 2 - 1) : "memory");  // X0 and G0
    __syncwarp();
    __syncthreads();
    uint32_t w0[4], a0[4], w1[4], a1[4];
    ldsm_x4_trans(wlane, w0);
    ldsm_x4(xlane, a0);

    int i = 0;                      // k-step relative to sa, even
    int x_left = kFChunk;           // steps left in the staged x chunk, counting step i
    uint32_t roff = 0;              // ring byte offset of step i
    uint32_t xcur = xlane;          // x fragment address of step i
    int64_t group = sa / spg;
    int seg_end = (int)min((int64_t)nsteps, (group + 1) * (int64_t)spg - sa);
    while (i < nsteps) {
        load_group(group);
        for (; i < seg_end; i += 2) {
            ldsm_x4_trans(wlane + roff + kStepBytes, w1);
            ldsm_x4(xcur + 32, a1);
            compute(w0, a0);
            // the copies of the next pair (and everything older) have landed, for this lane and the others of the warp
            asm volatile("cp.async.wait_group %0;" ::"n"(kDepth / 2 - 2) : "memory");
            __syncwarp();
            x_left -= 2;
            xcur += 64;
            if (x_left == 0 && i + 2 < nsteps) {
                // the staged x is used up (k ranges longer than kFChunk steps only): everyone finishes reading it, the
                // next piece is copied in, and the copies in flight are drained once
                __syncthreads();
                stage_x((i + 2) / kFChunk);
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                __syncthreads();
                x_left = kFChunk;
                xcur = xlane;
            }
            const uint32_t roff_next = (roff + 2 * kStepBytes == kDepth * kStepBytes) ? 0u : roff + 2 * kStepBytes;
            ldsm_x4_trans(wlane + roff_next, w0);  // stale bytes past the end of the range are loaded and never used
            ldsm_x4(xcur, a0);
            compute(w1, a1);
            __syncwarp();  // every lane has read steps i, i+1: their ring slots may be overwritten
            issue_pair(i + kDepth, cdst + roff);
            roff = roff_next;
        }
        finish_group();
        ++group;
        seg_end = min(nsteps, seg_end + spg);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    if (!a.cluster) {
        combine_and_store<kBf16, 1>(a, total, c, strip, warp, lane, tid, &s_reduce);
        return;
    }
    // ---- the strip's k-splits are one cluster: fragments go to each CTA's own shared memory (the warp's part of the ring, all
    // of whose copies have landed and been read), the first CTA sums them over distributed shared memory in split order ----
    const uint32_t frag = ring + (uint32_t)lane * 16;  // [tile][lane] float4, 4 KB of the warp's 6 KB
#pragma unroll
    for (int t = 0; t < kTiles; ++t)
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(frag + t * 512), "f"(total[t][0]), "f"(total[t][1]), "f"(total[t][2]),
                     "f"(total[t][3])
                     : "memory");
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (chunk == 0) {
        for (uint32_t j = 1; j < (uint32_t)a.splits; ++j) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(frag), "r"(j));
            float4 v[kTiles];
#pragma unroll
            for (int t = 0; t < kTiles; ++t)
                asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                             : "=f"(v[t].x), "=f"(v[t].y), "=f"(v[t].z), "=f"(v[t].w)
                             : "r"(remote + t * 512)
                             : "memory");
#pragma unroll
            for (int t = 0; t < kTiles; ++t) {
                total[t][0] += v[t].x; total[t][1] += v[t].y; total[t][2] += v[t].z; total[t][3] += v[t].w;
            }
        }
    }
    // nobody leaves (and frees its shared memory) before the first CTA has read everything
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (chunk == 0) store_tile_y<kBf16, 1>(a, total, strip, warp, lane);
}

int g_fast_ctas_per_sm[8] = {0, 0, 0, 0, 0, 0, 0, 0};
std::atomic<uint64_t> g_fast_configured[8];

template <bool kBf16, bool kHasOffset, bool kExact>
int fast_grid(int variant)
{
    once_per_device(g_fast_configured[variant], [&] {
        return cudaFuncSetAttribute(wqbmm_decode_fast_kernel<kBf16, kHasOffset, kExact>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFastSmem);
    });
    if (g_fast_ctas_per_sm[variant] == 0) {
        int nb = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, wqbmm_decode_fast_kernel<kBf16, kHasOffset, kExact>, kThreads, kFastSmem);
        g_fast_ctas_per_sm[variant] = nb > 0 ? nb : 1;
    }
    return current_sm_count() * g_fast_ctas_per_sm[variant];
}

constexpr int kFastMaxGrid = 148 * 4 * 2;  // same workspace layout and bound as the default decode kernel

}  // namespace

bool wqbmm_decode_eligible(const OpsnnWqbmmParams* p);
uint64_t wqbmm_decode_workspace_size(const OpsnnWqbmmParams* p);

bool wqbmm_decode_fast_eligible(const OpsnnWqbmmParams* p)
{
    if (!wqbmm_decode_eligible(p)) return false;
    if (p->n % 32 != 0 || p->w_ld % 32 != 0) return false;                // 16-byte pieces of 32 columns, 16-byte aligned rows
    if ((reinterpret_cast<uintptr_t>(p->w) % 16) != 0) return false;
    if (p->scale_sn == 1 && (p->scale_sg % 8 != 0)) return false;
    if (p->k % 32 != 0 || (p->group_size != 0 && p->group_size % 32 != 0)) return false;  // step pairs never straddle a group
    return true;
}

// exact = false: group-wise high-performance mode; exact = true: the default arithmetic on the same data path.
int32_t wqbmm_decode_ring_launch(const OpsnnWqbmmParams* p, cudaStream_t stream, bool exact)
{
    DecodeArgs a{};
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
    a.m = (int32_t)p->m;
    a.n = p->n;
    a.k = p->k;
    a.strips = (p->n + kStripCols - 1) / kStripCols;
    a.ksteps = p->k / 16;
    a.steps_per_group = p->group_size > 0 ? p->group_size / 16 : a.ksteps;
    const bool bf16 = p->x_dtype == ACL_BF16, has_off = p->offset != nullptr;
    const int variant = (exact ? 4 : 0) + (bf16 ? 2 : 0) + (has_off ? 1 : 0);
    int resident = 0;
    switch (variant) {
        case 0: resident = fast_grid<false, false, false>(0); break;
        case 1: resident = fast_grid<false, true, false>(1); break;
        case 2: resident = fast_grid<true, false, false>(2); break;
        case 3: resident = fast_grid<true, true, false>(3); break;
        case 4: resident = fast_grid<false, false, true>(4); break;
        case 5: resident = fast_grid<false, true, true>(5); break;
        case 6: resident = fast_grid<true, false, true>(6); break;
        default: resident = fast_grid<true, true, true>(7); break;
    }
    int64_t splits = resident / a.strips;
    if (const char* e = getenv("OPSNN_WQ_DECODE_SPLITS")) {
        int v = atoi(e);
        if (v > 0) splits = v;
    }
    if (splits > a.ksteps) splits = a.ksteps;
    if (splits * a.strips > kFastMaxGrid) splits = kFastMaxGrid / a.strips;
    if (splits < 1) splits = 1;
    // k ranges of whole groups when every split gets at least two of them, else of step pairs
    a.k_align = (a.ksteps % a.steps_per_group == 0 && a.ksteps / a.steps_per_group >= 2 * splits) ? a.steps_per_group : 2;
    if (splits > a.ksteps / a.k_align) splits = a.ksteps / a.k_align;
    if (splits < 1) splits = 1;
    a.splits = splits;
    const int64_t grid64 = a.strips * splits;
    if (grid64 > 0x7FFFFFFF) return (int32_t)cudaErrorInvalidConfiguration;
    const int grid = (int)grid64;
    const uint64_t tag_bytes = (((uint64_t)kFastMaxGrid * 8 + 255) / 256) * 256;
    // Opt-in (OPSNN_WQ_DECODE_CLUSTER=1): measured equal to the workspace combine on the benchmark shape (the tail is set by the
    // slowest CTA's main loop, not by the combination), so the path that needs no cluster scheduling stays the default.
    const bool want_cluster = splits >= 2 && splits <= 8 && getenv("OPSNN_WQ_DECODE_CLUSTER") != nullptr;
    if (splits > 1 && !want_cluster && (p->workspace == nullptr || p->workspace_size < wqbmm_decode_workspace_size(p)))
        return (int32_t)cudaErrorInvalidValue;
    a.tags = reinterpret_cast<unsigned long long*>(p->workspace);
    a.partials = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(p->workspace) + tag_bytes);
    a.nonce = next_nonce();
    a.c_mask = 0x000F000Fu;
    a.c_magic = bf16 ? Num<true>::kMagic : Num<false>::kMagic;
    a.c_bias = bf16 ? Num<true>::kBias : Num<false>::kBias;
    // the k-splits of a strip as one thread-block cluster (portable sizes only): the combination then needs no global memory
    a.cluster = want_cluster ? 1 : 0;
    if (a.cluster) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)grid, 1, 1);
        cfg.blockDim = dim3(kThreads, 1, 1);
        cfg.dynamicSmemBytes = kFastSmem;
        cfg.stream = stream;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = (unsigned)splits;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        cudaError_t rc;
        switch (variant) {
            case 0: rc = cudaLaunchKernelEx(&cfg, wqbmm_decode_fast_kernel<false, false, false>, a); break;
            case 1: rc = cudaLaunchKernelEx(&cfg, wqbmm_decode_fast_kernel<false, true, false>, a); break;
            case 2: rc = cudaLaunchKernelEx(&cfg, wqbmm_decode_fast_kernel<true, false, false>, a); break;
            case 3: rc = cudaLaunchKernelEx(&cfg, wqbmm_decode_fast_kernel<true, true, false>, a); break;
            case 4: rc = cudaLaunchKernelEx(&cfg, wqbmm_decode_fast_kernel<false, false, true>, a); break;
            case 5: rc = cudaLaunchKernelEx(&cfg, wqbmm_decode_fast_kernel<false, true, true>, a); break;
            case 6: rc = cudaLaunchKernelEx(&cfg, wqbmm_decode_fast_kernel<true, false, true>, a); break;
            default: rc = cudaLaunchKernelEx(&cfg, wqbmm_decode_fast_kernel<true, true, true>, a); break;
        }
        note_launch(exact ? "wqbmm_decode" : "wqbmm_decode_fast");
        return (int32_t)rc;
    }
    switch (variant) {
        case 0: wqbmm_decode_fast_kernel<false, false, false><<<grid, kThreads, kFastSmem, stream>>>(a); break;
        case 1: wqbmm_decode_fast_kernel<false, true, false><<<grid, kThreads, kFastSmem, stream>>>(a); break;
        case 2: wqbmm_decode_fast_kernel<true, false, false><<<grid, kThreads, kFastSmem, stream>>>(a); break;
        case 3: wqbmm_decode_fast_kernel<true, true, false><<<grid, kThreads, kFastSmem, stream>>>(a); break;
        case 4: wqbmm_decode_fast_kernel<false, false, true><<<grid, kThreads, kFastSmem, stream>>>(a); break;
        case 5: wqbmm_decode_fast_kernel<false, true, true><<<grid, kThreads, kFastSmem, stream>>>(a); break;
        case 6: wqbmm_decode_fast_kernel<true, false, true><<<grid, kThreads, kFastSmem, stream>>>(a); break;
        default: wqbmm_decode_fast_kernel<true, true, true><<<grid, kThreads, kFastSmem, stream>>>(a); break;
    }
    note_launch(exact ? "wqbmm_decode" : "wqbmm_decode_fast");
    return (int32_t)cudaGetLastError();
}

int32_t wqbmm_decode_fast_launch(const OpsnnWqbmmParams* p, cudaStream_t stream) { return wqbmm_decode_ring_launch(p, stream, false); }

}  // namespace opsnn
