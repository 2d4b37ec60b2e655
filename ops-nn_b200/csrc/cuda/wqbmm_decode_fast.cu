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
// on another warp. The ring layout puts the four rows a lane needs ({2q, 2q+1, 2q+8, 2q+9}) 128 bytes apart and the
// eight 16-byte pieces of one such row set on distinct bank groups, so the fragment reads are conflict free.
#include "common.cuh"
#include "wqbmm_decode_common.cuh"

namespace opsnn {

namespace {

constexpr int kDepth = 16;                       // k-steps in a warp's ring (power of two)
constexpr int kStepBytes = 512;                  // 16 rows x 32 bytes
constexpr int kPending = kDepth / 2 - 1;         // commit groups (2 k-steps each) allowed in flight at a wait
constexpr int kFChunk = 16;                      // k-steps of x per staged chunk (double buffered)
constexpr int kFXPitch = kFChunk * 16 + 8;       // elements; +8 skews rows over the banks
constexpr int kRingBytes = kWarps * kDepth * kStepBytes;
constexpr int kFastSmem = kRingBytes + 2 * 16 * kFXPitch * 2;

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

__device__ __forceinline__ uint32_t lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

template <bool kBf16, bool kHasOffset>
__global__ void __launch_bounds__(kThreads, 2) wqbmm_decode_fast_kernel(const DecodeArgs a)
{
    using N = Num<kBf16>;
    using F = FastNum<kBf16>;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, q = lane & 3;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    __shared__ int s_reduce;
    extern __shared__ __align__(128) uint8_t dyn[];
    uint16_t(*xs)[16][kFXPitch] = reinterpret_cast<uint16_t(*)[16][kFXPitch]>(dyn + kRingBytes);

    const int64_t c = blockIdx.x;
    const int64_t strip = c % a.strips;
    const int64_t chunk = c / a.strips;
    const uint16_t* x16 = reinterpret_cast<const uint16_t*>(a.x);
    const int64_t sa = (chunk * a.ksteps) / a.splits;
    const int64_t sb = ((chunk + 1) * a.ksteps) / a.splits;
    const int nsteps = (int)(sb - sa);
    const int64_t warp_col = strip * kStripCols + warp * kWarpCols;

    float total[kTiles][4], part[kTiles][4], xsum[4];
#pragma unroll
    for (int t = 0; t < kTiles; ++t) {
        total[t][0] = total[t][1] = total[t][2] = total[t][3] = 0.f;
        part[t][0] = part[t][1] = part[t][2] = part[t][3] = 0.f;
    }
    xsum[0] = xsum[1] = xsum[2] = xsum[3] = 0.f;

    // ---- weight copies: lane L moves the 16-byte piece (row L/2, half L%2) of every k-step of this warp's 64 columns ----
    const int64_t pitch_b = a.w_ld32 * 4;
    const int crow = lane >> 1, chalf = lane & 1;
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(dyn) + (uint32_t)warp * (kDepth * kStepBytes);
    const uint32_t cdst = ring + (uint32_t)(((crow & 1) + 2 * (crow >> 3)) * 128 + ((crow & 7) >> 1) * 32 + chalf * 16);
    const bool c_ok = warp_col + chalf * 32 < a.n;
    const char* cptr = reinterpret_cast<const char*>(a.w) + (sa * 16 + crow) * pitch_b + (c_ok ? (warp_col + chalf * 32) / 2 : 0);
    const uint32_t csize = c_ok ? 16u : 0u;  // 0: the piece is zero-filled, nothing is read
    int issued = 0;
    auto issue_pair = [&]() {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (issued < nsteps) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(cdst + (uint32_t)(issued & (kDepth - 1)) * kStepBytes),
                             "l"(cptr), "r"(csize)
                             : "memory");
                cptr += 16 * pitch_b;
            }
            ++issued;
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // ---- x[:, this run's k range] through shared memory in chunks of kFChunk steps ----
    auto stage_x = [&](int chunk_idx) {
        const int64_t k_first = (sa + (int64_t)chunk_idx * kFChunk) * 16;
        const int64_t k_end = sb * 16;
        uint16_t(*dst)[kFXPitch] = xs[chunk_idx & 1];
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
    for (int i = 0; i < kDepth / 2; ++i) issue_pair();

    // ---- group bookkeeping: scale/offset of the lane's 16 output columns (tile t, fragment column e&1 -> 8*(e&1)+t) ----
    const int64_t scol = (warp_col + 16 * q < a.n) ? warp_col + 16 * q : 0;
    uint32_t raw_s[8], raw_o[8];
    int64_t group = sa / a.steps_per_group - 1;
    int first_skip = (int)(sa % a.steps_per_group);
    int group_left = 0;
    bool have_group = false;
    const int spg = (int)min(a.steps_per_group, (int64_t)0x7FFFFFFF);

    auto finish_group = [&]() {
#pragma unroll
        for (int idx = 0; idx < 16; ++idx) {
            const uint32_t rs = raw_s[idx >> 1];
            const float sf = (idx & 1) ? F::hi(rs) : F::lo(rs);
            float of = -F::kB;
            if (kHasOffset) {
                const uint32_t ro = raw_o[idx >> 1];
                of += (idx & 1) ? F::hi(ro) : F::lo(ro);
            }
            const int t = idx & 7, e0 = idx >> 3;  // fragment entries e0 (row g) and e0 + 2 (row g + 8)
            total[t][e0] = fmaf(sf, fmaf(of, xsum[0], part[t][e0]), total[t][e0]);
            total[t][e0 + 2] = fmaf(sf, fmaf(of, xsum[2], part[t][e0 + 2]), total[t][e0 + 2]);
        }
#pragma unroll
        for (int t = 0; t < kTiles; ++t) part[t][0] = part[t][1] = part[t][2] = part[t][3] = 0.f;
        xsum[0] = xsum[1] = xsum[2] = xsum[3] = 0.f;
    };
    auto load_group = [&]() {
        if (a.scale_sn != 0) {
            const uint16_t* sp = reinterpret_cast<const uint16_t*>(a.scale) + group * a.scale_sg + scol;
            const uint4 s0 = __ldg(reinterpret_cast<const uint4*>(sp)), s1 = __ldg(reinterpret_cast<const uint4*>(sp) + 1);
            raw_s[0] = s0.x; raw_s[1] = s0.y; raw_s[2] = s0.z; raw_s[3] = s0.w;
            raw_s[4] = s1.x; raw_s[5] = s1.y; raw_s[6] = s1.z; raw_s[7] = s1.w;
            if (kHasOffset) {
                const uint16_t* op = reinterpret_cast<const uint16_t*>(a.offset) + group * a.scale_sg + scol;
                const uint4 o0 = __ldg(reinterpret_cast<const uint4*>(op)), o1 = __ldg(reinterpret_cast<const uint4*>(op) + 1);
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

    const uint32_t rd = ring + (uint32_t)(q * 32 + (g >> 2) * 16 + (g & 3) * 4);
    for (int i = 0; i < nsteps; i += 2) {
        // the copies of steps i, i+1 (and everything older, the x chunk included) have landed for this lane ...
        asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
        __syncwarp();  // ... and for the other lanes of the warp
        if ((i & (kFChunk - 1)) == 0) {
            __syncthreads();  // chunk boundary: every thread's pieces of this x chunk are visible; the other buffer is free
            if (i + kFChunk < nsteps) stage_x(i / kFChunk + 1);
        }
        const uint16_t* xrow0 = &xs[(i / kFChunk) & 1][g][2 * q];
        const uint16_t* xrow1 = &xs[(i / kFChunk) & 1][g + 8][2 * q];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int s = i + j;
            if (s >= nsteps) break;
            if (group_left == 0) {
                if (have_group) finish_group();
                ++group;
                group_left = spg - first_skip;
                first_skip = 0;
                load_group();
                have_group = true;
            }
            --group_left;

            const uint32_t slot = rd + (uint32_t)(s & (kDepth - 1)) * kStepBytes;
            const uint32_t wa = lds32(slot), wb = lds32(slot + 128), wc = lds32(slot + 256), wd = lds32(slot + 384);
            uint32_t af[4];
            {
                const int ls = (s & (kFChunk - 1)) * 16;
                af[0] = *reinterpret_cast<const uint32_t*>(xrow0 + ls);
                af[1] = *reinterpret_cast<const uint32_t*>(xrow1 + ls);
                af[2] = *reinterpret_cast<const uint32_t*>(xrow0 + ls + 8);
                af[3] = *reinterpret_cast<const uint32_t*>(xrow1 + ls + 8);
            }
            // low half: nibbles 0..3 of row a | nibbles 0..3 of row b; high half: nibbles 4..7
            const uint32_t lo01 = prmt(wa, wb, 0x5410u), hi01 = prmt(wa, wb, 0x7632u);
            const uint32_t lo23 = prmt(wc, wd, 0x5410u), hi23 = prmt(wc, wd, 0x7632u);
            uint32_t b0[kTiles], b1[kTiles];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(b0[t]) : "r"(lo01 >> (4 * t)), "r"(a.c_mask), "r"(a.c_magic));
                asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(b1[t]) : "r"(lo23 >> (4 * t)), "r"(a.c_mask), "r"(a.c_magic));
                asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(b0[4 + t]) : "r"(hi01 >> (4 * t)), "r"(a.c_mask), "r"(a.c_magic));
                asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(b1[4 + t]) : "r"(hi23 >> (4 * t)), "r"(a.c_mask), "r"(a.c_magic));
            }
#pragma unroll
            for (int t = 0; t < kTiles; ++t) N::mma(part[t], af, b0[t], b1[t]);
            N::mma(xsum, af, F::kOnes, F::kOnes);
        }
        __syncwarp();  // every lane has read steps i, i+1: their ring slots may be overwritten
        issue_pair();
    }
    if (have_group) finish_group();
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    combine_and_store<kBf16>(a, total, c, strip, warp, lane, tid, &s_reduce);
}

int g_fast_ctas_per_sm[4] = {0, 0, 0, 0};
int g_fast_sm_count = 0;

template <bool kBf16, bool kHasOffset>
int fast_grid(int variant)
{
    if (g_fast_sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_fast_sm_count, cudaDevAttrMultiProcessorCount, dev);
    }
    if (g_fast_ctas_per_sm[variant] == 0) {
        cudaFuncSetAttribute(wqbmm_decode_fast_kernel<kBf16, kHasOffset>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFastSmem);
        int nb = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, wqbmm_decode_fast_kernel<kBf16, kHasOffset>, kThreads, kFastSmem);
        g_fast_ctas_per_sm[variant] = nb > 0 ? nb : 1;
    }
    return g_fast_sm_count * g_fast_ctas_per_sm[variant];
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
    return true;
}

int32_t wqbmm_decode_fast_launch(const OpsnnWqbmmParams* p, cudaStream_t stream)
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
    const int variant = (bf16 ? 2 : 0) + (has_off ? 1 : 0);
    int resident = 0;
    switch (variant) {
        case 0: resident = fast_grid<false, false>(0); break;
        case 1: resident = fast_grid<false, true>(1); break;
        case 2: resident = fast_grid<true, false>(2); break;
        default: resident = fast_grid<true, true>(3); break;
    }
    int64_t splits = resident / a.strips;
    if (const char* e = getenv("OPSNN_WQ_DECODE_SPLITS")) {
        int v = atoi(e);
        if (v > 0) splits = v;
    }
    if (splits > a.ksteps) splits = a.ksteps;
    if (splits * a.strips > kFastMaxGrid) splits = kFastMaxGrid / a.strips;
    if (splits < 1) splits = 1;
    a.splits = splits;
    const int64_t grid64 = a.strips * splits;
    if (grid64 > 0x7FFFFFFF) return (int32_t)cudaErrorInvalidConfiguration;
    const int grid = (int)grid64;
    const uint64_t tag_bytes = (((uint64_t)kFastMaxGrid * 8 + 255) / 256) * 256;
    if (splits > 1 && (p->workspace == nullptr || p->workspace_size < wqbmm_decode_workspace_size(p))) return (int32_t)cudaErrorInvalidValue;
    a.tags = reinterpret_cast<unsigned long long*>(p->workspace);
    a.partials = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(p->workspace) + tag_bytes);
    a.nonce = next_nonce();
    a.c_mask = 0x000F000Fu;
    a.c_magic = bf16 ? Num<true>::kMagic : Num<false>::kMagic;
    a.c_bias = 0;
    switch (variant) {
        case 0: wqbmm_decode_fast_kernel<false, false><<<grid, kThreads, kFastSmem, stream>>>(a); break;
        case 1: wqbmm_decode_fast_kernel<false, true><<<grid, kThreads, kFastSmem, stream>>>(a); break;
        case 2: wqbmm_decode_fast_kernel<true, false><<<grid, kThreads, kFastSmem, stream>>>(a); break;
        default: wqbmm_decode_fast_kernel<true, true><<<grid, kThreads, kFastSmem, stream>>>(a); break;
    }
    note_launch("wqbmm_decode_fast");
    return (int32_t)cudaGetLastError();
}

}  // namespace opsnn
