// Weight-only quant matmul, decode kernel: y[m<=16, n] = x[m,k] @ dequant(w_int4[k,n]) for the HBM-bound small-m regime.
//
// Replaces, for this regime, the reference's per-group "reg-base" kernel
// (weight_quant_batch_matmul_v2/op_kernel/arch35/weight_quant_batch_matmul_v2_reg_base_common.h:164-286 and
//  weight_quant_batch_matmul_v2_vf.h:345-442: vector cores dequantise int4 -> bf16 into L1, cube core multiplies) and
// its host tiling (op_host/op_tiling/arch35/weight_quant_batch_matmul_v2_reg_base_tiling.cpp:89-337).
//
// Data layout. w is int4 packed 8 per 32-bit word along n, element j of a word at bits [4j,4j+4), word (k,c) holds
// columns 8c..8c+7 (reference: aclnn_weight_quant_batch_matmul_v2.cpp:1482-1524). scale/offset are (groups, n) in x's
// dtype. The weight (k*n/2 bytes) is read exactly once from HBM with 8-byte loads, 128 contiguous bytes per row per
// warp-row; x (m*k*2 bytes) and the scales stay in L2/L1.
//
// Mapping. One warp owns 128 columns. Lane (g = lane/4, q = lane%4) loads the word pair 2g,2g+1 (16 columns) of the four
// rows {2q, 2q+1, 2q+8, 2q+9} of every 16-row k-step: exactly the rows an m16n8k16 B fragment wants from this lane.
// A byte permute pairs the two rows' words so that one mask-xor turns nibble j of both rows into a bf16x2 {136+w_k,
// 136+w_k+1} (0x4300 | (nibble ^ 8) == 128 + 8 + w, exact); then, per the reference's rounding points,
//     w' = hmul2( hadd2( hsub2(v, 136), offset ), scale )          // each a single bf16 (fp16) rounding, no FMA
// feeds mma.sync.m16n8k16 (fp32 accumulate). Nibble j of word h of the pair is MMA tile 8h+j, so no data is shuffled
// between lanes; the column permutation this implies is undone when y is written.
//
// Work split. The (column strip of 512) x (k-step of 16) space is cut into equal contiguous runs, one per CTA, with
// gridDim = SMs x resident CTAs, so every SM streams the same number of bytes regardless of n and k. A strip whose k
// range is shared by several CTAs is summed through workspace: every contributor stores its fp32 fragment, then a
// launch nonce; whichever contributor observes all nonces present (at least one does: store, fence.sc, load) adds
// the fragments in CTA order - so the result does not depend on arrival order - and writes y, then zeroes the strip's
// nonces. No atomics, no spinning, no zero-initialised workspace (stale bytes never equal a fresh 64-bit nonce), and a
// replayed launch with an unchanged nonce still works because the previous run retired its tags. Two launches must
// not share one workspace concurrently.
#include <atomic>
#include <chrono>

#include "common.cuh"

namespace opsnn {

namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kStripCols = kWarps * 128;  // 512
constexpr int kPrefetch = 4;              // k-steps of weight words held in registers ahead of use
constexpr int kTiles = 16;                // m16n8 tiles per warp

struct DecodeArgs {
    const uint32_t* w;     // packed words
    int64_t w_ld32;        // words per k row
    const void* x;
    int64_t x_ld;
    const void* scale;
    const void* offset;
    int64_t scale_sg;      // elements between groups
    int32_t scale_sn;      // 1 per-channel/-group, 0 per-tensor
    const void* bias;
    int32_t bias_dtype;
    void* y;
    int64_t y_ld;
    int32_t m;
    int64_t n, k;
    int64_t strips, ksteps, total, steps_per_group;
    unsigned long long* tags;  // [gridDim + strips]
    float4* partials;          // [gridDim + strips][kWarps][kTiles][32]
    unsigned long long nonce;
};

__device__ __forceinline__ uint2 ldg_stream(const uint2* p)
{
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

template <bool kBf16>
struct Num;
template <>
struct Num<true> {
    using T2 = __nv_bfloat162;
    static constexpr uint32_t kMagic = 0x43084308u;  // (nibble ^ 8) | 0x4300  ->  128 + 8 + w
    static constexpr uint32_t kBias = 0x43084308u;   // bf16x2 {136, 136}
    __device__ static void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
    {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
template <>
struct Num<false> {
    using T2 = __half2;
    static constexpr uint32_t kMagic = 0x64086408u;  // (nibble ^ 8) | 0x6400  ->  1024 + 8 + w
    static constexpr uint32_t kBias = 0x64086408u;   // half2 {1032, 1032}
    __device__ static void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
    {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

template <class T2>
__device__ __forceinline__ T2 as_t2(uint32_t v)
{
    return *reinterpret_cast<T2*>(&v);
}
template <class T2>
__device__ __forceinline__ uint32_t as_u32(T2 v)
{
    return *reinterpret_cast<uint32_t*>(&v);
}

// Two nibbles (bits [3:0] and [19:16] of t) -> dequantised 16-bit pair, with the reference's two roundings.
template <bool kBf16, bool kHasOffset>
__device__ __forceinline__ uint32_t dequant_pair(uint32_t t, uint32_t scale2, uint32_t off2)
{
    using N = Num<kBf16>;
    using T2 = typename N::T2;
    T2 v = as_t2<T2>((t & 0x000F000Fu) ^ N::kMagic);
    v = __hsub2(v, as_t2<T2>(N::kBias));                       // exact: w in [-8, 7]
    if (kHasOffset) v = __hadd2(v, as_t2<T2>(off2));           // rounding #1
    v = __hmul2(v, as_t2<T2>(scale2));                         // rounding #2
    return as_u32(v);
}

template <bool kBf16, bool kHasOffset>
__global__ void __launch_bounds__(kThreads, 3) wqbmm_decode_kernel(const DecodeArgs a)
{
    using N = Num<kBf16>;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q = lane & 3;
    __shared__ int s_reduce;

    const int64_t P = gridDim.x, c = blockIdx.x;
    int64_t t0 = (c * a.total) / P;
    const int64_t t1 = ((c + 1) * a.total) / P;
    const uint16_t* x16 = reinterpret_cast<const uint16_t*>(a.x);

    while (t0 < t1) {
        const int64_t strip = t0 / a.ksteps;
        const int64_t sa = t0 % a.ksteps;
        const int64_t sb = min(a.ksteps, sa + (t1 - t0));
        t0 += sb - sa;

        const int64_t col0 = strip * kStripCols + warp * 128 + 16 * g;  // first of this lane's 16 columns
        const bool col_ok = col0 < a.n;
        const uint2* wp = reinterpret_cast<const uint2*>(a.w + (col_ok ? col0 / 8 : 0));

        float acc[kTiles][4];
#pragma unroll
        for (int t = 0; t < kTiles; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;

        uint32_t sc[16], of[16];
        int64_t cur_group = -1;

        uint2 wbuf[kPrefetch][4];
        auto fetch = [&](uint2(&dst)[4], int64_t step) {
            const bool ok = col_ok && step < sb;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int64_t row = step * 16 + 2 * q + (r & 1) + (r >> 1) * 8;
                dst[r] = ok ? ldg_stream(wp + row * (a.w_ld32 / 2)) : make_uint2(0u, 0u);
            }
        };
#pragma unroll
        for (int i = 0; i < kPrefetch; ++i) fetch(wbuf[i], sa + i);

        for (int64_t base = sa; base < sb; base += kPrefetch) {
#pragma unroll
            for (int i = 0; i < kPrefetch; ++i) {
                const int64_t step = base + i;
                uint2 cur[4] = {wbuf[i][0], wbuf[i][1], wbuf[i][2], wbuf[i][3]};
                fetch(wbuf[i], step + kPrefetch);
                if (step >= sb) continue;

                const int64_t group = step / a.steps_per_group;
                if (group != cur_group) {
                    cur_group = group;
                    // 16 consecutive columns of scale (and offset) -> one duplicated 16-bit pair per column
                    uint32_t raw_s[8], raw_o[8];
                    if (a.scale_sn != 0) {
                        const int64_t sidx = group * a.scale_sg + (col_ok ? col0 : 0);
                        const uint4* ps = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.scale) + sidx);
                        uint4 s0 = __ldg(ps), s1 = __ldg(ps + 1);
                        raw_s[0] = s0.x; raw_s[1] = s0.y; raw_s[2] = s0.z; raw_s[3] = s0.w;
                        raw_s[4] = s1.x; raw_s[5] = s1.y; raw_s[6] = s1.z; raw_s[7] = s1.w;
                        if (kHasOffset) {
                            const uint4* po = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.offset) + sidx);
                            uint4 o0 = __ldg(po), o1 = __ldg(po + 1);
                            raw_o[0] = o0.x; raw_o[1] = o0.y; raw_o[2] = o0.z; raw_o[3] = o0.w;
                            raw_o[4] = o1.x; raw_o[5] = o1.y; raw_o[6] = o1.z; raw_o[7] = o1.w;
                        }
                    } else {
                        const uint32_t s = reinterpret_cast<const uint16_t*>(a.scale)[group * a.scale_sg];
                        const uint32_t o = kHasOffset ? reinterpret_cast<const uint16_t*>(a.offset)[group * a.scale_sg] : 0u;
#pragma unroll
                        for (int i2 = 0; i2 < 8; ++i2) {
                            raw_s[i2] = s | (s << 16);
                            raw_o[i2] = o | (o << 16);
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const uint32_t sel = (e & 1) ? 0x3232u : 0x1010u;
                        sc[e] = prmt(raw_s[e >> 1], raw_s[e >> 1], sel);
                        if (kHasOffset) of[e] = prmt(raw_o[e >> 1], raw_o[e >> 1], sel);
                    }
                }

                // A fragment: x[rows g, g+8][k0 + 2q .. +1, +8 .. +9]
                uint32_t af[4];
                {
                    const int64_t k0 = step * 16 + 2 * q;
                    const uint32_t* r0 = reinterpret_cast<const uint32_t*>(x16 + (int64_t)g * a.x_ld + k0);
                    const uint32_t* r1 = reinterpret_cast<const uint32_t*>(x16 + (int64_t)(g + 8) * a.x_ld + k0);
                    af[0] = g < a.m ? __ldg(r0) : 0u;
                    af[1] = g + 8 < a.m ? __ldg(r1) : 0u;
                    af[2] = g < a.m ? __ldg(r0 + 4) : 0u;
                    af[3] = g + 8 < a.m ? __ldg(r1 + 4) : 0u;
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t wa = h ? cur[0].y : cur[0].x, wb = h ? cur[1].y : cur[1].x;
                    const uint32_t wc = h ? cur[2].y : cur[2].x, wd = h ? cur[3].y : cur[3].x;
                    // low half: nibbles 0..3 of row a | nibbles 0..3 of row b; high half: nibbles 4..7
                    const uint32_t lo01 = prmt(wa, wb, 0x5410u), hi01 = prmt(wa, wb, 0x7632u);
                    const uint32_t lo23 = prmt(wc, wd, 0x5410u), hi23 = prmt(wc, wd, 0x7632u);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        {
                            const int t = h * 8 + j;
                            const uint32_t b0 = dequant_pair<kBf16, kHasOffset>(lo01 >> (4 * j), sc[t], of[t]);
                            const uint32_t b1 = dequant_pair<kBf16, kHasOffset>(lo23 >> (4 * j), sc[t], of[t]);
                            N::mma(acc[t], af, b0, b1);
                        }
                        {
                            const int t = h * 8 + 4 + j;
                            const uint32_t b0 = dequant_pair<kBf16, kHasOffset>(hi01 >> (4 * j), sc[t], of[t]);
                            const uint32_t b1 = dequant_pair<kBf16, kHasOffset>(hi23 >> (4 * j), sc[t], of[t]);
                            N::mma(acc[t], af, b0, b1);
                        }
                    }
                }
            }
        }

        // ---- this CTA's share of the strip is in acc; combine with the other contributors if there are any ----
        const bool whole = (sa == 0 && sb == a.ksteps);
        bool do_write = whole;
        int64_t c_lo = c, c_hi = c;
        if (!whole) {
            float4* mine = a.partials + (((c + strip) * kWarps + warp) * kTiles) * 32 + lane;
#pragma unroll
            for (int t = 0; t < kTiles; ++t) mine[t * 32] = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
            asm volatile("fence.sc.gpu;" ::: "memory");
            __syncthreads();
            if (tid == 0) {
                // contributors: CTAs whose run intersects [strip*ksteps, (strip+1)*ksteps)
                const int64_t first = strip * a.ksteps, last = first + a.ksteps - 1;
                c_lo = (first * P) / a.total;
                while (c_lo > 0 && (c_lo * a.total) / P > first) --c_lo;
                while (((c_lo + 1) * a.total) / P <= first) ++c_lo;
                c_hi = (last * P) / a.total;
                while (c_hi > 0 && (c_hi * a.total) / P > last) --c_hi;
                while (((c_hi + 1) * a.total) / P <= last) ++c_hi;
                asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(a.tags + c + strip), "l"(a.nonce) : "memory");
                asm volatile("fence.sc.gpu;" ::: "memory");
                int all = 1;
                for (int64_t cc = c_lo; cc <= c_hi; ++cc) {
                    unsigned long long seen;
                    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(seen) : "l"(a.tags + cc + strip) : "memory");
                    all &= (seen == a.nonce);
                }
                asm volatile("fence.sc.gpu;" ::: "memory");
                s_reduce = all;
            }
            __syncthreads();
            do_write = s_reduce != 0;
            if (do_write) {
                // every thread recomputes the contributor range (cheap) and sums in CTA order
                const int64_t first = strip * a.ksteps, last = first + a.ksteps - 1;
                c_lo = (first * P) / a.total;
                while (c_lo > 0 && (c_lo * a.total) / P > first) --c_lo;
                while (((c_lo + 1) * a.total) / P <= first) ++c_lo;
                c_hi = (last * P) / a.total;
                while (c_hi > 0 && (c_hi * a.total) / P > last) --c_hi;
                while (((c_hi + 1) * a.total) / P <= last) ++c_hi;
#pragma unroll
                for (int t = 0; t < kTiles; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
                for (int64_t cc = c_lo; cc <= c_hi; ++cc) {
                    const float4* theirs = a.partials + (((cc + strip) * kWarps + warp) * kTiles) * 32 + lane;
#pragma unroll
                    for (int t = 0; t < kTiles; ++t) {
                        const float4 v = __ldcg(theirs + t * 32);
                        acc[t][0] += v.x; acc[t][1] += v.y; acc[t][2] += v.z; acc[t][3] += v.w;
                    }
                }
            }
            __syncthreads();  // s_reduce is reused by the next strip of this CTA
            if (do_write && tid == 0) {
                // every contributor's fragment has been consumed: retire the strip's tags, so that a replay of this very
                // launch (same nonce, e.g. from a captured CUDA graph) starts from a clean slate
                for (int64_t cc = c_lo; cc <= c_hi; ++cc)
                    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(a.tags + cc + strip), "l"(0ull) : "memory");
            }
        }
        if (do_write) {
            // D fragment: rows g, g+8; tile-local columns 2q, 2q+1 = lane groups 2q, 2q+1 of the loader
            const int64_t colw = strip * kStripCols + warp * 128;
#pragma unroll
            for (int t = 0; t < kTiles; ++t) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int row = g + (e >> 1) * 8;
                    const int64_t col = colw + 16 * (2 * q + (e & 1)) + t;
                    if (row < a.m && col < a.n) {
                        float f = acc[t][e];
                        if (a.bias != nullptr) f = __fadd_rn(f, load_as_float(a.bias, col, a.bias_dtype));
                        store_out(a.y, (int64_t)row * a.y_ld + col, f, kBf16 ? ACL_BF16 : ACL_FLOAT16);
                    }
                }
            }
        }
    }
}

int g_decode_ctas_per_sm[4] = {0, 0, 0, 0};
int g_sm_count = 0;

template <bool kBf16, bool kHasOffset>
int decode_grid(int variant)
{
    if (g_sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
    }
    if (g_decode_ctas_per_sm[variant] == 0) {
        int nb = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, wqbmm_decode_kernel<kBf16, kHasOffset>, kThreads, 0);
        g_decode_ctas_per_sm[variant] = nb > 0 ? nb : 1;
    }
    return g_sm_count * g_decode_ctas_per_sm[variant];
}

unsigned long long next_nonce()
{
    static std::atomic<unsigned long long> ctr{
        (unsigned long long)std::chrono::steady_clock::now().time_since_epoch().count() * 0x9E3779B97F4A7C15ull + 1};
    unsigned long long z = ctr.fetch_add(0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z ? z : 1;
}

constexpr int kMaxGrid = 148 * 4 * 2;  // workspace is sized for at most this many CTAs

}  // namespace

// Upper bound used by phase 1, which runs without a device: tags + fragments for (max grid + strips) slots.
uint64_t wqbmm_decode_workspace_size(const OpsnnWqbmmParams* p)
{
    const int64_t strips = (p->n + kStripCols - 1) / kStripCols;
    const uint64_t slots = (uint64_t)kMaxGrid + (uint64_t)strips;
    const uint64_t tags = ((slots * 8 + 255) / 256) * 256;
    return tags + slots * kWarps * kTiles * 32 * sizeof(float4);
}

bool wqbmm_decode_eligible(const OpsnnWqbmmParams* p)
{
    if (p->w_dtype != ACL_INT4 || p->trans_w != 0) return false;
    if (p->m < 1 || p->m > 16) return false;
    if (p->k % 16 != 0 || p->n % 16 != 0 || p->w_ld % 16 != 0 || p->x_ld % 2 != 0) return false;
    if (p->group_size != 0 && p->group_size % 16 != 0) return false;
    if (p->scale_sn != 0 && p->scale_sn != 1) return false;
    if (p->scale_sn == 1 && (p->scale_sg % 8 != 0)) return false;
    auto aligned = [](const void* q, uintptr_t a) { return (reinterpret_cast<uintptr_t>(q) % a) == 0; };
    if (!aligned(p->w, 8) || !aligned(p->x, 4)) return false;
    if (p->scale_sn == 1 && (!aligned(p->scale, 16) || (p->offset && !aligned(p->offset, 16)))) return false;
    return true;
}

int32_t wqbmm_decode_launch(const OpsnnWqbmmParams* p, cudaStream_t stream)
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
    a.total = a.strips * a.ksteps;
    a.steps_per_group = p->group_size > 0 ? p->group_size / 16 : a.ksteps;
    const bool bf16 = p->x_dtype == ACL_BF16, has_off = p->offset != nullptr;
    const int variant = (bf16 ? 2 : 0) + (has_off ? 1 : 0);
    int grid = 0;
    switch (variant) {
        case 0: grid = decode_grid<false, false>(0); break;
        case 1: grid = decode_grid<false, true>(1); break;
        case 2: grid = decode_grid<true, false>(2); break;
        default: grid = decode_grid<true, true>(3); break;
    }
    if (grid > kMaxGrid) grid = kMaxGrid;
    if ((int64_t)grid > a.total) grid = (int)a.total;
    if (const char* e = getenv("OPSNN_WQ_DECODE_GRID")) {
        int v = atoi(e);
        if (v > 0 && v <= kMaxGrid && v <= a.total) grid = v;
    }
    const uint64_t slots = (uint64_t)kMaxGrid + (uint64_t)a.strips;
    const uint64_t tag_bytes = ((slots * 8 + 255) / 256) * 256;
    if (p->workspace == nullptr || p->workspace_size < wqbmm_decode_workspace_size(p)) return (int32_t)cudaErrorInvalidValue;
    a.tags = reinterpret_cast<unsigned long long*>(p->workspace);
    a.partials = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(p->workspace) + tag_bytes);
    a.nonce = next_nonce();
    switch (variant) {
        case 0: wqbmm_decode_kernel<false, false><<<grid, kThreads, 0, stream>>>(a); break;
        case 1: wqbmm_decode_kernel<false, true><<<grid, kThreads, 0, stream>>>(a); break;
        case 2: wqbmm_decode_kernel<true, false><<<grid, kThreads, 0, stream>>>(a); break;
        default: wqbmm_decode_kernel<true, true><<<grid, kThreads, 0, stream>>>(a); break;
    }
    note_launch("wqbmm_decode");
    return (int32_t)cudaGetLastError();
}

}  // namespace opsnn
