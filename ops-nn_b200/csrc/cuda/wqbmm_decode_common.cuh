// Pieces shared by the W4A16 decode kernels (the one that reproduces the reference's two roundings per weight, and the
// group-wise scaling one): launch arguments, 16-bit pair arithmetic, and the cross-CTA combination of k-split partial sums.
#pragma once
#include <atomic>
#include <chrono>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace opsnn {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kWarpCols = 64;               // one packed word (8 columns) per lane-group g
constexpr int kStripCols = kWarps * kWarpCols;  // 512
#ifndef OPSNN_DECODE_PF
#define OPSNN_DECODE_PF 8
#endif
#ifndef OPSNN_DECODE_MINB
#define OPSNN_DECODE_MINB 2
#endif
constexpr int kPrefetch = OPSNN_DECODE_PF;  // k-steps of weight words held in registers ahead of use
constexpr int kTiles = 8;                 // m16n8 tiles per warp: nibble j of the lane's word is tile j
constexpr int kChunk = 32;                // k-steps of x staged in shared memory at a time (double buffered)
constexpr int kXPitch = kChunk * 16 + 8;  // elements; the +8 skews rows over the banks so fragment reads do not conflict

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
    int64_t strips, ksteps, splits, steps_per_group;
    int32_t cluster;       // != 0: the k-splits of a strip form a thread-block cluster (CTA index = strip * splits + split)
    int64_t k_align;       // group-wise kernel only: k ranges start and end on multiples of this many k-steps (even)
    unsigned long long* tags;  // [gridDim]
    float4* partials;          // [gridDim][kWarps][kTiles][32]
    unsigned long long nonce;
    uint32_t c_mask, c_magic, c_bias;  // 0x000F000F, Num::kMagic, Num::kBias
    PeerBinding peers;         // bulk-copy kernels: count > 0 stores every element into each rank's full output as well
};

__device__ __forceinline__ uint32_t ldg_stream(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// 16-bit pair arithmetic on raw 32-bit registers (no type punning through memory): each op rounds once, to nearest even.
template <bool kBf16>
struct Num;
template <>
struct Num<true> {
    static constexpr uint32_t kMagic = 0x43084308u;  // (nibble ^ 8) | 0x4300  ->  bf16 128 + 8 + w
    static constexpr uint32_t kBias = 0x43084308u;   // bf16x2 {136, 136}
    __device__ __forceinline__ static uint32_t sub(uint32_t a, uint32_t b)
    {
        uint32_t d;
        asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
        return d;
    }
    __device__ __forceinline__ static uint32_t add(uint32_t a, uint32_t b)
    {
        uint32_t d;
        asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
        return d;
    }
    __device__ __forceinline__ static uint32_t mul(uint32_t a, uint32_t b)
    {
        uint32_t d;
        asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
        return d;
    }
    // same instruction, not volatile: the compiler may interleave it with the logic ops of the next k-step
    __device__ __forceinline__ static void mma_free(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
    {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ __forceinline__ static void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
    {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
template <>
struct Num<false> {
    static constexpr uint32_t kMagic = 0x64086408u;  // (nibble ^ 8) | 0x6400  ->  fp16 1024 + 8 + w
    static constexpr uint32_t kBias = 0x64086408u;   // half2 {1032, 1032}
    __device__ __forceinline__ static uint32_t sub(uint32_t a, uint32_t b)
    {
        uint32_t d;
        asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
        return d;
    }
    __device__ __forceinline__ static uint32_t add(uint32_t a, uint32_t b)
    {
        uint32_t d;
        asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
        return d;
    }
    __device__ __forceinline__ static uint32_t mul(uint32_t a, uint32_t b)
    {
        uint32_t d;
        asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
        return d;
    }
    __device__ __forceinline__ static void mma_free(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
    {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ __forceinline__ static void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
    {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

// The element (row, col of the shard) into every bound rank's full output.
template <bool kBf16>
__device__ __forceinline__ void store_to_peers(const DecodeArgs& a, int row, int64_t col, float f)
{
    const int64_t idx = (int64_t)row * a.peers.ld + a.peers.col0 + col;
    for (int r = 0; r < a.peers.count; ++r) store_out(a.peers.full[r], idx, f, kBf16 ? ACL_BF16 : ACL_FLOAT16);
}

// Writes one warp's 16 x 64 block of y from its accumulator fragments (+ bias), undoing the column permutation of the MMA tiles.
template <bool kBf16, int kLayout>
__device__ __forceinline__ void store_tile_y(const DecodeArgs& a, float (&acc)[kTiles][4], int64_t strip, int warp, int lane)
{
    const int g = lane >> 2, q = lane & 3;

                // D fragment: rows g, g+8; tile-local columns 2q, 2q+1 = lane groups 2q, 2q+1 of the loader
                const int64_t colw = strip * kStripCols + warp * kWarpCols;
    #pragma unroll
                for (int t = 0; t < kTiles; ++t) {
    #pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int row = g + (e >> 1) * 8;
                        // kLayout 0: tile t is nibble t of the lane group's word; 1: the ldmatrix layout of the ring / TMA int4 kernels;
                        // 2: the 8-bit kernel, tile t = (16-column chunk t / 2, even / odd columns of it); 3: tile t = columns 8 t .. 8 t + 7
                const int64_t col = colw + (kLayout == 0   ? 8 * (2 * q + (e & 1)) + t
                                            : kLayout == 1 ? 32 * (t >> 2) + 4 * (2 * q + (e & 1)) + (t & 3)
                                            : kLayout == 2 ? 16 * (t >> 1) + 2 * (2 * q + (e & 1)) + (t & 1)
                                                           : 8 * t + 2 * q + (e & 1));
                        if (row < a.m && col < a.n) {
                            float f = acc[t][e];
                            if (a.bias != nullptr) f = __fadd_rn(f, load_as_float(a.bias, col, a.bias_dtype));
                            store_out(a.y, (int64_t)row * a.y_ld + col, f, kBf16 ? ACL_BF16 : ACL_FLOAT16);
                            if (a.peers.count > 0) store_to_peers<kBf16>(a, row, col, f);
                        }
                    }
                }
}

// Cross-CTA combination of a strip's k-split contributors, then the write of y. Every contributor stores its fp32
// fragments, then a launch nonce; whichever contributor observes all nonces present (at least one does: store, fence.sc,
// load) adds the fragments in CTA order - so the result does not depend on arrival order - writes y and zeroes the
// strip's nonces. No atomics, no spinning, no zero-initialised workspace.
template <bool kBf16, int kLayout = 0>
__device__ __forceinline__ void combine_and_store(const DecodeArgs& a, float (&acc)[kTiles][4], int64_t c, int64_t strip, int warp,
                                                  int lane, int tid, int* s_reduce_ptr)
{
    const int g = lane >> 2, q = lane & 3;
    int& s_reduce = *s_reduce_ptr;
            // ---- this CTA's share of the strip is in acc; combine with the other contributors if there are any ----
            const bool whole = a.splits == 1;
            bool do_write = whole;
            if (!whole) {
                float4* mine = a.partials + ((c * kWarps + warp) * kTiles) * 32 + lane;
    #pragma unroll
                for (int t = 0; t < kTiles; ++t) mine[t * 32] = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
                __syncthreads();  // every thread's fragment stores are ordered before warp 0's release below
                if (warp == 0) {
                    if (lane == 0) asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(a.tags + c), "l"(a.nonce) : "memory");
                    __syncwarp();
                    // own tag, then a sequentially consistent fence, then the others' tags: of two contributors at least
                    // the later one sees the other's tag. The lanes look at 32 tags at a time.
                    asm volatile("fence.sc.gpu;" ::: "memory");
                    int all = 1;
                    for (int64_t j0 = 0; j0 < a.splits; j0 += 32) {
                        unsigned long long seen = a.nonce;
                        if (j0 + lane < a.splits)
                            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(seen) : "l"(a.tags + strip + (j0 + lane) * a.strips) : "memory");
                        all &= (seen == a.nonce);
                    }
                    all = __all_sync(0xffffffffu, all);
                    if (lane == 0) s_reduce = all;
                }
                __syncthreads();
                do_write = s_reduce != 0;
                if (do_write) {
    #pragma unroll
                    for (int t = 0; t < kTiles; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
                    // two contributors' fragments are fetched per round trip; the sums stay in contributor order
                    for (int64_t j = 0; j < a.splits; j += 2) {
                        const bool two = j + 1 < a.splits;
                        const float4* pa = a.partials + (((strip + j * a.strips) * kWarps + warp) * kTiles) * 32 + lane;
                        const float4* pb = a.partials + (((strip + (two ? j + 1 : j) * a.strips) * kWarps + warp) * kTiles) * 32 + lane;
                        float4 va[kTiles], vb[kTiles];
    #pragma unroll
                        for (int t = 0; t < kTiles; ++t) va[t] = __ldcg(pa + t * 32);
    #pragma unroll
                        for (int t = 0; t < kTiles; ++t) vb[t] = __ldcg(pb + t * 32);
    #pragma unroll
                        for (int t = 0; t < kTiles; ++t) {
                            acc[t][0] += va[t].x; acc[t][1] += va[t].y; acc[t][2] += va[t].z; acc[t][3] += va[t].w;
                            if (two) {
                                acc[t][0] += vb[t].x; acc[t][1] += vb[t].y; acc[t][2] += vb[t].z; acc[t][3] += vb[t].w;
                            }
                        }
                    }
                }
                __syncthreads();
                if (do_write && warp == 0) {
                    // every contributor's fragment has been consumed: retire the strip's tags, so that a replay of this very
                    // launch (same nonce, e.g. from a captured CUDA graph) starts from a clean slate
                    for (int64_t j = lane; j < a.splits; j += 32)
                        asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(a.tags + strip + j * a.strips), "l"(0ull) : "memory");
                }
            }
            if (do_write) store_tile_y<kBf16, kLayout>(a, acc, strip, warp, lane);
}

// The same combination for k-splits launched as one thread-block cluster (CTA index = strip * splits + split): every CTA leaves
// its fp32 fragments in its own shared memory at `frag` ([warp][tile][lane] float4, 32 KB, + one word "fragments valid"), and
// after a cluster barrier CTA r sums the r-th slice of the strip's 2048 float4 over all CTAs, in CTA order (the same order,
// hence the same bits, as combine_and_store), and writes those elements of y. No global scratch, no tags, and the summing is
// spread over the cluster instead of falling on one CTA. `valid` is false for a CTA whose main loop gave up a wait: it still
// joins both barriers (nobody waits for a CTA that left), and nobody writes that strip.
template <bool kBf16, int kLayout>
__device__ __forceinline__ void cluster_combine_and_store(const DecodeArgs& a, float (&acc)[kTiles][4], int64_t strip, int warp, int lane,
                                                          int tid, uint32_t frag, bool valid)
{
    constexpr uint32_t kFragVec = (uint32_t)kWarps * kTiles * 32;  // float4 per CTA
    const uint32_t mine = frag + (uint32_t)((warp * kTiles) * 32 + lane) * 16u;
#pragma unroll
    for (int t = 0; t < kTiles; ++t)
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(mine + t * 512), "f"(acc[t][0]), "f"(acc[t][1]), "f"(acc[t][2]),
                     "f"(acc[t][3])
                     : "memory");
    if (tid == 0) asm volatile("st.shared.u32 [%0], %1;" ::"r"(frag + kFragVec * 16u), "r"(valid ? 1u : 0u) : "memory");
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const uint32_t S = (uint32_t)a.splits;
    // thread j looks at CTA j's "valid" word: one round trip for all of them
    uint32_t flag = 1u;
    if ((uint32_t)tid < S) {
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(frag + kFragVec * 16u), "r"((uint32_t)tid));
        asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(flag) : "r"(remote) : "memory");
    }
    const uint32_t all_valid = __syncthreads_and(flag != 0u) ? 1u : 0u;
    // the slice of this CTA: at most two float4 per thread (2048 / S <= 1024 only for S = 2, 3: the loop covers that)
    const uint32_t per = (kFragVec + S - 1) / S;
    const uint32_t lo = rank * per, hi = min(kFragVec, lo + per);
    constexpr int kMaxSplits = 16;
    bool arrived = false;
    for (uint32_t i0 = lo; i0 < hi && all_valid != 0u; i0 += (uint32_t)kThreads) {
        const uint32_t i = i0 + (uint32_t)tid;
        const bool active = i < hi;
        float4 v[kMaxSplits];
        // all loads first (they do not depend on one another), then the sum in CTA order
#pragma unroll
        for (uint32_t j = 0; j < (uint32_t)kMaxSplits; ++j) {
            if (active && j < S) {
                uint32_t remote;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(frag + i * 16u), "r"(j));
                asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                             : "=f"(v[j].x), "=f"(v[j].y), "=f"(v[j].z), "=f"(v[j].w)
                             : "r"(remote)
                             : "memory");
            } else {
                v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (uint32_t j = 0; j < (uint32_t)kMaxSplits; ++j) {
            if (j < S) { s.x += v[j].x; s.y += v[j].y; s.z += v[j].z; s.w += v[j].w; }
        }
        if (i0 + (uint32_t)kThreads >= hi) {
            // the last of this CTA's reads of the other CTAs' shared memory are in registers: tell the cluster before writing y
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            arrived = true;
        }
        if (active) {
            // float4 i is tile t of lane l of warp w: rows g, g + 8, columns as in store_tile_y
            const int w = (int)(i >> 8), t = (int)((i >> 5) & 7u), l = (int)(i & 31u);
            const int g = l >> 2, q = l & 3;
            const int64_t colw = strip * kStripCols + w * kWarpCols;
            const float f4[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = g + (e >> 1) * 8;
                const int64_t col = colw + (kLayout == 0   ? 8 * (2 * q + (e & 1)) + t
                                            : kLayout == 1 ? 32 * (t >> 2) + 4 * (2 * q + (e & 1)) + (t & 3)
                                            : kLayout == 2 ? 16 * (t >> 1) + 2 * (2 * q + (e & 1)) + (t & 1)
                                                           : 8 * t + 2 * q + (e & 1));
                if (row < a.m && col < a.n) {
                    float f = f4[e];
                    if (a.bias != nullptr) f = __fadd_rn(f, load_as_float(a.bias, col, a.bias_dtype));
                    store_out(a.y, (int64_t)row * a.y_ld + col, f, kBf16 ? ACL_BF16 : ACL_FLOAT16);
                    if (a.peers.count > 0) store_to_peers<kBf16>(a, row, col, f);
                }
            }
        }
    }
    // nobody leaves (and frees its shared memory) before every CTA has read what it needs
    if (!arrived) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

}  // namespace

// How many clusters of s CTAs of `kernel` the current device keeps resident at once under a cluster scheduling policy
// (cudaClusterSchedulingPolicy*: 0 default / 1 spread / 2 load balancing). Answers are cached per (kernel, device, s, policy).
inline int max_active_clusters(const void* kernel, int threads, int smem_bytes, int s, int policy)
{
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, int, int>, int> cache;
    int dev = 0;
    cudaGetDevice(&dev);
    const auto key = std::make_tuple(kernel, dev, s, policy);
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) return it->second;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(s * 64), 1, 1);
    cfg.blockDim = dim3((unsigned)threads, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cudaLaunchAttribute attr[2]{};
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)s;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeClusterSchedulingPolicyPreference;
    attr[1].val.clusterSchedulingPolicyPreference = static_cast<cudaClusterSchedulingPolicy>(policy);
    cfg.attrs = attr;
    cfg.numAttrs = policy != 0 ? 2 : 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    std::lock_guard<std::mutex> lock(mu);
    cache[key] = n;
    return n;
}

// Largest cluster size S in [2, max_s] for which `clusters` clusters of S CTAs of `kernel` are all resident at once on the
// current device (default scheduling policy), 0 when there is none.
inline int pick_cluster_size(const void* kernel, int threads, int smem_bytes, int64_t clusters, int max_s)
{
    for (int s = max_s; s >= 2; --s)
        if ((int64_t)max_active_clusters(kernel, threads, smem_bytes, s, 0) >= clusters) return s;
    return 0;
}

// One sequence for the whole library (inline with external linkage: a single counter across translation units).
inline unsigned long long next_nonce()
{
    static std::atomic<unsigned long long> ctr{
        (unsigned long long)std::chrono::steady_clock::now().time_since_epoch().count() * 0x9E3779B97F4A7C15ull + 1};
    unsigned long long z = ctr.fetch_add(0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z ? z : 1;
}

}  // namespace opsnn
