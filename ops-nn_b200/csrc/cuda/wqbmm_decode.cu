// Weight-only quant matmul, decode kernel: y[m<=16, n] = x[m,k] @ dequant(w_int4[k,n]) for the HBM-bound small-m regime.
//
// Replaces, for this regime, the reference's per-group "reg-base" kernel
// (weight_quant_batch_matmul_v2/op_kernel/arch35/weight_quant_batch_matmul_v2_reg_base_common.h:164-286 and
//  weight_quant_batch_matmul_v2_vf.h:345-442: vector cores dequantise int4 -> bf16 into L1, cube core multiplies) and
// its host tiling (op_host/op_tiling/arch35/weight_quant_batch_matmul_v2_reg_base_tiling.cpp:89-337).
//
// Data layout. w is int4 packed 8 per 32-bit word along n, element j of a word at bits [4j,4j+4), word (k,c) holds
// columns 8c..8c+7 (reference: aclnn_weight_quant_batch_matmul_v2.cpp:1482-1524). scale/offset are (groups, n) in x's
// dtype. The weight (k*n/2 bytes) is read exactly once from HBM; x (m*k*2 bytes) is staged through shared memory with
// cp.async (double buffered, 512 k at a time); the scales stay in L2/L1.
//
// Mapping. One warp owns 64 columns, one CTA (8 warps) a strip of 512. Lane (g = lane/4, q = lane%4) loads word g of
// the warp (8 columns) of the four rows {2q, 2q+1, 2q+8, 2q+9} of every 16-row k-step: exactly the rows an m16n8k16 B
// fragment wants from this lane. Eight k-steps of words are kept in flight in registers. A byte permute pairs the two
// rows' words so that one three-input logic op turns nibble j of both rows into a bf16x2 {136+w_k, 136+w_k+1}
// (0x4300 | (nibble ^ 8) == 128 + 8 + w, exact); then, per the reference's rounding points,
//     w' = mul.rn( add.rn( sub.rn(v, 136), offset ), scale )       // each a single bf16 (fp16) rounding, no FMA
// feeds mma.sync.m16n8k16 (fp32 accumulate). Nibble j of the word is MMA tile j, so no data is shuffled between
// lanes; the column permutation this implies is undone when y is written.
//
// Work split. gridDim = strips x Q: CTA c owns column strip (c % strips) of 512 columns and the q-th of Q equal k ranges,
// q = c / strips, with Q = resident CTAs / strips. CTAs that run side by side therefore read side-by-side 256-byte pieces
// of the same weight rows, so DRAM sees whole rows being streamed instead of hundreds of narrow strided streams.
// A strip's Q contributors are summed through workspace: every contributor stores its fp32 fragment, then a launch
// nonce; whichever contributor observes all nonces present (at least one does: store, fence.sc, load) adds the
// fragments in CTA order - so the result does not depend on arrival order - and writes y, then zeroes the strip's
// nonces. No atomics, no spinning, no zero-initialised workspace (stale bytes never equal a fresh 64-bit nonce), and a
// replayed launch with an unchanged nonce still works because the previous run retired its tags. Two launches must
// not share one workspace concurrently.
#include <atomic>
#include <chrono>

#include "common.cuh"
#include "wqbmm_decode_common.cuh"

namespace opsnn {

namespace {

// Two nibbles (bits [3:0] and [19:16] of t) -> dequantised 16-bit pair, with the reference's two roundings.
// mask / magic / bias come from kernel parameters, i.e. the constant bank, so that they cost neither a register nor a
// re-materialising move in front of every use; (t & mask) ^ magic is a single three-input logic op.
template <bool kBf16, bool kHasOffset>
__device__ __forceinline__ uint32_t dequant_pair(uint32_t t, uint32_t scale2, uint32_t off2, uint32_t mask, uint32_t magic,
                                                 uint32_t bias)
{
    using N = Num<kBf16>;
    uint32_t v;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(v) : "r"(t), "r"(mask), "r"(magic));
    v = N::sub(v, bias);                      // exact: w in [-8, 7]
    if (kHasOffset) v = N::add(v, off2);      // rounding #1
    return N::mul(v, scale2);                 // rounding #2
}

template <bool kBf16, bool kHasOffset>
__global__ void __launch_bounds__(kThreads, OPSNN_DECODE_MINB) wqbmm_decode_kernel(const DecodeArgs a)
{
    using N = Num<kBf16>;
    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, q = lane & 3;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // tells the compiler the warp index is warp-uniform
    __shared__ int s_reduce;
    __shared__ __align__(16) uint16_t xs[2][16][kXPitch];

    const int64_t c = blockIdx.x;
    const int64_t strip = c % a.strips;
    const int64_t chunk = c / a.strips;
    const uint16_t* x16 = reinterpret_cast<const uint16_t*>(a.x);
    {
        const int64_t sa = (chunk * a.ksteps) / a.splits;
        const int64_t sb = ((chunk + 1) * a.ksteps) / a.splits;

        const int64_t col0 = strip * kStripCols + warp * kWarpCols + 8 * g;  // first of this lane's 8 columns
        const bool col_ok = col0 < a.n;

        float acc[kTiles][4];
#pragma unroll
        for (int t = 0; t < kTiles; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;

        uint32_t sc[kTiles], of[kTiles];

        // Next step to fetch = warp-uniform 64-bit base (advances 16 rows per fetch, clamped to the last k-step of this
        // CTA's range, which the prefetch running ahead of the compute then merely re-reads from L1/L2) + per-lane 32-bit
        // offsets of the lane's four rows and its 4-byte column slot (lanes past n re-read column 0 and are discarded).
        const int64_t pitch_b = a.w_ld32 * 4;  // row pitch in bytes
        const int64_t warp_col = strip * kStripCols + warp * kWarpCols;
        const char* wbase = reinterpret_cast<const char*>(a.w) + (warp_col < a.n ? warp_col : 0) / 2;
        const char* ubase = wbase + sa * 16 * pitch_b;
        const char* ulast = wbase + (sb - 1) * 16 * pitch_b;
        uint32_t loff[4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
            loff[r] = (uint32_t)((2 * q + (r & 1) + (r >> 1) * 8) * pitch_b) + (col_ok ? 4 * g : 0);
        const int nsteps = (int)(sb - sa);
        uint32_t wbuf[kPrefetch][4];
        auto fetch = [&](uint32_t(&dst)[4]) {
#pragma unroll
            for (int r = 0; r < 4; ++r) dst[r] = ldg_stream(reinterpret_cast<const uint32_t*>(ubase + loff[r]));
            ubase = (ubase + 16 * pitch_b <= ulast) ? ubase + 16 * pitch_b : ulast;
        };
#pragma unroll
        for (int i = 0; i < kPrefetch; ++i) fetch(wbuf[i]);

        // x[:, this run's k range] goes through shared memory in chunks of kChunk steps, double buffered with cp.async:
        // a fragment read is then a 30-cycle shared load instead of an L2 round trip in front of every MMA group.
        auto stage_x = [&](int chunk_idx) {
            const int64_t k_first = (sa + (int64_t)chunk_idx * kChunk) * 16;
            const int64_t k_end = sb * 16;
            uint16_t(*dst)[kXPitch] = xs[chunk_idx & 1];
            for (int e = tid; e < 16 * (kChunk * 2); e += kThreads) {  // 16-byte pieces: 16 rows x (kChunk*16/8)
                const int row = e / (kChunk * 2), piece = e % (kChunk * 2);
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
        const int nchunks = (nsteps + kChunk - 1) / kChunk;
        stage_x(0);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();

        // k-group bookkeeping without a per-step division: `group_left` steps remain in the current group
        int64_t group = sa / a.steps_per_group - 1;
        int first_skip = (int)(sa % a.steps_per_group);  // steps of the first group that precede this run
        int group_left = 0;                              // 0 forces the scale load on the first step
        const int spg = (int)min(a.steps_per_group, (int64_t)0x7FFFFFFF);
        for (int chunk_idx = 0; chunk_idx < nchunks; ++chunk_idx) {
          if (chunk_idx + 1 < nchunks) stage_x(chunk_idx + 1);
          const uint16_t* xrow0 = &xs[chunk_idx & 1][g][2 * q];
          const uint16_t* xrow1 = &xs[chunk_idx & 1][g + 8][2 * q];
          const int chunk_end = min(nsteps, (chunk_idx + 1) * kChunk);
          for (int base = chunk_idx * kChunk; base < chunk_end; base += kPrefetch) {
#pragma unroll
            for (int i = 0; i < kPrefetch; ++i) {
                const int step_rel = base + i;
                const uint32_t wa = wbuf[i][0], wb = wbuf[i][1], wc = wbuf[i][2], wd = wbuf[i][3];
                fetch(wbuf[i]);
                if (step_rel >= nsteps) continue;

                if (group_left == 0) {
                    ++group;
                    group_left = spg - first_skip;
                    first_skip = 0;
                    // 8 consecutive columns of scale (and offset) -> one duplicated 16-bit pair per column
                    uint32_t raw_s[4], raw_o[4];
                    if (a.scale_sn != 0) {
                        const int64_t sidx = group * a.scale_sg + (col_ok ? col0 : 0);
                        const uint4 s0 = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.scale) + sidx));
                        raw_s[0] = s0.x; raw_s[1] = s0.y; raw_s[2] = s0.z; raw_s[3] = s0.w;
                        if (kHasOffset) {
                            const uint4 o0 = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.offset) + sidx));
                            raw_o[0] = o0.x; raw_o[1] = o0.y; raw_o[2] = o0.z; raw_o[3] = o0.w;
                        }
                    } else {
                        const uint32_t sv = reinterpret_cast<const uint16_t*>(a.scale)[group * a.scale_sg];
                        const uint32_t ov = kHasOffset ? reinterpret_cast<const uint16_t*>(a.offset)[group * a.scale_sg] : 0u;
#pragma unroll
                        for (int i2 = 0; i2 < 4; ++i2) {
                            raw_s[i2] = sv | (sv << 16);
                            raw_o[i2] = ov | (ov << 16);
                        }
                    }
#pragma unroll
                    for (int e = 0; e < kTiles; ++e) {
                        const uint32_t sel = (e & 1) ? 0x3232u : 0x1010u;
                        sc[e] = prmt(raw_s[e >> 1], raw_s[e >> 1], sel);
                        if (kHasOffset) of[e] = prmt(raw_o[e >> 1], raw_o[e >> 1], sel);
                    }
                }
                --group_left;

                // A fragment: x[rows g, g+8][k0 + 2q .. +1, +8 .. +9] from the staged chunk
                uint32_t af[4];
                {
                    const int ls = (step_rel - chunk_idx * kChunk) * 16;
                    af[0] = *reinterpret_cast<const uint32_t*>(xrow0 + ls);
                    af[1] = *reinterpret_cast<const uint32_t*>(xrow1 + ls);
                    af[2] = *reinterpret_cast<const uint32_t*>(xrow0 + ls + 8);
                    af[3] = *reinterpret_cast<const uint32_t*>(xrow1 + ls + 8);
                }
                // low half: nibbles 0..3 of row a | nibbles 0..3 of row b; high half: nibbles 4..7
                const uint32_t lo01 = prmt(wa, wb, 0x5410u), hi01 = prmt(wa, wb, 0x7632u);
                const uint32_t lo23 = prmt(wc, wd, 0x5410u), hi23 = prmt(wc, wd, 0x7632u);
                // dequantise all 16 pairs first (independent chains the scheduler can interleave), then issue the 8 MMAs
                uint32_t b0[kTiles], b1[kTiles];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    b0[j] = dequant_pair<kBf16, kHasOffset>(lo01 >> (4 * j), sc[j], of[j], a.c_mask, a.c_magic, a.c_bias);
                    b1[j] = dequant_pair<kBf16, kHasOffset>(lo23 >> (4 * j), sc[j], of[j], a.c_mask, a.c_magic, a.c_bias);
                    b0[4 + j] = dequant_pair<kBf16, kHasOffset>(hi01 >> (4 * j), sc[4 + j], of[4 + j], a.c_mask, a.c_magic, a.c_bias);
                    b1[4 + j] = dequant_pair<kBf16, kHasOffset>(hi23 >> (4 * j), sc[4 + j], of[4 + j], a.c_mask, a.c_magic, a.c_bias);
                }
#pragma unroll
                for (int t = 0; t < kTiles; ++t) N::mma(acc[t], af, b0[t], b1[t]);
            }
          }
          asm volatile("cp.async.wait_group 0;" ::: "memory");
          __syncthreads();
        }

        combine_and_store<kBf16>(a, acc, c, strip, warp, lane, tid, &s_reduce);
    }
}

int g_decode_ctas_per_sm[4] = {0, 0, 0, 0};  // a property of the kernel image and the architecture: the same on every device of a box

template <bool kBf16, bool kHasOffset>
int decode_grid(int variant)
{
    if (g_decode_ctas_per_sm[variant] == 0) {
        int nb = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, wqbmm_decode_kernel<kBf16, kHasOffset>, kThreads, 0);
        g_decode_ctas_per_sm[variant] = nb > 0 ? nb : 1;
    }
    return current_sm_count() * g_decode_ctas_per_sm[variant];
}

constexpr int kMaxGrid = 148 * 4 * 2;  // workspace is sized for at most this many CTAs

}  // namespace

// Upper bound used by phase 1, which runs without a device: one tag + one fp32 fragment set per CTA of the largest grid
// that ever splits k (a grid with more strips than that runs one CTA per strip and needs no workspace).
uint64_t wqbmm_decode_workspace_size(const OpsnnWqbmmParams* p)
{
    (void)p;
    const uint64_t slots = (uint64_t)kMaxGrid;
    const uint64_t tags = ((slots * 8 + 255) / 256) * 256;
    return tags + slots * kWarps * kTiles * 32 * sizeof(float4);
}

bool wqbmm_decode_eligible(const OpsnnWqbmmParams* p)
{
    if (p->w_dtype != ACL_INT4 || p->trans_w != 0) return false;
    if (p->scale_dtype == ACL_FLOAT8_E8M0) return false;  // the decode kernels read scale as 16-bit elements of x's dtype
    if (p->m < 1 || p->m > 16) return false;
    if (p->k < 16) return false;                            // at least one k-step: the prefetch reads 16 weight rows unconditionally
    if (p->k % 16 != 0 || p->n % 8 != 0 || p->w_ld % 8 != 0 || p->x_ld % 8 != 0) return false;
    if (p->group_size != 0 && p->group_size % 16 != 0) return false;
    if (p->scale_sn != 0 && p->scale_sn != 1) return false;
    if (p->scale_sn == 1 && (p->scale_sg % 8 != 0)) return false;
    auto aligned = [](const void* q, uintptr_t a) { return (reinterpret_cast<uintptr_t>(q) % a) == 0; };
    if (!aligned(p->w, 4) || !aligned(p->x, 16)) return false;
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
    a.steps_per_group = p->group_size > 0 ? p->group_size / 16 : a.ksteps;
    const bool bf16 = p->x_dtype == ACL_BF16, has_off = p->offset != nullptr;
    const int variant = (bf16 ? 2 : 0) + (has_off ? 1 : 0);
    int resident = 0;
    switch (variant) {
        case 0: resident = decode_grid<false, false>(0); break;
        case 1: resident = decode_grid<false, true>(1); break;
        case 2: resident = decode_grid<true, false>(2); break;
        default: resident = decode_grid<true, true>(3); break;
    }
    // host tile selection: as many equal k ranges per strip as keep every CTA resident at once
    int64_t splits = resident / a.strips;
    if (const char* e = getenv("OPSNN_WQ_DECODE_SPLITS")) {
        int v = atoi(e);
        if (v > 0) splits = v;
    }
    if (splits > a.ksteps) splits = a.ksteps;
    if (splits * a.strips > kMaxGrid) splits = kMaxGrid / a.strips;
    if (splits < 1) splits = 1;
    a.splits = splits;
    const int64_t grid64 = a.strips * splits;
    if (grid64 > 0x7FFFFFFF) return (int32_t)cudaErrorInvalidConfiguration;
    const int grid = (int)grid64;
    const uint64_t tag_bytes = (((uint64_t)kMaxGrid * 8 + 255) / 256) * 256;
    if (splits > 1 && (p->workspace == nullptr || p->workspace_size < wqbmm_decode_workspace_size(p))) return (int32_t)cudaErrorInvalidValue;
    a.tags = reinterpret_cast<unsigned long long*>(p->workspace);
    a.partials = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(p->workspace) + tag_bytes);
    a.nonce = next_nonce();
    a.c_mask = 0x000F000Fu;
    a.c_magic = bf16 ? Num<true>::kMagic : Num<false>::kMagic;
    a.c_bias = bf16 ? Num<true>::kBias : Num<false>::kBias;
    switch (variant) {
        case 0: wqbmm_decode_kernel<false, false><<<grid, kThreads, 0, stream>>>(a); break;
        case 1: wqbmm_decode_kernel<false, true><<<grid, kThreads, 0, stream>>>(a); break;
        case 2: wqbmm_decode_kernel<true, false><<<grid, kThreads, 0, stream>>>(a); break;
        default: wqbmm_decode_kernel<true, true><<<grid, kThreads, 0, stream>>>(a); break;
    }
    note_launch("wqbmm_decode");
    return (int32_t)cudaGetLastError();
}

// ---- entry point that allocates nothing -----------------------------------------------------------------------------
//
// Same kernel, same split selection, but the cross-CTA scratch (tags + fp32 fragments) is a fixed array in this module's
// device image instead of caller-provided workspace. Meant for callers that hold no allocator at the point of the call.
// The array covers kStaticGrid CTAs: two resident CTAs per SM on 148 SMs, rounded up.
namespace {

constexpr int kStaticGrid = 304;
constexpr size_t kStaticTagBytes = (((size_t)kStaticGrid * 8 + 255) / 256) * 256;
constexpr size_t kStaticBytes = kStaticTagBytes + (size_t)kStaticGrid * kWarps * kTiles * 32 * sizeof(float4);  // 9,964,032

}  // namespace

static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticBytes];

namespace {

constexpr int kMaxDevices = 64;
std::atomic<void*> g_static_scratch_ptr[kMaxDevices];

}  // namespace

void set_err(const char* fmt, ...);  // thread-local text behind aclGetRecentErrMsg (host library)

int32_t wqbmm_decode_static_launch(const OpsnnWqbmmParams* p, cudaStream_t stream)
{
    if (p->nz_k0 != 0) {
        set_err("opsnn_wqbmm_decode_static_launch: a FRACTAL_NZ weight needs workspace for its row-major copy");
        return (int32_t)cudaErrorInvalidValue;
    }
    if (p->n > (int64_t)kStaticGrid * kStripCols) {
        set_err("opsnn_wqbmm_decode_static_launch: n=%lld exceeds the %lld columns the built-in scratch covers", (long long)p->n,
                (long long)kStaticGrid * kStripCols);
        return (int32_t)cudaErrorInvalidValue;
    }
    // set-up, once per device with that device current: resolve the scratch array's address
    int dev = -1;
    cudaError_t rc = cudaGetDevice(&dev);
    if (rc != cudaSuccess) return (int32_t)rc;
    if (dev < 0 || dev >= kMaxDevices) {
        set_err("opsnn_wqbmm_decode_static_launch: device ordinal %d out of range (max %d)", dev, kMaxDevices - 1);
        return (int32_t)cudaErrorInvalidDevice;
    }
    void* scratch = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
    if (scratch == nullptr) {
        rc = cudaGetSymbolAddress(&scratch, g_decode_static_scratch);
        if (rc != cudaSuccess || scratch == nullptr) {
            set_err("opsnn_wqbmm_decode_static_launch: cudaGetSymbolAddress failed: %s", cudaGetErrorString(rc));
            return (int32_t)(rc != cudaSuccess ? rc : cudaErrorInvalidSymbol);
        }
        g_static_scratch_ptr[dev].store(scratch, std::memory_order_release);
    }

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
        case 0: resident = decode_grid<false, false>(0); break;
        case 1: resident = decode_grid<false, true>(1); break;
        case 2: resident = decode_grid<true, false>(2); break;
        default: resident = decode_grid<true, true>(3); break;
    }
    int64_t splits = resident / a.strips;
    if (splits > a.ksteps) splits = a.ksteps;
    if (splits * a.strips > kStaticGrid) splits = kStaticGrid / a.strips;
    if (splits < 1) splits = 1;
    a.splits = splits;
    const int grid = (int)(a.strips * splits);  // <= kStaticGrid by the checks above
    a.tags = reinterpret_cast<unsigned long long*>(scratch);
    a.partials = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(scratch) + kStaticTagBytes);
    a.nonce = next_nonce();
    a.c_mask = 0x000F000Fu;
    a.c_magic = bf16 ? Num<true>::kMagic : Num<false>::kMagic;
    a.c_bias = bf16 ? Num<true>::kBias : Num<false>::kBias;
    switch (variant) {
        case 0: wqbmm_decode_kernel<false, false><<<grid, kThreads, 0, stream>>>(a); break;
        case 1: wqbmm_decode_kernel<false, true><<<grid, kThreads, 0, stream>>>(a); break;
        case 2: wqbmm_decode_kernel<true, false><<<grid, kThreads, 0, stream>>>(a); break;
        default: wqbmm_decode_kernel<true, true><<<grid, kThreads, 0, stream>>>(a); break;
    }
    note_launch("wqbmm_decode_static");
    return (int32_t)cudaGetLastError();
}

}  // namespace opsnn

extern "C" __attribute__((visibility("default"))) int32_t opsnn_wqbmm_decode_static_launch(const OpsnnWqbmmParams* p, void* stream)
{
    if (p == nullptr) return (int32_t)cudaErrorInvalidValue;
    if (p->m <= 0 || p->n <= 0) return 0;
    if (!opsnn::wqbmm_decode_eligible(p)) {
        opsnn::set_err("opsnn_wqbmm_decode_static_launch: parameters outside the decode kernel's range (int4 weight stored (k,n), "
                       "m <= 16, k %% 16 == 0, n %% 8 == 0, 16-byte aligned x/scale rows)");
        return (int32_t)cudaErrorInvalidValue;
    }
    return opsnn::wqbmm_decode_static_launch(p, static_cast<cudaStream_t>(stream));
}
