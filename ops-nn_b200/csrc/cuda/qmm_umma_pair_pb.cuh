// Per-block (1x128 / 128x128 fp32 scales) fp8 and int8 matmul on CTA pairs (tcgen05 cta_group::2). Included by qmm_umma.cu.
//
// Why. The single-CTA per-block kernel uses 128 x 128 tiles (the promotion epilogue keeps 128 fp32 sums per thread), which
// pull 32 KB of operands from L2 per 128-deep k-block; with the epilogue switched off the main loop still needs ~700 cycles
// per k-block against 256 of tensor work: it is bound by the L2 -> SM operand feed. A CTA pair shares a 256 x 128 tile: each
// CTA loads its own 128 rows of A and 64 of the 128 rows of B (24 KB per k-block), keeps a 128 x 128 accumulator in its own
// TMEM and runs the same promotion on it.
//
// B per CTA is half of the tile's 128 columns. k-major (x2 stored (n,k)): 64 rows of 128 swizzled bytes. n-major (x2 stored
// (k,n)): half a 128-byte swizzle row is not a legal operand, so the 64 columns x 128 k rows are loaded and described in the
// 64-byte swizzle (TMA box 64 x 128, descriptor layout type 4, 512 bytes per 8 rows).
//
// Choreography per k-block (= one accumulation group), four TMEM buffers of 128 columns:
//   producers (both CTAs) : wait own empty[s]; even CTA arms full[s] for both CTAs' bytes; each loads A (128 rows) and B (64 rows)
//   MMA warp (even CTA)   : wait tempty[buf] (all epilogue warps of the pair), wait full[s], 4 pair MMAs (first overwrites),
//                           commit -> empty[s] and tfull[buf] of both CTAs
//   epilogue (both CTAs)  : wait own tfull[buf]; TMEM -> registers; acc += part * (s1 * s2); arrive on the even CTA's tempty[buf]
// All waits bounded, teardown through a cluster barrier, as in qmm_umma_pair.cuh.
namespace {

// 256-column tiles: 128 sums per epilogue thread need more registers than an even split of the register file over the CTA's
// warps gives (168 with ten warps), so the block is three whole warpgroups - epilogue warps 0..7, then {producer, MMA issuer, two
// idle warps} - and setmaxnreg moves registers from the third group (40 each) to the first two (232 each): per scheduler
// 2 x 232 + 40 = 504 of the 512 registers per lane.
#ifdef OPSNN_PB_DIAG
// Diagnostic builds only: clocks the MMA issuer spent waiting for a free accumulator buffer / for operands, and its total; clocks
// epilogue warp 0 spent waiting for a full buffer, and its total. [CTA][5]
__device__ unsigned long long g_pb_diag[1024 * 5];
#define OPSNN_PB_T(var) const long long var = clock64()
#define OPSNN_PB_ADD(acc, t0) acc += clock64() - (t0)
#else
#define OPSNN_PB_T(var) do { } while (0)
#define OPSNN_PB_ADD(acc, t0) do { } while (0)
#endif

// (Code that runs under setmaxnreg cannot call an out-of-line function: the bounded spin is inlined for those instances.)
template <bool kInline>
__device__ __forceinline__ bool pb_wait(uint32_t bar_addr, uint32_t parity, volatile uint32_t* abort_flag)
{
    if (!kInline) return ptx::mbar_wait_a(bar_addr, parity, abort_flag);
    if (ptx::mbar_try_wait_a(bar_addr, parity)) return true;
    const uint32_t limit = ptx::g_spin_limit;
    for (uint32_t i = 0; i < limit; ++i) {
        if (ptx::mbar_try_wait_a(bar_addr, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag != 0u) return false;
    }
    *abort_flag = 1u;
    return false;
}

template <int EW, int BN>
constexpr int pair_pb_threads() { return (EW + (BN == 256 ? 4 : 2)) * 32; }

// kAsym: INT4 x INT4 asymmetric per-group (quant_batch_matmul_v4_pertoken_pergroup.h; golden qbmmv4_kernel_golden.py:328-395), both
// operands widened to INT8 beforehand. An accumulation group is two k-blocks (256 of k); per group and element
// tot += (part - rowsum(x1 over the group)[m] * x2Offset[g, n]) * x2Scale[g, n], four separately rounded fp32 operations as in
// the golden, and at the end out = tot * x1Scale[m]. x2Offset / x2Scale of the tile's columns are staged in shared memory one
// group ahead (three buffers, one named barrier per group whose reduced predicate also carries the abort flag, so that the
// epilogue warps can only leave together).
template <ptx::MmaKind kKind, int EW, int BN, bool kAsym = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair_pb_threads<EW, BN>(), 1)
qmm_umma_pair_pb_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const UmmaArgs a)
{
    static_assert(BN == 128 || (BN == 256 && EW == 8), "256-column tiles keep 128 sums per thread: eight epilogue warps");
    static_assert(!kAsym || (BN == 128 && EW == 4 && kKind == ptx::MmaKind::kI8), "the asymmetric per-group epilogue: int8, 128 columns, four warps");
    __shared__ float s_cols[kAsym ? 3 * 2 * BN : 1];  // kAsym: [buffer][offset | scale][column]
    constexpr int NBUF = 512 / BN;              // accumulator buffers in the 512 TMEM columns
    constexpr int kCols = BN * 4 / EW;          // accumulator columns per epilogue thread
    constexpr uint32_t kBHalf = (BN / 2) * BK;  // this CTA's half of the B tile
    constexpr uint32_t kStage = kATile + kBHalf;
    constexpr uint32_t kTmemCols = 512;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)a.stages * kStage);
    uint64_t* full = bars;                    // [stages]  used in the even CTA only
    uint64_t* empty = bars + a.stages;        // [stages]
    uint64_t* tfull = bars + 2 * a.stages;    // [NBUF]
    uint64_t* tempty = tfull + NBUF;          // [NBUF]    used in the even CTA only
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tempty + NBUF);
    volatile uint32_t* abort_flag = tmem_ptr + 1;

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < NBUF; ++b) {
            ptx::mbar_init(&tfull[b], 1);
            ptx::mbar_init(&tempty[b], 2 * EW);
        }
        *abort_flag = 0u;
        ptx::fence_mbar_init();
    }
    if (warp == EW + 1) ptx::tmem_alloc_pair(tmem_ptr, kTmemCols);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;

    const uint32_t tiles_per_batch = (uint32_t)a.tiles_m * (uint32_t)a.tiles_n;
    const uint32_t ntiles = (uint32_t)a.num_tiles;
    const uint32_t pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const uint32_t smem0 = ptx::smem_u32(smem), full0 = ptx::smem_u32(full), empty0 = ptx::smem_u32(empty);
    const uint32_t tfull0 = ptx::smem_u32(tfull), tempty0 = ptx::smem_u32(tempty);
    const uint32_t stages = (uint32_t)a.stages;
    const int kblocks = a.kblocks;

    if (warp == EW) {
        // ======================= TMA producer (both CTAs) =======================
        if (BN == 256) asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (lane == 0) {
            ptx::tma_prefetch_desc(&map_a);
            ptx::tma_prefetch_desc(&map_b);
        }
        __syncwarp();
        uint32_t s = 0, par = 0;
        bool ok = true;
        const bool a_mn = a.a_mn_major != 0, b_mn = a.b_mn_major != 0;
        const uint32_t lead_full0 = full0 & ptx::kPeerBitMask;
        for (uint32_t tile = pair; tile < ntiles && ok; tile += npairs) {
            const uint32_t b = tile / tiles_per_batch, r = tile % tiles_per_batch;
            uint32_t tm, tn;
            tile_of<8>(r, (uint32_t)a.tiles_m, (uint32_t)a.tiles_n, tm, tn);
            const int32_t m0 = (int32_t)tm * 256 + (int32_t)rank * 128;
            const int32_t n0 = (int32_t)tn * BN + (int32_t)rank * (BN / 2);
            const int32_t ba = a.a_batched ? (int32_t)b : 0, bb = a.b_batched ? (int32_t)b : 0;
            int32_t kk = 0;
            for (int kb = 0; kb < kblocks; ++kb) {
                if (!pb_wait<BN == 256>(empty0 + 8u * s, par ^ 1u, abort_flag)) {
                    report(abort_flag, (1u << 8) | 1u);
                    ok = false;
                    break;
                }
                if (ptx::elect_one()) {
                    const uint32_t fb = lead_full0 + 8u * s, sa = smem0 + s * kStage, sb = sa + (uint32_t)kATile;
                    if (leader) ptx::mbar_expect_tx_a(full0 + 8u * s, 2u * kStage);
                    ptx::tma_load_3d_pair(sa, &map_a, fb, a_mn ? m0 : kk, a_mn ? kk : m0, ba);
                    if (b_mn) ptx::tma_load_3d_pair(sb, &map_b, fb, n0, kk, bb);  // BN / 2 columns x 128 k rows (64 columns: 64-byte swizzle)
                    else ptx::tma_load_3d_pair(sb, &map_b, fb, kk, n0, bb);
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
        // ======================= MMA issuer (even CTA only): every k-block is its own accumulation group =======================
        if (BN == 256) asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (leader) {
            uint32_t s = 0, par = 0, buf = 0, bpar = 0;
            bool ok = true;
            const uint64_t da0 = a.a_mn_major ? ptx::make_smem_desc(smem0, 128 * BK, 1024, 2) : ptx::make_smem_desc(smem0, 0, 1024, 2);
            // B k-major: 64 rows of 128 swizzled bytes. B n-major (x2 stored (k,n)): 128 k rows of this CTA's 64 columns in the
            // 64-byte swizzle (layout type 4): 8 rows = 512 bytes (stride byte offset), one MMA = 32 rows = 2 KB
            // 128 columns (BN = 256) are whole 128-byte swizzle rows, described like an m-major A
            const uint64_t db0 = !a.b_mn_major ? ptx::make_smem_desc(smem0 + kATile, 0, 1024, 2)
                                 : (BN == 128 ? ptx::make_smem_desc(smem0 + kATile, 64 * BK, 512, 4)
                                              : ptx::make_smem_desc(smem0 + kATile, 128 * BK, 1024, 2));
            const uint32_t a_lo = (uint32_t)da0, b_lo = (uint32_t)db0;
            const uint64_t a_hi = da0 & 0xFFFFFFFF00000000ull, b_hi = db0 & 0xFFFFFFFF00000000ull;
            const uint32_t a_k1 = a.a_mn_major ? 256u : 2u, b_k1 = a.b_mn_major ? (BN == 128 ? 128u : 256u) : 2u;
            const uint32_t idesc = a.idesc;
            long long d_tempty = 0, d_full = 0;
            OPSNN_PB_T(d_start);
            for (uint32_t tile = pair; tile < ntiles && ok; tile += npairs) {
                for (int kb = 0; kb < kblocks; ++kb) {
                    // kAsym: k-blocks 2g and 2g + 1 accumulate into one buffer; otherwise every k-block is its own group
                    const bool first = !kAsym || (kb & 1) == 0, last = !kAsym || (kb & 1) == 1 || kb == kblocks - 1;
                    OPSNN_PB_T(d_t0);
                    if (first && !pb_wait<BN == 256>(tempty0 + 8u * buf, bpar ^ 1u, abort_flag)) {
                        report(abort_flag, (2u << 8) | 1u);
                        ok = false;
                        break;
                    }
                    OPSNN_PB_ADD(d_tempty, d_t0);
                    OPSNN_PB_T(d_t1);
                    if (!pb_wait<BN == 256>(full0 + 8u * s, par, abort_flag)) {
                        report(abort_flag, (2u << 8) | 2u);
                        ok = false;
                        break;
                    }
                    OPSNN_PB_ADD(d_full, d_t1);
                    ptx::tc_fence_after();
                    if (ptx::elect_one()) {
                        const uint32_t stage_off = (s * kStage) >> 4;
                        const uint32_t d = tmem_base + buf * BN;
                        const uint32_t al = a_lo + stage_off, bl = b_lo + stage_off;
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            ptx::umma_pair<kKind>(d, a_hi | (uint64_t)(al + k * a_k1), b_hi | (uint64_t)(bl + k * b_k1), idesc,
                                                  (k == 0 && first) ? 0u : 1u);
                        ptx::umma_commit_pair(empty0 + 8u * s, (uint16_t)3);
                        if (last) ptx::umma_commit_pair(tfull0 + 8u * buf, (uint16_t)3);
                    }
                    __syncwarp();
                    if (++s == stages) {
                        s = 0;
                        par ^= 1u;
                    }
                    if (last && ++buf == NBUF) {
                        buf = 0;
                        bpar ^= 1u;
                    }
                }
            }
#ifdef OPSNN_PB_DIAG
            if (lane == 0) {
                g_pb_diag[blockIdx.x * 5 + 0] = (unsigned long long)d_tempty;
                g_pb_diag[blockIdx.x * 5 + 1] = (unsigned long long)d_full;
                g_pb_diag[blockIdx.x * 5 + 2] = (unsigned long long)(clock64() - d_start);
            }
#endif
            (void)d_tempty;
            (void)d_full;
        }
    } else if (warp < EW) {
        // ======================= epilogue warps (both CTAs): own 128 rows, kCols columns each =======================
        if (BN == 256) asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        const int quad = warp & 3, part = warp >> 2;
        const uint32_t lane_addr = ((uint32_t)(quad * 32) << 16) + (uint32_t)(part * kCols);
        const uint32_t lead_tempty0 = tempty0 & ptx::kPeerBitMask;
        uint32_t buf = 0, bpar = 0;
        bool ok = true;
        long long d_tfull = 0;
        OPSNN_PB_T(d_estart);
        for (uint32_t tile = pair; tile < ntiles && ok; tile += npairs) {
            const uint32_t b = tile / tiles_per_batch, r = tile % tiles_per_batch;
            uint32_t tm, tn;
            tile_of<8>(r, (uint32_t)a.tiles_m, (uint32_t)a.tiles_n, tm, tn);
            const int64_t m0 = (int64_t)tm * 256 + (int64_t)rank * 128, n0 = (int64_t)tn * BN;
            const int64_t row = m0 + quad * 32 + lane;
            const bool row_ok = row < a.m;
            uint8_t* out = reinterpret_cast<uint8_t*>(a.out) + b * a.out_bs * out_elem_bytes(a.out_dtype);
            const int64_t colbase = n0 + part * kCols;
            float acc[kCols];
#pragma unroll
            for (int i = 0; i < kCols; ++i) acc[i] = 0.f;
            if constexpr (kAsym) {
                const int groups = a.groups;
                const float* rsp = a.row_sums + (row_ok ? row : 0) * (int64_t)groups;
                const __half* offp = reinterpret_cast<const __half*>(a.b_offset);
                const float* scp = reinterpret_cast<const float*>(a.scale_b);
                const int tcol = quad * 32 + lane;  // the column of the tile whose offset and scale this thread stages
                const int64_t gcol = n0 + tcol;
                auto stage_cols = [&](int g) {
                    float o = 0.f, sc = 0.f;
                    if (g < groups && gcol < a.n) {
                        o = __half2float(offp[(int64_t)g * a.n + gcol]);
                        sc = __ldg(scp + (int64_t)g * a.n + gcol);
                    }
                    float* dst = s_cols + (g % 3) * 2 * BN;
                    dst[tcol] = o;
                    dst[BN + tcol] = sc;
                };
                asm volatile("bar.sync 1, 128;" ::: "memory");  // the previous tile's readers of the column buffers are done
                stage_cols(0);
                float rs_next = __ldg(rsp);
                for (int g = 0; g < groups; ++g) {
                    const float rsg = rs_next;
                    if (g + 1 < groups) rs_next = __ldg(rsp + g + 1);
                    stage_cols(g + 1);  // buffer (g + 1) % 3: last read in group g - 2, which every warp has left (barrier of g - 1)
                    const bool arrived = pb_wait<false>(tfull0 + 8u * buf, bpar, abort_flag);
                    if (!arrived) report(abort_flag, (3u << 8) | 2u);
                    // One barrier per group: group g's columns are visible to all four warps, and its reduced predicate tells every
                    // warp the same thing about a give-up anywhere in the CTA - they can only leave together.
                    const int bad = (!arrived || *abort_flag != 0u) ? 1 : 0;
                    int any_bad;
                    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.s32 q, %1, 0;\n\tbar.red.or.pred p, 1, 128, q;\n\tselp.s32 %0, 1, 0, p;\n\t}"
                                 : "=r"(any_bad)
                                 : "r"(bad)
                                 : "memory");
                    if (any_bad != 0) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const float* cur = s_cols + (g % 3) * 2 * BN;
                    const uint32_t t0 = tmem_base + lane_addr + buf * BN;
                    // (part - rowsum * offset) * scale, then the running sum: four roundings, none fused, as in the golden
                    auto fold = [&](const uint32_t(&v)[16], int c) {
#pragma unroll
                        for (int i = 0; i < 16; i += 4) {
                            const float4 o4 = *reinterpret_cast<const float4*>(cur + c + i);
                            const float4 s4 = *reinterpret_cast<const float4*>(cur + BN + c + i);
                            const float oo[4] = {o4.x, o4.y, o4.z, o4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float f = __fsub_rn(__uint_as_float(v[i + j] + 0x4B400000u), 12582912.f);  // exact int -> float, |part| < 2^22
                                const float w = __fmul_rn(__fsub_rn(f, __fmul_rn(rsg, oo[j])), ss[j]);
                                acc[c + i + j] = __fadd_rn(acc[c + i + j], w);
                            }
                        }
                    };
                    uint32_t va[16], vb[16];
                    ptx::tmem_ld16(t0, va);
#pragma unroll
                    for (int c = 0; c < kCols; c += 32) {
                        ptx::tmem_ld_wait();
                        ptx::tmem_ld16(t0 + c + 16, vb);
                        fold(va, c);
                        ptx::tmem_ld_wait();
                        if (c + 32 < kCols) {
                            ptx::tmem_ld16(t0 + c + 32, va);
                        } else {
                            ptx::tc_fence_before();
                            __syncwarp();
                            if (lane == 0) ptx::mbar_arrive_cluster(lead_tempty0 + 8u * buf);
                        }
                        fold(vb, c + 16);
                    }
                    if (++buf == NBUF) {
                        buf = 0;
                        bpar ^= 1u;
                    }
                }
                if (row_ok) {  // out = tot * x1Scale[m]
                    const float sa = __ldg(reinterpret_cast<const float*>(a.scale_a) + row);
#pragma unroll
                    for (int i = 0; i < kCols; ++i) acc[i] = __fmul_rn(acc[i], sa);
                }
            } else {
                const float* s1 = reinterpret_cast<const float*>(a.scale_a) + b * a.sa_bs;
                const float* s2 = reinterpret_cast<const float*>(a.scale_b) + b * a.sb_bs;
                const int64_t mg = (row_ok ? row : 0) / a.group_m;
                const int64_t n_mg = (a.m + a.group_m - 1) / a.group_m, n_ng = (a.n + 127) / 128;
                const int64_t ng = min(colbase / 128, n_ng - 1);
                auto load_s1 = [&](int kb) {
                    kb = min(kb, a.kblocks - 1);
                    return a.trans_a ? __ldg(s1 + kb * n_mg + mg) : __ldg(s1 + mg * a.kblocks + kb);
                };
                auto load_s2 = [&](int kb) {
                    kb = min(kb, a.kblocks - 1);
                    return a.trans_b ? __ldg(s2 + ng * a.kblocks + kb) : __ldg(s2 + kb * n_ng + ng);
                };
                float s1_next[4], s2_next[4];  // raw scales of the next four k-blocks; multiplied when their turn comes
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
                        const float sc = sc_cur[j];
                        OPSNN_PB_T(d_t2);
                        if (!pb_wait<BN == 256>(tfull0 + 8u * buf, bpar, abort_flag)) {
                            report(abort_flag, (3u << 8) | 2u);
                            ok = false;
                            break;
                        }
                        OPSNN_PB_ADD(d_tfull, d_t2);
                        ptx::tc_fence_after();
    #if defined(OPSNN_PB_EXPERIMENT) && OPSNN_PB_EXPERIMENT == 1
                        // diagnostic build: the buffer is released unread (main loop alone)
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive_cluster(lead_tempty0 + 8u * buf);
                        if (++buf == NBUF) {
                            buf = 0;
                            bpar ^= 1u;
                        }
                        acc[0] += sc;
                        continue;
    #endif
    #ifndef OPSNN_PB256_W
    #define OPSNN_PB256_W 16
    #endif
                        constexpr int W = BN == 256 ? OPSNN_PB256_W : 16;  // staging registers per TMEM load (two sets in flight)
                        const uint32_t t0 = tmem_base + lane_addr + buf * BN;
                        uint32_t va[W], vb[W];
                        ptx::tmem_ld_n(t0, va);
    #pragma unroll
                        for (int c = 0; c < kCols; c += 2 * W) {
                            ptx::tmem_ld_wait();
                            ptx::tmem_ld_n(t0 + c + W, vb);
    #pragma unroll
                            for (int i = 0; i < W; ++i) acc[c + i] = promote<kKind>(va[i], sc, acc[c + i]);
                            ptx::tmem_ld_wait();
                            if (c + 2 * W < kCols) {
                                ptx::tmem_ld_n(t0 + c + 2 * W, va);
                            } else {
                                ptx::tc_fence_before();
                                __syncwarp();
                                if (lane == 0) ptx::mbar_arrive_cluster(lead_tempty0 + 8u * buf);
                            }
    #pragma unroll
                            for (int i = 0; i < W; ++i) acc[c + W + i] = promote<kKind>(vb[i], sc, acc[c + W + i]);
                        }
                        if (++buf == NBUF) {
                            buf = 0;
                            bpar ^= 1u;
                        }
                    }
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
#ifdef OPSNN_PB_DIAG
        if (warp == 0 && lane == 0) {
            g_pb_diag[blockIdx.x * 5 + 3] = (unsigned long long)d_tfull;
            g_pb_diag[blockIdx.x * 5 + 4] = (unsigned long long)(clock64() - d_estart);
        }
#endif
        (void)d_tfull;
    }
    else if (BN == 256) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");  // the two idle warps of the third warpgroup
    }
#ifdef OPSNN_PB_DIAG
    // (epilogue warp 0's counters are written from inside its branch)
#endif
    // ---- teardown ----
    if (*abort_flag != 0u) __nanosleep(200000);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();
    if (warp == EW + 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

template <ptx::MmaKind KIND, int EW, int BN = 128, bool ASYM = false>
int32_t launch_pair_pb(const CUtensorMap& ma, const CUtensorMap& mb, UmmaArgs& a, cudaStream_t stream)
{
    constexpr int kStage = kATile + (BN / 2) * BK;
    constexpr int kDynMax = 227 * 1024 - (ASYM ? 4096 : 0);  // the asymmetric epilogue keeps 3 KB of static shared memory for its column buffers
    int stages = (kDynMax - 2048) / kStage;
    if (stages > 8) stages = 8;
    if (stages > a.kblocks + 1) stages = a.kblocks + 1 > 2 ? a.kblocks + 1 : 2;
    a.stages = stages;
    const size_t smem = (size_t)stages * kStage + 1024 + 256;
    auto kern = qmm_umma_pair_pb_kernel<KIND, EW, BN, ASYM>;
    static std::atomic<uint64_t> configured{0};
    if (once_per_device(configured, [&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kDynMax); }) != cudaSuccess)
        return (int32_t)cudaGetLastError();
    int64_t pairs = sm_count() / 2;
    if (a.num_tiles < pairs) pairs = a.num_tiles;
    kern<<<(unsigned)(2 * pairs), pair_pb_threads<EW, BN>(), smem, stream>>>(ma, mb, a);
    note_launch(ASYM ? "qmm_umma_pair_pergroup_asym" : "qmm_umma_pair_perblock");
    return (int32_t)cudaGetLastError();
}

// Sums of x1's rows over each k-group, as floats (exact: at most 256 values of magnitude <= 128), for the asymmetric per-group
// epilogue. One thread per (row, group); x1 is the widened INT8 operand, stored (m,k) or, transposed, (k,m).
__global__ void row_sums_kernel(const int8_t* __restrict__ x1, int64_t ld, int trans, int64_t m, int64_t k, int32_t groups, int32_t group_k,
                                float* __restrict__ out)
{
    const int64_t total = m * groups;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        // transposed storage: consecutive threads take consecutive rows (contiguous in memory); else consecutive groups of one row
        const int64_t row = trans ? i % m : i / groups;
        const int g = (int)(trans ? i / m : i % groups);
        const int64_t k0 = (int64_t)g * group_k, k1 = min(k, k0 + group_k);
        int sum = 0;
        if (trans) {
            for (int64_t kk = k0; kk < k1; ++kk) sum += x1[kk * ld + row];
        } else {
            for (int64_t kk = k0; kk < k1; ++kk) sum += x1[row * ld + kk];
        }
        out[row * groups + g] = (float)sum;
    }
}

// Pair tiles for per-block problems: worthwhile once there are enough 256 x 128 tiles to fill the pairs.
bool pair_pb_worthwhile(const OpsnnQmmParams* p)
{
    if (p->mode != OPSNN_QMM_PERBLOCK) return false;
    if (const char* e = getenv("OPSNN_QMM_PAIR")) return atoi(e) != 0;
    const int64_t tiles = p->batch * ((p->m + 255) / 256) * ((p->n + 127) / 128);
    return p->m >= 256 && tiles >= 74;
}

// Tile width of the per-block pair kernel: 256 columns (32 KB of operands per CTA and k-block for twice the tensor work of the
// 128-column tile's 24 KB: the L2 -> SM feed is what bounds the main loop) once there are enough such tiles for every pair.
// OPSNN_QMM_PB_BN=128|256 fixes it.
int pair_pb_bn(const OpsnnQmmParams* p)
{
    if (const char* e = getenv("OPSNN_QMM_PB_BN")) return atoi(e) == 256 ? 256 : 128;
    const int64_t tiles = p->batch * ((p->m + 255) / 256) * ((p->n + 255) / 256);
    return tiles >= sm_count() / 2 ? 256 : 128;
}

}  // namespace
