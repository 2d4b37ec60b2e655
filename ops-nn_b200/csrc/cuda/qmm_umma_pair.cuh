// int8 / fp8 dequant matmul on CTA pairs (tcgen05 cta_group::2). Included by qmm_umma.cu (same translation unit).
//
// Why pairs. With one CTA per tile (128 x 256) every SM pulls 48 KB of operands from L2 per 512 tensor-core cycles; 148 SMs
// at full rate ask for more than the L2 -> SM path delivers, so the tensor pipe waits for operands. Two CTAs of a cluster
// that share one 256 x 256 tile each load their own 128 rows of A and only HALF of B (128 columns); the MMA, issued by the
// even CTA, reads A and B from both CTAs' shared memory and writes rows 0-127 / 128-255 of the accumulator to the even / odd
// CTA's TMEM. Per SM that is 32 KB per 512 cycles: a third less traffic for the same arithmetic.
//
// Choreography (each CTA waits only on its own barriers):
//   producer warp, both CTAs : wait own empty[s]; the even CTA arms its full[s] with both CTAs' byte count; both issue their two
//                              TMA loads into their own shared memory, counted on the EVEN CTA's full[s]
//   MMA warp, even CTA only  : wait tempty[buf] (all 8 epilogue warps of the pair arrive there), wait full[s], 4 pair MMAs,
//                              commit to empty[s] of both CTAs; after the last k-block commit to tfull[buf] of both CTAs
//   epilogue warps, both CTAs: wait own tfull[buf], dequantise own 128 rows from own TMEM, arrive on the even CTA's tempty[buf]
// No load is multicast; the only cluster-wide signals are barrier arrivals. All waits are bounded as in the single-CTA kernel;
// the two CTAs meet at a cluster barrier before the first remote signal and before TMEM is freed.
namespace {

template <ptx::MmaKind kKind>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
qmm_umma_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const UmmaArgs a)
{
    constexpr int BN = 256, EW = 4;         // pair tile 256 x 256; each CTA: 128 rows of A, 128 columns of B, 128 x 256 accumulator
    constexpr uint32_t kBHalf = 128 * BK;   // this CTA's half of the B tile
    constexpr uint32_t kStage = kATile + kBHalf;
    constexpr uint32_t kTmemCols = 512;     // two accumulator buffers of 256 columns

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)a.stages * kStage);
    uint64_t* full = bars;                    // [stages]  used in the even CTA only
    uint64_t* empty = bars + a.stages;        // [stages]
    uint64_t* tfull = bars + 2 * a.stages;    // [2]
    uint64_t* tempty = tfull + 2;             // [2]       used in the even CTA only
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile uint32_t* abort_flag = tmem_ptr + 1;
    float* s_scale = reinterpret_cast<float*>(tmem_ptr + 4);
    uint32_t* s_bias = reinterpret_cast<uint32_t*>(s_scale + BN);

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();  // 0: even CTA (issues the MMAs), 1: odd
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(&tfull[b], 1);
            ptx::mbar_init(&tempty[b], 2 * EW);  // one arrival per epilogue warp of either CTA
        }
        *abort_flag = 0u;
        ptx::fence_mbar_init();
    }
    if (warp == EW + 1) ptx::tmem_alloc_pair(tmem_ptr, kTmemCols);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();  // both CTAs' barriers are initialised before anybody signals across the pair
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
        if (lane == 0) {
            ptx::tma_prefetch_desc(&map_a);
            ptx::tma_prefetch_desc(&map_b);
        }
        __syncwarp();
        uint32_t s = 0, par = 0;
        bool ok = true;
        const bool a_mn = a.a_mn_major != 0, b_mn = a.b_mn_major != 0;
        const uint32_t lead_full0 = full0 & ptx::kPeerBitMask;  // the even CTA's full barriers, from either CTA
        for (uint32_t tile = pair; tile < ntiles && ok; tile += npairs) {
            const uint32_t b = tile / tiles_per_batch, r = tile % tiles_per_batch;
            uint32_t tm, tn;
            tile_of<8>(r, (uint32_t)a.tiles_m, (uint32_t)a.tiles_n, tm, tn);
            const int32_t m0 = (int32_t)tm * 256 + (int32_t)rank * 128;
            const int32_t n0 = (int32_t)tn * BN + (int32_t)rank * 128;
            const int32_t ba = a.a_batched ? (int32_t)b : 0, bb = a.b_batched ? (int32_t)b : 0;
            int32_t kk = 0;
            for (int kb = 0; kb < kblocks; ++kb) {
                if (!ptx::mbar_wait_a(empty0 + 8u * s, par ^ 1u, abort_flag)) {
                    report(abort_flag, (1u << 8) | 1u);
                    ok = false;
                    break;
                }
                if (ptx::elect_one()) {
                    const uint32_t fb = lead_full0 + 8u * s, sa = smem0 + s * kStage, sb = sa + (uint32_t)kATile;
                    if (leader) ptx::mbar_expect_tx_a(full0 + 8u * s, 2u * kStage);
                    ptx::tma_load_3d_pair(sa, &map_a, fb, a_mn ? m0 : kk, a_mn ? kk : m0, ba);
                    ptx::tma_load_3d_pair(sb, &map_b, fb, b_mn ? n0 : kk, b_mn ? kk : n0, bb);
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
        // ======================= MMA issuer (even CTA only) =======================
        if (leader) {
            uint32_t s = 0, par = 0, grp = 0;
            bool ok = true;
            const uint64_t da0 = a.a_mn_major ? ptx::make_smem_desc(smem0, 128 * BK, 1024, 2) : ptx::make_smem_desc(smem0, 0, 1024, 2);
            const uint64_t db0 = a.b_mn_major ? ptx::make_smem_desc(smem0 + kATile, 128 * BK, 1024, 2)
                                              : ptx::make_smem_desc(smem0 + kATile, 0, 1024, 2);
            const uint32_t a_lo = (uint32_t)da0, b_lo = (uint32_t)db0;
            const uint64_t a_hi = da0 & 0xFFFFFFFF00000000ull, b_hi = db0 & 0xFFFFFFFF00000000ull;
            const uint32_t a_k1 = a.a_mn_major ? 256u : 2u, b_k1 = a.b_mn_major ? 256u : 2u;
            const uint32_t idesc = a.idesc;
            for (uint32_t tile = pair; tile < ntiles && ok; tile += npairs) {
                uint32_t acc = 0u;
                if (!ptx::mbar_wait_a(tempty0 + 8u * (grp & 1u), ((grp >> 1) & 1u) ^ 1u, abort_flag)) {
                    report(abort_flag, (2u << 8) | 1u);
                    ok = false;
                    break;
                }
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!ptx::mbar_wait_a(full0 + 8u * s, par, abort_flag)) {
                        report(abort_flag, (2u << 8) | 2u);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    if (ptx::elect_one()) {
                        const uint32_t stage_off = (s * kStage) >> 4;
                        const uint32_t d = tmem_base + (grp & 1u) * BN;
                        const uint32_t al = a_lo + stage_off, bl = b_lo + stage_off;
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            ptx::umma_pair<kKind>(d, a_hi | (uint64_t)(al + k * a_k1), b_hi | (uint64_t)(bl + k * b_k1), idesc,
                                                  k == 0 ? acc : 1u);
                        ptx::umma_commit_pair(empty0 + 8u * s, (uint16_t)3);
                    }
                    __syncwarp();
                    acc = 1u;
                    if (++s == stages) {
                        s = 0;
                        par ^= 1u;
                    }
                }
                if (ok) {
                    if (ptx::elect_one()) ptx::umma_commit_pair(tfull0 + 8u * (grp & 1u), (uint16_t)3);
                    __syncwarp();
                    ++grp;
                }
            }
        }
    } else {
        // ======================= epilogue warps (both CTAs): own 128 rows x 256 columns =======================
        const int quad = warp & 3;
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        const uint32_t lead_tempty0 = tempty0 & ptx::kPeerBitMask;
        uint32_t grp = 0;
        bool ok = true;
        for (uint32_t tile = pair; tile < ntiles && ok; tile += npairs) {
            const uint32_t b = tile / tiles_per_batch, r = tile % tiles_per_batch;
            uint32_t tm, tn;
            tile_of<8>(r, (uint32_t)a.tiles_m, (uint32_t)a.tiles_n, tm, tn);
            const int64_t m0 = (int64_t)tm * 256 + (int64_t)rank * 128, n0 = (int64_t)tn * BN;
            const int64_t row = m0 + quad * 32 + lane;
            const bool row_ok = row < a.m;
            const int out_bytes = (a.out_dtype == ACL_FLOAT || a.out_dtype == ACL_INT32) ? 4 : 2;
            uint8_t* out = reinterpret_cast<uint8_t*>(a.out) + b * a.out_bs * out_bytes;
            const uint32_t buf = grp & 1, gpar = (grp >> 1) & 1;
            const uint8_t* bias = reinterpret_cast<const uint8_t*>(a.bias);
            if (bias != nullptr) bias += b * a.bias_bs * ((a.bias_dtype == ACL_FLOAT || a.bias_dtype == ACL_INT32) ? 4 : 2);
            const bool has_sa = a.scale_a != nullptr;
            const float sav = (has_sa && row_ok) ? reinterpret_cast<const float*>(a.scale_a)[a.scale_a_len == 1 ? 0 : row] : 1.f;
            const bool has_fbias = bias != nullptr && a.bias_dtype != ACL_INT32;
            const bool has_ibias = bias != nullptr && a.bias_dtype == ACL_INT32;
            asm volatile("bar.sync 1, 128;" ::: "memory");  // the previous tile's readers of the staged columns are done
            deq_stage_cols<BN>(a, bias, has_ibias, has_fbias, n0, s_scale, s_bias);
            if (!ptx::mbar_wait_relaxed(&tfull[buf], gpar, abort_flag)) report(abort_flag, (3u << 8) | 1u);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*abort_flag != 0u) {
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            deq_store_cols<BN>(a, tmem_base + lane_addr + buf * BN, out, row, row_ok, n0, s_scale, s_bias, sav, has_sa, has_fbias, has_ibias);
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(lead_tempty0 + 8u * buf);
            ++grp;
        }
    }
    // ---- teardown: both CTAs meet (the even CTA's MMAs read the odd CTA's shared memory until the very end), then free TMEM ----
    if (*abort_flag != 0u) __nanosleep(200000);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();
    if (warp == EW + 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

template <ptx::MmaKind KIND>
int32_t launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, UmmaArgs& a, cudaStream_t stream)
{
    constexpr int kStage = kATile + 128 * BK;
    int stages = (227 * 1024 - 2048) / kStage;
    if (stages > 6) stages = 6;
    if (stages > a.kblocks + 1) stages = a.kblocks + 1 > 2 ? a.kblocks + 1 : 2;
    a.stages = stages;
    const size_t smem = (size_t)stages * kStage + 1024 + 256 + 2 * 256 * 4;
    auto kern = qmm_umma_pair_kernel<KIND>;
    static std::atomic<uint64_t> configured{0};
    if (once_per_device(configured, [&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); }) != cudaSuccess)
        return (int32_t)cudaGetLastError();
    int64_t pairs = sm_count() / 2;
    if (a.num_tiles < pairs) pairs = a.num_tiles;
    kern<<<(unsigned)(2 * pairs), 192, smem, stream>>>(ma, mb, a);
    note_launch("qmm_umma_pair_deq");
    return (int32_t)cudaGetLastError();
}

// Pairs pay off when there is a 256 x 256 tile for about every pair of SMs; small problems keep the single-CTA kernel.
bool pair_worthwhile(const OpsnnQmmParams* p)
{
    if (const char* e = getenv("OPSNN_QMM_PAIR")) return atoi(e) != 0;
    if (p->mode != OPSNN_QMM_DEQ) return false;
    const int64_t tiles = p->batch * ((p->m + 255) / 256) * ((p->n + 255) / 256);
    return p->m >= 256 && p->n >= 256 && tiles >= 74;
}

}  // namespace
