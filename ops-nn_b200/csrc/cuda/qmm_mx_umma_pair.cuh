// Block-scaled (MX) quant matmul on CTA pairs: the choreography of qmm_umma_pair.cuh with the scale handling of
// qmm_mx_umma.cuh. Included by qmm_umma.cu after both.
//
// Pair tile 256 x 224: each CTA loads its own 128 rows of A, half of B (112 columns), the scale atoms of its own A rows and
// the scale atoms of ALL 224 B columns (every CTA's tensor core multiplies its 128 rows by the whole width, so both need B's
// scales; they are 1-2 KB per stage). The atoms come through tensor maps over the workspace (rows of one 512-byte atom): an
// untiled bulk copy can only signal a barrier of the CTA it writes to, the cta_group::2 tensor copy can signal the pair's. The even CTA issues tcgen05.cp.cta_group::2, which moves each CTA's atoms from its own
// shared memory into its own TMEM, then the pair MMAs. TMEM per CTA: accumulators at columns 0 and 256 (224 wide), two sets
// of scale slots at 224.. and 480.. used by alternate k-blocks. (Issuing the scale copies from a warp of their own, ahead of
// the MMA warp, was tried and lost: the extra handshake per k-block costs more than the three to six copy instructions.)
namespace {

template <bool kF4>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
qmm_mx_umma_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb, const UmmaArgs a)
{
    constexpr int BN = 224, HALF = 112, EW = 4;
    constexpr int kAtoms = kF4 ? 2 : 1;
    constexpr int RA = 2;
    constexpr uint32_t kSfaBytes = kAtoms * 512, kSfbBytes = kAtoms * RA * 512;
    constexpr uint32_t kBHalf = 128 * BK;  // reserved: 112 k-major rows (14336 B) or one 128-column n-major box (16384 B)
    constexpr uint32_t kStage = kATile + kBHalf + kSfaBytes + kSfbBytes;
    constexpr uint32_t kSfaCol = 224u, kSfbCol = kSfaCol + 4 * kAtoms, kAcc1 = 256u;
    constexpr uint32_t kTmemCols = 512;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)a.stages * kStage);
    uint64_t* full = bars;
    uint64_t* empty = bars + a.stages;
    uint64_t* tfull = bars + 2 * a.stages;
    uint64_t* tempty = tfull + 2;
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile uint32_t* abort_flag = tmem_ptr + 1;
    float* s_bias = reinterpret_cast<float*>(tmem_ptr + 4);  // [256]

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const bool leader = rank == 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
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
    const int kstages = a.kblocks;
    const int64_t tiles_m128 = (a.m + 127) / 128;  // the A scale atoms in workspace are indexed by 128-row tiles

    if (warp == EW) {
        // ======================= producer (both CTAs) =======================
        if (lane == 0) {
            ptx::tma_prefetch_desc(&map_a);
            ptx::tma_prefetch_desc(&map_b);
            ptx::tma_prefetch_desc(&map_sfa);
            ptx::tma_prefetch_desc(&map_sfb);
        }
        __syncwarp();
        uint32_t s = 0, par = 0;
        bool ok = true;
        const bool b_mn = a.b_mn_major != 0, a_mn = a.a_mn_major != 0;
        const uint32_t lead_full0 = full0 & ptx::kPeerBitMask;
        // bytes one CTA's copies deliver per stage; the even CTA arms the barrier with both CTAs' share
        const uint32_t tx = (uint32_t)kATile + (b_mn ? kBHalf : (uint32_t)(HALF * BK)) + kSfaBytes + kSfbBytes;
        for (uint32_t tile = pair; tile < ntiles && ok; tile += npairs) {
            const uint32_t b = tile / tiles_per_batch, r = tile % tiles_per_batch;
            uint32_t tmp, tn;
            tile_of<8>(r, (uint32_t)a.tiles_m, (uint32_t)a.tiles_n, tmp, tn);
            const int64_t tm128 = (int64_t)tmp * 2 + rank;
            const int32_t m0 = (int32_t)tm128 * 128, n0 = (int32_t)tn * BN + (int32_t)rank * HALF;
            const int32_t ba = a.a_batched ? (int32_t)b : 0, bb = a.b_batched ? (int32_t)b : 0;
            // atom row indices in workspace; a 128-row tile past m has no atoms: reuse the last one (its data is zero-filled)
            const int64_t sa_b = a.sfa_bs != 0 ? (int64_t)b : 0, sb_b = a.sfb_bs != 0 ? (int64_t)b : 0;
            int32_t sfa_row = (int32_t)(((sa_b * tiles_m128 + min(tm128, tiles_m128 - 1)) * kstages) * kAtoms);
            int32_t sfb_row = (int32_t)(((sb_b * a.tiles_n + tn) * kstages) * (kAtoms * RA));
            int32_t kk = 0;
            for (int kb = 0; kb < kstages; ++kb) {
                if (!ptx::mbar_wait_a(empty0 + 8u * s, par ^ 1u, abort_flag)) {
                    report(abort_flag, (1u << 8) | 1u);
                    ok = false;
                    break;
                }
                if (ptx::elect_one()) {
                    const uint32_t fb = lead_full0 + 8u * s, sa = smem0 + s * kStage, sb = sa + (uint32_t)kATile;
                    if (leader) ptx::mbar_expect_tx_a(full0 + 8u * s, 2u * tx);
                    ptx::tma_load_3d_pair(sa, &map_a, fb, a_mn ? m0 : kk, a_mn ? kk : m0, ba);
                    ptx::tma_load_3d_pair(sb, &map_b, fb, b_mn ? n0 : kk, b_mn ? kk : n0, bb);
                    ptx::tma_load_2d_pair(sb + kBHalf, &map_sfa, fb, 0, sfa_row);
                    ptx::tma_load_2d_pair(sb + kBHalf + kSfaBytes, &map_sfb, fb, 0, sfb_row);
                }
                __syncwarp();
                sfa_row += kAtoms;
                sfb_row += kAtoms * RA;
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
            uint32_t s = 0, par = 0, grp = 0, kbg = 0;  // kbg: k-blocks issued so far, over all tiles
            bool ok = true;
            const uint64_t da0 = a.a_mn_major ? ptx::make_smem_desc(smem0, 128 * BK, 1024, 2) : ptx::make_smem_desc(smem0, 0, 1024, 2);
            const uint64_t db0 = a.b_mn_major ? ptx::make_smem_desc(smem0 + kATile, 128 * BK, 1024, 2)
                                              : ptx::make_smem_desc(smem0 + kATile, 0, 1024, 2);
            const uint64_t dsf0 = ptx::make_smem_desc(smem0 + kATile + kBHalf, 0, 128, 0);  // 32 rows x 16 bytes, no swizzle
            const uint32_t a_lo = (uint32_t)da0, b_lo = (uint32_t)db0, sf_lo = (uint32_t)dsf0;
            const uint64_t a_hi = da0 & 0xFFFFFFFF00000000ull, b_hi = db0 & 0xFFFFFFFF00000000ull, sf_hi = dsf0 & 0xFFFFFFFF00000000ull;
            const uint32_t a_k1 = a.a_mn_major ? 256u : 2u, b_k1 = a.b_mn_major ? 256u : 2u;
            const uint32_t idesc = a.idesc;
            for (uint32_t tile = pair; tile < ntiles && ok; tile += npairs) {
                uint32_t acc = 0u;
                if (!ptx::mbar_wait_a(tempty0 + 8u * (grp & 1u), ((grp >> 1) & 1u) ^ 1u, abort_flag)) {
                    report(abort_flag, (2u << 8) | 1u);
                    ok = false;
                    break;
                }
                for (int kb = 0; kb < kstages; ++kb) {
                    if (!ptx::mbar_wait_a(full0 + 8u * s, par, abort_flag)) {
                        report(abort_flag, (2u << 8) | 2u);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    if (ptx::elect_one()) {
                        const uint32_t stage_off = (s * kStage) >> 4;
                        const uint32_t d = tmem_base + (grp & 1u) * kAcc1;
                        const uint32_t al = a_lo + stage_off, bl = b_lo + stage_off, sl = sf_lo + stage_off;
                        // scale atoms shared -> TMEM (each CTA's own atoms into its own TMEM), two slot sets used alternately
                        const uint32_t sfa_t = tmem_base + ((kbg & 1u) ? 480u : kSfaCol), sfb_t = sfa_t + 4 * kAtoms;
#pragma unroll
                        for (int at = 0; at < kAtoms; ++at) ptx::tmem_cp_sf_pair(sfa_t + 4 * at, sf_hi | (uint64_t)(sl + at * 32));
#pragma unroll
                        for (int at = 0; at < kAtoms * RA; ++at)
                            ptx::tmem_cp_sf_pair(sfb_t + 4 * at, sf_hi | (uint64_t)(sl + (kAtoms + at) * 32));
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint32_t sf_id = kF4 ? (uint32_t)(k & 1) * 2u : (uint32_t)k;
                            const uint32_t katom = kF4 ? (uint32_t)(k >> 1) : 0u;
                            const uint32_t id = idesc | (sf_id << 29) | (sf_id << 4);
                            const uint64_t da = a_hi | (uint64_t)(al + k * a_k1), db = b_hi | (uint64_t)(bl + k * b_k1);
                            const uint32_t ta = sfa_t + 4u * katom, tb = sfb_t + 4u * RA * katom;
                            if (kF4) ptx::umma_mxf4_pair(d, da, db, id, ta, tb, k == 0 ? acc : 1u);
                            else ptx::umma_mxf8f6f4_pair(d, da, db, id, ta, tb, k == 0 ? acc : 1u);
                        }
                        ptx::umma_commit_pair(empty0 + 8u * s, (uint16_t)3);
                    }
                    __syncwarp();
                    acc = 1u;
                    ++kbg;
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
        // ======================= epilogue warps (both CTAs): own 128 rows x 224 columns =======================
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
            const int out_bytes = a.out_dtype == ACL_FLOAT ? 4 : 2;
            uint8_t* out = reinterpret_cast<uint8_t*>(a.out) + b * a.out_bs * out_bytes;
            const uint32_t buf = grp & 1, gpar = (grp >> 1) & 1;
            const uint8_t* bias = reinterpret_cast<const uint8_t*>(a.bias);
            if (bias != nullptr) bias += b * a.bias_bs * (a.bias_dtype == ACL_FLOAT ? 4 : 2);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            for (int c = threadIdx.x; c < BN; c += 128)
                s_bias[c] = bias != nullptr ? load_as_float(bias, min(n0 + c, a.n - 1), a.bias_dtype) : 0.f;
            if (!ptx::mbar_wait_relaxed(&tfull[buf], gpar, abort_flag)) report(abort_flag, (3u << 8) | 1u);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*abort_flag != 0u) {
                ok = false;
                break;
            }
            ptx::tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t v[32];
                ptx::tmem_ld32(tmem_base + lane_addr + buf * kAcc1 + c, v);
                ptx::tmem_ld_wait();
                const int64_t col = n0 + c;
                const int valid = (int)min((int64_t)32, a.n - col);
                if (row_ok && valid > 0) {
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const float4 b4 = *reinterpret_cast<const float4*>(s_bias + c + i);
                        f[i] = __fadd_rn(__uint_as_float(v[i]), b4.x);
                        f[i + 1] = __fadd_rn(__uint_as_float(v[i + 1]), b4.y);
                        f[i + 2] = __fadd_rn(__uint_as_float(v[i + 2]), b4.z);
                        f[i + 3] = __fadd_rn(__uint_as_float(v[i + 3]), b4.w);
                    }
                    store_row32(a, out, row, col, f, valid);
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(lead_tempty0 + 8u * buf);
            ++grp;
        }
    }
    if (*abort_flag != 0u) __nanosleep(200000);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();
    if (warp == EW + 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// Workspace atoms as a 2-D tensor: rows of one 512-byte atom (128 x uint32), box = the atoms one stage needs.
bool make_map_atoms(CUtensorMap* map, const void* base, uint64_t total_atoms, uint32_t box_atoms)
{
    EncodeFn enc = get_encode();
    if (enc == nullptr) return false;
    cuuint64_t dims[2] = {128, total_atoms};
    cuuint64_t strides[1] = {512};
    cuuint32_t box[2] = {128, box_atoms};
    cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool kF4>
int32_t mx_launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, UmmaArgs& a, cudaStream_t stream)
{
    constexpr uint32_t kAtoms = kF4 ? 2 : 1;
    const uint64_t nb_a = a.sfa_bs != 0 ? (uint64_t)a.batch : 1, nb_b = a.sfb_bs != 0 ? (uint64_t)a.batch : 1;
    const uint64_t tiles_m128 = (uint64_t)((a.m + 127) / 128);
    CUtensorMap msa, msb;
    if (!make_map_atoms(&msa, a.sfa, nb_a * tiles_m128 * (uint64_t)a.kblocks * kAtoms, kAtoms) ||
        !make_map_atoms(&msb, a.sfb, nb_b * (uint64_t)a.tiles_n * (uint64_t)a.kblocks * kAtoms * 2, kAtoms * 2))
        return (int32_t)cudaErrorInvalidValue;
    constexpr uint32_t stage = (uint32_t)kATile + 128 * BK + (kF4 ? 2 : 1) * 512 * 3;
    int stages = (227 * 1024 - 2048) / (int)stage;
    if (stages > 6) stages = 6;
    if (stages > a.kblocks + 1) stages = a.kblocks + 1 > 2 ? a.kblocks + 1 : 2;
    a.stages = stages;
    const size_t smem = (size_t)stages * stage + 1024 + 256 + 256 * 4;
    static std::atomic<uint64_t> configured{0};
    {
        const cudaError_t rc = once_per_device(
            configured, [&] { return cudaFuncSetAttribute(qmm_mx_umma_pair_kernel<kF4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); });
        if (rc != cudaSuccess) return (int32_t)rc;
    }
    int64_t pairs = sm_count() / 2;
    if (a.num_tiles < pairs) pairs = a.num_tiles;
    qmm_mx_umma_pair_kernel<kF4><<<(unsigned)(2 * pairs), 192, smem, stream>>>(ma, mb, msa, msb, a);
    note_launch(kF4 ? "qmm_umma_pair_mxfp4" : "qmm_umma_pair_mxfp8");
    return (int32_t)cudaGetLastError();
}

}  // namespace
