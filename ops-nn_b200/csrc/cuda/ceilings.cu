// Measured ceilings the roofline fractions can be read against ("fraction of achievable" beside "fraction of peak").
//
//   opsnn_probe_umma   one CTA per SM issues tcgen05.mma of one kind back to back on operands resident in shared memory (garbage
//                      bytes: the tensor core's timing does not depend on values), no loads, no epilogue: the instruction-issue
//                      ceiling of that kind and tile width in clocks per MMA. Kinds: i8, f8f6f4, mxf8f6f4 (block scaled, fp8),
//                      mxf4 (block scaled, fp4). One MMA is 128 x bn x 32 bytes of k.
//   opsnn_probe_mix    the three execution pipes the weight-only decode kernels live on - integer (lop3), 16-bit-pair arithmetic
//                      (add.bf16x2) and legacy mma.sync m16n8k16 - issued from independent registers in the per-k-step proportions of
//                      the decode kernels: clocks per k-step per scheduler when nothing else is in the way. Separately each pipe takes
//                      2, 2 and 8 clocks per warp instruction; together they overlap only in part, which is what bounds those kernels.
// Every wait is bounded. Nothing here is on a product path; bench.py --workload ceilings prints the figures.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace opsnn {

namespace {

// KIND 0: i8, 1: f8f6f4, 2: mxf8f6f4, 3: mxf4
template <int KIND>
__global__ void __launch_bounds__(64) umma_rate_kernel(int iters, uint32_t bn, long long* out, unsigned int* status)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t done;
    __shared__ uint32_t tmem_ptr;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&done, 1);
        ptx::fence_mbar_init();
    }
    if (warp == 0) ptx::tmem_alloc(&tmem_ptr, 512);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = tmem_ptr;
    if (warp == 0) {
        const uint32_t smem0 = ptx::smem_u32(smem);
        const uint64_t da0 = ptx::make_smem_desc(smem0, 0, 1024, 2), db0 = ptx::make_smem_desc(smem0 + 16384, 0, 1024, 2);
        uint32_t idesc;
        if (KIND == 0) idesc = make_idesc(2, 1, 1, 0, 0, 128, bn);
        else if (KIND == 1) idesc = make_idesc(1, 0, 0, 0, 0, 128, bn);
        else if (KIND == 2) idesc = make_idesc_block_scaled(0, 0, 0, 0, 128, bn);
        else idesc = make_idesc_block_scaled(1, 1, 0, 0, 128, bn);
        const long long t0 = clock64();
        for (int i = 0; i < iters; ++i) {
            if (ptx::elect_one()) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    if (KIND == 0) ptx::umma<ptx::MmaKind::kI8>(tmem, da0 + 2 * kk, db0 + 2 * kk, idesc, 1u);
                    else if (KIND == 1) ptx::umma<ptx::MmaKind::kF8F6F4>(tmem, da0 + 2 * kk, db0 + 2 * kk, idesc, 1u);
                    else if (KIND == 2) ptx::umma_mxf8f6f4(tmem, da0 + 2 * kk, db0 + 2 * kk, idesc | (kk << 29) | (kk << 4), tmem + 300, tmem + 320, 1u);
                    else ptx::umma_mxf4(tmem, da0 + 2 * kk, db0 + 2 * kk, idesc | ((kk & 1) * 2 << 29) | ((kk & 1) * 2 << 4), tmem + 300, tmem + 320, 1u);
                }
            }
            __syncwarp();
        }
        if (ptx::elect_one()) ptx::umma_commit(&done);
        __syncwarp();
        bool ok = false;
        for (uint32_t it = 0; it < 50u * 1000u * 1000u && !ok; ++it) ok = ptx::mbar_try_wait(&done, 0);
        if (lane == 0) {
            out[blockIdx.x] = clock64() - t0;
            if (!ok) atomicExch(status, 1u);
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) ptx::tmem_dealloc(tmem, 512);
}

template <int NI, int NH, int NM>
__global__ void __launch_bounds__(256) pipe_mix_kernel(int iters, uint32_t c0, uint32_t c1, float* sink, long long* cyc)
{
    uint32_t ri[16], rh[16];
    float d[8][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        ri[i] = threadIdx.x + i + c0;
        rh[i] = 0x3F803F80u + i;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) d[i][0] = d[i][1] = d[i][2] = d[i][3] = 0.f;
    const uint32_t a[4] = {c0, c0 + 1, c0 + 2, c0 + 3};
    __syncthreads();
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {  // one eighth of a k-step's instructions per pass, interleaved
#pragma unroll
            for (int i = 0; i < NI / 8; ++i) asm volatile("lop3.b32 %0, %0, %1, %2, 0x6A;" : "+r"(ri[(u * (NI / 8) + i) & 15]) : "r"(c0), "r"(c1));
#pragma unroll
            for (int i = 0; i < NH / 8; ++i) asm volatile("add.rn.bf16x2 %0, %0, %1;" : "+r"(rh[(u * (NH / 8) + i) & 15]) : "r"(c1));
            if (u < NM)
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(d[u][0]), "+f"(d[u][1]), "+f"(d[u][2]), "+f"(d[u][3])
                             : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(rh[u]), "r"(rh[u + 8]));
        }
    }
    __syncthreads();
    const long long t1 = clock64();
    float s = 0.f;
    uint32_t x = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += d[i][0] + d[i][1] + d[i][2] + d[i][3];
#pragma unroll
    for (int i = 0; i < 16; ++i) x ^= ri[i] ^ rh[i];
    if (s == 1.2345f || x == 0x12345678u) sink[0] = s + x;
    if (threadIdx.x == 0) cyc[blockIdx.x] = t1 - t0;
}

long long max_of(const long long* dev, int n)
{
    long long h[1024], m = 0;
    cudaMemcpy(h, dev, (size_t)n * sizeof(long long), cudaMemcpyDeviceToHost);
    for (int i = 0; i < n; ++i) m = h[i] > m ? h[i] : m;
    return m;
}


// TMEM -> register read rate. `warps` warps (4 or 8; warp w reads lane quarter w % 4, column half w / 4 when there are 8) each read
// 128 columns of their 32 lanes per iteration, 2000 times, in one of these forms:
//   0: 32x32b.x16, wait after every load        1: 32x32b.x32, wait after every load      2: 32x32b.x64, wait after every load
//   3: two 32x32b.x16 in flight per wait        4: 16x256b.x8 (16 lanes x 64 columns), two per wait (both lane halves)
//   5: four 32x32b.x32 in flight per wait (all 128 columns)
// Contents of TMEM are whatever the allocation holds; the values only feed an xor that keeps the loads alive.
template <int FORM>
__global__ void __launch_bounds__(256) tmem_read_kernel(int iters, long long* out, uint32_t* sink)
{
    __shared__ uint32_t tmem_ptr;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    if (warp == 0) ptx::tmem_alloc(&tmem_ptr, 512);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t base = tmem_ptr + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)((warp >> 2) * 128);
    uint32_t x = 0;
    __syncthreads();
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
        const uint32_t b = base + (uint32_t)((it & 1) * 256);
        if (FORM == 0) {
#pragma unroll
            for (int c = 0; c < 128; c += 16) {
                uint32_t v[16];
                ptx::tmem_ld16(b + c, v);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) x ^= v[i];
            }
        } else if (FORM == 1 || FORM == 5) {
            uint32_t v[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                ptx::tmem_ld32(b + c * 32, v[c]);
                if (FORM == 1) ptx::tmem_ld_wait();
            }
            if (FORM == 5) ptx::tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) x ^= v[c][i];
        } else if (FORM == 2) {
#pragma unroll
            for (int c = 0; c < 128; c += 64) {
                uint32_t v[64];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, "
                    "%27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, "
                    "%52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                      "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                      "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                      "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]), "=r"(v[32]), "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]),
                      "=r"(v[37]), "=r"(v[38]), "=r"(v[39]), "=r"(v[40]), "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]),
                      "=r"(v[46]), "=r"(v[47]), "=r"(v[48]), "=r"(v[49]), "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]),
                      "=r"(v[55]), "=r"(v[56]), "=r"(v[57]), "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
                    : "r"(b + c)
                    : "memory");
                ptx::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 64; ++i) x ^= v[i];
            }
        } else if (FORM == 3) {
#pragma unroll
            for (int c = 0; c < 128; c += 32) {
                uint32_t v[16], w[16];
                ptx::tmem_ld16(b + c, v);
                ptx::tmem_ld16(b + c + 16, w);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) x ^= v[i] ^ w[i];
            }
        } else {
#pragma unroll
            for (int c = 0; c < 128; c += 64) {
                uint32_t v[2][32];
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    asm volatile(
                        "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, "
                        "%26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(v[h][0]), "=r"(v[h][1]), "=r"(v[h][2]), "=r"(v[h][3]), "=r"(v[h][4]), "=r"(v[h][5]), "=r"(v[h][6]), "=r"(v[h][7]),
                          "=r"(v[h][8]), "=r"(v[h][9]), "=r"(v[h][10]), "=r"(v[h][11]), "=r"(v[h][12]), "=r"(v[h][13]), "=r"(v[h][14]),
                          "=r"(v[h][15]), "=r"(v[h][16]), "=r"(v[h][17]), "=r"(v[h][18]), "=r"(v[h][19]), "=r"(v[h][20]), "=r"(v[h][21]),
                          "=r"(v[h][22]), "=r"(v[h][23]), "=r"(v[h][24]), "=r"(v[h][25]), "=r"(v[h][26]), "=r"(v[h][27]), "=r"(v[h][28]),
                          "=r"(v[h][29]), "=r"(v[h][30]), "=r"(v[h][31])
                        : "r"(b + c + ((uint32_t)(h * 16) << 16))
                        : "memory");
                ptx::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) x ^= v[0][i] ^ v[1][i];
            }
        }
    }
    const long long t1 = clock64();
    if (lane == 0) atomicMax(reinterpret_cast<unsigned long long*>(out + blockIdx.x), (unsigned long long)(t1 - t0));
    if (x == 0x12345678u) sink[0] = x;
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) ptx::tmem_dealloc(tmem_ptr, 512);
    (void)nwarps;
}

template <int KIND>
cudaError_t run_umma(int iters, uint32_t bn, int grid, long long* out, unsigned int* status)
{
    cudaError_t rc = cudaFuncSetAttribute(umma_rate_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
    if (rc != cudaSuccess) return rc;
    for (int rep = 0; rep < 2; ++rep) umma_rate_kernel<KIND><<<grid, 64, 65536>>>(iters, bn, out, status);
    return cudaDeviceSynchronize();
}

template <int NI, int NH, int NM>
cudaError_t run_mix(int iters, int grid, float* sink, long long* cyc)
{
    pipe_mix_kernel<NI, NH, NM><<<grid, 256>>>(16, 0x3F803F80u, 0x3C003C00u, sink, cyc);
    pipe_mix_kernel<NI, NH, NM><<<grid, 256>>>(iters, 0x3F803F80u, 0x3C003C00u, sink, cyc);
    return cudaDeviceSynchronize();
}

}  // namespace
}  // namespace opsnn

using namespace opsnn;

// kind 0 i8 | 1 f8f6f4 | 2 mxf8f6f4 | 3 mxf4; bn 128 | 224 | 256 (224 only for the block-scaled kinds' tile). Writes the clocks per
// MMA of the slowest SM (all SMs issue at once). Synchronises the device; allocates and frees a few KB of device memory (a probe).
extern "C" __attribute__((visibility("default"))) int32_t opsnn_probe_umma(int32_t kind, int32_t bn, double* clocks_per_mma)
{
    if (clocks_per_mma == nullptr || kind < 0 || kind > 3 || (bn != 128 && bn != 224 && bn != 256)) return (int32_t)cudaErrorInvalidValue;
    const int grid = current_sm_count() < 1024 ? current_sm_count() : 1024, iters = 2000;
    long long* out = nullptr;
    unsigned int* status = nullptr;
    cudaError_t rc = cudaMalloc(&out, 1024 * sizeof(long long));
    if (rc == cudaSuccess) rc = cudaMalloc(&status, sizeof(unsigned int));
    if (rc != cudaSuccess) return (int32_t)rc;
    cudaMemset(status, 0, sizeof(unsigned int));
    switch (kind) {
        case 0: rc = run_umma<0>(iters, (uint32_t)bn, grid, out, status); break;
        case 1: rc = run_umma<1>(iters, (uint32_t)bn, grid, out, status); break;
        case 2: rc = run_umma<2>(iters, (uint32_t)bn, grid, out, status); break;
        default: rc = run_umma<3>(iters, (uint32_t)bn, grid, out, status); break;
    }
    unsigned int st = 0;
    if (rc == cudaSuccess) {
        cudaMemcpy(&st, status, sizeof(st), cudaMemcpyDeviceToHost);
        *clocks_per_mma = (double)max_of(out, grid) / iters / 4.0;
    }
    cudaFree(out);
    cudaFree(status);
    if (rc == cudaSuccess && st != 0) return (int32_t)cudaErrorLaunchFailure;
    return (int32_t)rc;
}

// mix 0 integer only | 1 16-bit-pair arithmetic only | 2 mma.sync only | 3 the default decode arithmetic's mix (32 + 48 + 8 per k-step) |
// 4 the group-wise arithmetic's mix (32 + 8 + 8). Sixteen warps per SM, as in the decode kernels. Writes clocks per k-step per scheduler.
extern "C" __attribute__((visibility("default"))) int32_t opsnn_probe_mix(int32_t mix, double* clocks_per_kstep)
{
    if (clocks_per_kstep == nullptr || mix < 0 || mix > 4) return (int32_t)cudaErrorInvalidValue;
    const int sms = current_sm_count() < 512 ? current_sm_count() : 512, grid = sms * 2, iters = 2000;
    long long* cyc = nullptr;
    float* sink = nullptr;
    cudaError_t rc = cudaMalloc(&cyc, 1024 * sizeof(long long));
    if (rc == cudaSuccess) rc = cudaMalloc(&sink, 64);
    if (rc != cudaSuccess) return (int32_t)rc;
    switch (mix) {
        case 0: rc = run_mix<32, 0, 0>(iters, grid, sink, cyc); break;
        case 1: rc = run_mix<0, 48, 0>(iters, grid, sink, cyc); break;
        case 2: rc = run_mix<0, 0, 8>(iters, grid, sink, cyc); break;
        case 3: rc = run_mix<32, 48, 8>(iters, grid, sink, cyc); break;
        default: rc = run_mix<32, 8, 8>(iters, grid, sink, cyc); break;
    }
    if (rc == cudaSuccess) *clocks_per_kstep = (double)max_of(cyc, grid) / iters / 4.0;  // 16 warps per SM = 4 per scheduler
    cudaFree(cyc);
    cudaFree(sink);
    return (int32_t)rc;
}

// form: see tmem_read_kernel; warps 4 or 8. One CTA per SM, all SMs at once. Writes the bytes a whole SM reads from TMEM per clock.
extern "C" __attribute__((visibility("default"))) int32_t opsnn_probe_tmem_read(int32_t form, int32_t warps, double* bytes_per_clock)
{
    if (bytes_per_clock == nullptr || form < 0 || form > 5 || (warps != 4 && warps != 8)) return (int32_t)cudaErrorInvalidValue;
    const int grid = current_sm_count() < 1024 ? current_sm_count() : 1024, iters = 2000;
    long long* out = nullptr;
    uint32_t* sink = nullptr;
    cudaError_t rc = cudaMalloc(&out, 1024 * sizeof(long long));
    if (rc == cudaSuccess) rc = cudaMalloc(&sink, 64);
    if (rc != cudaSuccess) return (int32_t)rc;
    for (int rep = 0; rep < 2 && rc == cudaSuccess; ++rep) {
        cudaMemset(out, 0, 1024 * sizeof(long long));
        switch (form) {
            case 0: tmem_read_kernel<0><<<grid, warps * 32>>>(iters, out, sink); break;
            case 1: tmem_read_kernel<1><<<grid, warps * 32>>>(iters, out, sink); break;
            case 2: tmem_read_kernel<2><<<grid, warps * 32>>>(iters, out, sink); break;
            case 3: tmem_read_kernel<3><<<grid, warps * 32>>>(iters, out, sink); break;
            case 4: tmem_read_kernel<4><<<grid, warps * 32>>>(iters, out, sink); break;
            default: tmem_read_kernel<5><<<grid, warps * 32>>>(iters, out, sink); break;
        }
        rc = cudaDeviceSynchronize();
    }
    if (rc == cudaSuccess) *bytes_per_clock = (double)warps * 32.0 * 128.0 * 4.0 * iters / (double)max_of(out, grid);
    cudaFree(out);
    cudaFree(sink);
    return (int32_t)rc;
}
