// FRACTAL_NZ weight -> row-major (aclnnWeightQuantBatchMatmulNz). The fractal layout stores the (k, n) matrix as
// [ceil(n / n0)][ceil(k / k0)][k0][n0] elements (nz_to_nd of matmul/common/tests/st/arch35/matmul_golden_util.py:76-114 in the
// reference): it feeds the Ascend cube unit and has no use here, so the weight is copied once per call into the head of the
// workspace as plain (k, n) and the row-major kernels run on it. Pure copy: runs of n0 elements are contiguous on both sides.
#include "common.cuh"

namespace opsnn {

namespace {

// One thread moves `piece` bytes (16 when n0's byte length, the row length and both addresses allow it, else 1).
template <typename T>
__global__ void __launch_bounds__(256) nz_to_nd_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t k, int64_t n_bytes,
                                                       int64_t k0, int64_t n0_bytes, int64_t k1)
{
    const int64_t per_row = n_bytes / (int64_t)sizeof(T), total = k * per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t kk = i / per_row, nb = (i % per_row) * (int64_t)sizeof(T);  // row, byte column
        const int64_t blk = nb / n0_bytes, in_blk = nb % n0_bytes;
        const int64_t off = ((blk * k1 + kk / k0) * k0 + kk % k0) * n0_bytes + in_blk;
        *reinterpret_cast<T*>(dst + kk * n_bytes + nb) = *reinterpret_cast<const T*>(src + off);
    }
}

}  // namespace

uint64_t wq_nz_bytes(const OpsnnWqbmmParams* p)
{
    if (p->nz_k0 == 0) return 0;
    const int bits = p->w_dtype == ACL_INT8 ? 8 : 4;
    return (((uint64_t)p->k * (uint64_t)p->n * bits / 8) + 255u) & ~(uint64_t)255u;
}

// The row-major problem the copy leaves behind.
void wq_nz_view(const OpsnnWqbmmParams* p, OpsnnWqbmmParams* q, void* dst)
{
    *q = *p;
    const uint64_t used = wq_nz_bytes(p);
    q->w = dst;
    q->w_ld = p->n;
    q->trans_w = 0;
    q->nz_k0 = q->nz_n0 = 0;
    q->workspace = dst == nullptr ? nullptr : static_cast<uint8_t*>(dst) + used;
    q->workspace_size = p->workspace_size > used ? p->workspace_size - used : 0;
}

int32_t wq_nz_launch(const OpsnnWqbmmParams* p, void* dst, cudaStream_t stream)
{
    const int bits = p->w_dtype == ACL_INT8 ? 8 : 4;
    if ((p->w_dtype != ACL_INT8 && p->w_dtype != ACL_INT4) || p->nz_k0 <= 0 || p->nz_n0 <= 0) return (int32_t)cudaErrorInvalidValue;
    if ((p->n * bits) % 8 != 0 || (p->nz_n0 * bits) % 8 != 0) return (int32_t)cudaErrorInvalidValue;
    const int64_t n_bytes = p->n * bits / 8, n0_bytes = (int64_t)p->nz_n0 * bits / 8, k1 = (p->k + p->nz_k0 - 1) / p->nz_k0;
    const bool wide = n_bytes % 16 == 0 && n0_bytes % 16 == 0 && ((reinterpret_cast<uintptr_t>(p->w) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
    const int64_t work = p->k * (wide ? n_bytes / 16 : n_bytes);
    if (work == 0) return 0;
    int64_t grid = (work + 255) / 256;
    if (grid > 148 * 32) grid = 148 * 32;
    const uint8_t* src = static_cast<const uint8_t*>(p->w);
    if (wide) nz_to_nd_kernel<uint4><<<(unsigned)grid, 256, 0, stream>>>(src, static_cast<uint8_t*>(dst), p->k, n_bytes, p->nz_k0, n0_bytes, k1);
    else nz_to_nd_kernel<uint8_t><<<(unsigned)grid, 256, 0, stream>>>(src, static_cast<uint8_t*>(dst), p->k, n_bytes, p->nz_k0, n0_bytes, k1);
    note_launch("nz_to_nd");
    return (int32_t)cudaGetLastError();
}

}  // namespace opsnn

// Any 2-D byte matrix stored FRACTAL_NZ, [ceil(row_bytes / c0_bytes)][ceil(rows / r0)][r0][c0_bytes], -> row-major (rows, row_bytes).
extern "C" __attribute__((visibility("default"))) int32_t opsnn_nz_to_nd_launch(const void* src, void* dst, int64_t rows, int64_t row_bytes,
                                                                                int64_t r0, int64_t c0_bytes, void* stream)
{
    using namespace opsnn;
    if (src == nullptr || dst == nullptr || rows < 0 || row_bytes < 0 || r0 <= 0 || c0_bytes <= 0) return (int32_t)cudaErrorInvalidValue;
    const int64_t r1 = (rows + r0 - 1) / r0;
    const bool wide = row_bytes % 16 == 0 && c0_bytes % 16 == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
    const int64_t work = rows * (wide ? row_bytes / 16 : row_bytes);
    if (work == 0) return 0;
    int64_t grid = (work + 255) / 256;
    if (grid > 148 * 32) grid = 148 * 32;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (wide) nz_to_nd_kernel<uint4><<<(unsigned)grid, 256, 0, s>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), rows, row_bytes, r0, c0_bytes, r1);
    else nz_to_nd_kernel<uint8_t><<<(unsigned)grid, 256, 0, s>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), rows, row_bytes, r0, c0_bytes, r1);
    note_launch("nz_to_nd");
    return (int32_t)cudaGetLastError();
}
