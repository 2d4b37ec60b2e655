/*
 * Thin C-ABI launch layer between the C++ host code (validation, plan, tile selection) and the CUDA kernels.
 *
 * Plain pointers and sizes only. Every launcher enqueues on `stream` (a cudaStream_t passed as void*), never
 * synchronises, never allocates, and returns 0 or a cudaError_t value. All pointers are device pointers.
 * There is no CPU implementation behind any of these: without a CUDA device they return an error.
 *
 * The aclnn entry points (include/aclnnop/) are the public surface; these are what they call in phase 2, and they
 * are exported so that a host written in another language can bind the kernels directly.
 */
#ifndef OPSNN_B200_KERNELS_H_
#define OPSNN_B200_KERNELS_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OPSNN_API __attribute__((visibility("default")))

/* Element type codes = aclDataType values (include/aclnn_compat/acl_base.h). */

/* ---- full-quant matmul (aclnnQuantMatmulV5 path) --------------------------------------------------------- */

typedef enum {
    OPSNN_QMM_DEQ = 0,      /* int8 (or fp8 with fp32 scales): out = f32(acc [+ibias]) * sB[n|0] [* sA[m|0]] [+ fbias] */
    OPSNN_QMM_PERBLOCK = 1, /* out = sum_kb part_kb * (sA[m/gm,kb] * sB[kb,n/gn]), fp32 */
    OPSNN_QMM_MX = 2,       /* e8m0 scale per 32 along k on both operands, + fp32 bias */
    OPSNN_QMM_PERGROUP_ASYM = 3 /* INT4 x INT4 asymmetric per-group (qbmmv4_kernel_golden.py:328-395):
                                  out = sA[m] * sum_g (part_g - rowsum_g(a)[m] * b_offset[g,n]) * sB[g,n], g = group_k rows of k */
} OpsnnQmmMode;

/* The reference's fixpipe keeps only the top 19 bits of some fp32 scales
 * (matmul/common/tests/st/arch35/matmul_quant_util.py:50-72, qbmmv3_kernel_golden.py:435-443). */
#define OPSNN_DEQ_TRUNC_SCALE_B 1 /* x2Scale &= 0xFFFFE000 before use */
#define OPSNN_DEQ_MERGE_TRUNC 2   /* (x2Scale * x1Scale) &= 0xFFFFE000, one multiply */
#define OPSNN_DEQ_FBIAS_BEFORE_SCALE 4 /* a float bias is added to the fp32 accumulator before the scale multiply */
#define OPSNN_DEQ_REQUANT 8        /* INT8 out (qbmmv3_kernel_golden.py:465-487): clip(rint(acc * scale), -256, 255), then clip to int8 */
#define OPSNN_DEQ_REQUANT_OFFSET 16 /* with REQUANT: add the signed 9-bit offset held in bits 37..45 of the packed UINT64 scale */

typedef enum {
    OPSNN_KERNEL_AUTO = 0,    /* host tile selection decides */
    OPSNN_KERNEL_GENERIC = 1, /* CUDA-core kernel: any shape, stride and transpose */
    OPSNN_KERNEL_UMMA = 2     /* TMA + tcgen05 kernel: needs 16-byte aligned rows */
} OpsnnKernelChoice;

typedef struct OpsnnQmmParams {
    int32_t mode;
    int32_t a_dtype, b_dtype, out_dtype;
    int32_t bias_dtype;     /* ACL_DT_UNDEFINED (-1) when bias == NULL */
    int32_t scale_b_dtype;  /* ACL_FLOAT, ACL_BF16, ACL_UINT64 (packed: low 32 bits & 0xFFFFE000 is the fp32 scale), ACL_FLOAT8_E8M0 */
    int32_t trans_a;        /* 0: a is (m,k) row-major; 1: a is stored (k,m) */
    int32_t trans_b;        /* 0: b is (k,n) row-major; 1: b is stored (n,k) */
    int64_t batch, m, n, k;
    const void* a;
    const void* b;
    int64_t a_ld, b_ld;     /* elements between consecutive stored rows */
    int64_t a_bs, b_bs;     /* elements between batches; 0 broadcasts the operand over the batch */
    const void* scale_a;    /* x1Scale: NULL | fp32 (m,) or (1,) | fp32 per-block | e8m0 */
    const void* scale_b;    /* x2Scale */
    int64_t scale_a_len;    /* DEQ: 1 or m */
    int64_t scale_b_len;    /* DEQ: 1 or n */
    int64_t sa_bs, sb_bs;   /* elements between batches of the scales (PERBLOCK / MX); 0 broadcasts */
    int32_t group_m, group_n, group_k; /* PERBLOCK: 1|128,128,128; MX: 1,1,32 */
    int32_t deq_flags;      /* DEQ only: OPSNN_DEQ_* bits */
    const void* bias;
    int64_t bias_bs;        /* 0: (n,) shared by all batches; n: (batch,1,n) */
    void* out;
    int64_t out_ld, out_bs;
    void* workspace;
    uint64_t workspace_size;
    /* A8W4 (fp8 x fp4, aclnn_quant_matmul_v5.cpp:193-243): b is FLOAT4_E2M1 and is rewritten as fp8 into the head of
       the workspace before the matmul runs on it.
       OPSNN_B_PREPASS_WIDEN: every e2m1 value as the same value in e4m3 (exact); the mx scales apply unchanged.
       OPSNN_B_PREPASS_GROUP_SCALE: T-CG of qbmmv4_kernel_golden.py:189-255: value * pre_scale[group] rounded to
       pre_scale_dtype (BF16 | FLOAT16), then rounded to a_dtype; pre_scale is stored like b with one entry per
       pre_group elements of k: (n, k/pre_group) for b (n,k), (k/pre_group, n) for b (k,n). */
    int32_t b_prepass;
    int32_t pre_scale_dtype;
    const void* pre_scale;
    int32_t pre_group;
    /* INT4 x INT4 (per-tensor / per-channel / per-token modes): OPSNN_PREPASS_WIDEN_INT4 in a_prepass and b_prepass
       sign-extends the packed nibbles of that operand to INT8 in the workspace (exact), then the INT8 kernels run. */
    int32_t a_prepass;
    const void* b_offset;   /* PERGROUP_ASYM: x2Offset (k/group_k, n), FLOAT16 */
    /* MX mode, x2 prepared once by opsnn_qmm_prepare_b_launch (all three zero: nothing prepared, every call does its own layout work):
       prep_b   x2 rewritten k-contiguous (n,k) for all batches (used instead of b, which stays the caller's tensor), or NULL when x2
                is already stored (n,k);
       prep_sfb x2Scale in the tensor core's scale-atom order, laid out for tiles of prep_bn columns; ignored (the call relays the
                scales itself) when host tile selection picks another width for this call's m. */
    const void* prep_b;
    const void* prep_sfb;
    int32_t prep_bn;
} OpsnnQmmParams;

enum { OPSNN_B_PREPASS_NONE = 0, OPSNN_B_PREPASS_WIDEN = 1, OPSNN_B_PREPASS_GROUP_SCALE = 2, OPSNN_PREPASS_WIDEN_INT4 = 3 };

/* Bytes of device workspace `opsnn_qmm_launch` needs for these parameters with this kernel choice. */
OPSNN_API uint64_t opsnn_qmm_workspace_size(const OpsnnQmmParams* p, int32_t kernel_choice);
/* Returns the OpsnnKernelChoice the host tile selection resolves AUTO to (never AUTO). */
OPSNN_API int32_t opsnn_qmm_select_kernel(const OpsnnQmmParams* p);
OPSNN_API int32_t opsnn_qmm_launch(const OpsnnQmmParams* p, int32_t kernel_choice, void* stream);

/* Prepare-once form of a static x2 (a weight) for the MX modes. The layout work that does not depend on x1 - x2Scale into scale-atom
 * order, and x2 stored (k,n) rewritten k-contiguous (fp4 must be, fp8 runs faster so) - is done one time into caller memory
 * `storage` (opsnn_qmm_prepare_b_size bytes; the library allocates nothing) and described by three values to put into prep_b /
 * prep_sfb / prep_bn of later calls on the same x2. p describes a representative call: its m and batch select the tile width the
 * scale atoms are laid out for; x1, x1Scale and out are not touched. Returns 0 and leaves *prep_bn = 0 when p's mode or layout has
 * nothing to prepare. The reference's precedent for offline weight re-layout is aclnnConvertWeightToINT4Pack
 * (matmul/convert_weight_to_int4_pack/op_host/op_api/aclnn_convert_weight_to_int4_pack.cpp:318-358, ND -> NZ). */
OPSNN_API uint64_t opsnn_qmm_prepare_b_size(const OpsnnQmmParams* p);
OPSNN_API int32_t opsnn_qmm_prepare_b_launch(const OpsnnQmmParams* p, void* storage, uint64_t storage_size, const void** prep_b,
                                             const void** prep_sfb, int32_t* prep_bn, void* stream);

/* ---- weight-only quant matmul (aclnnWeightQuantBatchMatmulV2/V3 path) ------------------------------------ */

typedef enum {
    OPSNN_WQ_KERNEL_AUTO = 0,
    OPSNN_WQ_KERNEL_GENERIC = 1, /* coverage kernel: any layout and stride, dequantisation fused, CUDA-core fp32 products */
    OPSNN_WQ_KERNEL_DECODE = 2,  /* fused streaming kernel for small m: int4 (n-packed) per-group/-channel; reproduces
                                    the reference's two roundings per dequantised weight */
    OPSNN_WQ_KERNEL_DECODE_FAST = 3, /* same regime, "high performance" precision mode (inner_precise = 1): scale and
                                    offset applied per k-group after the MMA in fp32; not bit-identical to DECODE */
    OPSNN_WQ_KERNEL_PREFILL = 4  /* m beyond the decode range: the weight is dequantised (the reference's two roundings)
                                    into workspace as (n,k) in x's dtype, then a tcgen05 bf16/fp16 matmul */
} OpsnnWqKernelChoice;

typedef struct OpsnnWqbmmParams {
    int32_t x_dtype;        /* ACL_BF16 | ACL_FLOAT16; y has the same dtype */
    int32_t w_dtype;        /* ACL_INT4 / ACL_FLOAT4_E2M1 (packed nibbles, low first, along the stored inner axis) | ACL_INT8 |
                               ACL_FLOAT8_E4M3FN | ACL_FLOAT8_E5M2 */
    int32_t bias_dtype;     /* -1 | x_dtype | ACL_FLOAT */
    int32_t trans_w;        /* 0: weight stored (k,n); 1: stored (n,k) */
    int64_t m, n, k;
    const void* x;          /* (m,k) row-major, x_ld elements per row */
    int64_t x_ld;
    const void* w;
    int64_t w_ld;           /* elements (int4 count for ACL_INT4) between consecutive stored rows */
    const void* scale;      /* x_dtype */
    const void* offset;     /* x_dtype or NULL */
    int64_t group_size;     /* 0: per-channel/-tensor; else k-group length */
    int64_t scale_sg;       /* elements between consecutive k-groups of scale/offset (0 when group_size == 0) */
    int64_t scale_sn;       /* elements between consecutive n of scale/offset (0: per-tensor) */
    const void* bias;
    void* y;
    int64_t y_ld;
    void* workspace;
    uint64_t workspace_size;
    int32_t inner_precise;  /* innerPrecise of aclnnWeightQuantBatchMatmulV3: 0 high precision (default), 1 high performance */
    /* aclnnWeightQuantBatchMatmulNz: the (k,n) weight is stored FRACTAL_NZ, [ceil(n/nz_n0)][ceil(k/nz_k0)][nz_k0][nz_n0] elements
       (matmul/common/tests/st/arch35/matmul_golden_util.py:76-114 of the reference). 0, 0: plain row-major storage. It is
       rewritten row-major into the head of the workspace before the matmul runs. */
    int32_t nz_k0, nz_n0;
    int32_t scale_dtype;    /* 0 or x_dtype: scale in x's dtype; ACL_FLOAT8_E8M0: mx antiquant (group_size 32, no offset) */
    /* Optional: the weight as the prefill path would dequantise it (opsnn_wqbmm_prepare_launch wrote it, once, into caller
       memory). With it set, calls on the prefill path (m > 16) skip the dequantisation pre-pass and need no workspace; results
       are identical. Ignored by the decode kernels, which stream the packed weight. */
    const void* prep_w;
} OpsnnWqbmmParams;

OPSNN_API uint64_t opsnn_wqbmm_workspace_size(const OpsnnWqbmmParams* p, int32_t kernel_choice);
/* Prepare-once form of the prefill path's weight: bytes of caller storage (0: this weight / layout has no prefill path), and the
 * pre-pass alone, writing the dequantised 16-bit weight of p (x_dtype says bf16 or fp16) into `storage` (256-byte aligned). p->x, p->y
 * and p->m are not read. Afterwards set p->prep_w = storage in calls on the same weight, scale, offset and x dtype. */
OPSNN_API uint64_t opsnn_wqbmm_prepare_size(const OpsnnWqbmmParams* p);
OPSNN_API int32_t opsnn_wqbmm_prepare_launch(const OpsnnWqbmmParams* p, void* storage, uint64_t storage_size, void* stream);
OPSNN_API int32_t opsnn_wqbmm_select_kernel(const OpsnnWqbmmParams* p);
OPSNN_API int32_t opsnn_wqbmm_launch(const OpsnnWqbmmParams* p, int32_t kernel_choice, void* stream);

/* The decode kernel again, for callers that cannot hand over workspace and must not cause a device allocation at the
 * call: a hook running inside another runtime's memory-planned region, or a serving loop whose memory pool is frozen
 * after warm-up, where a cudaMalloc would either fail the plan or synchronise the device. This entry point has no
 * counterpart in the reference (there every operator gets its scratch through the two-phase workspace contract).
 *
 *   - The cross-CTA scratch is a 9,964,032-byte array inside the library's device image; p->workspace and
 *     p->workspace_size are ignored. Neither this function nor anything it calls allocates host-visible device memory.
 *   - Limits: the parameters must satisfy the decode kernel's range (opsnn_wqbmm_select_kernel(p) ==
 *     OPSNN_WQ_KERNEL_DECODE with inner_precise = 0; inner_precise is ignored here) and n <= 155,648 columns (304 CTAs x 512). Anything else returns cudaErrorInvalidValue
 *     and leaves the reason in aclGetRecentErrMsg().
 *   - The first call on each device (with that device current) resolves the array's address; this may load the
 *     library's device code. Make that first call during start-up, before any stream capture begins.
 *   - The array is shared by every call on the device and keeps its last contents. Nothing in it has to start at
 *     zero: each launch stamps its scratch with a fresh 64-bit nonce and clears its own stamps before it ends.
 *   - Two calls that overlap in time on one device (two streams, two threads) race on the array and give wrong
 *     results; order them on one stream or with events. The workspace entry point above has no such restriction.
 */
OPSNN_API int32_t opsnn_wqbmm_decode_static_launch(const OpsnnWqbmmParams* p, void* stream);

/* A 2-D byte matrix stored FRACTAL_NZ, [ceil(row_bytes / c0_bytes)][ceil(rows / r0)][r0][c0_bytes] (nz_to_nd of
 * matmul/common/tests/st/arch35/matmul_golden_util.py:76-114 in the reference), rewritten row-major (rows, row_bytes) into dst.
 * What aclnnWeightQuantBatchMatmulNz and aclnnQuantMatmulWeightNz run before their matmul. */
OPSNN_API int32_t opsnn_nz_to_nd_launch(const void* src, void* dst, int64_t rows, int64_t row_bytes, int64_t r0, int64_t c0_bytes,
                                        void* stream);

/* ---- dynamic MX quant (aclnnDynamicMxQuant path)---------------------------------------------------------- */

typedef struct OpsnnMxQuantParams {
    int32_t x_dtype;   /* ACL_BF16 | ACL_FLOAT16 */
    int32_t y_dtype;   /* ACL_FLOAT8_E4M3FN | ACL_FLOAT8_E5M2 | ACL_FLOAT4_E2M1 */
    int64_t rows, k;   /* x is (rows,k) contiguous; blocks of 32 along k */
    const void* x;
    void* y;           /* (rows,k) fp8, or (rows, k/2) bytes for fp4 */
    void* scale;       /* (rows, 2*ceil(ceil(k/32)/2)) e8m0 bytes */
    int64_t inner;     /* 0 or 1: blocks along the last axis. > 1: x is (rows, k, inner) contiguous with the blocks along k (a
                          non-last axis); y has x's shape (fp4 packed along inner, inner even), scale is
                          (rows, ceil(ceil(k/32)/2), inner, 2) with block b of a pair at [.., b / 2, i, b % 2] */
    int32_t scale_alg;  /* 0: OCP shared exponent floor(log2 amax) - emax; 1 (fp8 outputs): exponent of amax / max_norm rounded up
                           to a power of two (quant/dynamic_mx_quant/tests/assets/golden.py:157-177) */
    int32_t round_mode; /* fp4 outputs: 0 rint (ties to even), 1 round (ties away from zero), 2 floor; fp8 outputs: 0 */
} OpsnnMxQuantParams;

OPSNN_API int32_t opsnn_mx_quant_launch(const OpsnnMxQuantParams* p, void* stream);

/* ---- 4-bit weight packing (aclnnConvertWeightToINT4Pack path) --------------------------------------------------- */

typedef struct OpsnnPackB4Params {
    int32_t src_dtype;  /* ACL_INT32: one 4-bit integer per word (low nibble used) | ACL_FLOAT: one e2m1 value per float */
    int64_t count;      /* elements; even */
    const void* src;    /* contiguous */
    void* dst;          /* count / 2 bytes: element 2i in the low nibble of byte i, element 2i+1 in the high nibble */
} OpsnnPackB4Params;

OPSNN_API int32_t opsnn_pack_b4_launch(const OpsnnPackB4Params* p, void* stream);

/* ---- misc ---------------------------------------------------------------------------------------------------- */

/* Number of kernel launches issued through this library since load (all streams, all threads). */
OPSNN_API uint64_t opsnn_launch_count(void);
/* Name of the last kernel family launched on the calling thread (static string; "" if none). */
OPSNN_API const char* opsnn_last_kernel_name(void);
/* Error word of the tensor-core (tcgen05) quant matmul kernels on the current device: 0 when every bounded wait
 * inside them completed; otherwise the code of the first wait that gave up (the kernel then returned early and its
 * output is undefined). Synchronises the device. reset != 0 clears the word after reading it.
 * The same condition also reaches the caller without polling: the word is mirrored into pinned host memory, and every later
 * tensor-core launch of the process (opsnn_qmm_launch, and through it aclnnQuantMatmulV3/V4/V5 and the prefill path of
 * aclnnWeightQuantBatchMatmul*) first looks at the mirror and, while it is non-zero, refuses with cudaErrorLaunchFailure
 * (ACLNN_ERR_RUNTIME_ERROR at the aclnn level, reason in aclGetRecentErrMsg) until this function is called with reset != 0. */
OPSNN_API uint32_t opsnn_qmm_umma_status(int32_t reset);
/* The same for the streaming W4A16 decode kernel that feeds shared memory with bulk tensor copies: 0, or 1 (a stage of
 * operands never arrived) / 2 (a stage buffer was never released). Synchronises the device. */
OPSNN_API uint32_t opsnn_wqbmm_decode_status(int32_t reset);
/* How the calling thread's last streaming decode launch (W4A16 / W8A16, bulk-copy kernels) cut the problem: strips of 512
 * columns, k-ranges per strip, and whether the k-ranges of a strip ran as one thread-block cluster (summed over distributed
 * shared memory) or were summed through the workspace. Any pointer may be null. */
OPSNN_API void opsnn_wqbmm_decode_last_plan(int32_t* strips, int32_t* splits, int32_t* cluster);

/* ---- measured ceilings (diagnostics; not on any product path) --------------------------------------------------------------
 * opsnn_probe_umma: clocks per tcgen05.mma (128 x bn x 32 bytes of k) when one CTA per SM issues them back to back on operands
 * resident in shared memory; kind 0 i8, 1 f8f6f4, 2 mxf8f6f4, 3 mxf4; bn 128, 224 or 256. opsnn_probe_mix: clocks per k-step per
 * scheduler of the decode kernels' instruction mixes (0 integer only, 1 16-bit-pair arithmetic only, 2 mma.sync only, 3 default
 * arithmetic, 4 group-wise arithmetic). Both synchronise the device and use a few KB of their own device memory for the duration of
 * the call. opsnn_probe_tmem_read: bytes per clock a whole SM moves from tensor memory to registers with tcgen05.ld (form 0:
 * 32x32b.x16, 1: .x32, 2: .x64, each waited for; 3: two .x16 per wait; 4: 16x256b.x8, two per wait; 5: four 32x32b.x32 per wait;
 * warps 4 or 8) - the rate that bounds the per-block promotion. No counterpart in the reference. */
OPSNN_API int32_t opsnn_probe_umma(int32_t kind, int32_t bn, double* clocks_per_mma);
OPSNN_API int32_t opsnn_probe_mix(int32_t mix, double* clocks_per_kstep);
OPSNN_API int32_t opsnn_probe_tmem_read(int32_t form, int32_t warps, double* bytes_per_clock);

#ifdef __cplusplus
}
#endif
#endif /* OPSNN_B200_KERNELS_H_ */
