// C-ABI launch layer (include/opsnn_b200_kernels.h): host-side tile/kernel selection and dispatch.
//
// This is what is left of the reference's host tiling framework (common/inc/op_host/tiling_base.h:70-103: an ordered list
// of tiling templates, each with IsCapable(); the first capable one wins) once the target is a single GPU
// architecture: a capability test per kernel family, tried fastest first.
#include <atomic>
#include <cstdlib>

#include "common.cuh"

namespace opsnn {

void set_err(const char* fmt, ...);

static std::atomic<uint64_t> g_launches{0};
static thread_local const char* g_last_kernel = "";

void note_launch(const char* name, uint64_t n)
{
    g_launches.fetch_add(n, std::memory_order_relaxed);
    g_last_kernel = name;
}

static thread_local int32_t g_decode_plan[3] = {0, 0, 0};
void note_decode_plan(int64_t strips, int64_t splits, int32_t cluster)
{
    g_decode_plan[0] = (int32_t)strips;
    g_decode_plan[1] = (int32_t)splits;
    g_decode_plan[2] = cluster;
}

int32_t qmm_generic_launch(const OpsnnQmmParams* p, cudaStream_t stream);
bool qmm_umma_eligible(const OpsnnQmmParams* p);
uint64_t qmm_umma_workspace_size(const OpsnnQmmParams* p);
int32_t qmm_umma_launch(const OpsnnQmmParams* p, cudaStream_t stream);
uint64_t qmm_mx_prepare_b_size(const OpsnnQmmParams* p);
int32_t qmm_mx_prepare_b_launch(const OpsnnQmmParams* p, void* storage, uint64_t storage_size, const void** prep_b, const void** prep_sfb,
                                int32_t* prep_bn, cudaStream_t stream);
uint64_t qmm_a8w4_prepass_bytes(const OpsnnQmmParams* p);
void qmm_a8w4_view(const OpsnnQmmParams* p, OpsnnQmmParams* q, void* dst);
int32_t qmm_a8w4_prepass_launch(const OpsnnQmmParams* p, void* dst, cudaStream_t stream);
uint64_t qmm_int4_prepass_bytes(const OpsnnQmmParams* p);
void qmm_int4_view(const OpsnnQmmParams* p, OpsnnQmmParams* q, void* dst);
int32_t qmm_int4_prepass_launch(const OpsnnQmmParams* p, void* dst, cudaStream_t stream);

int32_t wqbmm_generic_launch(const OpsnnWqbmmParams* p, cudaStream_t stream);
bool wqbmm_decode_eligible(const OpsnnWqbmmParams* p);
uint64_t wqbmm_decode_workspace_size(const OpsnnWqbmmParams* p);
int32_t wqbmm_decode_launch(const OpsnnWqbmmParams* p, cudaStream_t stream);
bool wqbmm_decode_fast_eligible(const OpsnnWqbmmParams* p);
int32_t wqbmm_decode_fast_launch(const OpsnnWqbmmParams* p, cudaStream_t stream);
int32_t wqbmm_decode_ring_launch(const OpsnnWqbmmParams* p, cudaStream_t stream, bool exact);
bool wqbmm_decode_tma_eligible(const OpsnnWqbmmParams* p);
int32_t wqbmm_decode_tma_launch(const OpsnnWqbmmParams* p, cudaStream_t stream, bool exact);

// The streaming decode kernels that share one data layout condition, newest data path first: bulk tensor copies (TMA) into
// swizzled stages, else the per-warp cp.async ring. OPSNN_WQ_DECODE_PATH=ring forces the second.
static int32_t decode_stream_launch(const OpsnnWqbmmParams* p, cudaStream_t stream, bool exact)
{
    const char* e = getenv("OPSNN_WQ_DECODE_PATH");
    const bool ring_only = e != nullptr && e[0] == 'r';
    if (!ring_only && wqbmm_decode_tma_eligible(p)) return wqbmm_decode_tma_launch(p, stream, exact);
    return wqbmm_decode_ring_launch(p, stream, exact);
}

bool wqbmm_decode_tma_nk_eligible(const OpsnnWqbmmParams* p);
bool wqbmm_decode8_eligible(const OpsnnWqbmmParams* p);
int32_t wqbmm_decode8_launch(const OpsnnWqbmmParams* p, cudaStream_t stream);
bool wqbmm_prefill_eligible(const OpsnnWqbmmParams* p);
uint64_t wqbmm_prefill_workspace_size(const OpsnnWqbmmParams* p);
int32_t wqbmm_prefill_launch(const OpsnnWqbmmParams* p, cudaStream_t stream);
uint64_t wqbmm_prefill_image_size(const OpsnnWqbmmParams* p);
int32_t wqbmm_prefill_prepass(const OpsnnWqbmmParams* p, uint8_t* ws, cudaStream_t stream);

uint64_t wq_nz_bytes(const OpsnnWqbmmParams* p);
void wq_nz_view(const OpsnnWqbmmParams* p, OpsnnWqbmmParams* q, void* dst);
int32_t wq_nz_launch(const OpsnnWqbmmParams* p, void* dst, cudaStream_t stream);

int32_t mx_quant_launch(const OpsnnMxQuantParams* p, cudaStream_t stream);
int32_t pack_b4_launch(const OpsnnPackB4Params* p, cudaStream_t stream);

}  // namespace opsnn

using namespace opsnn;

extern "C" {

// A8W4: kernel selection and workspace are those of the fp8 problem the pre-pass leaves behind. For planning (no
// workspace yet) the rewritten operand is given a stand-in address with the alignment every device allocation has.
static const OpsnnQmmParams* after_prepass(const OpsnnQmmParams* p, OpsnnQmmParams* q, void* dst)
{
    if (p->a_prepass == OPSNN_PREPASS_WIDEN_INT4 || p->b_prepass == OPSNN_PREPASS_WIDEN_INT4) {
        qmm_int4_view(p, q, dst);
        return q;
    }
    if (p->b_prepass == OPSNN_B_PREPASS_NONE) return p;
    qmm_a8w4_view(p, q, dst);
    return q;
}

int32_t opsnn_qmm_select_kernel(const OpsnnQmmParams* p)
{
    if (p == nullptr) return OPSNN_KERNEL_GENERIC;
    OpsnnQmmParams q;
    p = after_prepass(p, &q, reinterpret_cast<void*>(uintptr_t(256)));
    return qmm_umma_eligible(p) ? OPSNN_KERNEL_UMMA : OPSNN_KERNEL_GENERIC;
}

uint64_t opsnn_qmm_workspace_size(const OpsnnQmmParams* p, int32_t kernel_choice)
{
    if (p == nullptr) return 0;
    if (kernel_choice == OPSNN_KERNEL_AUTO) kernel_choice = opsnn_qmm_select_kernel(p);
    const uint64_t pre = qmm_a8w4_prepass_bytes(p) + qmm_int4_prepass_bytes(p);
    OpsnnQmmParams q;
    p = after_prepass(p, &q, reinterpret_cast<void*>(uintptr_t(256)));
    return pre + (kernel_choice == OPSNN_KERNEL_UMMA ? qmm_umma_workspace_size(p) : 0);
}

// Only the plain MX modes have x1-independent layout work worth keeping: the A8W4 and INT4 forms rewrite x2 through their own
// pre-passes, the dequant and per-block modes feed x2 to the tensor core as stored.
static bool preparable(const OpsnnQmmParams* p)
{
    return p != nullptr && p->mode == OPSNN_QMM_MX && p->a_prepass == OPSNN_B_PREPASS_NONE && p->b_prepass == OPSNN_B_PREPASS_NONE &&
           p->b != nullptr && p->scale_b != nullptr && p->m > 0 && p->n > 0 && p->batch > 0;
}

uint64_t opsnn_qmm_prepare_b_size(const OpsnnQmmParams* p) { return preparable(p) ? qmm_mx_prepare_b_size(p) : 0; }

int32_t opsnn_qmm_prepare_b_launch(const OpsnnQmmParams* p, void* storage, uint64_t storage_size, const void** prep_b, const void** prep_sfb,
                                   int32_t* prep_bn, void* stream)
{
    if (prep_b == nullptr || prep_sfb == nullptr || prep_bn == nullptr) return (int32_t)cudaErrorInvalidValue;
    *prep_b = *prep_sfb = nullptr;
    *prep_bn = 0;
    if (!preparable(p)) return 0;
    return qmm_mx_prepare_b_launch(p, storage, storage_size, prep_b, prep_sfb, prep_bn, static_cast<cudaStream_t>(stream));
}

int32_t opsnn_qmm_launch(const OpsnnQmmParams* p, int32_t kernel_choice, void* stream)
{
    if (p == nullptr) return (int32_t)cudaErrorInvalidValue;
    if (p->m <= 0 || p->n <= 0 || p->batch <= 0) return 0;
    OpsnnQmmParams q;
    if (p->a_prepass != OPSNN_B_PREPASS_NONE || p->b_prepass != OPSNN_B_PREPASS_NONE) {
        const bool i4 = p->a_prepass == OPSNN_PREPASS_WIDEN_INT4 || p->b_prepass == OPSNN_PREPASS_WIDEN_INT4;
        if (p->workspace == nullptr || p->workspace_size < qmm_a8w4_prepass_bytes(p) + qmm_int4_prepass_bytes(p))
            return (int32_t)cudaErrorInvalidValue;
        const int32_t rc = i4 ? qmm_int4_prepass_launch(p, p->workspace, static_cast<cudaStream_t>(stream))
                              : qmm_a8w4_prepass_launch(p, p->workspace, static_cast<cudaStream_t>(stream));
        if (rc != 0) return rc;
        p = after_prepass(p, &q, p->workspace);
        if (kernel_choice == OPSNN_KERNEL_UMMA && !qmm_umma_eligible(p)) kernel_choice = OPSNN_KERNEL_GENERIC;  // odd workspace address
    }
    if (kernel_choice == OPSNN_KERNEL_AUTO) kernel_choice = opsnn_qmm_select_kernel(p);
    if (kernel_choice == OPSNN_KERNEL_UMMA) {
        if (!qmm_umma_eligible(p)) return (int32_t)cudaErrorInvalidValue;
        return qmm_umma_launch(p, static_cast<cudaStream_t>(stream));
    }
    return qmm_generic_launch(p, static_cast<cudaStream_t>(stream));
}

// 16 < m <= 48 against a large enough weight: the streaming decode kernel once per 16 rows of x (the weight is re-read from
// HBM for every chunk, 62 us each on the m16 k8192 n28672 shape) still beats dequantising the whole weight into workspace
// first (0.19 ms for that weight before the matmul starts).
static bool decode_in_chunks(const OpsnnWqbmmParams* p, OpsnnWqbmmParams* chunk)
{
    // Measured against dequantise-then-matmul (int4, bf16): 4096 x 4096 at m = 32 31 us against 38; 4096 x 14336 44 against 89 at
    // m = 32 and 63 against 89 at m = 48. Two launches pay from 2^24 weights on, three from 3 x 2^24.
    // OPSNN_WQ_CHUNK_MIN_LOG2 replaces both thresholds by 2^value (tuning).
    int64_t min_kn = (p->m <= 32 ? 1 : 3) * ((int64_t)1 << 24);
    if (const char* e = getenv("OPSNN_WQ_CHUNK_MIN_LOG2")) {
        const int v = atoi(e);
        if (v > 0 && v < 62) min_kn = (int64_t)1 << v;
    }
    if (p->m <= 16 || p->m > 48 || p->k * p->n < min_kn) return false;
    *chunk = *p;
    chunk->m = 16;
    if (wqbmm_decode_eligible(chunk)) return true;
    // the 8-bit kernels and the (n,k) int4 kernel the same way: three launches of 55-65 us still beat the 0.3 ms of
    // dequantise-then-matmul on such a weight
    if (wqbmm_decode8_eligible(chunk) && getenv("OPSNN_WQ_NO_DECODE8") == nullptr) return true;
    return wqbmm_decode_tma_nk_eligible(chunk) && getenv("OPSNN_WQ_NO_DECODE_NK") == nullptr;
}

// One decode launch per 16 rows; `fast` = the group-wise kernel of inner_precise = 1.
static int32_t decode_chunk_launches(const OpsnnWqbmmParams* p, cudaStream_t stream, int which)
{
    const size_t esz = 2;  // bf16 / fp16
    for (int64_t r0 = 0; r0 < p->m; r0 += 16) {
        OpsnnWqbmmParams q = *p;
        q.m = p->m - r0 < 16 ? p->m - r0 : 16;
        q.x = static_cast<const uint8_t*>(p->x) + (size_t)r0 * (size_t)p->x_ld * esz;
        q.y = static_cast<uint8_t*>(p->y) + (size_t)r0 * (size_t)p->y_ld * esz;
        int32_t rc;
        if (q.w_dtype == ACL_INT8 || q.w_dtype == ACL_FLOAT8_E4M3FN) rc = wqbmm_decode8_launch(&q, stream);
        else if (q.trans_w != 0) rc = wqbmm_decode_tma_launch(&q, stream, true);
        else if (which == OPSNN_WQ_KERNEL_DECODE_FAST) rc = decode_stream_launch(&q, stream, false);
        else if (wqbmm_decode_fast_eligible(&q) && getenv("OPSNN_WQ_DECODE_LEGACY") == nullptr) rc = decode_stream_launch(&q, stream, true);
        else rc = wqbmm_decode_launch(&q, stream);
        if (rc != 0) return rc;
    }
    return 0;
}

int32_t opsnn_wqbmm_select_kernel(const OpsnnWqbmmParams* p)
{
    if (p == nullptr) return OPSNN_WQ_KERNEL_GENERIC;
    OpsnnWqbmmParams nd;
    if (p->nz_k0 != 0) {  // FRACTAL_NZ weight: selection is that of the row-major copy (stand-in address with allocation alignment)
        wq_nz_view(p, &nd, reinterpret_cast<void*>(uintptr_t(256)));
        p = &nd;
    }
    if (p->inner_precise == 1 && wqbmm_decode_fast_eligible(p)) return OPSNN_WQ_KERNEL_DECODE_FAST;
    if (wqbmm_decode_eligible(p)) return OPSNN_WQ_KERNEL_DECODE;
    // 8-bit weights (int8, e4m3) at small m: their own streaming kernel once the weight is large enough to be worth a k-split grid
    if (wqbmm_decode8_eligible(p) && p->k * p->n >= ((int64_t)1 << 20) && getenv("OPSNN_WQ_NO_DECODE8") == nullptr) return OPSNN_WQ_KERNEL_DECODE;
    // 4-bit weights stored (n,k) at small m: the (n,k) form of the bulk-copy decode kernel, same threshold
    if (wqbmm_decode_tma_nk_eligible(p) && p->k * p->n >= ((int64_t)1 << 20) && getenv("OPSNN_WQ_NO_DECODE_NK") == nullptr) return OPSNN_WQ_KERNEL_DECODE;
    // a weight prepared for the prefill path (dequantised once, kept by the caller): beyond the decode range the tensor-core matmul
    // alone beats streaming the packed weight once per 16 rows
    if (p->prep_w != nullptr && p->m > 16 && wqbmm_prefill_eligible(p)) return OPSNN_WQ_KERNEL_PREFILL;
    OpsnnWqbmmParams chunk;
    if (getenv("OPSNN_WQ_NO_CHUNKS") == nullptr && decode_in_chunks(p, &chunk))
        return (p->inner_precise == 1 && wqbmm_decode_fast_eligible(&chunk)) ? OPSNN_WQ_KERNEL_DECODE_FAST : OPSNN_WQ_KERNEL_DECODE;
    // m beyond the decode range: dequantise once, multiply on the tensor cores; tiny problems stay on the one-launch coverage kernel
    // (also small m when no streaming decode kernel takes the layout - fp4 weights, unaligned pitches, odd group sizes - and the
    // weight is large: 0.95 ms against 4.7 ms of the coverage kernel for an 8-bit 8192 x 28672 weight at m = 16)
    if ((p->m > 16 || p->k * p->n >= ((int64_t)1 << 22)) && wqbmm_prefill_eligible(p)) return OPSNN_WQ_KERNEL_PREFILL;
    return OPSNN_WQ_KERNEL_GENERIC;
}

uint64_t opsnn_wqbmm_workspace_size(const OpsnnWqbmmParams* p, int32_t kernel_choice)
{
    if (p == nullptr) return 0;
    if (kernel_choice == OPSNN_WQ_KERNEL_AUTO) kernel_choice = opsnn_wqbmm_select_kernel(p);
    OpsnnWqbmmParams nd;
    if (p->nz_k0 != 0) {
        const uint64_t pre = wq_nz_bytes(p);
        wq_nz_view(p, &nd, reinterpret_cast<void*>(uintptr_t(256)));
        return pre + opsnn_wqbmm_workspace_size(&nd, kernel_choice);
    }
    if (kernel_choice == OPSNN_WQ_KERNEL_PREFILL) return wqbmm_prefill_workspace_size(p);
    return (kernel_choice == OPSNN_WQ_KERNEL_DECODE || kernel_choice == OPSNN_WQ_KERNEL_DECODE_FAST) ? wqbmm_decode_workspace_size(p) : 0;
}

// A stand-in view for the questions that do not depend on the activations (is there a prefill path for this weight, how large is
// its dequantised image): one aligned row of x.
static void prepare_view(const OpsnnWqbmmParams* p, OpsnnWqbmmParams* v)
{
    *v = *p;
    v->m = 32;
    v->x = reinterpret_cast<const void*>(uintptr_t(256));
    v->x_ld = (p->k + 7) / 8 * 8;
    v->y = reinterpret_cast<void*>(uintptr_t(256));
    v->y_ld = p->n;
    v->prep_w = nullptr;
}

uint64_t opsnn_wqbmm_prepare_size(const OpsnnWqbmmParams* p)
{
    if (p == nullptr || p->nz_k0 != 0 || p->n <= 0 || p->k <= 0) return 0;
    OpsnnWqbmmParams v;
    prepare_view(p, &v);
    return wqbmm_prefill_eligible(&v) ? wqbmm_prefill_image_size(&v) : 0;
}

int32_t opsnn_wqbmm_prepare_launch(const OpsnnWqbmmParams* p, void* storage, uint64_t storage_size, void* stream)
{
    const uint64_t need = opsnn_wqbmm_prepare_size(p);
    if (need == 0 || storage == nullptr || storage_size < need || (reinterpret_cast<uintptr_t>(storage) & 255) != 0 || p->w == nullptr ||
        p->scale == nullptr)
        return (int32_t)cudaErrorInvalidValue;
    OpsnnWqbmmParams v;
    prepare_view(p, &v);
    return wqbmm_prefill_prepass(&v, static_cast<uint8_t*>(storage), static_cast<cudaStream_t>(stream));
}

int32_t opsnn_wqbmm_launch(const OpsnnWqbmmParams* p, int32_t kernel_choice, void* stream)
{
    if (p == nullptr) return (int32_t)cudaErrorInvalidValue;
    if (p->m <= 0 || p->n <= 0) return 0;
    OpsnnWqbmmParams nd;
    if (p->nz_k0 != 0) {
        if (p->workspace == nullptr || p->workspace_size < wq_nz_bytes(p)) return (int32_t)cudaErrorInvalidValue;
        const int32_t rc = wq_nz_launch(p, p->workspace, static_cast<cudaStream_t>(stream));
        if (rc != 0) return rc;
        wq_nz_view(p, &nd, p->workspace);
        return opsnn_wqbmm_launch(&nd, kernel_choice, stream);
    }
    if (kernel_choice == OPSNN_WQ_KERNEL_AUTO) kernel_choice = opsnn_wqbmm_select_kernel(p);
    {
        // An output bound to a communicator (opsnn_comm_bind_columns) is written into every rank's full copy by the bulk-copy
        // decode kernels only; a call that would run elsewhere must not silently skip that.
        PeerBinding pb;
        if (lookup_peer_binding(p->y, &pb)) {
            const char* e = getenv("OPSNN_WQ_DECODE_PATH");
            const bool ring_only = e != nullptr && e[0] == 'r';
            const bool tma4 = (kernel_choice == OPSNN_WQ_KERNEL_DECODE || kernel_choice == OPSNN_WQ_KERNEL_DECODE_FAST) && p->w_dtype != ACL_INT8 &&
                              p->m <= 16 && !ring_only && wqbmm_decode_fast_eligible(p) && wqbmm_decode_tma_eligible(p) &&
                              getenv("OPSNN_WQ_DECODE_LEGACY") == nullptr;
            const bool tma8 = kernel_choice == OPSNN_WQ_KERNEL_DECODE && wqbmm_decode8_eligible(p);
            const bool tma4nk = kernel_choice == OPSNN_WQ_KERNEL_DECODE && wqbmm_decode_tma_nk_eligible(p);
            if (!tma4 && !tma8 && !tma4nk) {
                set_err("opsnn_wqbmm_launch: y is bound to a communicator, but this call does not run on a streaming decode kernel that "
                        "stores into the peers' outputs (m <= 16, int4, int8 or e4m3 weight stored (k,n), aligned rows)");
                return (int32_t)cudaErrorNotSupported;
            }
        }
    }
    OpsnnWqbmmParams chunk;
    if (p->m > 16 && (kernel_choice == OPSNN_WQ_KERNEL_DECODE || kernel_choice == OPSNN_WQ_KERNEL_DECODE_FAST)) {
        if (!decode_in_chunks(p, &chunk)) return (int32_t)cudaErrorInvalidValue;
        if (kernel_choice == OPSNN_WQ_KERNEL_DECODE_FAST && !wqbmm_decode_fast_eligible(&chunk)) return (int32_t)cudaErrorInvalidValue;
        return decode_chunk_launches(p, static_cast<cudaStream_t>(stream), kernel_choice);
    }
    if (kernel_choice == OPSNN_WQ_KERNEL_DECODE && p->w_dtype == ACL_INT4 && p->trans_w != 0) {
        if (!wqbmm_decode_tma_nk_eligible(p)) return (int32_t)cudaErrorInvalidValue;
        return wqbmm_decode_tma_launch(p, static_cast<cudaStream_t>(stream), true);
    }
    if (kernel_choice == OPSNN_WQ_KERNEL_DECODE && (p->w_dtype == ACL_INT8 || p->w_dtype == ACL_FLOAT8_E4M3FN)) {
        if (!wqbmm_decode8_eligible(p)) return (int32_t)cudaErrorInvalidValue;
        return wqbmm_decode8_launch(p, static_cast<cudaStream_t>(stream));
    }
    if (kernel_choice == OPSNN_WQ_KERNEL_DECODE) {
        if (!wqbmm_decode_eligible(p)) return (int32_t)cudaErrorInvalidValue;
        // same arithmetic, two data paths: shared-memory ring + ldmatrix where the layout allows it (32-column pieces, 16-byte
        // aligned rows, groups of whole step pairs), register prefetch otherwise
        if (wqbmm_decode_fast_eligible(p) && getenv("OPSNN_WQ_DECODE_LEGACY") == nullptr)
            return decode_stream_launch(p, static_cast<cudaStream_t>(stream), true);
        return wqbmm_decode_launch(p, static_cast<cudaStream_t>(stream));
    }
    if (kernel_choice == OPSNN_WQ_KERNEL_DECODE_FAST) {
        if (!wqbmm_decode_fast_eligible(p)) return (int32_t)cudaErrorInvalidValue;
        return decode_stream_launch(p, static_cast<cudaStream_t>(stream), false);
    }
    if (kernel_choice == OPSNN_WQ_KERNEL_PREFILL) {
        if (!wqbmm_prefill_eligible(p)) return (int32_t)cudaErrorInvalidValue;
        return wqbmm_prefill_launch(p, static_cast<cudaStream_t>(stream));
    }
    return wqbmm_generic_launch(p, static_cast<cudaStream_t>(stream));
}

int32_t opsnn_mx_quant_launch(const OpsnnMxQuantParams* p, void* stream)
{
    if (p == nullptr) return (int32_t)cudaErrorInvalidValue;
    return mx_quant_launch(p, static_cast<cudaStream_t>(stream));
}

int32_t opsnn_pack_b4_launch(const OpsnnPackB4Params* p, void* stream)
{
    if (p == nullptr || p->src == nullptr || p->dst == nullptr) return (int32_t)cudaErrorInvalidValue;
    return pack_b4_launch(p, static_cast<cudaStream_t>(stream));
}

uint64_t opsnn_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
const char* opsnn_last_kernel_name(void) { return g_last_kernel; }

}  // extern "C"

extern "C" OPSNN_API void opsnn_wqbmm_decode_last_plan(int32_t* strips, int32_t* splits, int32_t* cluster)
{
    if (strips != nullptr) *strips = opsnn::g_decode_plan[0];
    if (splits != nullptr) *splits = opsnn::g_decode_plan[1];
    if (cluster != nullptr) *cluster = opsnn::g_decode_plan[2];
}
