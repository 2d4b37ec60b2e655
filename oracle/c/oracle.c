/* CPU restatement, in plain C, of the two reference goldens the benchmark times. TEST INFRASTRUCTURE ONLY: the shipped
 * library never links or calls this file; tests and the benchmark's CPU-baseline leg do.
 *
 *   oracle_qmm_int8_kc      int8 x int8 -> int32, + int32 bias, -> fp32 (RNE), * x2Scale[n], * x1Scale[m], -> bf16 (RNE)
 *                           follows matmul/quant_batch_matmul_v3/tests/assets/qbmmv3_kernel_golden.py:361-387
 *                           (compute_pertoken) and the kernel epilogue order of
 *                           matmul/quant_batch_matmul_v3/op_kernel/arch35/qbmm_mix_online_dynamic.h:646-736
 *   oracle_wq_w4a16_group   y = x @ bf16(bf16(w + offset) * scale), fp32 accumulate, -> bf16
 *                           follows matmul/weight_quant_batch_matmul_v2/tests/assets/wqbmmv2_kernel_golden.py:242-297
 *                           (_compute_pergroup); int4 unpack as wqbmmv2_aclnn_golden.py:128-144 (low nibble first)
 *
 * Both split their outer loop over `threads` POSIX threads (pass 1 for a scalar run).
 */
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef void (*range_fn)(void* ctx, int64_t begin, int64_t end);
typedef struct {
    range_fn fn;
    void* ctx;
    int64_t begin, end;
} job_t;
static void* job_main(void* p)
{
    job_t* j = (job_t*)p;
    j->fn(j->ctx, j->begin, j->end);
    return NULL;
}
static void parallel_for(range_fn fn, void* ctx, int64_t total, int threads)
{
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    if ((int64_t)threads > total) threads = total > 0 ? (int)total : 1;
    pthread_t tid[256];
    job_t jobs[256];
    for (int t = 0; t < threads; ++t) {
        jobs[t].fn = fn;
        jobs[t].ctx = ctx;
        jobs[t].begin = total * t / threads;
        jobs[t].end = total * (t + 1) / threads;
        if (t > 0) pthread_create(&tid[t], NULL, job_main, &jobs[t]);
    }
    job_main(&jobs[0]);
    for (int t = 1; t < threads; ++t) pthread_join(tid[t], NULL);
}

static inline float bf16_to_f32(uint16_t h)
{
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_bf16_rne(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return (uint16_t)((u >> 16) | 0x0040u); /* NaN */
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16_rne(f)); }

typedef struct {
    const int8_t *x1, *x2;
    int64_t m, k, n;
    const float *s2, *s1;
    const int32_t* bias;
    uint16_t* out;
    int32_t* acc_out;
} qmm_ctx;

static void qmm_rows(void* p, int64_t r0, int64_t r1)
{
    const qmm_ctx* c = (const qmm_ctx*)p;
    const int64_t k = c->k, n = c->n;
    int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)n);
    for (int64_t i = r0; i < r1; ++i) {
        memset(acc, 0, sizeof(int32_t) * (size_t)n);
        for (int64_t q = 0; q < k; ++q) {
            const int32_t a = c->x1[i * k + q];
            const int8_t* row = c->x2 + q * n;
            for (int64_t j = 0; j < n; ++j) acc[j] += a * (int32_t)row[j];
        }
        for (int64_t j = 0; j < n; ++j) {
            int32_t v = acc[j];
            if (c->acc_out) c->acc_out[i * n + j] = v;
            if (c->bias) v += c->bias[j];
            float f = (float)v; /* RNE */
            f = f * c->s2[j];
            if (c->s1) f = f * c->s1[i];
            c->out[i * n + j] = f32_to_bf16_rne(f);
        }
    }
    free(acc);
}

/* x1 (m,k) row-major, x2 (k,n) row-major. s1/bias may be NULL. acc_out (m,n) int32 may be NULL. */
void oracle_qmm_int8_kc(const int8_t* x1, const int8_t* x2, int64_t m, int64_t k, int64_t n, const float* s2,
                        const float* s1, const int32_t* bias, uint16_t* out_bf16, int32_t* acc_out, int threads)
{
    qmm_ctx c = {x1, x2, m, k, n, s2, s1, bias, out_bf16, acc_out};
    parallel_for(qmm_rows, &c, m, threads);
}

/* x (m,k) bf16; words (k, n/8) int32, nibble j of word c = column 8c+j; scale/offset (k/g, n) bf16 (offset may be NULL);
 * computes columns [col_begin, col_end) of y (m, n) bf16. m <= 64. */
typedef struct {
    const float* xf;
    const int32_t* words;
    const uint16_t *scale, *offset;
    int64_t m, k, n, g, col_begin, col_end;
    uint16_t* y;
} wq_ctx;

static void wq_words(void* p, int64_t c0, int64_t c1)
{
    const wq_ctx* a = (const wq_ctx*)p;
    const int64_t n = a->n, nw = n / 8, first = a->col_begin / 8;
    for (int64_t c = first + c0; c < first + c1; ++c) {
        float acc[64][8];
        for (int64_t i = 0; i < a->m; ++i)
            for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
        for (int64_t q = 0; q < a->k; ++q) {
            const uint32_t wv = (uint32_t)a->words[q * nw + c];
            const int64_t gi = q / a->g;
            float wd[8];
            for (int j = 0; j < 8; ++j) {
                const int nib = (int)((wv >> (4 * j)) & 0xFu);
                float w = (float)((nib ^ 8) - 8);
                const int64_t col = 8 * c + j;
                if (a->offset) w = round_bf16(w + bf16_to_f32(a->offset[gi * n + col]));
                wd[j] = round_bf16(w * bf16_to_f32(a->scale[gi * n + col]));
            }
            for (int64_t i = 0; i < a->m; ++i) {
                const float xv = a->xf[i * a->k + q];
                for (int j = 0; j < 8; ++j) acc[i][j] += xv * wd[j];
            }
        }
        for (int64_t i = 0; i < a->m; ++i)
            for (int j = 0; j < 8; ++j) {
                const int64_t col = 8 * c + j;
                if (col >= a->col_begin && col < a->col_end) a->y[i * n + col] = f32_to_bf16_rne(acc[i][j]);
            }
    }
}

void oracle_wq_w4a16_group(const uint16_t* x, const int32_t* words, const uint16_t* scale, const uint16_t* offset, int64_t m,
                           int64_t k, int64_t n, int64_t g, int64_t col_begin, int64_t col_end, uint16_t* y, int threads)
{
    if (m > 64 || col_end <= col_begin) return;
    float* xf = (float*)malloc(sizeof(float) * (size_t)(m * k));
    for (int64_t i = 0; i < m * k; ++i) xf[i] = bf16_to_f32(x[i]);
    wq_ctx c = {xf, words, scale, offset, m, k, n, g, col_begin, col_end, y};
    parallel_for(wq_words, &c, (col_end + 7) / 8 - col_begin / 8, threads);
    free(xf);
}
