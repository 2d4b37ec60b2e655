// aclnnQuantMatmulV5: phase-1 validation + plan, phase-2 dispatch.
//
// Behavioural mirror (Ascend 950 column only) of the reference's
//   matmul/quant_batch_matmul_v4/op_host/op_api/aclnn_quant_matmul_v5.cpp:245-283 (input existence),
//   :285-325 (dim range), :967-1016 (pre-process), :1063-1183 (common process / routing), :1189-1227 (entry points)
//   matmul/quant_batch_matmul_v3/op_api/quant_matmul_checker.cpp:597-722 (groupSize inference), :724-967 (shape),
//   :1137-1195 (groupSize / CheckShape), :1574-1916 (dtype tables, CheckParams order).
// The rule order is kept (dtype -> shape -> format -> empty tensor) so the first failure yields the same status.
#include <algorithm>
#include <map>
#include <memory>
#include <mutex>
#include <shared_mutex>

#include "aclnnop/aclnn_quant_matmul_v4.h"
#include "aclnnop/aclnn_quant_matmul_v5.h"
#include "aclnnop/aclnn_quant_matmul_weight_nz.h"
#include "opsnn_b200_prepare.h"
#include "internal.h"

using namespace opsnn;

namespace {

constexpr uint64_t kGroupMask = 0xFFFF;

struct Group {
    uint64_t m = 0, n = 0, k = 0;
};
Group decode_group(int64_t g)
{
    Group r;
    r.k = (uint64_t)g & kGroupMask;
    r.n = ((uint64_t)g >> 16) & kGroupMask;
    r.m = ((uint64_t)g >> 32) & kGroupMask;
    return r;
}
int64_t encode_group(const Group& g) { return (int64_t)((g.m << 32) | (g.n << 16) | g.k); }

bool is_fp8(int dt) { return dt == ACL_FLOAT8_E4M3FN || dt == ACL_FLOAT8_E5M2; }
bool in(int dt, std::initializer_list<int> l) { return std::find(l.begin(), l.end(), dt) != l.end(); }

// Working copy of the arguments; views are normalised in place like the reference's executor->CreateView.
struct Ctx {
    aclTensor x1, x2, out;
    bool has_x1s = false, has_x2o = false, has_bias = false, has_ys = false, has_yo = false;
    aclTensor x1s, x2s, x2o, bias, ys, yo;
    bool t1 = false, t2 = false;
    int64_t group = 0;
    int64_t m = 0, n = 0, k1 = 0, k2 = 0;

    bool int8_in() const { return x1.dtype == ACL_INT8 && x2.dtype == ACL_INT8; }
    bool int4_in() const { return x1.dtype == ACL_INT4 && x2.dtype == ACL_INT4; }
    bool fp8_in() const { return is_fp8(x1.dtype) && is_fp8(x2.dtype); }
    bool hif8_in() const { return x1.dtype == ACL_HIFLOAT8 && x2.dtype == ACL_HIFLOAT8; }
    bool fp4_in() const { return x1.dtype == ACL_FLOAT4_E2M1 && x2.dtype == ACL_FLOAT4_E2M1; }
    bool mx() const { return has_x1s && x1s.dtype == ACL_FLOAT8_E8M0 && x2s.dtype == ACL_FLOAT8_E8M0; }
    bool perblock() const
    {
        return has_x1s && (int8_in() || fp8_in() || hif8_in()) && x1s.dtype == ACL_FLOAT && x1s.rank() > 1 &&
               x2s.dtype == ACL_FLOAT && x2s.rank() > 1;
    }
    void dims()
    {
        size_t r1 = x1.rank(), r2 = x2.rank();
        if (r1 >= 2 && r2 >= 2) {
            k1 = t1 ? x1.shape[r1 - 2] : x1.shape[r1 - 1];
            m = t1 ? x1.shape[r1 - 1] : x1.shape[r1 - 2];
            k2 = t2 ? x2.shape[r2 - 1] : x2.shape[r2 - 2];
            n = t2 ? x2.shape[r2 - 2] : x2.shape[r2 - 1];
        }
    }
};

// quant_matmul_common_check.cpp:106-123 — a strided-transposed view flips the flag instead of being copied.
void normalise_view(aclTensor& t, bool* transpose)
{
    if (is_transposed_last_two(&t)) {
        size_t r = t.rank();
        std::swap(t.shape[r - 1], t.shape[r - 2]);
        std::swap(t.strides[r - 1], t.strides[r - 2]);
        if (transpose) *transpose = !*transpose;
    }
}

// quant_matmul_checker.cpp:354-395
bool a4w4_pergroup_nonsym(const Ctx& c, uint64_t gk)
{
    if (!c.has_x1s || !c.has_x2o) return false;
    if (c.x1s.dtype != ACL_FLOAT || c.x1s.rank() <= 1) return false;
    if (c.x2s.dtype != ACL_FLOAT || c.x2s.rank() <= 1) return false;
    if (c.x2o.dtype != ACL_FLOAT16 || c.x2o.rank() <= 1) return false;
    if (c.has_bias) return false;
    int64_t m = c.t1 ? c.x1.shape[1] : c.x1.shape[0];
    int64_t k = c.t2 ? c.x2.shape[1] : c.x2.shape[0];
    int64_t n = c.t2 ? c.x2.shape[0] : c.x2.shape[1];
    if (k % 1024 != 0 || n % 256 != 0) return false;
    return c.int4_in() && c.x1s.shape[0] == m && c.x1s.shape[1] == 1 && c.x2s.shape[0] == ceil_div(k, (int64_t)gk) &&
           c.x2s.shape[1] == n && c.x2o.shape[0] == ceil_div(k, (int64_t)gk) && c.x2o.shape[1] == n;
}

// quant_matmul_checker.cpp:597-722
bool recalc_group(int64_t input, int64_t scale, uint64_t& g, const char* which)
{
    if (scale == 0) {
        set_err("aclnnQuantMatmulV5: the %s dimension of the scale is 0", which);
        return false;
    }
    if (g == 0) {
        if (input % scale != 0) {
            set_err("aclnnQuantMatmulV5: groupSize %s cannot be inferred: %ld is not divisible by %ld", which,
                    (long)input, (long)scale);
            return false;
        }
        g = (uint64_t)(input / scale);
    }
    return true;
}

bool infer_group(const Ctx& c, int64_t& group)
{
    if (!c.has_x1s || c.x1s.rank() < 2 || c.x2s.rank() < 2) return true;
    Group g = decode_group(group);
    size_t r1 = c.x1.rank(), r2 = c.x2.rank(), s1 = c.x1s.rank(), s2 = c.x2s.rank();
    int64_t in_m = c.t1 ? c.x1.shape[r1 - 1] : c.x1.shape[r1 - 2];
    int64_t in_k = c.t1 ? c.x1.shape[r1 - 2] : c.x1.shape[r1 - 1];
    int64_t in_n = c.t2 ? c.x2.shape[r2 - 2] : c.x2.shape[r2 - 1];
    int64_t sm, sk, sn;
    if (c.mx()) {
        if (s1 < 3 || s2 < 3) return true;  // rejected later by the dim-range check
        size_t b1 = s1 - 3, b2 = s2 - 3;
        sm = c.x1s.shape[b1 + (c.t1 ? 1 : 0)];
        sk = c.x1s.shape[b1 + (c.t1 ? 0 : 1)] * 2;
        sn = c.x2s.shape[b2 + (c.t2 ? 0 : 1)];
        int64_t d0 = c.x2s.shape[b2], d1 = c.x2s.shape[b2 + 1];
        if ((d0 == 1 && d1 == in_n) || (d0 == in_n && d1 == 1) || (in_n == 1 && (d0 == 1 || d1 == 1))) sn = in_n;
    } else {
        sm = c.t1 ? c.x1s.shape[s1 - 1] : c.x1s.shape[s1 - 2];
        sk = c.t1 ? c.x1s.shape[s1 - 2] : c.x1s.shape[s1 - 1];
        if (a4w4_pergroup_nonsym(c, g.k)) sn = c.t2 ? c.x2s.shape[s2 - 1] : c.x2s.shape[s2 - 2];
        else sn = c.t2 ? c.x2s.shape[s2 - 2] : c.x2s.shape[s2 - 1];
    }
    if (!recalc_group(in_m, sm, g.m, "m")) return false;
    if (!recalc_group(in_k, sk, g.k, "k")) return false;
    if (!recalc_group(in_n, sn, g.n, "n")) return false;
    group = encode_group(g);
    return true;
}

#define FAIL(...)             \
    do {                      \
        set_err(__VA_ARGS__); \
        return false;         \
    } while (0)

// ---- dtype rules, quant_matmul_checker.cpp:1574-1852 (DAV_3510 branch) ---------------------------------------
bool check_dtype(const Ctx& c)
{
    const int out = c.out.dtype, s2 = c.x2s.dtype;
    const int bias = c.has_bias ? (int)c.bias.dtype : -1;
    if (out == ACL_INT32 && c.has_x1s) FAIL("out INT32 does not take x1Scale");
    if (!c.has_x1s) {  // per-tensor / per-channel
        if (out == ACL_INT32 && !c.int8_in()) FAIL("out INT32 needs INT8 x1/x2");
        if (c.int8_in() || c.int4_in()) {
            if (out == ACL_BF16) {
                if (!in(s2, {ACL_UINT64, ACL_INT64, ACL_FLOAT, ACL_BF16})) FAIL("x2Scale dtype %s not supported for BF16 out", dtype_name(s2));
            } else if (out == ACL_INT8 || out == ACL_FLOAT16) {
                if (!in(s2, {ACL_UINT64, ACL_INT64})) FAIL("x2Scale must be UINT64/INT64 for %s out", dtype_name(out));
            } else if (out == ACL_INT32) {
                if (!in(s2, {ACL_FLOAT, ACL_BF16})) FAIL("x2Scale must be FLOAT/BF16 for INT32 out");
            }
            if (c.has_bias) {
                if (out == ACL_INT32 && bias != ACL_INT32) FAIL("bias must be INT32 for INT32 out");
                if (out == ACL_BF16 && (s2 == ACL_FLOAT || s2 == ACL_BF16) && !in(bias, {ACL_INT32, ACL_BF16, ACL_FLOAT}))
                    FAIL("bias dtype %s not supported", dtype_name(bias));
                if ((out == ACL_INT8 || out == ACL_FLOAT16 || out == ACL_BF16) && (s2 == ACL_UINT64 || s2 == ACL_INT64) &&
                    bias != ACL_INT32)
                    FAIL("bias must be INT32 with a packed UINT64 scale");
            }
            if (c.has_x2o) {
                if (out != ACL_INT8) FAIL("x2Offset only with INT8 out");
                if (c.x2o.dtype != ACL_FLOAT) FAIL("x2Offset must be FLOAT");
            }
            if (!in(out, {ACL_INT8, ACL_FLOAT16, ACL_BF16, ACL_INT32})) FAIL("out dtype %s not supported", dtype_name(out));
        } else if (c.hif8_in() || c.fp8_in()) {
            if (!in(s2, {ACL_UINT64, ACL_INT64})) FAIL("x2Scale must be UINT64/INT64 for fp8 per-tensor/per-channel");
            if (c.has_bias && bias != ACL_FLOAT) FAIL("bias must be FLOAT");
            if (c.has_x2o) FAIL("x2Offset not supported");
            if (!in(out, {ACL_FLOAT16, ACL_BF16, ACL_FLOAT})) FAIL("out dtype %s not supported", dtype_name(out));
        } else {
            FAIL("x1/x2 dtype combination %s/%s not supported", dtype_name(c.x1.dtype), dtype_name(c.x2.dtype));
        }
    } else if (c.mx()) {
        if (!c.fp4_in() && !c.fp8_in()) FAIL("mx needs fp8 x fp8 or fp4 x fp4 inputs");
        // the reference takes a FLOAT bias only in this mode (quant_matmul_checker.cpp:1685-1687); a BF16 bias is accepted here as
        // an extension (widened to fp32 exactly before the add), because serving stacks keep the bias in the activation dtype
        if (c.has_bias && bias != ACL_FLOAT && bias != ACL_BF16) FAIL("mx bias must be FLOAT (or BF16, an extension of this library)");
        if (!in(out, {ACL_FLOAT16, ACL_BF16, ACL_FLOAT})) FAIL("out dtype %s not supported", dtype_name(out));
        if (c.has_x2o) FAIL("x2Offset not supported");
    } else if (c.int4_in() && c.has_x2o) {  // per-token per-group asymmetric int4
        if (!in(out, {ACL_FLOAT16, ACL_BF16})) FAIL("out dtype not supported");
        if (c.x1s.dtype != ACL_FLOAT || s2 != ACL_FLOAT || c.x2o.dtype != ACL_FLOAT16) FAIL("scale/offset dtype not supported");
        if (c.t1 || !c.t2) FAIL("A4W4 per-group needs transposeX1=false, transposeX2=true");
    } else if (c.int8_in() || c.int4_in()) {  // per-token
        if (!in(out, {ACL_FLOAT16, ACL_BF16})) FAIL("per-token out dtype %s not supported", dtype_name(out));
        if (c.x1s.dtype != ACL_FLOAT) FAIL("x1Scale must be FLOAT");
        if (c.has_x2o) FAIL("x2Offset not supported");
        if (out == ACL_BF16) {
            if (!in(s2, {ACL_BF16, ACL_FLOAT})) FAIL("x2Scale must be BF16/FLOAT");
            if (c.has_bias && !in(bias, {ACL_INT32, ACL_BF16, ACL_FLOAT})) FAIL("bias dtype not supported");
        } else {
            if (s2 != ACL_FLOAT) FAIL("x2Scale must be FLOAT for FLOAT16 out");
            if (c.has_bias && !in(bias, {ACL_INT32, ACL_FLOAT16, ACL_FLOAT})) FAIL("bias dtype not supported");
        }
    } else if (c.hif8_in() || c.fp8_in()) {  // double scale, fp8 per-token, per-block
        if (c.x1s.dtype != ACL_FLOAT) FAIL("x1Scale must be FLOAT");
        if (s2 != ACL_FLOAT) FAIL("x2Scale must be FLOAT");
        if (!in(out, {ACL_FLOAT16, ACL_BF16, ACL_FLOAT})) FAIL("out dtype not supported");
        if (c.perblock() && c.has_bias) FAIL("per-block does not take bias");
        if (c.has_bias && bias != ACL_FLOAT) FAIL("bias must be FLOAT");
        if (c.has_x2o) FAIL("x2Offset not supported");
    } else {
        FAIL("x1/x2 dtype combination %s/%s not supported", dtype_name(c.x1.dtype), dtype_name(c.x2.dtype));
    }
    return true;
}

// ---- shape rules, quant_matmul_checker.cpp:477-967, 1008-1195 ----------------------------------------------
bool check_mx_dims(const Ctx& c)
{
    size_t b1 = c.x1s.rank() - 3, b2 = c.x2s.rank() - 3;
    int64_t s1m = c.x1s.shape[b1 + (c.t1 ? 1 : 0)], s1k = c.x1s.shape[b1 + (c.t1 ? 0 : 1)];
    int64_t s2n = c.x2s.shape[b2 + (c.t2 ? 0 : 1)], s2k = c.x2s.shape[b2 + (c.t2 ? 1 : 0)];
    int64_t kq1 = ceil_div(c.k1, 64), kq2 = ceil_div(c.k2, 64);
    bool one1 = (s1m == 1 && s1k == c.m) || (s1m == c.m && s1k == 1) || (s1m == 1 && s1k == kq1) || (s1m == kq1 && s1k == 1);
    bool one2 = (s2n == 1 && s2k == c.n) || (s2n == c.n && s2k == 1) || (s2n == 1 && s2k == kq2) || (s2n == kq2 && s2k == 1);
    if ((!one1 && s1m != c.m) || (!one2 && s2n != c.n)) FAIL("mx: scale M/N dimension does not match x1/x2");
    if ((!one1 && kq1 != s1k) || (!one2 && kq2 != s2k)) FAIL("mx: scale K dimension must be ceil(k/64)");
    if (c.x1s.dim(-1) != 2 || c.x2s.dim(-1) != 2) FAIL("mx: last dimension of the scales must be 2");
    if (c.fp4_in()) {
        // fp4 packs two values per byte along the inner axis (CheckMXFP4FP8ParamsNDOrNZ, :453-475)
        if (c.k1 % 2 != 0) FAIL("mxfp4: k must be even");
        if (c.t1 && c.m % 2 != 0) FAIL("mxfp4: inner axis m must be even when x1 is transposed");
        if (!c.t2 && c.n % 2 != 0) FAIL("mxfp4: inner axis n must be even when x2 is not transposed");
    }
    return true;
}

bool check_perblock_dims(const Ctx& c)
{
    size_t r1 = c.x1.rank(), r2 = c.x2.rank();
    uint64_t gm = std::max<uint64_t>(((uint64_t)c.group >> 32) & kGroupMask, 1);
    if (c.x1s.rank() != r1 || c.x2s.rank() != r2) FAIL("per-block: scale rank must equal input rank");
    for (int64_t i = (int64_t)r1 - 3; i >= 0; --i)
        if (c.x1s.shape[i] != c.x1.shape[i]) FAIL("per-block: x1Scale batch dims must equal x1's");
    for (int64_t i = (int64_t)r2 - 3; i >= 0; --i)
        if (c.x2s.shape[i] != c.x2.shape[i]) FAIL("per-block: x2Scale batch dims must equal x2's");
    size_t mi = r1 - (c.t1 ? 1 : 2), k1i = r1 - (c.t1 ? 2 : 1), ni = r2 - (c.t2 ? 2 : 1), k2i = r2 - (c.t2 ? 1 : 2);
    if (ceil_div(c.x1.shape[mi], (int64_t)gm) != c.x1s.shape[mi]) FAIL("per-block: x1Scale m dim must be ceil(m/groupSizeM)");
    if (ceil_div(c.x1.shape[k1i], 128) != c.x1s.shape[k1i]) FAIL("per-block: x1Scale k dim must be ceil(k/128)");
    if (ceil_div(c.x2.shape[ni], 128) != c.x2s.shape[ni]) FAIL("per-block: x2Scale n dim must be ceil(n/128)");
    if (ceil_div(c.x2.shape[k2i], 128) != c.x2s.shape[k2i]) FAIL("per-block: x2Scale k dim must be ceil(k/128)");
    return true;
}

bool check_shape(const Ctx& c)
{
    const Group g = decode_group(c.group);
    // scale dim range (:1115-1135)
    if (!c.has_x1s) {
        if (c.x2s.rank() != 1) FAIL("x2Scale must be 1-D without x1Scale");
    } else if (c.mx()) {
        size_t s1 = c.x1s.rank(), s2 = c.x2s.rank();
        if (s1 < 3 || s2 < 3) FAIL("mx: scales must have at least 3 dims");
        size_t ib1 = c.x1.rank() > 2 ? c.x1.rank() - 2 : 0, ib2 = c.x2.rank() > 2 ? c.x2.rank() - 2 : 0;
        if (s1 - 3 != ib1 || s2 - 3 != ib2) FAIL("mx: scale batch dim count must match the input's");
        for (size_t i = 0; i < s1 - 3; ++i)
            if (c.x1s.shape[i] != c.x1.shape[i]) FAIL("mx: x1Scale batch dims must equal x1's");
        for (size_t i = 0; i < s2 - 3; ++i)
            if (c.x2s.shape[i] != c.x2.shape[i]) FAIL("mx: x2Scale batch dims must equal x2's");
    } else if (a4w4_pergroup_nonsym(c, g.k)) {
    } else {
        bool pb = c.perblock();
        if ((pb && c.x1s.rank() != c.x1.rank()) || (!pb && c.x1s.rank() != 1)) FAIL("x1Scale rank not supported");
        if ((pb && c.x2s.rank() != c.x2.rank()) || (!pb && c.x2s.rank() != 1)) FAIL("x2Scale rank not supported");
    }
    // groupSize (:1137-1159)
    if (a4w4_pergroup_nonsym(c, g.k)) {
        if (g.k != 256) FAIL("A4W4 per-group: groupSizeK must be 256");
    } else if (c.mx()) {
        if (g.k != 32 || g.m != 1 || g.n != 1) FAIL("mx: groupSize must resolve to [1,1,32] (4295032864), got [%lu,%lu,%lu]", g.m, g.n, g.k);
    } else if (c.perblock()) {
        if (g.k != 128 || g.n != 128 || (g.m != 128 && g.m != 1)) FAIL("per-block: groupSize must be [1|128,128,128], got [%lu,%lu,%lu]", g.m, g.n, g.k);
    } else if (c.group != 0) {
        FAIL("groupSize must be 0 for this quantization mode");
    }
    if (c.int4_in()) {
        // CheckShapeInt4 (:969-1006): the packed inner axis must be even
        if (c.x1.dim(-1) % 2 != 0 || c.x2.dim(-1) % 2 != 0) FAIL("int4 inner axis must be even");
    }
    if (c.k1 != c.k2) FAIL("k of x1 (%ld) and x2 (%ld) differ", (long)c.k1, (long)c.k2);
    // CheckDimValue (:805-852)
    bool skip_rest = false;
    if (c.has_x1s) {
        if (c.mx()) {
            if (!check_mx_dims(c)) return false;
            skip_rest = true;
        } else if (c.perblock()) {
            if (!check_perblock_dims(c)) return false;
            skip_rest = true;
        } else {
            int64_t s0 = c.x1s.shape[0];
            if (c.m == 1) {
                if (s0 != 1) FAIL("x1Scale must have 1 element when m is 1");
            } else if (s0 == 1 && !c.int8_in()) {
                if (c.x2s.shape[0] != 1 && c.x2s.shape[0] != c.n) FAIL("x2Scale must have 1 or n elements");
            } else if (s0 != c.m) {
                FAIL("x1Scale must have m (%ld) elements, got %ld", (long)c.m, (long)s0);
            }
        }
    }
    if (!skip_rest) {
        bool a4 = a4w4_pergroup_nonsym(c, g.k);
        if (!a4 && c.x2s.shape[0] != c.n && c.x2s.shape[0] != 1) FAIL("x2Scale must have 1 or n (%ld) elements", (long)c.n);
        if (c.has_x2o && !a4) {
            if (c.x2o.rank() != 1) FAIL("x2Offset must be 1-D");
            if (c.x2o.shape[0] != c.n && c.x2o.shape[0] != 1) FAIL("x2Offset must have 1 or n elements");
        }
    }
    // output batch inference (:854-877)
    std::vector<int64_t> batch;
    int64_t batch_prod = 1;
    {
        size_t r1 = c.x1.rank(), r2 = c.x2.rank(), ro = std::max(r1, r2), off = ro - std::min(r1, r2);
        const aclTensor& lg = r1 > r2 ? c.x1 : c.x2;
        const aclTensor& sh = r1 > r2 ? c.x2 : c.x1;
        for (size_t i = 0; i + 2 < ro; ++i) {
            int64_t a = lg.shape[i], b = i < off ? 1 : sh.shape[i - off];
            if (a > 1 && b > 1 && a != b) FAIL("batch dims of x1 and x2 cannot be broadcast");
            batch.push_back(std::max(a, b));
            batch_prod *= std::max(a, b);
        }
    }
    if (c.has_bias) {  // :879-927
        size_t br = c.bias.rank();
        if (br != 3 && br != 1) FAIL("bias must be 1-D or 3-D");
        if (br == 1) {
            if (c.bias.shape[0] != c.n) FAIL("bias must have n (%ld) elements", (long)c.n);
        } else {
            if (batch.size() != 1) FAIL("3-D bias needs exactly one output batch dim");
            if (c.bias.shape[1] != 1) FAIL("bias second dim must be 1");
            if (c.bias.shape[2] != c.n) FAIL("bias third dim must be n");
            if (c.bias.shape[0] != batch_prod) FAIL("bias first dim must equal the output batch");
        }
    }
    {  // :929-967
        size_t ro = c.out.rank();
        int64_t om = c.out.shape[ro - 2], on = c.out.shape[ro - 1];
        size_t inferred = batch.size() + 2;
        bool two_d = c.x1.rank() == 2 && c.x2.rank() == 2;
        if (om == 1 && inferred == 2 && ro == 3 && two_d) {
            ro -= 1;
            om = c.out.shape[0];
        }
        if (inferred != ro) FAIL("out rank %zu does not match the inferred rank %zu", ro, inferred);
        if (om != c.m) FAIL("out m (%ld) must equal x1 m (%ld)", (long)om, (long)c.m);
        if (on != c.n) FAIL("out n (%ld) must equal x2 n (%ld)", (long)on, (long)c.n);
        for (size_t i = 0; i + 2 < ro; ++i)
            if (c.out.shape[i] != batch[i]) FAIL("out batch dim %zu must be %ld", i, (long)batch[i]);
    }
    return true;
}

// ---- A8W4 (fp8 x fp4) rules, aclnn_quant_matmul_v5.cpp:193-243, 327-398, 414-480, 560-760 -------------------------
aclnnStatus check_a8w4_float(const Ctx& c, const aclTensor* x1Scale, int64_t group_k)
{
    bool is_mx = c.mx();
    bool is_tcg = !c.has_x1s && (c.x2s.dtype == ACL_BF16 || c.x2s.dtype == ACL_FLOAT16);
    if (!is_mx && !is_tcg) {
        set_err("A8W4: neither mx (e8m0 scales) nor T-CG (x1Scale null, x2Scale BF16/FLOAT16)");
        return ACLNN_ERR_PARAM_INVALID;
    }
    (void)x1Scale;
    if (c.t1) { set_err("A8W4: transposeX1 must be false"); return ACLNN_ERR_PARAM_INVALID; }
    if (!c.t2) { set_err("A8W4 ND: transposeX2 must be true"); return ACLNN_ERR_PARAM_INVALID; }
    if (group_k != 32) { set_err("A8W4: groupSizeK must be 32"); return ACLNN_ERR_PARAM_INVALID; }
    // dim range
    if (c.x1.rank() != 2 || c.x2.rank() != 2 || c.out.rank() != 2) { set_err("A8W4: x1, x2, out must be 2-D"); return ACLNN_ERR_PARAM_INVALID; }
    if (c.has_bias && c.bias.rank() != 2) { set_err("A8W4: bias must be 2-D"); return ACLNN_ERR_PARAM_INVALID; }
    size_t want = is_mx ? 3 : 2;
    if (c.has_x1s && c.x1s.rank() != want) { set_err("A8W4: x1Scale rank"); return ACLNN_ERR_PARAM_INVALID; }
    if (c.x2s.rank() != want) { set_err("A8W4: x2Scale rank"); return ACLNN_ERR_PARAM_INVALID; }
    if (c.has_ys && c.ys.rank() != 2) { set_err("A8W4: yScale must be 2-D"); return ACLNN_ERR_PARAM_INVALID; }
    if (c.has_yo && c.yo.rank() != 1) { set_err("A8W4: yOffset must be 1-D"); return ACLNN_ERR_PARAM_INVALID; }
    // dtype
    if (!is_fp8(c.x1.dtype) || c.x2.dtype != ACL_FLOAT4_E2M1 || !in(c.out.dtype, {ACL_BF16, ACL_FLOAT16})) {
        set_err("A8W4: dtype combination not supported");
        return ACLNN_ERR_PARAM_INVALID;
    }
    if (c.x1.dtype != ACL_FLOAT8_E4M3FN) { set_err("A8W4: x1 must be FLOAT8_E4M3FN"); return ACLNN_ERR_PARAM_INVALID; }
    if (!c.has_x1s) {
        if (c.has_bias) { set_err("A8W4 T-CG: bias must be null"); return ACLNN_ERR_PARAM_INVALID; }
        if (!c.has_ys) { set_err("A8W4 T-CG: yScale is required"); return ACLNN_ERR_PARAM_INVALID; }
        if (!in(c.ys.dtype, {ACL_UINT64, ACL_INT64})) { set_err("A8W4 T-CG: yScale must be UINT64"); return ACLNN_ERR_PARAM_INVALID; }
    } else {
        if (c.has_bias && c.bias.dtype != c.out.dtype) { set_err("MxA8W4: bias dtype must equal out dtype"); return ACLNN_ERR_PARAM_INVALID; }
        if (c.has_ys) { set_err("MxA8W4: yScale must be null"); return ACLNN_ERR_PARAM_INVALID; }
    }
    // shape
    if (c.m <= 0 || c.k1 <= 0 || c.n <= 0 || c.k1 != c.k2) { set_err("A8W4: bad m/k/n"); return ACLNN_ERR_PARAM_INVALID; }
    if (is_tcg && (c.k1 % 32 != 0 || c.k1 <= 32)) { set_err("A8W4 T-CG: k must be a multiple of 32 and > 32"); return ACLNN_ERR_PARAM_INVALID; }
    if (is_mx && c.k1 % 8 != 0) { set_err("MxA8W4: k must be a multiple of 8"); return ACLNN_ERR_PARAM_INVALID; }
    int64_t gd = ceil_div(c.k2, 32);
    if (is_mx) {
        if (c.x1s.shape[0] != c.m || c.x1s.shape[1] != ceil_div(gd, 2) || c.x1s.shape[2] != 2) { set_err("MxA8W4: x1Scale shape"); return ACLNN_ERR_PARAM_INVALID; }
        if (c.x2s.shape[0] != c.n || c.x2s.shape[1] != ceil_div(gd, 2) || c.x2s.shape[2] != 2) { set_err("MxA8W4: x2Scale shape"); return ACLNN_ERR_PARAM_INVALID; }
    } else {
        if (c.x2s.shape[0] != c.n || c.x2s.shape[1] != gd) { set_err("A8W4 T-CG: x2Scale must be (n, k/32)"); return ACLNN_ERR_PARAM_INVALID; }
    }
    if (c.has_ys && (c.ys.shape[0] != 1 || c.ys.shape[1] != c.n)) { set_err("A8W4: yScale must be (1,n)"); return ACLNN_ERR_PARAM_INVALID; }
    if (c.has_bias && (c.bias.shape[0] != 1 || c.bias.shape[1] != c.n)) { set_err("A8W4: bias must be (1,n)"); return ACLNN_ERR_PARAM_INVALID; }
    if (c.out.shape[0] != c.m || c.out.shape[1] != c.n) { set_err("A8W4: out must be (m,n)"); return ACLNN_ERR_PARAM_INVALID; }
    return ACLNN_SUCCESS;
}

// Batch stride (elements) of an operand whose leading dims either equal the output batch dims or are absent/1.
bool operand_batch(const aclTensor& t, size_t core_rank, const std::vector<int64_t>& out_batch, int64_t core_elems,
                   int64_t* bs)
{
    size_t nb = t.rank() - core_rank;
    bool all_one = true;
    for (size_t i = 0; i < nb; ++i) all_one &= (t.shape[i] == 1);
    if (all_one) {
        *bs = 0;
        return true;
    }
    // must match the trailing out_batch dims exactly and be dense
    if (nb > out_batch.size()) return false;
    size_t off = out_batch.size() - nb;
    for (size_t i = 0; i < off; ++i)
        if (out_batch[i] != 1) return false;
    for (size_t i = 0; i < nb; ++i)
        if (t.shape[i] != out_batch[off + i]) return false;
    *bs = core_elems;
    return true;
}

// ---- prepared x2 registry (opsnnQuantMatmulPrepareX2) --------------------------------------------------------------------
// Keyed by x2's device address. An entry is used only by calls whose x2 and x2Scale describe the very tensors that were
// prepared (same addresses, extents, strides, orientation); anything else runs unprepared.
struct PreparedX2 {
    OpsnnQmmParams key{};  // the plan fields of the prepared call that must match
    const void* prep_b = nullptr;
    const void* prep_sfb = nullptr;
    int32_t prep_bn = 0;
};
std::shared_mutex g_prepared_mu;
std::map<const void*, PreparedX2> g_prepared;

bool same_x2(const OpsnnQmmParams& a, const OpsnnQmmParams& b)
{
    return a.mode == b.mode && a.b == b.b && a.scale_b == b.scale_b && a.b_dtype == b.b_dtype && a.a_dtype == b.a_dtype &&
           a.trans_b == b.trans_b && a.n == b.n && a.k == b.k && a.b_ld == b.b_ld && a.b_bs == b.b_bs && a.sb_bs == b.sb_bs &&
           (a.b_bs == 0 || a.batch == b.batch) && a.group_k == b.group_k && a.b_prepass == b.b_prepass;
}

void attach_prepared(OpsnnQmmParams* p)
{
    if (p->mode != OPSNN_QMM_MX || p->b == nullptr) return;
    std::shared_lock<std::shared_mutex> lk(g_prepared_mu);
    auto it = g_prepared.find(p->b);
    if (it == g_prepared.end() || !same_x2(it->second.key, *p)) return;
    p->prep_b = it->second.prep_b;
    p->prep_sfb = it->second.prep_sfb;
    p->prep_bn = it->second.prep_bn;
}

// A stand-in x1 / x1Scale / out of mHint rows for planning a call on x2 alone (stand-in addresses: nothing of them is read).
struct HintTensors {
    aclTensor x1, x1s, out;
};
void make_hint(const aclTensor* x2, const aclTensor* x2Scale, bool transposeX2, int64_t m_hint, HintTensors* h)
{
    const size_t r = x2->rank();
    const int64_t k = transposeX2 ? x2->dim(-1) : x2->dim(-2), n = transposeX2 ? x2->dim(-2) : x2->dim(-1);
    std::vector<int64_t> batch(x2->shape.begin(), x2->shape.begin() + (r >= 2 ? r - 2 : 0));
    auto contiguous = [](aclTensor* t) {
        t->strides.assign(t->shape.size(), 1);
        for (int i = (int)t->shape.size() - 2; i >= 0; --i) t->strides[i] = t->strides[i + 1] * t->shape[i + 1];
        t->storage_shape = t->shape;
        t->offset = 0;
        t->format = ACL_FORMAT_ND;
        t->data = reinterpret_cast<void*>(uintptr_t(256));  // stand-in with allocation alignment: kernel selection looks at it, nothing reads it
    };
    h->x1.shape = batch; h->x1.shape.push_back(m_hint); h->x1.shape.push_back(k);
    h->x1.dtype = x2->dtype;
    contiguous(&h->x1);
    h->x1s.shape = batch; h->x1s.shape.push_back(m_hint); h->x1s.shape.push_back((k + 63) / 64); h->x1s.shape.push_back(2);
    h->x1s.dtype = x2Scale->dtype;
    contiguous(&h->x1s);
    h->out.shape = batch; h->out.shape.push_back(m_hint); h->out.shape.push_back(n);
    h->out.dtype = ACL_BF16;
    contiguous(&h->out);
}

}  // namespace

extern "C" {

aclnnStatus aclnnQuantMatmulV5GetWorkspaceSize(const aclTensor* x1, const aclTensor* x2, const aclTensor* x1Scale,
                                               const aclTensor* x2Scale, const aclTensor* yScale,
                                               const aclTensor* x1Offset, const aclTensor* x2Offset,
                                               const aclTensor* yOffset, const aclTensor* bias, bool transposeX1,
                                               bool transposeX2, int64_t groupSize, aclTensor* out,
                                               uint64_t* workspaceSize, aclOpExecutor** executor)
{
    OPSNN_DFX_RANGE("aclnnQuantMatmulV5GetWorkspaceSize");
    clear_err();
    if (workspaceSize == nullptr || executor == nullptr) {
        set_err("aclnnQuantMatmulV5GetWorkspaceSize: workspaceSize/executor is nullptr");
        return ACLNN_ERR_PARAM_NULLPTR;
    }
    // Extension (no counterpart in the reference, whose checker refuses 16-bit x1 here): BF16 / FLOAT16 x1 with no x1Scale against an
    // MX weight = "dynamic activation quantisation fused ahead". x1 is quantised with aclnnDynamicMxQuant's arithmetic (OCP shared
    // exponent per 32 along k, round to nearest even; quant/dynamic_mx_quant/tests/assets/golden.py:141-217) to x2's element type
    // into the workspace, then the MX matmul runs: one call pair, results bit-identical to the two-call chain.
    if (x1 != nullptr && x2 != nullptr && x2Scale != nullptr && x1Scale == nullptr && out != nullptr &&
        (x1->dtype == ACL_BF16 || x1->dtype == ACL_FLOAT16) && x2Scale->dtype == ACL_FLOAT8_E8M0 &&
        (x2->dtype == ACL_FLOAT8_E4M3FN || x2->dtype == ACL_FLOAT8_E5M2 || x2->dtype == ACL_FLOAT4_E2M1)) {
        const char* api = "aclnnQuantMatmulV5GetWorkspaceSize";
        if (transposeX1 || x1->rank() < 2 || !is_contiguous(x1)) {
            set_err("%s: a 16-bit x1 (quantised on the fly) must be contiguous, at least 2-D and not transposed", api);
            return ACLNN_ERR_PARAM_INVALID;
        }
        const int64_t k = x1->dim(-1);
        if (x2->dtype == ACL_FLOAT4_E2M1 && (k & 1)) {
            set_err("%s: fp4 quantisation needs an even k", api);
            return ACLNN_ERR_PARAM_INVALID;
        }
        aclTensor q = *x1, sc = *x1;
        q.dtype = x2->dtype;
        q.data = reinterpret_cast<void*>(uintptr_t(256));  // stand-ins with allocation alignment; replaced by workspace addresses in phase 2
        q.offset = 0;
        sc.shape.back() = (k + 63) / 64;
        sc.shape.push_back(2);
        sc.dtype = ACL_FLOAT8_E8M0;
        sc.strides.assign(sc.shape.size(), 1);
        for (int i = (int)sc.shape.size() - 2; i >= 0; --i) sc.strides[i] = sc.strides[i + 1] * sc.shape[i + 1];
        sc.storage_shape = sc.shape;
        sc.data = reinterpret_cast<void*>(uintptr_t(256));
        sc.offset = 0;
        const aclnnStatus st = aclnnQuantMatmulV5GetWorkspaceSize(&q, x2, &sc, x2Scale, yScale, x1Offset, x2Offset, yOffset, bias, false,
                                                                  transposeX2, groupSize, out, workspaceSize, executor);
        if (st != ACLNN_SUCCESS) return st;
        aclOpExecutor* exec = *executor;
        if (exec->nothing_to_do) return ACLNN_SUCCESS;
        exec->dyn_quant = true;
        OpsnnMxQuantParams& mq = exec->mxq;
        mq.x_dtype = x1->dtype;
        mq.y_dtype = x2->dtype;
        mq.k = k;
        mq.rows = k > 0 ? x1->numel() / k : 0;
        mq.x = x1->data == nullptr ? nullptr : data_ptr(x1);
        mq.inner = 0;
        mq.scale_alg = 0;
        mq.round_mode = 0;
        const uint64_t bits = (uint64_t)dtype_bits(x2->dtype);
        exec->dq_q_bytes = (((uint64_t)x1->numel() * bits / 8) + 255u) & ~(uint64_t)255u;
        exec->dq_s_bytes = (((uint64_t)mq.rows * 2u * (uint64_t)((k + 63) / 64)) + 255u) & ~(uint64_t)255u;
        exec->qmm.a = nullptr;
        exec->qmm.scale_a = nullptr;
        exec->workspace_size += exec->dq_q_bytes + exec->dq_s_bytes;
        *workspaceSize = exec->workspace_size;
        return ACLNN_SUCCESS;
    }
    if (x2 == nullptr) {
        set_err("aclnnQuantMatmulV5GetWorkspaceSize: x2 is nullptr");
        return ACLNN_ERR_PARAM_NULLPTR;
    }
    if (x2->format == ACL_FORMAT_FRACTAL_NZ || x2->format == ACL_FORMAT_FRACTAL_NZ_C0_32) {
        set_err("aclnnQuantMatmulV5GetWorkspaceSize: x2 format FRACTAL_NZ is not accepted by this entry point, use ND");
        return ACLNN_ERR_PARAM_INVALID;
    }
    // CheckInputExistence (:245-283)
    if (x1 == nullptr || x2Scale == nullptr || out == nullptr) {
        set_err("aclnnQuantMatmulV5GetWorkspaceSize: x1, x2Scale and out are required");
        return ACLNN_ERR_PARAM_NULLPTR;
    }
    const bool a8w4f = is_fp8(x1->dtype) && x2->dtype == ACL_FLOAT4_E2M1;
    const bool a8w4i = x1->dtype == ACL_INT8 && x2->dtype == ACL_INT32;
    const bool a8w4 = a8w4f || a8w4i;
    if (!a8w4 && yScale != nullptr && !yScale->empty()) {
        set_err("aclnnQuantMatmulV5GetWorkspaceSize: yScale must be nullptr or empty");
        return ACLNN_ERR_PARAM_NULLPTR;
    }
    if (x1Offset != nullptr && !x1Offset->empty()) {
        set_err("aclnnQuantMatmulV5GetWorkspaceSize: x1Offset must be nullptr or empty");
        return ACLNN_ERR_PARAM_NULLPTR;
    }
    if (a8w4 && x2Offset != nullptr) {
        set_err("aclnnQuantMatmulV5GetWorkspaceSize: x2Offset must be nullptr in A8W4 mode");
        return ACLNN_ERR_PARAM_NULLPTR;
    }
    if (yOffset != nullptr && !yOffset->empty() && !a8w4i) {
        set_err("aclnnQuantMatmulV5GetWorkspaceSize: yOffset must be nullptr or empty");
        return ACLNN_ERR_PARAM_NULLPTR;
    }
    int64_t group = groupSize;
    if (a8w4f) {  // A8W4InferGroupSize (:1045-1061)
        Group g = decode_group(group);
        if (!((g.m == 0 && g.n == 0) || (g.m == 1 && g.n == 1))) {
            set_err("A8W4: groupSizeM and groupSizeN must both be 0 or both be 1");
            return ACLNN_ERR_PARAM_INVALID;
        }
        group = (int64_t)g.k;
    }

    auto exec = std::make_unique<aclOpExecutor>();
    exec->kind = ExecKind::kQmm;

    // empty output short-cut (:1088-1108)
    if (!a8w4 && x1->rank() >= 2 && x2->rank() >= 2) {
        int64_t mm = transposeX1 ? x1->dim(-1) : x1->dim(-2);
        int64_t nn = transposeX2 ? x2->dim(-2) : x2->dim(-1);
        if (mm == 0 || nn == 0) {
            exec->nothing_to_do = true;
            *workspaceSize = 0;
            *executor = exec.release();
            return ACLNN_SUCCESS;
        }
    }

    Ctx c;
    c.x1 = *x1;
    c.x2 = *x2;
    c.out = *out;
    c.x2s = *x2Scale;
    if (x1Scale) { c.has_x1s = true; c.x1s = *x1Scale; }
    if (x2Offset) { c.has_x2o = true; c.x2o = *x2Offset; }
    if (bias) { c.has_bias = true; c.bias = *bias; }
    if (yScale && !yScale->empty()) { c.has_ys = true; c.ys = *yScale; }
    if (yOffset && !yOffset->empty()) { c.has_yo = true; c.yo = *yOffset; }
    if (yScale && yScale->empty() && a8w4) { c.has_ys = true; c.ys = *yScale; }
    c.t1 = transposeX1;
    c.t2 = transposeX2;
    c.group = group;
    if (c.x2s.dtype == ACL_INT64) c.x2s.dtype = ACL_UINT64;

    // PreMatmulCalcProcess (:967-1016): strided-transposed views flip the flags
    if (c.x1.rank() >= 2) normalise_view(c.x1, &c.t1);
    if (c.x2.rank() >= 2) normalise_view(c.x2, &c.t2);
    c.dims();

    if (a8w4f) {
        aclnnStatus st = check_a8w4_float(c, x1Scale, group);
        if (st != ACLNN_SUCCESS) return st;
        // Plan: the fp4 weight is rewritten as fp8 into the workspace, then the fp8 kernels run (mx: block-scaled matmul
        // on the widened weight; T-CG: group scale folded into the rewrite, yScale is the per-channel dequant scale).
        OpsnnQmmParams& p = exec->qmm;
        const bool is_mx = c.has_x1s && c.x2s.dtype == ACL_FLOAT8_E8M0;
        p.a_dtype = c.x1.dtype;
        p.b_dtype = c.x2.dtype;
        p.out_dtype = c.out.dtype;
        p.bias_dtype = c.has_bias ? (int)c.bias.dtype : -1;
        p.trans_a = 0;
        p.trans_b = 1;
        p.m = c.m; p.n = c.n; p.k = c.k1; p.batch = 1;
        int64_t ld = 0, bs = 0;
        auto why_unsupported = [&](const char* w) {
            exec->unsupported = true;
            exec->unsupported_why = w;
        };
        if (!row_strided_view(&c.x1, &ld, &bs)) why_unsupported("x1 is neither contiguous nor row-strided");
        p.a_ld = ld;
        if (!row_strided_view(&c.x2, &ld, &bs)) why_unsupported("x2 is neither contiguous nor row-strided");
        p.b_ld = ld;
        if (!row_strided_view(&c.out, &ld, &bs)) why_unsupported("out must be contiguous or row-strided");
        p.out_ld = ld;
        p.out_bs = c.m * ld;
        p.a = data_ptr(&c.x1);
        p.b = data_ptr(&c.x2);
        p.out = const_cast<uint8_t*>(data_ptr(&c.out));
        p.bias = c.has_bias ? data_ptr(&c.bias) : nullptr;
        for (const aclTensor* t : {&c.x2s, c.has_x1s ? &c.x1s : nullptr, c.has_bias ? &c.bias : nullptr, c.has_ys ? &c.ys : nullptr}) {
            if (t != nullptr && !is_contiguous(t)) why_unsupported("scale/bias tensors must be contiguous");
        }
        p.group_m = 1; p.group_n = 1; p.group_k = 32;
        if (is_mx) {
            p.mode = OPSNN_QMM_MX;
            p.b_prepass = OPSNN_B_PREPASS_WIDEN;
            p.scale_a = data_ptr(&c.x1s);
            p.scale_b = data_ptr(&c.x2s);
            p.scale_b_dtype = ACL_FLOAT8_E8M0;
            p.pre_scale_dtype = -1;
        } else {
            p.mode = OPSNN_QMM_DEQ;
            p.b_prepass = OPSNN_B_PREPASS_GROUP_SCALE;
            p.pre_scale = data_ptr(&c.x2s);
            p.pre_scale_dtype = c.x2s.dtype;
            p.pre_group = 32;
            p.scale_a = nullptr;
            p.scale_b = data_ptr(&c.ys);
            p.scale_b_dtype = ACL_UINT64;
            p.scale_b_len = c.n;
        }
        exec->kernel_choice = OPSNN_KERNEL_AUTO;
        if (const char* e = std::getenv("OPSNN_QMM_KERNEL")) exec->kernel_choice = std::atoi(e);
        if (!exec->unsupported) {
            if (exec->kernel_choice == OPSNN_KERNEL_AUTO) exec->kernel_choice = opsnn_qmm_select_kernel(&p);
            exec->workspace_size = opsnn_qmm_workspace_size(&p, exec->kernel_choice);
        }
        *workspaceSize = exec->workspace_size;
        log_info("aclnnQuantMatmulV5 plan: A8W4 %s m=%ld n=%ld k=%ld kernel=%d ws=%lu", is_mx ? "mx" : "T-CG", (long)p.m,
                 (long)p.n, (long)p.k, exec->kernel_choice, (unsigned long)exec->workspace_size);
        *executor = exec.release();
        return ACLNN_SUCCESS;
    }
    if (a8w4i) {
        // CheckParamsA8W4Int (:736-752): only Atlas A2/A3 implement int8 x packed-int4; other targets report a runtime error
        set_err("aclnnQuantMatmulV5GetWorkspaceSize: INT8 x INT32(int4) pseudo-quant is not implemented for this target");
        return ACLNN_ERR_RUNTIME_ERROR;
    }
    // CheckDimRange (:285-325)
    if (c.x2.storage_shape.size() < 2 || c.x2.storage_shape.size() > 6) {
        set_err("x2 must have 2..6 dims, got %zu", c.x2.storage_shape.size());
        return ACLNN_ERR_PARAM_INVALID;
    }
    if (c.x1.rank() < 2 || c.x1.rank() > 6) {
        set_err("x1 must have 2..6 dims, got %zu", c.x1.rank());
        return ACLNN_ERR_PARAM_INVALID;
    }
    if (c.out.rank() < 2 || c.out.rank() > 6) {
        set_err("out must have 2..6 dims, got %zu", c.out.rank());
        return ACLNN_ERR_PARAM_INVALID;
    }
    if (c.x2.rank() < 2 || c.x2.rank() > 6) {
        set_err("x2 must have 2..6 dims, got %zu", c.x2.rank());
        return ACLNN_ERR_PARAM_INVALID;
    }
    // A4W4CaseProcess: INT32 words are re-viewed as 8 INT4 along the inner axis (quant_matmul_common_check.cpp:140-169)
    for (aclTensor* t : {&c.x1, &c.x2}) {
        if (t->dtype == ACL_INT32) {
            t->shape.back() *= 8;
            for (size_t i = 0; i + 1 < t->rank(); ++i) t->strides[i] *= 8;
            t->offset *= 8;
            t->dtype = ACL_INT4;
        }
    }
    c.dims();
    if (!infer_group(c, c.group)) return ACLNN_ERR_PARAM_INVALID;
    if (!check_dtype(c)) return ACLNN_ERR_PARAM_INVALID;
    if (!check_shape(c)) return ACLNN_ERR_PARAM_INVALID;
    for (const aclTensor* t : {&c.x1, &c.x2s, &c.out}) {
        if (t->format != ACL_FORMAT_ND) {
            set_err("only ACL_FORMAT_ND tensors are accepted");
            return ACLNN_ERR_PARAM_INVALID;
        }
    }
    if (c.x1.empty() || c.x2.empty()) {
        set_err("x1 and x2 can not be empty");
        return ACLNN_ERR_PARAM_INVALID;
    }

    // ---------------- plan ----------------
    OpsnnQmmParams& p = exec->qmm;
    p.a_dtype = c.x1.dtype;
    p.b_dtype = c.x2.dtype;
    p.out_dtype = c.out.dtype;
    p.bias_dtype = c.has_bias ? (int)c.bias.dtype : -1;
    p.scale_b_dtype = c.x2s.dtype;
    p.trans_a = c.t1;
    p.trans_b = c.t2;
    p.m = c.m;
    p.n = c.n;
    p.k = c.k1;
    std::vector<int64_t> ob(c.out.shape.begin(), c.out.shape.end() - 2);
    if (c.out.rank() == 3 && c.x1.rank() == 2 && c.x2.rank() == 2 && c.out.shape[1] == 1 && c.m != 1) ob.clear();
    p.batch = 1;
    for (auto d : ob) p.batch *= d;
    auto why_unsupported = [&](const char* w) {
        exec->unsupported = true;
        exec->unsupported_why = w;
    };
    int64_t ld = 0, bs = 0;
    if (!row_strided_view(&c.x1, &ld, &bs)) why_unsupported("x1 is neither contiguous, row-strided nor a transposed view");
    p.a_ld = ld;
    if (!operand_batch(c.x1, 2, ob, bs, &p.a_bs)) why_unsupported("x1 batch dims broadcast partially");
    if (c.x1.rank() > 2 && p.a_bs != 0 && bs == 0) p.a_bs = c.x1.dim(-2) * ld;
    if (!row_strided_view(&c.x2, &ld, &bs)) why_unsupported("x2 is neither contiguous, row-strided nor a transposed view");
    p.b_ld = ld;
    if (!operand_batch(c.x2, 2, ob, bs, &p.b_bs)) why_unsupported("x2 batch dims broadcast partially");
    if (c.x2.rank() > 2 && p.b_bs != 0 && bs == 0) p.b_bs = c.x2.dim(-2) * ld;
    if (!row_strided_view(&c.out, &ld, &bs)) why_unsupported("out must be contiguous or row-strided");
    p.out_ld = ld;
    p.out_bs = bs != 0 ? bs : c.m * ld;
    p.a = data_ptr(&c.x1);
    p.b = data_ptr(&c.x2);
    p.out = const_cast<uint8_t*>(data_ptr(&c.out));
    p.scale_a = c.has_x1s ? data_ptr(&c.x1s) : nullptr;
    p.scale_b = data_ptr(&c.x2s);
    p.bias = c.has_bias ? data_ptr(&c.bias) : nullptr;
    p.bias_bs = (c.has_bias && c.bias.rank() == 3) ? c.n : 0;
    for (const aclTensor* t : {&c.x2s, c.has_x1s ? &c.x1s : nullptr, c.has_bias ? &c.bias : nullptr}) {
        if (t != nullptr && !is_contiguous(t)) why_unsupported("scale/bias tensors must be contiguous");
    }
    const Group g = decode_group(c.group);
    p.group_m = (int32_t)g.m;
    p.group_n = (int32_t)g.n;
    p.group_k = (int32_t)g.k;
    if (c.mx()) {
        p.mode = OPSNN_QMM_MX;
        // canonical layouts only: x1Scale follows transposeX1, x2Scale follows transposeX2
        size_t b1 = c.x1s.rank() - 3, b2 = c.x2s.rank() - 3;
        int64_t kq = ceil_div(c.k1, 64);
        bool ok1 = c.x1s.shape[b1 + (c.t1 ? 1 : 0)] == c.m && c.x1s.shape[b1 + (c.t1 ? 0 : 1)] == kq;
        bool ok2 = c.x2s.shape[b2 + (c.t2 ? 0 : 1)] == c.n && c.x2s.shape[b2 + (c.t2 ? 1 : 0)] == kq;
        if (!ok1 || !ok2) why_unsupported("mx scale stored with a transposition different from its operand");
        if (!operand_batch(c.x1s, 3, ob, c.m * kq * 2, &p.sa_bs)) why_unsupported("x1Scale batch dims");
        if (!operand_batch(c.x2s, 3, ob, c.n * kq * 2, &p.sb_bs)) why_unsupported("x2Scale batch dims");
    } else if (c.int4_in() && c.has_x2o) {
        // INT4 x INT4 asymmetric per-group: operands widened to INT8 in the workspace, per-group epilogue in the coverage kernel
        p.mode = OPSNN_QMM_PERGROUP_ASYM;
        p.a_prepass = OPSNN_PREPASS_WIDEN_INT4;
        p.b_prepass = OPSNN_PREPASS_WIDEN_INT4;
        p.group_k = 256;
        p.b_offset = data_ptr(&c.x2o);
        if (!is_contiguous(&c.x2o)) why_unsupported("x2Offset must be contiguous");
        if (p.batch != 1) why_unsupported("INT4 per-group asymmetric takes 2-D operands");
    } else if (c.perblock()) {
        p.mode = OPSNN_QMM_PERBLOCK;
        if (c.hif8_in()) why_unsupported("HIFLOAT8 has no implementation here");
        if (!operand_batch(c.x1s, 2, ob, c.x1s.dim(-1) * c.x1s.dim(-2), &p.sa_bs)) why_unsupported("x1Scale batch dims");
        if (!operand_batch(c.x2s, 2, ob, c.x2s.dim(-1) * c.x2s.dim(-2), &p.sb_bs)) why_unsupported("x2Scale batch dims");
    } else {
        p.mode = OPSNN_QMM_DEQ;
        p.scale_b_len = c.x2s.shape[0];
        p.scale_a_len = c.has_x1s ? c.x1s.shape[0] : 0;
        if (c.hif8_in()) why_unsupported("HIFLOAT8 has no implementation here");
        if (c.int4_in()) {
            {  // sign-extend both operands to INT8 in the workspace, then the INT8 kernels (same integers, same result)
                p.a_prepass = OPSNN_PREPASS_WIDEN_INT4;
                p.b_prepass = OPSNN_PREPASS_WIDEN_INT4;
            }
        }
        if (c.out.dtype == ACL_INT8) {
            // requantised output: the offset tensor only says that the packed scale carries one (QuantBatchMatmulV3TestSpec.golden,
            // qbmmv3_kernel_golden.py:726-731)
            p.deq_flags |= OPSNN_DEQ_REQUANT;
            if (c.has_x2o) p.deq_flags |= OPSNN_DEQ_REQUANT_OFFSET;
        }
        // Rounding-point rules of the reference golden (qbmmv3_kernel_golden.py:566-577, 641-692;
        // matmul_quant_util.py:62-72): which scales lose their low 13 bits, and where a float bias is added.
        const bool float_bias = c.has_bias && in(c.bias.dtype, {ACL_FLOAT, ACL_BF16, ACL_FLOAT16});
        const bool double_scale = c.fp8_in() && c.has_x1s && c.x1s.shape[0] == 1;
        if (c.int8_in() && !c.has_x1s && c.x2s.dtype != ACL_UINT64 && c.x2s.shape[0] == 1 &&
            !(c.has_bias && in(c.bias.dtype, {ACL_BF16, ACL_FLOAT})))
            p.deq_flags |= OPSNN_DEQ_TRUNC_SCALE_B;
        if (double_scale && c.x2s.shape[0] == 1 && !float_bias) p.deq_flags |= OPSNN_DEQ_MERGE_TRUNC;
        if (c.fp8_in() && !c.has_x1s && float_bias) p.deq_flags |= OPSNN_DEQ_FBIAS_BEFORE_SCALE;
    }
    exec->kernel_choice = OPSNN_KERNEL_AUTO;
    if (const char* e = std::getenv("OPSNN_QMM_KERNEL")) exec->kernel_choice = std::atoi(e);
    if (!exec->unsupported) {
        if (exec->kernel_choice == OPSNN_KERNEL_AUTO) exec->kernel_choice = opsnn_qmm_select_kernel(&p);
        if (exec->kernel_choice == OPSNN_KERNEL_UMMA) attach_prepared(&p);  // an x2 registered by opsnnQuantMatmulPrepareX2
        exec->workspace_size = opsnn_qmm_workspace_size(&p, exec->kernel_choice);
    }
    *workspaceSize = exec->workspace_size;
    log_info("aclnnQuantMatmulV5 plan: mode=%d b=%ld m=%ld n=%ld k=%ld tA=%d tB=%d kernel=%d ws=%lu%s", p.mode,
             (long)p.batch, (long)p.m, (long)p.n, (long)p.k, p.trans_a, p.trans_b, exec->kernel_choice,
             (unsigned long)exec->workspace_size, exec->unsupported ? " (no kernel)" : "");
    *executor = exec.release();
    return ACLNN_SUCCESS;
}

static aclnnStatus qmm_run(const char* api, void* workspace, uint64_t workspaceSize, aclOpExecutor* executor, aclrtStream stream)
{
    clear_err();
    if (executor == nullptr) {
        set_err("%s: executor is nullptr", api);
        return ACLNN_ERR_PARAM_NULLPTR;
    }
    std::unique_ptr<aclOpExecutor> exec(executor);  // phase 2 consumes the executor
    if (exec->magic != 0x4F50534E || exec->kind != ExecKind::kQmm) {
        exec.release();
        set_err("%s: executor was not created by the matching GetWorkspaceSize call", api);
        return ACLNN_ERR_PARAM_INVALID;
    }
    exec->magic = 0;
    if (exec->nothing_to_do) return ACLNN_SUCCESS;
    if (exec->unsupported) {
        set_err("%s: %s", api, exec->unsupported_why.c_str());
        return ACLNN_ERR_INNER_FIND_KERNEL_ERROR;
    }
    if (workspaceSize < exec->workspace_size || (exec->workspace_size > 0 && workspace == nullptr)) {
        set_err("%s: workspace too small (%lu < %lu)", api, (unsigned long)workspaceSize, (unsigned long)exec->workspace_size);
        return ACLNN_ERR_PARAM_INVALID;
    }
    if (exec->dyn_quant) {  // 16-bit x1: quantised into the head of the workspace first, the matmul reads it from there
        if (exec->mxq.x == nullptr) {
            set_err("%s: a tensor was created without a device address", api);
            return ACLNN_ERR_PARAM_NULLPTR;
        }
        uint8_t* ws = static_cast<uint8_t*>(workspace);
        exec->mxq.y = ws;
        exec->mxq.scale = ws + exec->dq_q_bytes;
        const int32_t rc = opsnn_mx_quant_launch(&exec->mxq, stream);
        if (rc != 0) {
            set_err("%s: the activation quantiser failed with CUDA error %d", api, rc);
            return ACLNN_ERR_RUNTIME_ERROR;
        }
        exec->qmm.a = ws;
        exec->qmm.scale_a = ws + exec->dq_q_bytes;
        workspace = ws + exec->dq_q_bytes + exec->dq_s_bytes;
        workspaceSize -= exec->dq_q_bytes + exec->dq_s_bytes;
    }
    if (exec->nz_bytes != 0) {  // FRACTAL_NZ x2: row-major copy into the head of the workspace, the matmul gets the rest
        if (exec->nz_src == nullptr) {
            set_err("%s: a tensor was created without a device address", api);
            return ACLNN_ERR_PARAM_NULLPTR;
        }
        const int32_t rc = opsnn_nz_to_nd_launch(exec->nz_src, workspace, exec->nz_rows, exec->nz_row_bytes, exec->nz_r0, exec->nz_c0_bytes, stream);
        if (rc != 0) {
            set_err("%s: the FRACTAL_NZ -> row-major copy failed with CUDA error %d", api, rc);
            return ACLNN_ERR_RUNTIME_ERROR;
        }
        exec->qmm.b = workspace;
        workspace = static_cast<uint8_t*>(workspace) + exec->nz_bytes;
        workspaceSize -= exec->nz_bytes;
    }
    if (exec->qmm.a == nullptr || exec->qmm.b == nullptr || exec->qmm.out == nullptr || exec->qmm.scale_b == nullptr) {
        set_err("%s: a tensor was created without a device address", api);
        return ACLNN_ERR_PARAM_NULLPTR;
    }
    exec->qmm.workspace = workspace;
    exec->qmm.workspace_size = workspaceSize;
    int32_t rc = opsnn_qmm_launch(&exec->qmm, exec->kernel_choice, stream);
    if (rc != 0) {
        const std::string why = aclGetRecentErrMsg() ? aclGetRecentErrMsg() : "";
        set_err("%s: kernel launch failed with CUDA error %d%s%s", api, rc, why.empty() ? "" : ": ", why.c_str());
        return ACLNN_ERR_RUNTIME_ERROR;
    }
    return ACLNN_SUCCESS;
}

aclnnStatus aclnnQuantMatmulV5(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor, aclrtStream stream)
{
    OPSNN_DFX_RANGE("aclnnQuantMatmulV5");
    return qmm_run("aclnnQuantMatmulV5", workspace, workspaceSize, executor, stream);
}

// ---- aclnnQuantMatmulWeightNz (matmul/quant_batch_matmul_v3/op_api/aclnn_quant_matmul_weight_nz.h:41-55): aclnnQuantMatmulV5's
// arguments with x2 stored FRACTAL_NZ. The fractal layout feeds the Ascend cube unit and has no use on this hardware, so phase 2
// first rewrites x2 row-major into the head of the workspace (one copy kernel) and the ND plan runs on that. ----

aclnnStatus aclnnQuantMatmulWeightNzGetWorkspaceSize(const aclTensor* x1, const aclTensor* x2, const aclTensor* x1Scale,
                                                     const aclTensor* x2Scale, const aclTensor* yScale, const aclTensor* x1Offset,
                                                     const aclTensor* x2Offset, const aclTensor* yOffset, const aclTensor* bias,
                                                     bool transposeX1, bool transposeX2, int64_t groupSize, aclTensor* out,
                                                     uint64_t* workspaceSize, aclOpExecutor** executor)
{
    OPSNN_DFX_RANGE("aclnnQuantMatmulWeightNzGetWorkspaceSize");
    const char* api = "aclnnQuantMatmulWeightNzGetWorkspaceSize";
    clear_err();
    if (workspaceSize == nullptr || executor == nullptr || x2 == nullptr) {
        set_err("%s: x2, workspaceSize and executor are required", api);
        return ACLNN_ERR_PARAM_NULLPTR;
    }
    if (x2->format != ACL_FORMAT_FRACTAL_NZ && x2->format != ACL_FORMAT_FRACTAL_NZ_C0_32) {  // aclnn_quant_matmul_v4.cpp:855
        set_err("%s: x2's storage format must be FRACTAL_NZ", api);
        return ACLNN_ERR_PARAM_INVALID;
    }
    // storage dims [ceil(cols / c0), ceil(rows / r0), r0, c0] over the 2-D matrix the view describes
    const auto& sd = x2->storage_shape;
    const int bits = dtype_bits(x2->dtype);
    if (x2->rank() != 2 || sd.size() != 4 || bits == 0) {
        set_err("%s: a FRACTAL_NZ x2 needs a 2-D view and 4 storage dims", api);
        return ACLNN_ERR_PARAM_INVALID;
    }
    const int64_t rows = x2->shape[0], cols = x2->shape[1], c1 = sd[0], r1 = sd[1], r0 = sd[2], c0 = sd[3];
    if (r0 <= 0 || c0 <= 0 || r0 > 4096 || c0 > 4096 || c1 != (cols + c0 - 1) / c0 || r1 != (rows + r0 - 1) / r0 || (cols * bits) % 8 != 0 ||
        (c0 * bits) % 8 != 0) {
        set_err("%s: storage dims [%ld,%ld,%ld,%ld] do not tile the (%ld,%ld) view", api, (long)c1, (long)r1, (long)r0, (long)c0, (long)rows,
                (long)cols);
        return ACLNN_ERR_PARAM_INVALID;
    }
    aclTensor nd = *x2;  // the plan sees the row-major matrix the pre-pass leaves in the workspace
    nd.format = ACL_FORMAT_ND;
    nd.strides = {cols, 1};
    nd.storage_shape = nd.shape;
    nd.offset = 0;
    nd.data = reinterpret_cast<void*>(uintptr_t(256));  // stand-in with allocation alignment: kernel selection looks at alignment only
    const aclnnStatus st = aclnnQuantMatmulV5GetWorkspaceSize(x1, &nd, x1Scale, x2Scale, yScale, x1Offset, x2Offset, yOffset, bias, transposeX1,
                                                              transposeX2, groupSize, out, workspaceSize, executor);
    if (st != ACLNN_SUCCESS) return st;
    aclOpExecutor* exec = *executor;
    exec->qmm.b = nullptr;
    exec->nz_src = x2->data == nullptr ? nullptr : data_ptr(x2);
    exec->nz_rows = rows;
    exec->nz_row_bytes = cols * bits / 8;
    exec->nz_r0 = r0;
    exec->nz_c0_bytes = c0 * bits / 8;
    exec->nz_bytes = (((uint64_t)rows * (uint64_t)exec->nz_row_bytes) + 255u) & ~(uint64_t)255u;
    if (exec->nothing_to_do) exec->nz_bytes = 0;
    exec->workspace_size += exec->nz_bytes;
    *workspaceSize = exec->workspace_size;
    return ACLNN_SUCCESS;
}

aclnnStatus aclnnQuantMatmulWeightNz(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor, aclrtStream stream)
{
    OPSNN_DFX_RANGE("aclnnQuantMatmulWeightNz");
    return qmm_run("aclnnQuantMatmulWeightNz", workspace, workspaceSize, executor, stream);
}

// ---- older entry points of the same operator (matmul/quant_batch_matmul_v3/op_api/aclnn_quant_matmul_v4.h:41-60,
// aclnn_quant_matmul_v3.h:40-58): argument order (scale, offset, pertokenScale, bias), no groupSize; same plans and kernels ----

aclnnStatus aclnnQuantMatmulV4GetWorkspaceSize(const aclTensor* x1, const aclTensor* x2, const aclTensor* scale,
                                               const aclTensor* offset, const aclTensor* pertokenScaleOptional,
                                               const aclTensor* bias, bool transposeX1, bool transposeX2, const aclTensor* out,
                                               uint64_t* workspaceSize, aclOpExecutor** executor)
{
    OPSNN_DFX_RANGE("aclnnQuantMatmulV4GetWorkspaceSize");
    return aclnnQuantMatmulV5GetWorkspaceSize(x1, x2, pertokenScaleOptional, scale, nullptr, nullptr, offset, nullptr, bias, transposeX1,
                                              transposeX2, 0, const_cast<aclTensor*>(out), workspaceSize, executor);
}

aclnnStatus aclnnQuantMatmulV4(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor, aclrtStream stream)
{
    OPSNN_DFX_RANGE("aclnnQuantMatmulV4");
    return aclnnQuantMatmulV5(workspace, workspaceSize, executor, stream);
}

aclnnStatus aclnnQuantMatmulV3GetWorkspaceSize(const aclTensor* x1, const aclTensor* x2, const aclTensor* scale,
                                               const aclTensor* offset, const aclTensor* bias, bool transposeX1, bool transposeX2,
                                               const aclTensor* out, uint64_t* workspaceSize, aclOpExecutor** executor)
{
    OPSNN_DFX_RANGE("aclnnQuantMatmulV3GetWorkspaceSize");
    return aclnnQuantMatmulV5GetWorkspaceSize(x1, x2, nullptr, scale, nullptr, nullptr, offset, nullptr, bias, transposeX1, transposeX2, 0,
                                              const_cast<aclTensor*>(out), workspaceSize, executor);
}

aclnnStatus aclnnQuantMatmulV3(void* workspace, uint64_t workspaceSize, aclOpExecutor* executor, aclrtStream stream)
{
    OPSNN_DFX_RANGE("aclnnQuantMatmulV3");
    return aclnnQuantMatmulV5(workspace, workspaceSize, executor, stream);
}

// ---- prepare-once x2 (include/opsnn_b200_prepare.h) ----------------------------------------------------------------------------

static aclnnStatus plan_on_x2(const char* api, const aclTensor* x2, const aclTensor* x2Scale, bool transposeX2, int64_t groupSize,
                              int64_t mHint, std::unique_ptr<aclOpExecutor>* exec_out)
{
    if (x2 == nullptr || x2Scale == nullptr) {
        set_err("%s: x2 and x2Scale are required", api);
        return ACLNN_ERR_PARAM_NULLPTR;
    }
    if (mHint < 1 || x2->rank() < 2) {
        set_err("%s: mHint must be >= 1 and x2 at least 2-D", api);
        return ACLNN_ERR_PARAM_INVALID;
    }
    HintTensors h;
    make_hint(x2, x2Scale, transposeX2, mHint, &h);
    uint64_t ws = 0;
    aclOpExecutor* ex = nullptr;
    const aclnnStatus st = aclnnQuantMatmulV5GetWorkspaceSize(&h.x1, x2, &h.x1s, x2Scale, nullptr, nullptr, nullptr, nullptr, nullptr, false,
                                                              transposeX2, groupSize, &h.out, &ws, &ex);
    if (st != ACLNN_SUCCESS) return st;
    exec_out->reset(ex);
    return ACLNN_SUCCESS;
}

aclnnStatus opsnnQuantMatmulPrepareX2GetStorageSize(const aclTensor* x2, const aclTensor* x2Scale, bool transposeX2, int64_t groupSize,
                                                    int64_t mHint, uint64_t* storageSize)
{
    OPSNN_DFX_RANGE("opsnnQuantMatmulPrepareX2GetStorageSize");
    const char* api = "opsnnQuantMatmulPrepareX2GetStorageSize";
    clear_err();
    if (storageSize == nullptr) {
        set_err("%s: storageSize is nullptr", api);
        return ACLNN_ERR_PARAM_NULLPTR;
    }
    *storageSize = 0;
    if (x2 != nullptr && x2Scale != nullptr && x2Scale->dtype != ACL_FLOAT8_E8M0) return ACLNN_SUCCESS;  // not an MX mode: nothing to prepare
    std::unique_ptr<aclOpExecutor> exec;
    const aclnnStatus st = plan_on_x2(api, x2, x2Scale, transposeX2, groupSize, mHint, &exec);
    if (st != ACLNN_SUCCESS) return st;
    if (!exec->unsupported && !exec->nothing_to_do && exec->kernel_choice == OPSNN_KERNEL_UMMA) {
        exec->qmm.prep_b = exec->qmm.prep_sfb = nullptr;  // size of a fresh preparation, also when one is registered already
        exec->qmm.prep_bn = 0;
        *storageSize = opsnn_qmm_prepare_b_size(&exec->qmm);
    }
    return ACLNN_SUCCESS;
}

aclnnStatus opsnnQuantMatmulPrepareX2(const aclTensor* x2, const aclTensor* x2Scale, bool transposeX2, int64_t groupSize, int64_t mHint,
                                      void* storage, uint64_t storageSize, aclrtStream stream)
{
    OPSNN_DFX_RANGE("opsnnQuantMatmulPrepareX2");
    const char* api = "opsnnQuantMatmulPrepareX2";
    clear_err();
    if (x2 != nullptr && x2Scale != nullptr && x2Scale->dtype != ACL_FLOAT8_E8M0) return ACLNN_SUCCESS;  // not an MX mode: nothing to prepare
    std::unique_ptr<aclOpExecutor> exec;
    const aclnnStatus st = plan_on_x2(api, x2, x2Scale, transposeX2, groupSize, mHint, &exec);
    if (st != ACLNN_SUCCESS) return st;
    if (exec->unsupported || exec->nothing_to_do || exec->kernel_choice != OPSNN_KERNEL_UMMA) return ACLNN_SUCCESS;  // nothing to prepare
    OpsnnQmmParams& p = exec->qmm;
    if (p.b == nullptr || p.scale_b == nullptr) {
        set_err("%s: x2 / x2Scale were created without a device address", api);
        return ACLNN_ERR_PARAM_NULLPTR;
    }
    p.prep_b = p.prep_sfb = nullptr;
    p.prep_bn = 0;
    PreparedX2 e;
    const int32_t rc = opsnn_qmm_prepare_b_launch(&p, storage, storageSize, &e.prep_b, &e.prep_sfb, &e.prep_bn, stream);
    if (rc != 0) {
        set_err("%s: preparation failed with CUDA error %d (storage of %lu bytes needed)", api, rc, (unsigned long)opsnn_qmm_prepare_b_size(&p));
        return rc == 1 /* cudaErrorInvalidValue */ ? ACLNN_ERR_PARAM_INVALID : ACLNN_ERR_RUNTIME_ERROR;
    }
    if (e.prep_bn == 0) return ACLNN_SUCCESS;
    e.key = p;
    std::unique_lock<std::shared_mutex> lk(g_prepared_mu);
    g_prepared[p.b] = e;
    return ACLNN_SUCCESS;
}

aclnnStatus opsnnQuantMatmulReleaseX2(const aclTensor* x2)
{
    OPSNN_DFX_RANGE("opsnnQuantMatmulReleaseX2");
    clear_err();
    if (x2 == nullptr) return ACLNN_ERR_PARAM_NULLPTR;
    std::unique_lock<std::shared_mutex> lk(g_prepared_mu);
    g_prepared.erase(data_ptr(x2));
    return ACLNN_SUCCESS;
}

}  // extern "C"
