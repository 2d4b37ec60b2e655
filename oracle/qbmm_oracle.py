"""numpy restatement of the reference's full-quant matmul golden (aclnnQuantMatmulV5 path).

Follows matmul/quant_batch_matmul_v3/tests/assets/qbmmv3_kernel_golden.py of the reference:
  determine_quant_mode :62-145, compute_mx :153-234, compute_perblock :237-358, compute_pertoken :361-387,
  compute_tc :390-462, compute_int32 :490-506, dispatch :509-699;
and matmul/common/tests/st/arch35/matmul_quant_util.py: scale_generate :50-54, needs_scale_generate :62-72,
u64_to_deq_scale :129-134, unpack_groupsize :179-190.

Test infrastructure only (see oracle/__init__.py).
"""
import ml_dtypes
import numpy as np

BF16 = ml_dtypes.bfloat16
E4M3 = ml_dtypes.float8_e4m3fn
E5M2 = ml_dtypes.float8_e5m2
E2M1 = ml_dtypes.float4_e2m1fn
E8M0 = ml_dtypes.float8_e8m0fnu
INT4 = ml_dtypes.int4

_OUT = {"bfloat16": BF16, "float16": np.float16, "float32": np.float32, "int32": np.int32}


def cast_out(arr, name):
    return arr.astype(_OUT[name])


def trunc19(a):
    """Keep the top 19 bits of an fp32 array (matmul_quant_util.py:50-54)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).copy()
    u &= np.uint32(0xFFFFE000)
    return u.view(np.float32)


def u64_to_deq_scale(u64):
    """matmul_quant_util.py:129-134"""
    lo = (np.asarray(u64).astype(np.uint64) & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    lo &= np.uint32(0xFFFFE000)
    return lo.view(np.float32).reshape(np.shape(u64))


def u64_to_offset(u64):
    """Signed 9-bit offset in bits 37..45 of the packed scale (matmul_quant_util.py:137-143)."""
    raw = ((np.asarray(u64).astype(np.uint64) >> np.uint64(37)) & np.uint64(0x1FF)).astype(np.int64)
    raw = np.where(raw & 0x100, raw - 0x200, raw)
    return raw.astype(np.float32).reshape(np.shape(u64))


def f32_2_s9(a):
    """Round half to even, clip to nine signed bits (matmul_quant_util.py:57-59)."""
    return np.clip(np.round(a), -256, 255)


def unpack_groupsize(g):
    gm, gn, gk = (g >> 32) & 0xFFFF, (g >> 16) & 0xFFFF, g & 0xFFFF
    return gm or 1, gn or 1, gk or 1


def _is_fp8(dt):
    return dt in (np.dtype(E4M3), np.dtype(E5M2))


def _t(a):
    return np.swapaxes(a, -1, -2)


def mx_scales_to_2d(x1_scale, x2_scale, transpose_x1, transpose_x2, k):
    """e8m0 scales in the reference's wire layout -> (m, groups) and (groups, n) fp32 (qbmmv3_kernel_golden.py:166-202).

    x1Scale is (m, ceil(k/64), 2), or (ceil(k/64), m, 2) when x1 is stored (k, m); x2Scale is (ceil(k/64), n, 2), or
    (n, ceil(k/64), 2) when x2 is stored (n, k). Group g = 2p + j sits at [.., p, .., j]. An odd group count means the
    last entry is padding.
    """
    s1 = x1_scale.astype(np.float32)
    s2 = x2_scale.astype(np.float32)
    if transpose_x1:  # (kq, m, 2) -> (m, 2kq)
        s1 = np.transpose(s1, (1, 0, 2)).reshape(s1.shape[1], -1)
    else:
        s1 = s1.reshape(s1.shape[0], -1)
    if transpose_x2:  # (n, kq, 2) -> (2kq, n)
        s2 = s2.reshape(s2.shape[0], -1).T
    else:  # (kq, n, 2) -> (2kq, n)
        s2 = np.transpose(s2, (0, 2, 1)).reshape(-1, s2.shape[1])
    if -(-k // 32) % 2 != 0:
        s1 = s1[:, :-1]
        s2 = s2[:-1, :]
    return s1, s2


def compute_mx(x1, x2, x1_scale, x2_scale, bias, transpose_x1, transpose_x2, out_dtype):
    """2-D operands (call per batch). qbmmv3_kernel_golden.py:153-234"""
    a = x1.astype(np.float32)
    b = x2.astype(np.float32)
    if transpose_x1:
        a = a.T
    if transpose_x2:
        b = b.T
    k = a.shape[-1]
    s1, s2 = mx_scales_to_2d(x1_scale, x2_scale, transpose_x1, transpose_x2, k)
    s1 = np.repeat(s1, 32, axis=-1)
    s2 = np.repeat(s2, 32, axis=-2)
    if s1.shape[-1] > k:
        a = np.pad(a, [(0, 0), (0, s1.shape[-1] - k)])
    if s2.shape[-2] > k:
        b = np.pad(b, [(0, s2.shape[-2] - k), (0, 0)])
    y = np.matmul(a * s1, b * s2)
    if bias is not None:
        y = y + bias.astype(np.float32)
    return cast_out(y, out_dtype)


def compute_t_cg(x1, x2, x2_scale, y_scale, transpose_x1, transpose_x2, group_k, out_dtype, bias=None):
    """A8W4 T-CG: fp8 x1, fp4 x2 with a bf16/fp16 scale per `group_k` elements of k, uint64 yScale per column.
    qbmmv4_kernel_golden.py:189-255: the weight is widened to the scale's dtype, multiplied by the scale in that dtype,
    rounded to x1's fp8 dtype, and only then multiplied; yScale (decoded as in matmul_quant_util.py:129-134) scales the
    fp32 product."""
    mid = x2_scale.dtype
    b = x2.astype(np.float32)
    s = x2_scale.astype(np.float32)
    if transpose_x2:
        b, s = b.T, s.T
    k = b.shape[0]
    s = np.repeat(s, group_k, axis=0)[:k]
    w = (b.astype(mid) * s.astype(mid)).astype(np.float32).astype(x1.dtype).astype(np.float32)
    a = x1.astype(np.float32)
    if transpose_x1:
        a = a.T
    y = np.matmul(a, w)
    if y_scale is not None:
        y = y * u64_to_deq_scale(y_scale).reshape(1, -1)[:, : y.shape[-1]]
    if bias is not None:
        y = y + bias.astype(np.float32)
    return cast_out(y, out_dtype)


def compute_int4_asym(x1, x2, x1_scale, x2_scale, x2_offset, transpose_x1, transpose_x2, out_dtype, group_k=256):
    """INT4 x INT4 asymmetric per-group (qbmmv4_kernel_golden.py:328-395):
    out = x1Scale[m] * sum_g (x1_g @ x2_g - rowsum(x1_g) * x2Offset[g, n]) * x2Scale[g, n], groups of 256 along k."""
    a = x1.astype(np.int32)
    b = x2.astype(np.int32)
    if transpose_x1:
        a = a.T
    if transpose_x2:
        b = b.T
    m, k = a.shape
    s2 = x2_scale.astype(np.float32)
    of = x2_offset.astype(np.float32)
    out = np.zeros((m, b.shape[1]), dtype=np.float32)
    for g in range(-(-k // group_k)):
        ag, bg = a[:, g * group_k:(g + 1) * group_k], b[g * group_k:(g + 1) * group_k]
        mm = np.matmul(ag, bg).astype(np.float32)
        rs = np.sum(ag.astype(np.float32), axis=-1, keepdims=True)
        out += (mm - rs * of[g:g + 1, :]) * s2[g:g + 1, :]
    out = out * x1_scale.astype(np.float32)[:, 0:1]
    return cast_out(out, out_dtype)


def compute_perblock(x1, x2, x1_scale, x2_scale, group, transpose_x1, transpose_x2, out_dtype, bias=None):
    """2-D operands. qbmmv3_kernel_golden.py:237-358"""
    gm, gn, gk = group
    a = x1.astype(np.float32)
    b = x2.astype(np.float32)
    s1 = x1_scale.astype(np.float32)
    s2 = x2_scale.astype(np.float32)
    if transpose_x1:
        a, s1 = a.T, s1.T
    if transpose_x2:
        b, s2 = b.T, s2.T
    m, k = a.shape
    n = b.shape[1]
    s1 = np.repeat(s1, gm, axis=0)[:m, :]
    s2 = np.repeat(s2, gn, axis=1)[:, :n]
    y = np.zeros((m, n), dtype=np.float32)
    for kb in range(-(-k // gk)):
        ks, ke = kb * gk, min((kb + 1) * gk, k)
        y += np.matmul(a[:, ks:ke], b[ks:ke, :]) * (s1[:, kb : kb + 1] * s2[kb : kb + 1, :])
    if bias is not None:
        y = y + bias.astype(np.float32)
    return cast_out(y, out_dtype)


def int_matmul(a, b):
    """Exact int32 matmul of int8 operands. numpy's integer matmul is not BLAS-backed and slow, so for larger shapes this
    goes through float64 BLAS, which is exact while |sum| < 2^53 (always true for int8 x int8 with k < 2^37)."""
    if a.shape[-1] * a.shape[-2] * b.shape[-1] > (1 << 24):
        return np.matmul(a.astype(np.float64), b.astype(np.float64)).astype(np.int64).astype(np.int32)
    return np.matmul(a.astype(np.int32), b.astype(np.int32))


def quant_matmul_v5(x1, x2, x1_scale, x2_scale, bias=None, transpose_x1=False, transpose_x2=False, group_size=0,
                    out_dtype="bfloat16", x2_scale_is_u64=False, y_scale=None, x2_offset=None):
    """aclnnQuantMatmulV5 for the modes this build implements; batch dims on x1/x2 are looped.

    Mode selection = qbmmv3_kernel_golden.py:62-145 (same tree as the reference's host tiling,
    quant_batch_matmul_v3_tiling_base.cpp:458-557).
    """
    if x1.dtype == np.dtype(INT4) and x2_offset is not None:
        return compute_int4_asym(x1, x2, x1_scale, x2_scale, x2_offset, transpose_x1, transpose_x2, out_dtype)
    if x1.dtype == np.dtype(INT4):  # int4 x int4: the golden widens both to int32 like int8 (qbmmv3_kernel_golden.py:612-615)
        x1, x2 = x1.astype(np.int8), x2.astype(np.int8)
    if x1.ndim > 2 or x2.ndim > 2:
        nb = max(x1.shape[0] if x1.ndim > 2 else 1, x2.shape[0] if x2.ndim > 2 else 1)
        outs = []
        for i in range(nb):
            def pick(t, core):
                if t is None or t.ndim <= core:
                    return t
                return t[i if t.shape[0] > 1 else 0]
            mx = x2_scale.dtype == np.dtype(E8M0)
            pb = (not mx) and x1_scale is not None and x1_scale.ndim > 1
            outs.append(quant_matmul_v5(pick(x1, 2), pick(x2, 2),
                                        pick(x1_scale, 3 if mx else (2 if pb else 1)),
                                        pick(x2_scale, 3 if mx else (2 if pb else 1)),
                                        pick(bias, 1) if bias is None or bias.ndim != 3 else bias[i, 0],
                                        transpose_x1, transpose_x2, group_size, out_dtype, x2_scale_is_u64))
        return np.stack(outs)

    if y_scale is not None and _is_fp8(x1.dtype) and x2.dtype == np.dtype(E2M1) and x1_scale is None:
        return compute_t_cg(x1, x2, x2_scale, y_scale, transpose_x1, transpose_x2, (group_size & 0xFFFF) or 32, out_dtype,
                            bias)
    if x2_scale.dtype == np.dtype(E8M0):
        return compute_mx(x1, x2, x1_scale, x2_scale, bias, transpose_x1, transpose_x2, out_dtype)
    is_int = x1.dtype == np.int8
    fp8 = _is_fp8(x1.dtype)
    # fp8 per-block (qbmmv3_kernel_golden.py:237-358) and int8 per-tile (qbmmv4_kernel_golden.py:258-325) share the formula:
    # int8 products and their 128-term sums are exact in fp32, so the float path restates the int32 matmul bit for bit
    if (fp8 or is_int) and x1_scale is not None and x1_scale.ndim > 1 and x2_scale.ndim > 1:
        return compute_perblock(x1, x2, x1_scale, x2_scale, unpack_groupsize(group_size), transpose_x1, transpose_x2,
                                out_dtype, bias)
    a = x1.T if transpose_x1 else x1
    b = x2.T if transpose_x2 else x2
    m = a.shape[0]
    acc = int_matmul(a, b) if is_int else np.matmul(a.astype(np.float32), b.astype(np.float32))
    bias_dt = None if bias is None else bias.dtype
    float_bias = bias is not None and bias_dt != np.int32
    if out_dtype == "int32":  # compute_int32 :490-506
        return (acc + bias).astype(np.int32) if bias is not None else acc.astype(np.int32)
    s2 = u64_to_deq_scale(x2_scale) if x2_scale_is_u64 else x2_scale.astype(np.float32)
    if out_dtype == "int8":  # compute_requant :465-487; the offset rides in bits 37..45 of the packed scale (:726-731)
        out = acc + bias if bias is not None and bias_dt == np.int32 else acc
        out = f32_2_s9(out.astype(np.float32) * s2)
        if x2_offset is not None:
            out = out + f32_2_s9(u64_to_offset(x2_scale))
        return np.clip(out, -128, 127).astype(np.int8)
    per_token = x1_scale is not None and x1_scale.ndim == 1 and x1_scale.shape[0] == m and not (
        fp8 and x1_scale.shape[0] == 1)
    double_scale = fp8 and x1_scale is not None and x1_scale.ndim == 1 and x1_scale.shape[0] == 1
    is_bias_vec = float_bias and (is_int or (fp8 and x1_scale is not None))
    if per_token and not double_scale:  # compute_pertoken :361-387
        out = acc
        if bias is not None and bias_dt == np.int32:
            out = out + bias
        out = out.astype(np.float32)
        out = out * s2 * x1_scale.astype(np.float32)[:, None]
        if float_bias:
            out = out + bias.astype(np.float32)
        return cast_out(out, out_dtype)
    # compute_tc :390-462
    out = acc
    if not is_bias_vec and bias is not None:
        out = out + bias if bias_dt == np.int32 else out.astype(np.float32) + bias.astype(np.float32)
    out = out.astype(np.float32)
    do_scale_gen = is_int and not x2_scale_is_u64 and s2.shape[0] == 1 and not (
        bias is not None and bias_dt in (np.dtype(BF16), np.dtype(np.float32)))
    if x1_scale is not None:
        s1 = x1_scale.astype(np.float32)
        if double_scale and s2.shape[0] == 1 and not is_bias_vec:  # merge + 19-bit truncation
            out = out * trunc19(s2 * s1)[None, :]
        else:
            if do_scale_gen:
                s2 = trunc19(s2)
            out = out * s2[None, :] * s1
    else:
        if do_scale_gen:
            s2 = trunc19(s2)
        out = out * s2[None, :]
    if is_bias_vec:
        out = out + bias.astype(np.float32)
    return cast_out(out, out_dtype)
