"""numpy restatement of the reference's weight-only quant matmul golden (aclnnWeightQuantBatchMatmulV2/V3 path).

Follows matmul/weight_quant_batch_matmul_v2/tests/assets/wqbmmv2_kernel_golden.py of the reference
(prepare_* :41-82, matmul_and_finalize/finalize :85-103, _compute_tc :199-239, _compute_pergroup :242-297) and the
int32 -> int4 unpack of wqbmmv2_aclnn_golden.py:128-144 / matmul_quant_util.py:228-273 (element j of a word at bits 4j).

Test infrastructure only (see oracle/__init__.py).
"""
import ml_dtypes
import numpy as np

BF16 = ml_dtypes.bfloat16


def unpack_int4_words(packed):
    """int32 (.., c) -> int8 (.., 8c), sign-extended nibbles, low nibble first."""
    u = np.ascontiguousarray(packed).view(np.uint32)
    out = np.empty(u.shape + (8,), dtype=np.int8)
    for j in range(8):
        nib = ((u >> np.uint32(4 * j)) & np.uint32(0xF)).astype(np.int8)
        out[..., j] = (nib ^ 8) - 8
    return out.reshape(u.shape[:-1] + (u.shape[-1] * 8,))


def pack_int4_words(vals):
    """int8 values in [-8,7], (.., 8c) -> int32 (.., c)."""
    v = (np.asarray(vals).astype(np.int64) & 0xF).reshape(vals.shape[:-1] + (vals.shape[-1] // 8, 8))
    out = np.zeros(v.shape[:-1], dtype=np.int64)
    for j in range(8):
        out |= v[..., j] << (4 * j)
    return out.astype(np.uint32).view(np.int32)


def dequant_weight(w, scale, offset, group_size, inter):
    """w (k,n) integer values; scale/offset (1|groups, 1|n) or (n,) in `inter` dtype. Two roundings in `inter`."""
    wf = w.astype(np.float32)  # int4/int8 values, or fp8 / fp4 (exact in either intermediate dtype)
    sf = np.atleast_2d(scale.astype(np.float32))
    if scale.dtype.name.startswith("float8_e8m0"):
        # mx antiquant (wqbmmv2_kernel_golden.py:298-352): e8m0 per 32 rows, row count padded to even; with fp16 activations
        # the scale passes through fp16 first
        if inter == np.float16:
            with np.errstate(over="ignore"):
                sf = sf.astype(np.float16).astype(np.float32)
        group_size = 32
        sf = sf[: -(-wf.shape[0] // 32)]
    of = None if offset is None else np.atleast_2d(offset.astype(np.float32))
    k = wf.shape[0]
    if group_size and group_size > 0:
        reps = -(-k // group_size)
        sf = np.repeat(sf, group_size, axis=0)[:k] if sf.shape[0] == reps else sf
        if of is not None:
            of = np.repeat(of, group_size, axis=0)[:k] if of.shape[0] == reps else of
    if of is not None:
        wf = (wf + of).astype(inter).astype(np.float32)
    return (wf * sf).astype(inter).astype(np.float32)


def weight_quant_batch_matmul(x, w, scale, offset=None, bias=None, group_size=0):
    """x (m,k) bf16|fp16; w (k,n) integer values (already unpacked, already in (k,n) orientation);
    scale/offset in (groups|1, n|1) orientation. Returns y in x's dtype."""
    inter = x.dtype.type
    wf = dequant_weight(w, scale, offset, group_size, inter)
    out = np.matmul(x.astype(np.float32), wf)
    if bias is not None:
        out = out + bias.astype(np.float32)
    return out.astype(inter)


def fp32_dequant_product(x, w, scale, offset=None, bias=None, group_size=0):
    """The tolerance yardstick: x @ ((w + offset) * scale) with no intermediate rounding, float64 accumulate."""
    wf = w.astype(np.float64)
    sf = np.atleast_2d(scale.astype(np.float64))
    of = None if offset is None else np.atleast_2d(offset.astype(np.float64))
    k = wf.shape[0]
    if group_size and group_size > 0:
        sf = np.repeat(sf, group_size, axis=0)[:k]
        if of is not None:
            of = np.repeat(of, group_size, axis=0)[:k]
    if of is not None:
        wf = wf + of
    out = np.matmul(x.astype(np.float64), wf * sf)
    if bias is not None:
        out = out + bias.astype(np.float64)
    return out


def convert_weight_to_b4_pack(weight):
    """aclnnConvertWeightToINT4Pack, ND output (aclnn_convert_weight_to_int4_pack.cpp:43-121 of the reference): `weight` holds one
    4-bit value per element - int32 (low nibble used) or float32 (an e2m1 value; anything else packs as code 0). Returns the
    packed bytes, element 2i in the low nibble of byte i, shaped (..., n / 2)."""
    w = np.ascontiguousarray(weight)
    if w.dtype == np.float32:
        bits = w.view(np.uint32) & np.uint32(0xFFC00000)
        table = {0x00000000: 0, 0x3F000000: 1, 0x3F800000: 2, 0x3FC00000: 3, 0x40000000: 4, 0x40400000: 5, 0x40800000: 6,
                 0x40C00000: 7, 0x80000000: 8, 0xBF000000: 9, 0xBF800000: 10, 0xBFC00000: 11, 0xC0000000: 12, 0xC0400000: 13,
                 0xC0800000: 14, 0xC0C00000: 15}
        codes = np.zeros(bits.shape, dtype=np.uint8)
        for k, v in table.items():
            codes[bits == np.uint32(k)] = v
    else:
        codes = (w.astype(np.int64) & 0xF).astype(np.uint8)
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def nd_to_nz(a, k0, n0):
    """(k, n) -> FRACTAL_NZ storage [ceil(n/n0), ceil(k/k0), k0, n0], zero padded: element (i, j) sits at
    [j // n0, i // k0, i % k0, j % n0] (inverse of nz_to_nd, matmul/common/tests/st/arch35/matmul_golden_util.py:76-114)."""
    k, n = a.shape
    k1, n1 = -(-k // k0), -(-n // n0)
    pad = np.zeros((k1 * k0, n1 * n0), dtype=a.dtype)
    pad[:k, :n] = a
    return np.ascontiguousarray(pad.reshape(k1, k0, n1, n0).transpose(2, 0, 1, 3))


def nz_to_nd(nz, shape):
    """FRACTAL_NZ storage [n1, k1, k0, n0] -> (k, n) (matmul_golden_util.py:76-114 of the reference)."""
    n1, k1, k0, n0 = nz.shape
    k, n = shape
    return np.ascontiguousarray(nz.transpose(1, 2, 0, 3).reshape(k1 * k0, n1 * n0)[:k, :n])
