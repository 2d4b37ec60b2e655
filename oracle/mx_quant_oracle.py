"""numpy restatement of the reference's dynamic MX quantisation golden (aclnnDynamicMxQuant, OCP scale).

Follows quant/dynamic_mx_quant/tests/assets/golden.py of the reference: shared exponent :141-154, element quantisation
:197-217, _mx_quantize :272-336 (scale padded to an even count with 2^-127, shaped (.., ceil(k/64), 2)).

Test infrastructure only (see oracle/__init__.py).
"""
import ml_dtypes
import numpy as np

_FMT = {
    "float8_e4m3fn": (ml_dtypes.float8_e4m3fn, 4, 3, 448.0),
    "float8_e5m2": (ml_dtypes.float8_e5m2, 5, 2, 57344.0),
    "float4_e2m1": (ml_dtypes.float4_e2m1fn, 2, 1, 6.0),
}


def dynamic_mx_quant(x, dst="float8_e4m3fn", block=32, axis=-1, scale_alg=0, round_mode="rint"):
    """x bf16|fp16|fp32, blocks of 32 along `axis` -> (y in dst dtype, x's shape; scale bytes uint8: x's shape with the axis
    replaced by ceil(ceil(len/32)/2), plus a trailing 2 holding the even/odd block of each pair - golden.py:320-331)."""
    ax = axis if axis >= 0 else x.ndim + axis
    if ax != x.ndim - 1:
        y, sc = dynamic_mx_quant(np.moveaxis(x, ax, -1), dst, block, -1, scale_alg, round_mode)
        # sc: (rest.., pairs, 2) -> pairs back to the axis position, the 2 stays last
        return np.ascontiguousarray(np.moveaxis(y, -1, ax)), np.ascontiguousarray(np.moveaxis(sc, -2, ax))
    np_dt, ebits, mbits, max_norm = _FMT[dst]
    xf = x.astype(np.float32)
    k = xf.shape[-1]
    nblk = -(-k // block)
    pad = nblk * block - k
    if pad:
        xf = np.pad(xf, [(0, 0)] * (xf.ndim - 1) + [(0, pad)])
    blk = xf.reshape(xf.shape[:-1] + (nblk, block))
    amax = np.max(np.abs(blk), axis=-1, keepdims=True)
    emax = int(np.log2(max_norm))
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(amax == 0, np.float32(2.0 ** -126), amax))) - emax
    if scale_alg == 1 and dst != "float4_e2m1":  # exponent of amax / max_norm, rounded up to a power of two (golden.py:157-177)
        bits = (amax.astype(np.float32) / np.float32(max_norm)).view(np.uint32)
        ex = ((bits & np.uint32(0x7F800000)) >> 23).astype(np.int16)
        mant = bits & np.uint32(0x007FFFFF)
        up = ((ex > 0) & (ex < 254) & (mant > 0)) | ((ex == 0) & (mant > 2 ** 22))
        e = (np.where(up, ex + 1, ex) - 127).astype(np.float32)
    e[amax == 0] = -np.inf
    e = np.where(e < -127, -127.0, e)
    r = blk / np.exp2(e).astype(np.float32)
    with np.errstate(divide="ignore"):
        pe = np.floor(np.log2(np.abs(r) + (r == 0)))
    pe = np.maximum(pe, -(2 ** (ebits - 1)) + 2)
    t = r / np.exp2(pe) * (2 ** mbits)
    if round_mode == "rint":
        t = np.rint(t)
    elif round_mode == "round":  # ties away from zero (golden.py:183-186)
        t = np.where(np.signbit(t), -np.floor(np.abs(t) + 0.5), np.floor(np.abs(t) + 0.5))
    else:  # "floor"
        t = np.floor(t)
    q = t / (2 ** mbits) * np.exp2(pe)
    q = np.clip(q, -max_norm, max_norm).astype(np.float32)
    y = q.reshape(xf.shape)[..., :k].astype(np_dt)
    sbytes = (e[..., 0] + 127).astype(np.uint8)
    if nblk % 2:
        sbytes = np.concatenate([sbytes, np.zeros(sbytes.shape[:-1] + (1,), np.uint8)], axis=-1)
    return y, sbytes.reshape(sbytes.shape[:-1] + (sbytes.shape[-1] // 2, 2))
