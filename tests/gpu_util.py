"""Helpers for the GPU parity tests: fixtures -> device tensors and aclnn descriptors, calls through the C ABI."""
import ml_dtypes
import numpy as np
import torch

from oracle import wqbmm_oracle

DEV = "cuda:0"


def np_name(a):
    names = {np.dtype(ml_dtypes.bfloat16): "bfloat16", np.dtype(ml_dtypes.float8_e4m3fn): "float8_e4m3fn",
             np.dtype(ml_dtypes.float8_e5m2): "float8_e5m2", np.dtype(ml_dtypes.float4_e2m1fn): "float4_e2m1",
             np.dtype(ml_dtypes.float8_e8m0fnu): "float8_e8m0", np.dtype(ml_dtypes.int4): "int4"}
    return names.get(a.dtype, a.dtype.name)


def to_dev_raw(a):
    """numpy array of any of the supported dtypes -> (torch tensor holding the raw bytes on the device, acl dtype name,
    logical shape). fp4 is packed two per byte along the last axis (low nibble first)."""
    name = np_name(a)
    a = np.ascontiguousarray(a)
    if name == "bfloat16":
        t = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    elif name in ("float8_e4m3fn", "float8_e5m2", "float8_e8m0"):
        t = torch.from_numpy(a.view(np.uint8).copy())
    elif name == "float4_e2m1":
        codes = a.view(np.uint8)
        assert codes.shape[-1] % 2 == 0
        t = torch.from_numpy((codes[..., 0::2] & 0xF) | ((codes[..., 1::2] & 0xF) << 4))
    elif name == "int4":
        codes = a.astype(np.int8).view(np.uint8)
        assert codes.shape[-1] % 2 == 0
        t = torch.from_numpy((codes[..., 0::2] & 0xF) | ((codes[..., 1::2] & 0xF) << 4))
    elif name == "uint64":
        t = torch.from_numpy(a.view(np.int64).copy())
    else:
        t = torch.from_numpy(a.copy())
    return t.to(DEV), name, tuple(a.shape)


def desc(aclnn, a, strides=None, shape=None):
    if a is None:
        return None
    t, name, lshape = to_dev_raw(a)
    return aclnn.Tensor(shape or lshape, name, t, strides)


def out_tensor(shape, name):
    dt = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32, "int32": torch.int32, "int8": torch.int8}[name]
    # poison so that an element the kernel fails to write is caught
    poison = {torch.int32: -7777, torch.int8: -77}.get(dt, -7777.0)
    t = torch.full(shape, poison, dtype=dt, device=DEV)
    return t


def out_to_np(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(ml_dtypes.bfloat16)
    return t.cpu().numpy()


def run_qmm_fixture(aclnn, a, meta, kernel=None):
    import os

    out = out_tensor(a["out"].shape, meta["out_dtype"])
    d_out = aclnn.Tensor(a["out"].shape, meta["out_dtype"], out)
    if kernel is not None:
        os.environ["OPSNN_QMM_KERNEL"] = str(kernel)
    try:
        aclnn.quant_matmul_v5(desc(aclnn, a["x1"]), desc(aclnn, a["x2"]), desc(aclnn, a.get("x1_scale")),
                              desc(aclnn, a["x2_scale"]), d_out, desc(aclnn, a.get("bias")), meta["transpose_x1"],
                              meta["transpose_x2"], meta["group_size"], y_scale=desc(aclnn, a.get("y_scale")),
                              x2_offset=desc(aclnn, a.get("x2_offset")))
    finally:
        os.environ.pop("OPSNN_QMM_KERNEL", None)
    torch.cuda.synchronize()
    status = aclnn.lib().opsnn_qmm_umma_status(1)
    assert status == 0, "tensor-core kernel reported a timed-out wait: 0x%x" % status
    return out_to_np(out)


def run_wq_fixture(aclnn, a, meta, kernel=None, api="v2", inner_precise=0):
    import os

    x = a["x"]
    w = a["w"]
    t = meta["transpose_weight"]
    out_name = np_name(a["out"])
    out = out_tensor(a["out"].shape, out_name)
    d_y = aclnn.Tensor(a["out"].shape, out_name, out)
    if meta.get("w_float"):
        d_w = desc(aclnn, w)  # fp8 bytes, or fp4 packed two per byte along n
    elif meta["w_is_int4"]:
        if meta.get("packed_int32"):
            words = wqbmm_oracle.pack_int4_words(w)  # packed along the stored inner axis
            wt = torch.from_numpy(words.copy()).to(DEV)
            if t:  # stored (n, k/8) viewed as (k/8, n)
                d_w = aclnn.Tensor((words.shape[1], words.shape[0]), "int32", wt, strides=(1, words.shape[1]))
            else:
                d_w = aclnn.Tensor(words.shape, "int32", wt)
        else:
            nib = (w.astype(np.uint8) & 0xF)
            packed = (nib[..., 0::2] | (nib[..., 1::2] << 4)).astype(np.uint8)
            wt = torch.from_numpy(packed).to(DEV)
            if t:  # stored (n,k) described as the (k,n) view
                d_w = aclnn.Tensor((w.shape[1], w.shape[0]), "int4", wt, strides=(1, w.shape[1]))
            else:
                d_w = aclnn.Tensor(w.shape, "int4", wt)
    else:
        wt = torch.from_numpy(w.copy()).to(DEV)
        d_w = aclnn.Tensor((w.shape[1], w.shape[0]), "int8", wt, strides=(1, w.shape[1])) if t else aclnn.Tensor(w.shape, "int8", wt)

    def sc_desc(s):
        if s is None:
            return None
        if t and s.ndim == 2:  # stored (n, groups) described as (groups, n)
            tt, name, _ = to_dev_raw(s)
            return aclnn.Tensor((s.shape[1], s.shape[0]), name, tt, strides=(1, s.shape[1]))
        return desc(aclnn, s)

    if kernel is not None:
        os.environ["OPSNN_WQ_KERNEL"] = str(kernel)
    try:
        aclnn.weight_quant_batch_matmul(desc(aclnn, x), d_w, sc_desc(a["scale"]), d_y, sc_desc(a.get("offset")),
                                        desc(aclnn, a.get("bias")), meta["group_size"], inner_precise=inner_precise if api == "v3" else None)
    finally:
        os.environ.pop("OPSNN_WQ_KERNEL", None)
    torch.cuda.synchronize()
    return out_to_np(out)


def check_close(got, want, ref32, out_name, exact=False, floor_rms=1e-3):
    """Parity criteria, all three reported in the assertion message:
      * exact: bit-equal (integer outputs, and the int8 dequant modes whose epilogue order is fully specified);
      * the reference's own system-test criterion: isclose(rtol 1e-3, atol 1e-3) on >= 99.9 % of the elements
        (matmul/common/tests/st/arch35/matmul_golden_util.py:340-380 of the reference), against the golden output;
      * the stated tolerance: max relative error <= 1e-2 (bf16) / 5e-3 (fp16, fp32) against the fp32 dequantised
        product `ref32`; the denominator is floored at `floor_rms` x rms(ref32) so that an output that cancels to ~0
        does not turn accumulation-order noise into an unbounded ratio.
    """
    g = np.asarray(got).astype(np.float64)
    w = np.asarray(want).astype(np.float64)
    assert g.shape == w.shape
    assert not np.any(g == -7777.0), "kernel left output elements unwritten"
    if exact:
        assert np.array_equal(np.asarray(got).view(np.uint8), np.asarray(want).view(np.uint8)), \
            "not bit-exact: %d of %d elements differ, max abs diff %g" % ((g != w).sum(), g.size, np.abs(g - w).max())
        return
    fin = np.isfinite(w)
    ok = np.isclose(g[fin], w[fin], rtol=1e-3, atol=1e-3)
    frac = ok.mean() if ok.size else 1.0
    r = np.asarray(ref32).astype(np.float64)
    rms = np.sqrt(np.mean(r[fin] ** 2)) if fin.any() else 0.0
    rel = np.abs(g - r)[fin] / np.maximum(np.abs(r[fin]), floor_rms * rms + 1e-30)
    tol = 1e-2 if out_name == "bfloat16" else 5e-3
    assert frac >= 0.999 and rel.max() <= tol, "isclose fraction %.5f (need 0.999), max rel err vs fp32 product %.3g (tol %g)" % (
        frac, rel.max() if rel.size else 0.0, tol)
