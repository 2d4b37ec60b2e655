"""CPU: phase 1 of aclnnWeightQuantBatchMatmulV2/V3 and aclnnDynamicMxQuant.

The first table is the reference's own Ascend950 parameter set
(matmul/weight_quant_batch_matmul_v2/tests/ut/op_host/op_api/test_aclnn_weight_quant_batch_matmul_v2_api.cpp:2471-2752:
casesParamsAscend950, fields in the order of its WeightQuantBatchMatmulV2TestParam struct) with the status each must give.
"""
import threading

import pytest

OK, INVALID, NULLPTR = 0, 161002, 161001
ND, NZ = 2, 29

# name, x, weight, aqScale, aqOffset(or None), group, y, xT, wT, sT, oT, wFormat, weight transposed view, expect
REF_950 = [
    ("nd_f8_offset_invalid", (96, 11264), (11264, 1664), (1, 1664), (1, 1664), 0, (96, 1664), "float16", "float8_e4m3fn", "float16", "float16", ND, False, INVALID),
    ("nd_w4_nz_transweight_error", (2, 64), (64, 128), (1, 128), (1, 128), 0, (2, 128), "float16", "int4", "float16", "float16", NZ, True, INVALID),
    ("nd_aqoffset_int32_invalid", (96, 11264), (11264, 1664), (1, 1664), (1, 1664), 0, (96, 1664), "float16", "int8", "float16", "int32", ND, False, INVALID),
    ("a16mxf4_nd_weight_fp4", (2, 64), (64, 128), (2, 128), None, 32, (2, 128), "float16", "float4_e2m1", "float8_e8m0", None, ND, False, OK),
    ("a16mxf4_nd_weight_fp32", (2, 64), (64, 16), (2, 128), None, 32, (2, 128), "float16", "float32", "float8_e8m0", None, ND, False, OK),
    ("a16mxf4_nd_invalid_group_size", (2, 64), (64, 128), (1, 128), None, 0, (2, 128), "float16", "float4_e2m1", "float8_e8m0", None, ND, False, INVALID),
    ("a16mxf4_nd_invalid_antiquant_offset", (2, 64), (64, 128), (2, 128), (2, 128), 32, (2, 128), "float16", "float4_e2m1", "float8_e8m0", "float16", ND, False, INVALID),
    ("nd_fp8_e4m3_offset_not_null_invalid", (2, 64), (64, 128), (2, 128), (2, 128), 32, (2, 128), "float16", "float8_e4m3fn", "float8_e8m0", "float8_e8m0", ND, False, INVALID),
    ("nd_hifloat8_offset_not_null_invalid", (2, 64), (64, 128), (2, 128), (2, 128), 32, (2, 128), "float16", "hifloat8", "float8_e8m0", "float8_e8m0", ND, False, INVALID),
    ("a16mxf4_nd_invalid_shape", (2, 64), (64, 129), (2, 129), (2, 129), 32, (2, 129), "float16", "float4_e2m1", "float8_e8m0", "float16", ND, False, INVALID),
]

# Rules of aclnn_weight_quant_batch_matmul_v2.cpp (:251-281 group size, :344-400 antiquant shapes, :439-576 dims,
# :1482-1524 int32 packing, :1584-1590 x layout) exercised with the shapes of the reference's system-test rows.
EXTRA = [
    ("st_v2_fp16_s4_pergroup_bias_int32packed", (672, 768), (768, 72), (12, 576), None, 64, (672, 576), "float16", "int32", "float16", None, ND, False, OK),
    ("st_v2_bf16_s4_perchannel_offset", (896, 640), (640, 96), (768,), (768,), 0, (896, 768), "bfloat16", "int32", "bfloat16", "bfloat16", ND, False, OK),
    ("decode_config", (16, 8192), (8192, 3584), (64, 28672), (64, 28672), 128, (16, 28672), "bfloat16", "int32", "bfloat16", "bfloat16", ND, False, OK),
    ("group_not_multiple_of_32", (16, 512), (512, 256), (11, 256), None, 48, (16, 256), "bfloat16", "int4", "bfloat16", None, ND, False, INVALID),
    ("group_equal_k", (16, 512), (512, 256), (1, 256), None, 512, (16, 256), "bfloat16", "int4", "bfloat16", None, ND, False, INVALID),
    ("group_160_k_384", (1, 384), (384, 4544), (3, 4544), None, 160, (1, 4544), "bfloat16", "int4", "bfloat16", None, ND, False, OK),
    ("scale_rows_wrong", (16, 512), (512, 256), (3, 256), None, 128, (16, 256), "bfloat16", "int4", "bfloat16", None, ND, False, INVALID),
    ("scale_dtype_differs_from_x", (16, 512), (512, 256), (4, 256), None, 128, (16, 256), "bfloat16", "int4", "float16", None, ND, False, INVALID),
    ("k_mismatch", (16, 500), (512, 256), (4, 256), None, 128, (16, 256), "bfloat16", "int4", "bfloat16", None, ND, False, INVALID),
    ("y_shape_wrong", (16, 512), (512, 256), (4, 256), None, 128, (16, 128), "bfloat16", "int4", "bfloat16", None, ND, False, INVALID),
    ("y_dtype_wrong", (16, 512), (512, 256), (4, 256), None, 128, (16, 256), "bfloat16", "int4", "bfloat16", None, ND, False, INVALID),
    ("int4_odd_n", (16, 512), (512, 255), (4, 255), None, 128, (16, 255), "bfloat16", "int4", "bfloat16", None, ND, False, INVALID),
    ("transposed_weight_view", (4, 64), (64, 2176), (2176,), None, 0, (4, 2176), "float16", "int4", "float16", None, ND, True, OK),
    ("per_tensor_1d", (9, 96), (96, 40), (1,), None, 0, (9, 40), "bfloat16", "int8", "bfloat16", None, ND, False, OK),
    ("x_dtype_fp32", (9, 96), (96, 40), (1,), None, 0, (9, 40), "float32", "int8", "float32", None, ND, False, INVALID),
    # an e8m0 (micro-scaling) antiquantScale goes with FLOAT4_E2M1 weights only (aclnn_weight_quant_batch_matmul_v2.cpp:766 refuses it
    # for fp8 weights; integer weights have no mx form): without this rule an INT4 weight would reach kernels that read 16-bit scales
    ("e8m0_scale_with_int4_weight", (16, 512), (512, 256), (16, 256), None, 32, (16, 256), "bfloat16", "int4", "float8_e8m0", None, ND, False, INVALID),
    ("e8m0_scale_with_int8_weight", (16, 512), (512, 256), (16, 256), None, 32, (16, 256), "bfloat16", "int8", "float8_e8m0", None, ND, False, INVALID),
    ("e8m0_scale_with_fp8_weight", (16, 512), (512, 256), (16, 256), None, 32, (16, 256), "bfloat16", "float8_e4m3fn", "float8_e8m0", None, ND, False, INVALID),
]


def _call(aclnn, row, inner_precise=None, y_dtype=None):
    name, x, w, s, o, g, y, xT, wT, sT, oT, wfmt, wtrans, expect = row
    tx = aclnn.Tensor(x, xT)
    tw = aclnn.Tensor(w, wT, 0, strides=(1, w[0]) if wtrans else None, fmt=wfmt)
    ts = aclnn.Tensor(s, sT)
    to = aclnn.Tensor(o, oT) if o is not None else None
    ty = aclnn.Tensor(y, y_dtype or xT)
    st, ws, ex = aclnn.weight_quant_batch_matmul_get_workspace_size(tx, tw, ts, to, None, None, None, g, ty, inner_precise)
    if st == 0:
        aclnn.destroy_executor(ex)
    return st, ws


@pytest.mark.parametrize("row", REF_950 + EXTRA, ids=[r[0] for r in REF_950 + EXTRA])
def test_phase1_status(aclnn, row):
    y_dtype = "float16" if row[0] == "y_dtype_wrong" else None
    st, _ = _call(aclnn, row, y_dtype=y_dtype)
    assert st == row[-1], "%s: got %d (%s)" % (row[0], st, aclnn.last_error())


def test_v3_inner_precise(aclnn):
    row = EXTRA[2]
    assert _call(aclnn, row, inner_precise=0)[0] == OK
    assert _call(aclnn, row, inner_precise=1)[0] == OK
    assert _call(aclnn, row, inner_precise=2)[0] == INVALID
    assert "innerPrecise" in aclnn.last_error()


def test_quant_scale_must_be_null_and_required_args(aclnn):
    x = aclnn.Tensor((16, 512), "bfloat16")
    w = aclnn.Tensor((512, 256), "int4")
    s = aclnn.Tensor((4, 256), "bfloat16")
    y = aclnn.Tensor((16, 256), "bfloat16")
    q = aclnn.Tensor((1, 256), "uint64")
    st, _, _ = aclnn.weight_quant_batch_matmul_get_workspace_size(x, w, s, None, q, None, None, 128, y)
    assert st == INVALID
    st, _, _ = aclnn.weight_quant_batch_matmul_get_workspace_size(x, None, s, None, None, None, None, 128, y)
    assert st == NULLPTR
    st, _, _ = aclnn.weight_quant_batch_matmul_get_workspace_size(x, w, None, None, None, None, None, 128, y)
    assert st == NULLPTR


def test_decode_config_reports_a_bounded_workspace(aclnn):
    st, ws = _call(aclnn, EXTRA[2])
    assert st == OK and 0 < ws <= 64 << 20  # the reference's own kernel uses a fixed 16 MiB workspace


def test_multi_thread(aclnn):
    """weight_quant_batch_matmul_v2 api UT `ascend950_multi_thread` (:2757-2802): three threads, same cases."""
    bad = []

    def worker():
        for row in REF_950:
            if _call(aclnn, row)[0] != row[-1]:
                bad.append(row[0])

    ts = [threading.Thread(target=worker) for _ in range(3)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not bad


def _mxq(aclnn, xshape, xT, dst, sshape, axis=-1, block=32, alg=0, mode=b"rint", yshape=None):
    import ctypes

    x = aclnn.Tensor(xshape, xT)
    y = aclnn.Tensor(yshape or xshape, dst)
    s = aclnn.Tensor(sshape, "float8_e8m0")
    ws, ex = ctypes.c_uint64(0), ctypes.c_void_p(0)
    st = aclnn.lib().aclnnDynamicMxQuantGetWorkspaceSize(x.handle, axis, mode, aclnn.DTYPE_BY_NAME[dst], block, alg, y.handle,
                                                         s.handle, ctypes.byref(ws), ctypes.byref(ex))
    if st == 0:
        aclnn.destroy_executor(ex)
    return st


def test_dynamic_mx_quant_phase1(aclnn):
    assert _mxq(aclnn, (2048, 4096), "bfloat16", "float8_e4m3fn", (2048, 64, 2)) == OK
    assert _mxq(aclnn, (5, 100), "bfloat16", "float8_e4m3fn", (5, 2, 2)) == OK          # 4 groups -> 2 pairs
    assert _mxq(aclnn, (5, 160), "float16", "float8_e5m2", (5, 3, 2)) == OK             # 5 groups padded to 6
    assert _mxq(aclnn, (5, 160), "float16", "float8_e5m2", (5, 5)) == INVALID           # wrong scale shape
    assert _mxq(aclnn, (5, 160), "float32", "float8_e5m2", (5, 3, 2)) == INVALID        # x dtype
    assert _mxq(aclnn, (5, 160), "bfloat16", "float8_e4m3fn", (5, 3, 2), block=64) == INVALID
    assert _mxq(aclnn, (5, 160), "bfloat16", "float8_e4m3fn", (5, 3, 2), mode=b"floor") == INVALID
    assert _mxq(aclnn, (8, 128), "bfloat16", "float4_e2m1", (8, 2, 2)) == OK
