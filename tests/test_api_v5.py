"""CPU: phase 1 of aclnnQuantMatmulV5 against the reference's own op_api unit-test table (84 Ascend950 rows with the
status each argument combination must produce), plus executor ownership rules. No device work happens in phase 1."""
import json
import os
import threading

import pytest

from conftest import GOLDEN

with open(os.path.join(GOLDEN, "api_v5_cases.json")) as fh:
    CASES = json.load(fh)

STATUS = {"ACLNN_SUCCESS": 0, "ACLNN_ERR_PARAM_NULLPTR": 161001, "ACLNN_ERR_PARAM_INVALID": 161002,
          "ACLNN_ERR_RUNTIME_ERROR": 361001}
FMT = {"ACL_FORMAT_ND": 2, "ACL_FORMAT_FRACTAL_NZ": 29, "ACL_FORMAT_FRACTAL_NZ_C0_32": 52}


def _mk(aclnn, spec, fmt="ACL_FORMAT_ND"):
    if spec is None:
        return None
    return aclnn.Tensor(spec["shape"], spec["dtype"], 0, spec.get("strides"), 0, FMT[fmt], spec.get("storage_shape"))


def _run_case(aclnn, c):
    t = c["tensors"]
    x1 = _mk(aclnn, t.get("x1"), c["x1Format"])
    x2 = _mk(aclnn, t.get("x2"), c["x2Format"])
    args = [_mk(aclnn, t.get(k)) for k in ("x1Scale", "x2Scale", "yScale", "x1Offset", "x2Offset", "yOffset", "bias")]
    out = _mk(aclnn, t.get("out"))
    st, ws, ex = aclnn.quant_matmul_v5_get_workspace_size(x1, x2, *args, c["transposeX1"], c["transposeX2"], c["groupSize"], out)
    if st == 0:
        aclnn.destroy_executor(ex)
    return st


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_phase1_status_matches_reference_table(aclnn, case):
    st = _run_case(aclnn, case)
    assert st == STATUS[case["expect"]], "%s: got %d (%s), reference expects %s" % (
        case["name"], st, aclnn.last_error(), case["expect"])


def test_null_workspace_or_executor_pointer(aclnn):
    import ctypes

    x1 = aclnn.Tensor((16, 32), "int8")
    x2 = aclnn.Tensor((32, 16), "int8")
    sc = aclnn.Tensor((16,), "float32")
    out = aclnn.Tensor((16, 16), "bfloat16")
    L = aclnn.lib()
    st = L.aclnnQuantMatmulV5GetWorkspaceSize(x1.handle, x2.handle, None, sc.handle, None, None, None, None, None, False,
                                              False, 0, out.handle, None, None)
    assert st == aclnn.ACLNN_ERR_PARAM_NULLPTR
    assert "nullptr" in aclnn.last_error()


def test_empty_m_or_n_is_success_and_launches_nothing(aclnn):
    x1 = aclnn.Tensor((0, 32), "int8")
    x2 = aclnn.Tensor((32, 16), "int8")
    sc = aclnn.Tensor((16,), "float32")
    out = aclnn.Tensor((0, 16), "bfloat16")
    st, ws, ex = aclnn.quant_matmul_v5_get_workspace_size(x1, x2, None, sc, None, None, None, None, None, False, False, 0, out)
    assert st == 0 and ws == 0
    before = aclnn.launch_count()
    assert aclnn.lib().aclnnQuantMatmulV5(None, 0, ex, None) == 0  # consumes the executor; nothing to launch
    assert aclnn.launch_count() == before


def test_strided_transposed_view_flips_the_flag(aclnn):
    # x2 given as a (k,n) view of (n,k) storage: same as passing the (n,k) tensor with transposeX2=true
    x1 = aclnn.Tensor((16, 32), "int8")
    x2 = aclnn.Tensor((32, 48), "int8", 0, strides=(1, 32))
    sc = aclnn.Tensor((48,), "float32")
    out = aclnn.Tensor((16, 48), "bfloat16")
    st, ws, ex = aclnn.quant_matmul_v5_get_workspace_size(x1, x2, None, sc, None, None, None, None, None, False, False, 0, out)
    assert st == 0, aclnn.last_error()
    aclnn.destroy_executor(ex)


def test_group_size_inference_mx_and_perblock(aclnn):
    # mx: groupSize 0 -> [1,1,32]; explicit wrong K field is rejected
    x1 = aclnn.Tensor((64, 256), "float8_e4m3fn")
    x2 = aclnn.Tensor((256, 96), "float8_e4m3fn")
    s1 = aclnn.Tensor((64, 4, 2), "float8_e8m0")
    s2 = aclnn.Tensor((4, 96, 2), "float8_e8m0")
    out = aclnn.Tensor((64, 96), "bfloat16")
    for g, want in ((0, 0), (4295032864, 0), (64, 161002), ((2 << 32) | (1 << 16) | 32, 161002)):
        st, _, ex = aclnn.quant_matmul_v5_get_workspace_size(x1, x2, s1, s2, None, None, None, None, None, False, False, g, out)
        assert st == want, (g, aclnn.last_error())
        if st == 0:
            aclnn.destroy_executor(ex)
    # per-block G-B
    x1 = aclnn.Tensor((256, 384), "float8_e4m3fn")
    x2 = aclnn.Tensor((384, 256), "float8_e4m3fn")
    s1 = aclnn.Tensor((256, 3), "float32")
    s2 = aclnn.Tensor((3, 2), "float32")
    out = aclnn.Tensor((256, 256), "bfloat16")
    for g, want in ((0, 0), (4303356032, 0), ((1 << 32) | (64 << 16) | 128, 161002)):
        st, _, ex = aclnn.quant_matmul_v5_get_workspace_size(x1, x2, s1, s2, None, None, None, None, None, False, False, g, out)
        assert st == want, (g, aclnn.last_error())
        if st == 0:
            aclnn.destroy_executor(ex)


def test_int8_perblock_is_accepted(aclnn):
    """int8 x int8 with (m, k/128) and (k/128, n/128) fp32 scales: the PER_TILE mode of
    matmul/quant_batch_matmul_v4/tests/assets/qbmmv4_kernel_golden.py:258-325; bias allowed, groupSizeN must be 128."""
    x1 = aclnn.Tensor((256, 384), "int8")
    x2 = aclnn.Tensor((384, 256), "int8")
    s1 = aclnn.Tensor((256, 3), "float32")
    s2 = aclnn.Tensor((3, 2), "float32")
    bias = aclnn.Tensor((256,), "float32")
    out = aclnn.Tensor((256, 256), "bfloat16")
    for g, b, want in ((4303356032, None, 0), (4303356032, bias, 0), ((1 << 32) | (64 << 16) | 128, None, 161002)):
        st, _, ex = aclnn.quant_matmul_v5_get_workspace_size(x1, x2, s1, s2, None, None, None, None, b, False, False, g, out)
        assert st == want, (g, aclnn.last_error())
        if st == 0:
            aclnn.destroy_executor(ex)


def test_a8w4_plans_reserve_the_rewritten_weight(aclnn):
    """fp8 x fp4 (mx and T-CG): phase 1 succeeds and asks for at least n * k bytes, the fp8 copy of the weight."""
    m, k, n = 16, 128, 128
    x1 = aclnn.Tensor((m, k), "float8_e4m3fn")
    x2 = aclnn.Tensor((n, k), "float4_e2m1")
    out = aclnn.Tensor((m, n), "float16")
    s1 = aclnn.Tensor((m, 2, 2), "float8_e8m0")
    s2 = aclnn.Tensor((n, 2, 2), "float8_e8m0")
    st, ws, ex = aclnn.quant_matmul_v5_get_workspace_size(x1, x2, s1, s2, None, None, None, None, None, False, True, 32, out)
    assert st == 0 and ws >= n * k, (st, ws, aclnn.last_error())
    aclnn.destroy_executor(ex)
    s2g = aclnn.Tensor((n, 4), "bfloat16")
    ys = aclnn.Tensor((1, n), "uint64")
    st, ws, ex = aclnn.quant_matmul_v5_get_workspace_size(x1, x2, None, s2g, ys, None, None, None, None, False, True, 32, out)
    assert st == 0 and ws >= n * k, (st, ws, aclnn.last_error())
    aclnn.destroy_executor(ex)


def test_phase1_is_thread_safe(aclnn):
    """The reference drives phase 1 from three threads at once
    (weight_quant_batch_matmul_v2/tests/ut/op_host/op_api/test_aclnn_weight_quant_batch_matmul_v2_api.cpp:2757-2802)."""
    errors = []

    def worker():
        try:
            for c in CASES[:40]:
                if _run_case(aclnn, c) != STATUS[c["expect"]]:
                    errors.append(c["name"])
        except Exception as e:  # noqa: BLE001
            errors.append(repr(e))

    ts = [threading.Thread(target=worker) for _ in range(3)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errors, errors


def test_older_entry_points_share_the_v5_validator(aclnn):
    """aclnnQuantMatmulV4 / V3 (argument order scale, offset, pertokenScale, bias) go through the same phase 1."""
    import ctypes

    L = aclnn.lib()
    ws, ex = ctypes.c_uint64(7), ctypes.c_void_p(0)
    x1 = aclnn.Tensor((128, 256), "int8")
    x2 = aclnn.Tensor((256, 64), "int8")
    sc = aclnn.Tensor((64,), "float32")
    pt = aclnn.Tensor((128,), "float32")
    out = aclnn.Tensor((128, 64), "bfloat16")
    st = L.aclnnQuantMatmulV4GetWorkspaceSize(x1.handle, x2.handle, sc.handle, None, pt.handle, None, False, False, out.handle,
                                              ctypes.byref(ws), ctypes.byref(ex))
    assert st == aclnn.ACLNN_SUCCESS and ws.value == 0 and ex.value
    aclnn.destroy_executor(ex)
    st = L.aclnnQuantMatmulV3GetWorkspaceSize(x1.handle, x2.handle, sc.handle, None, None, False, False, out.handle,
                                              ctypes.byref(ws), ctypes.byref(ex))
    assert st == aclnn.ACLNN_SUCCESS
    aclnn.destroy_executor(ex)
    st = L.aclnnQuantMatmulV4GetWorkspaceSize(x1.handle, None, sc.handle, None, pt.handle, None, False, False, out.handle,
                                              ctypes.byref(ws), ctypes.byref(ex))
    assert st == aclnn.ACLNN_ERR_PARAM_NULLPTR
    bad = aclnn.Tensor((128, 65), "bfloat16")
    st = L.aclnnQuantMatmulV4GetWorkspaceSize(x1.handle, x2.handle, sc.handle, None, pt.handle, None, False, False, bad.handle,
                                              ctypes.byref(ws), ctypes.byref(ex))
    assert st == aclnn.ACLNN_ERR_PARAM_INVALID
