"""GPU parity: aclnnQuantMatmulV5 through the C ABI against the reference-golden fixtures and the oracle."""
import numpy as np
import pytest

from conftest import golden_names, load_golden
from oracle import qbmm_oracle

pytestmark = pytest.mark.gpu

# int8 dequant modes: the accumulator is exact and the epilogue's rounding points are fully specified -> bit-exact
EXACT = {n for n in golden_names("qmm_") if "_int8_" in n or "_int4_" in n}


def _ref32(a, meta):
    u64 = meta["dtypes"].get("x2_scale") == "uint64"
    g = meta["group_size"]
    out = meta["out_dtype"] if meta["out_dtype"] in ("int32", "int8") else "float32"
    bias = a.get("bias")
    if bias is not None and bias.ndim == 2:
        bias = bias.reshape(-1)  # the A8W4 modes take bias as (1, n)
    return qbmm_oracle.quant_matmul_v5(a["x1"], a["x2"], a.get("x1_scale"), a["x2_scale"], bias, meta["transpose_x1"],
                                       meta["transpose_x2"], g, out, x2_scale_is_u64=u64, y_scale=a.get("y_scale"),
                                       x2_offset=a.get("x2_offset"))


@pytest.mark.parametrize("kernel", [1, 0], ids=["generic", "auto"])
@pytest.mark.parametrize("name", golden_names("qmm_"))
def test_fixture(aclnn, name, kernel):
    from gpu_util import check_close, run_qmm_fixture

    a, meta = load_golden(name)
    got = run_qmm_fixture(aclnn, a, meta, kernel=kernel)
    check_close(got, a["out"], _ref32(a, meta), meta["out_dtype"], exact=name in EXACT)


def test_c1_shape_int32_accumulator_bit_exact(aclnn):
    """The int8 benchmark shape (m128 k4096 n4096): int32 accumulator (+ int32 bias) bit-exact, bf16 output bit-exact."""
    import torch

    from gpu_util import DEV, out_tensor, out_to_np

    rng = np.random.default_rng(1001)
    m, k, n = 128, 4096, 4096
    x1 = rng.integers(-127, 128, (m, k), dtype=np.int8)
    x2 = rng.integers(-127, 128, (k, n), dtype=np.int8)
    s2 = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    s1 = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    bias = rng.integers(-1000, 1001, n).astype(np.int32)
    acc = qbmm_oracle.quant_matmul_v5(x1, x2, None, s2, bias, out_dtype="int32")
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, bias, out_dtype="bfloat16")
    tx1, tx2 = torch.from_numpy(x1).to(DEV), torch.from_numpy(x2).to(DEV)
    ts1, ts2, tb = torch.from_numpy(s1).to(DEV), torch.from_numpy(s2).to(DEV), torch.from_numpy(bias).to(DEV)
    o32 = out_tensor((m, n), "int32")
    aclnn.quant_matmul_v5(aclnn.from_torch(tx1), aclnn.from_torch(tx2), None, aclnn.from_torch(ts2), aclnn.from_torch(o32),
                          aclnn.from_torch(tb))
    obf = out_tensor((m, n), "bfloat16")
    aclnn.quant_matmul_v5(aclnn.from_torch(tx1), aclnn.from_torch(tx2), aclnn.from_torch(ts1), aclnn.from_torch(ts2),
                          aclnn.from_torch(obf), aclnn.from_torch(tb))
    torch.cuda.synchronize()
    assert np.array_equal(o32.cpu().numpy(), acc)
    assert np.array_equal(out_to_np(obf).view(np.uint16), want.view(np.uint16))


def test_row_strided_n_shard_views(aclnn):
    """N-sharding hands the kernel column slices of x2/x2Scale/bias/out without copying: row-strided views."""
    import torch

    from gpu_util import DEV, out_to_np

    rng = np.random.default_rng(7)
    m, k, n, r = 48, 256, 512, 4
    x1 = rng.integers(-127, 128, (m, k), dtype=np.int8)
    x2 = rng.integers(-127, 128, (k, n), dtype=np.int8)
    s2 = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    s1 = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, None, out_dtype="bfloat16")
    tx1, tx2 = torch.from_numpy(x1).to(DEV), torch.from_numpy(x2).to(DEV)
    ts1, ts2 = torch.from_numpy(s1).to(DEV), torch.from_numpy(s2).to(DEV)
    out = torch.zeros((m, n), dtype=torch.bfloat16, device=DEV)
    for i in range(r):
        sl = slice(i * n // r, (i + 1) * n // r)
        aclnn.quant_matmul_v5(aclnn.from_torch(tx1), aclnn.from_torch(tx2[:, sl]), aclnn.from_torch(ts1),
                              aclnn.from_torch(ts2[sl]), aclnn.from_torch(out[:, sl]))
    torch.cuda.synchronize()
    assert np.array_equal(out_to_np(out).view(np.uint16), want.view(np.uint16))


def test_phase2_rejects_small_workspace_and_reused_executor(aclnn):
    import ctypes

    import torch

    from gpu_util import DEV

    x1 = torch.zeros((16, 32), dtype=torch.int8, device=DEV)
    x2 = torch.zeros((32, 16), dtype=torch.int8, device=DEV)
    sc = torch.ones((16,), dtype=torch.float32, device=DEV)
    out = torch.zeros((16, 16), dtype=torch.bfloat16, device=DEV)
    st, ws, ex = aclnn.quant_matmul_v5_get_workspace_size(aclnn.from_torch(x1), aclnn.from_torch(x2), None, aclnn.from_torch(sc),
                                                          None, None, None, None, None, False, False, 0, aclnn.from_torch(out))
    assert st == 0
    L = aclnn.lib()
    assert L.aclnnQuantMatmulV5(None, 0, None, None) == aclnn.ACLNN_ERR_PARAM_NULLPTR
    assert L.aclnnQuantMatmulV5(None, ctypes.c_uint64(ws), ex, None) == 0
    torch.cuda.synchronize()


ASYM_CASES = [
    # m, k, n, transpose_x1, transpose_x2, out dtype
    # (the reference takes this mode with x1 (m,k), x2 stored (n,k), k a multiple of 1024 and n of 256 only: quant_matmul_checker.cpp:354-395)
    (512, 1024, 768, False, True, "bfloat16"),
    (300, 2048, 512, False, True, "float16"),     # ragged m
    (64, 1024, 256, False, True, "bfloat16"),     # less than one tile of rows
    (1000, 2048, 1280, False, True, "bfloat16"),  # several tiles per CTA pair
]


@pytest.mark.parametrize("case", ASYM_CASES, ids=[str(c) for c in ASYM_CASES])
def test_int4_asymmetric_per_group_on_the_tensor_core(aclnn, case, monkeypatch):
    """INT4 x INT4 with a per-group (256 of k) x2Scale and x2Offset and a per-token x1Scale (qbmmv4_kernel_golden.py:328-395):
    operands widened to INT8, then the CTA-pair tensor-core kernel with two k-blocks per accumulation group and the golden's four
    roundings per group in the epilogue. Bit-identical to the oracle and to the coverage kernel."""
    import ml_dtypes
    import torch

    from gpu_util import desc, out_tensor, out_to_np

    m, k, n, t1, t2, out_name = case
    rng = np.random.default_rng(m * 7 + n)
    groups = -(-k // 256)
    x1 = rng.integers(-8, 8, (k, m) if t1 else (m, k)).astype(ml_dtypes.int4)
    x2 = rng.integers(-8, 8, (n, k) if t2 else (k, n)).astype(ml_dtypes.int4)
    s1 = rng.uniform(0.01, 0.1, (m, 1)).astype(np.float32)
    s2 = rng.uniform(0.01, 0.1, (groups, n)).astype(np.float32)
    off = rng.uniform(-4, 4, (groups, n)).astype(np.float16)
    group = 256
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, None, t1, t2, group, out_name, x2_offset=off)

    def run():
        out = out_tensor((m, n), out_name)
        aclnn.quant_matmul_v5(desc(aclnn, x1), desc(aclnn, x2), desc(aclnn, s1), desc(aclnn, s2), aclnn.Tensor(out.shape, out_name, out), None,
                              t1, t2, group, x2_offset=desc(aclnn, off))
        torch.cuda.synchronize()
        assert aclnn.lib().opsnn_qmm_umma_status(1) == 0
        return out_to_np(out), aclnn.last_kernel_name()

    got, name = run()
    assert name == "qmm_umma_pair_pergroup_asym", name
    bits = lambda a: a.view(np.uint16) if a.dtype.itemsize == 2 else a.view(np.uint32)  # noqa: E731
    assert np.array_equal(bits(got), bits(want))
    monkeypatch.setenv("OPSNN_QMM_ASYM_GENERIC", "1")
    ref, ref_name = run()
    assert ref_name != name and np.array_equal(bits(ref), bits(got))
