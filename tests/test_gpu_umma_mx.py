"""GPU parity of the block-scaled (MX) tcgen05 kernels against the oracle restatement of the reference golden
(quant_batch_matmul_v3/tests/assets/qbmmv3_kernel_golden.py:153-234): MXFP8 via kind::mxf8f6f4, MXFP4 via kind::mxf4.

Every product e4m3*e4m3*2^e (or e2m1*e2m1*2^e) is exact in fp32 and the sums here stay far below 2^24 ulps of cancellation,
so the only differences from the golden are fp32 summation order; the stated tolerance (max relative error <= 1e-2 for
bf16, 5e-3 for fp16/fp32, against the fp32 dequantised product) is asserted, and in fact a much tighter one holds."""
import ml_dtypes
import numpy as np
import pytest

from conftest import case_seed, load_golden
from oracle import qbmm_oracle

pytestmark = pytest.mark.gpu

E4M3, E5M2, E2M1, E8M0 = ml_dtypes.float8_e4m3fn, ml_dtypes.float8_e5m2, ml_dtypes.float4_e2m1fn, ml_dtypes.float8_e8m0fnu
GROUP_MX = (1 << 32) | (1 << 16) | 32


def _e8m0(rng, shape, lo=-3, hi=3):
    return np.exp2(rng.integers(lo, hi + 1, shape).astype(np.float32)).astype(E8M0)


def _q(rng, shape, dt):
    return (rng.standard_normal(shape).astype(np.float32) * (2.0 if dt == E2M1 else 1.0)).astype(dt)


def _run(aclnn, x1, x2, s1, s2, bias, t1, t2, out_name, expect_kernel, bn=None):
    """bn: 128 | 224 (host tile selection override) | "pair" (224-column tiles on CTA pairs, tcgen05 cta_group::2)."""
    import os

    import torch

    from gpu_util import desc, out_tensor, out_to_np

    m = x1.shape[-1] if t1 else x1.shape[-2]
    n = x2.shape[-2] if t2 else x2.shape[-1]
    batch = tuple(x1.shape[:-2])
    out = out_tensor(batch + (m, n), out_name)
    if bn == "pair":
        os.environ["OPSNN_QMM_MX_BN"] = "224"
        os.environ["OPSNN_QMM_PAIR"] = "1"
        expect_kernel = expect_kernel.replace("qmm_umma_", "qmm_umma_pair_")
    elif bn:
        os.environ["OPSNN_QMM_MX_BN"] = str(bn)  # host tile selection override: 128- or 224-column tiles
        os.environ["OPSNN_QMM_PAIR"] = "0"
    try:
        aclnn.quant_matmul_v5(desc(aclnn, x1), desc(aclnn, x2), desc(aclnn, s1), desc(aclnn, s2),
                              aclnn.Tensor(out.shape, out_name, out), desc(aclnn, bias), t1, t2, GROUP_MX)
    finally:
        os.environ.pop("OPSNN_QMM_MX_BN", None)
        os.environ.pop("OPSNN_QMM_PAIR", None)
    torch.cuda.synchronize()
    assert aclnn.last_kernel_name() == expect_kernel, aclnn.last_kernel_name()
    assert aclnn.lib().opsnn_qmm_umma_status(1) == 0
    return out_to_np(out)


def _oracle(x1, x2, s1, s2, bias, t1, t2, out_name):
    if x1.ndim == 2:
        return qbmm_oracle.compute_mx(x1, x2, s1, s2, bias, t1, t2, out_name)
    return np.stack([qbmm_oracle.compute_mx(x1[i], x2[i], s1[i], s2[i], bias, t1, t2, out_name) for i in range(x1.shape[0])])


def _check(got, want, out_name):
    g, w = np.asarray(got).astype(np.float64), np.asarray(want).astype(np.float64)
    assert not np.any(g == -7777.0)
    rms = np.sqrt(np.mean(w ** 2))
    rel = np.max(np.abs(g - w) / np.maximum(np.abs(w), 1e-3 * rms))
    assert rel <= (1e-2 if out_name == "bfloat16" else 5e-3), rel
    # summation order only: about one output ulp for the 16-bit outputs, up to a few hundred fp32 ulps where the terms cancel (3e-5 has been seen) for fp32
    tight = {"bfloat16": 2.1 * 2.0 ** -8, "float16": 2.1 * 2.0 ** -11, "float32": 1e-4}[out_name]
    assert np.max(np.abs(g - w) / np.maximum(np.abs(w), 0.05 * rms)) <= tight


MX8_CASES = [
    # batch, m, k, n, t1, t2, a dtype, b dtype, bias, out
    ((), 128, 128, 128, False, True, E4M3, E4M3, None, "float32"),
    ((), 128, 512, 128, False, False, E4M3, E4M3, None, "float32"),           # mn-major B
    ((), 200, 640, 328, False, True, E4M3, E5M2, "f32", "bfloat16"),         # tails in m, n; k not a multiple of 128
    ((), 200, 608, 336, False, False, E5M2, E4M3, "f32", "bfloat16"),        # k = 19 blocks of 32 (odd), mn-major B
    ((), 144, 384, 208, True, True, E4M3, E4M3, None, "float16"),            # mn-major A
    ((3,), 130, 256, 272, False, False, E4M3, E4M3, "f32", "bfloat16"),      # batched
    ((), 1024, 2048, 1536, False, False, E4M3, E4M3, "f32", "bfloat16"),     # many tiles per CTA, deep k
    ((), 256, 512, 1344, False, True, E4M3, E4M3, "f32", "bfloat16"),        # n = 6 x 224
    ((), 256, 512, 1008, False, False, E4M3, E4M3, None, "float32"),         # n-major B, ragged last 224-tile
    ((), 2500, 256, 464, False, True, E4M3, E4M3, "f32", "bfloat16"),        # 20 tile rows / 10 pair-tile rows: ragged last band
]


@pytest.mark.parametrize("bn", [128, 224, "pair"])
@pytest.mark.parametrize("case", MX8_CASES, ids=[str(c[:6]) for c in MX8_CASES])
def test_mxfp8_tcgen05(aclnn, case, bn):
    batch, m, k, n, t1, t2, da, db, bias_kind, out_name = case
    rng = np.random.default_rng(case_seed(str(case)))
    kq = -(-k // 64)
    x1 = _q(rng, batch + ((k, m) if t1 else (m, k)), da)
    x2 = _q(rng, batch + ((n, k) if t2 else (k, n)), db)
    s1 = _e8m0(rng, batch + ((kq, m, 2) if t1 else (m, kq, 2)))
    s2 = _e8m0(rng, batch + ((n, kq, 2) if t2 else (kq, n, 2)))
    bias = None if bias_kind is None else rng.uniform(-2, 2, n).astype(np.float32)  # the API takes only fp32 bias in mx mode
    got = _run(aclnn, x1, x2, s1, s2, bias, t1, t2, out_name, "qmm_umma_mxfp8", bn)
    _check(got, _oracle(x1, x2, s1, s2, bias, t1, t2, out_name), out_name)


MX4_CASES = [
    ((), 128, 256, 128, None, "float32"),
    ((), 128, 64, 128, None, "float32"),                # a quarter of a stage
    ((), 197, 960, 154, "f32", "bfloat16"),
    ((), 256, 1024, 384, None, "float16"),
    ((2,), 140, 512, 264, "f32", "bfloat16"),
    ((), 1024, 4096, 1280, None, "bfloat16"),
]


@pytest.mark.parametrize("bn", [128, 224, "pair"])
@pytest.mark.parametrize("case", MX4_CASES, ids=[str(c[:4]) for c in MX4_CASES])
def test_mxfp4_tcgen05(aclnn, case, bn):
    batch, m, k, n, bias_kind, out_name = case
    rng = np.random.default_rng(case_seed(str(case)))
    kq = -(-k // 64)
    x1 = _q(rng, batch + (m, k), E2M1)
    x2 = _q(rng, batch + (n, k), E2M1)  # stored (n,k): transposeX2 = true
    s1 = _e8m0(rng, batch + (m, kq, 2))
    s2 = _e8m0(rng, batch + (n, kq, 2))
    bias = None if bias_kind is None else rng.uniform(-2, 2, n).astype(np.float32)
    got = _run(aclnn, x1, x2, s1, s2, bias, False, True, out_name, "qmm_umma_mxfp4", bn)
    _check(got, _oracle(x1, x2, s1, s2, bias, False, True, out_name), out_name)


def test_mx_fixtures_run_on_the_tensor_core_kernels(aclnn):
    from gpu_util import run_qmm_fixture

    for name, kern in (("qmm_mxfp8_bias_bf16", "qmm_umma_mxfp8"), ("qmm_mxfp8_transB_oddgroups", "qmm_umma_mxfp8"),
                       ("qmm_mxfp4_transB_fp32", "qmm_umma_mxfp4")):
        a, meta = load_golden(name)
        got = run_qmm_fixture(aclnn, a, meta, kernel=0)
        assert aclnn.last_kernel_name() == kern, (name, aclnn.last_kernel_name())
        _check(got, a["out"], meta["out_dtype"])


@pytest.mark.parametrize("dst", ["float8_e4m3fn", "float8_e5m2", "float4_e2m1"])
@pytest.mark.parametrize("xdt", ["bfloat16", "float16"])
def test_dynamic_mx_quant_streaming_kernel_matches_oracle(aclnn, dst, xdt):
    """The coalesced quantiser (rows a multiple of 32 long) against the oracle of quant/dynamic_mx_quant/tests/assets/golden.py,
    bit for bit, on inputs with outliers, zero blocks, subnormals and huge values."""
    import torch

    from gpu_util import DEV, desc
    from oracle import mx_quant_oracle

    rng = np.random.default_rng(77)
    x = rng.standard_normal((96, 1024)).astype(np.float32)
    x[rng.integers(0, 96, 200), rng.integers(0, 1024, 200)] *= 50.0
    x[3, 64:96] = 0.0
    x[4, :32] = 1e-30
    x[5, 32:64] = 3e4
    xs = x.astype(ml_dtypes.bfloat16 if xdt == "bfloat16" else np.float16)
    want_y, want_s = mx_quant_oracle.dynamic_mx_quant(xs, dst)
    ybytes = xs.shape[:-1] + ((xs.shape[-1] // 2,) if dst == "float4_e2m1" else (xs.shape[-1],))
    y = torch.full(ybytes, 0xAA, dtype=torch.uint8, device=DEV)
    s = torch.full(want_s.shape, 0xAA, dtype=torch.uint8, device=DEV)
    aclnn.dynamic_mx_quant(desc(aclnn, xs), aclnn.Tensor(xs.shape, dst, y), aclnn.Tensor(want_s.shape, "float8_e8m0", s), dst)
    torch.cuda.synchronize()
    assert aclnn.last_kernel_name() == "mx_quant_stream"
    assert np.array_equal(s.cpu().numpy(), np.asarray(want_s).view(np.uint8))
    wy = np.asarray(want_y)
    if dst == "float4_e2m1":
        codes = wy.view(np.uint8)
        wy_bytes = (codes[..., 0::2] & 0xF) | ((codes[..., 1::2] & 0xF) << 4)
    else:
        wy_bytes = wy.view(np.uint8)
    assert np.array_equal(y.cpu().numpy(), wy_bytes)


MX4_LAYOUT_CASES = [
    # batch, m, k, n, x1 stored (k,m), x2 stored (n,k)
    ((), 128, 256, 160, False, False),     # x2 given as (k,n): rewritten k-contiguous by the pre-pass
    ((), 192, 512, 352, True, True),       # x1 given as (k,m)
    ((2,), 160, 384, 224, True, False),    # both, batched
    ((), 256, 320, 384, True, False),      # whole 64 x 128 tiles: the word-wise form of the pre-pass, both operands
    ((3,), 128, 192, 256, False, False),   # the same, batched
]


@pytest.mark.parametrize("case", MX4_LAYOUT_CASES, ids=[str(c) for c in MX4_LAYOUT_CASES])
def test_mxfp4_operands_stored_along_m_or_n(aclnn, case):
    """kind::mxf4 only takes k-contiguous operands; the other storage orders the API allows go through a transpose pre-pass
    into workspace and must give the same result as the oracle."""
    batch, m, k, n, t1, t2 = case
    rng = np.random.default_rng(case_seed(str(case)))
    kq = -(-k // 64)
    x1 = _q(rng, batch + ((k, m) if t1 else (m, k)), E2M1)
    x2 = _q(rng, batch + ((n, k) if t2 else (k, n)), E2M1)
    s1 = _e8m0(rng, batch + ((kq, m, 2) if t1 else (m, kq, 2)))
    s2 = _e8m0(rng, batch + ((n, kq, 2) if t2 else (kq, n, 2)))
    got = _run(aclnn, x1, x2, s1, s2, None, t1, t2, "bfloat16", "qmm_umma_mxfp4", 128)
    _check(got, _oracle(x1, x2, s1, s2, None, t1, t2, "bfloat16"), "bfloat16")


MX8_MOVED_WEIGHT_CASES = [
    # batch, m, k, n: x2 stored (k,n), one copy of it serving >= 4096 output rows, 224-column tiles
    ((), 8200, 160, 208),     # ragged m; k = 2.5 tiles of 64; n below one 256-column tile of the pre-pass
    ((), 8192, 96, 528),      # n = 2 tiles + 16
    ((2,), 8192, 64, 272),    # per-batch weights
]


@pytest.mark.parametrize("case", MX8_MOVED_WEIGHT_CASES, ids=[str(c) for c in MX8_MOVED_WEIGHT_CASES])
def test_mxfp8_weight_stored_along_n_is_moved_k_contiguous(aclnn, case, monkeypatch):
    """An 8-bit x2 stored (k,n) that serves thousands of rows is first rewritten (n,k) into workspace (one more launch);
    the result must equal the one the n-contiguous operand path gives (same kernel, same summation order: bit for bit)
    and agree with the oracle."""
    batch, m, k, n = case
    rng = np.random.default_rng(case_seed(str(case)))
    kq = -(-k // 64)
    x1, x2 = _q(rng, batch + (m, k), E4M3), _q(rng, batch + (k, n), E4M3)
    s1, s2 = _e8m0(rng, batch + (m, kq, 2)), _e8m0(rng, batch + (kq, n, 2))
    bias = rng.uniform(-2, 2, n).astype(np.float32)
    before = aclnn.launch_count()
    got = _run(aclnn, x1, x2, s1, s2, bias, False, False, "bfloat16", "qmm_umma_mxfp8", 224)
    moved = aclnn.launch_count() - before
    monkeypatch.setenv("OPSNN_MX_NO_TRANSPOSE", "1")
    before = aclnn.launch_count()
    plain = _run(aclnn, x1, x2, s1, s2, bias, False, False, "bfloat16", "qmm_umma_mxfp8", 224)
    assert moved == aclnn.launch_count() - before + 1
    assert np.array_equal(got.view(np.uint16), plain.view(np.uint16))
    _check(got, _oracle(x1, x2, s1, s2, bias, False, False, "bfloat16"), "bfloat16")


A8W4_CASES = [
    # m, k, n, mode, out
    (256, 512, 448, "mx", "bfloat16"),
    (130, 1024, 300, "mx", "float16"),      # tails in m and n
    (256, 512, 448, "tcg-bf16", "bfloat16"),
    (130, 1024, 304, "tcg-fp16", "float16"),
]


@pytest.mark.parametrize("case", A8W4_CASES, ids=[str(c) for c in A8W4_CASES])
def test_a8w4_fp8_x_fp4(aclnn, case):
    """fp8 x fp4 (qbmmv4_kernel_golden.py:119-255): the weight is rewritten as fp8 by a pre-pass, then the mx kernel
    (e8m0 scales) or the fp8 dequant kernel (T-CG: group scale folded into the rewrite, uint64 yScale per column) runs."""
    import torch

    from gpu_util import desc, out_tensor, out_to_np

    m, k, n, mode, out_name = case
    rng = np.random.default_rng(case_seed(case))
    x1, x2 = _q(rng, (m, k), E4M3), _q(rng, (n, k), E2M1)
    out = out_tensor((m, n), out_name)
    if mode == "mx":
        s1, s2 = _e8m0(rng, (m, k // 64, 2)), _e8m0(rng, (n, k // 64, 2))
        bias = rng.standard_normal((1, n)).astype(ml_dtypes.bfloat16 if out_name == "bfloat16" else np.float16)
        ys, expect = None, "qmm_umma_mxfp8"
        want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, bias.reshape(-1), False, True, 32, out_name)
    else:
        s1, bias = None, None
        s2 = rng.uniform(0.25, 4, (n, k // 32)).astype(ml_dtypes.bfloat16 if mode == "tcg-bf16" else np.float16)
        sc = rng.uniform(0.01, 0.1, (1, n)).astype(np.float32)
        ys = (sc.view(np.uint32) & np.uint32(0xFFFFE000)).astype(np.uint64)
        expect = "qmm_umma_deq"
        want = qbmm_oracle.quant_matmul_v5(x1, x2, None, s2, None, False, True, 32, out_name, y_scale=ys)
    ws = aclnn.quant_matmul_v5(desc(aclnn, x1), desc(aclnn, x2), desc(aclnn, s1), desc(aclnn, s2),
                               aclnn.Tensor(out.shape, out_name, out), desc(aclnn, bias), False, True, 32, y_scale=desc(aclnn, ys))
    torch.cuda.synchronize()
    assert ws >= n * k  # the rewritten weight lives in the caller's workspace
    assert aclnn.last_kernel_name().startswith(expect), aclnn.last_kernel_name()
    assert aclnn.lib().opsnn_qmm_umma_status(1) == 0
    _check(out_to_np(out), want, out_name)


@pytest.mark.parametrize("dst", [E4M3, E2M1], ids=["mxfp8", "mxfp4"])
def test_16bit_x1_is_quantised_on_the_fly_like_the_two_call_chain(aclnn, dst):
    """aclnnQuantMatmulV5 with a BF16 x1 and no x1Scale against an MX weight (an extension: "dynamic activation quantisation fused
    ahead"): one call pair must give exactly what aclnnDynamicMxQuant followed by the MX matmul gives, and the quantised operand
    must be the quantiser oracle's bit for bit (checked through the two-call chain's buffers)."""
    import torch

    from gpu_util import DEV, desc, out_tensor, out_to_np
    from oracle import mx_quant_oracle

    rng = np.random.default_rng(case_seed("dynq" + str(dst)))
    b, m, k, n = 2, 192, 512, 448
    act = (rng.standard_normal((b, m, k)).astype(np.float32) * np.where(rng.random((b, m, k)) < 1e-3, 50.0, 1.0)).astype(ml_dtypes.bfloat16)
    x2 = _q(rng, (b, n, k), dst)
    s2 = _e8m0(rng, (b, n, k // 64, 2))
    bias = rng.uniform(-2, 2, n).astype(np.float32)
    name = "float4_e2m1" if dst == E2M1 else "float8_e4m3fn"
    yq, sq = mx_quant_oracle.dynamic_mx_quant(act, name)
    d_act, d_x2, d_s2, d_bias = desc(aclnn, act), desc(aclnn, x2), desc(aclnn, s2), desc(aclnn, bias)
    # two calls
    two = out_tensor((b, m, n), "bfloat16")
    aclnn.quant_matmul_v5(desc(aclnn, yq), d_x2, desc(aclnn, sq.view(E8M0)), d_s2, aclnn.Tensor(two.shape, "bfloat16", two), d_bias, False, True,
                          GROUP_MX)
    # one call
    one = out_tensor((b, m, n), "bfloat16")
    before = aclnn.launch_count()
    aclnn.quant_matmul_v5(d_act, d_x2, None, d_s2, aclnn.Tensor(one.shape, "bfloat16", one), d_bias, False, True, GROUP_MX)
    torch.cuda.synchronize()
    assert aclnn.launch_count() - before >= 2 and aclnn.last_kernel_name().startswith("qmm_umma")
    assert np.array_equal(out_to_np(one).view(np.uint16), out_to_np(two).view(np.uint16))
    _check(out_to_np(one), _oracle(yq, x2, sq.view(E8M0), s2, bias, False, True, "bfloat16"), "bfloat16")
