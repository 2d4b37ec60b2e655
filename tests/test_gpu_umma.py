"""GPU parity of the tcgen05 (TMA + tensor-memory) kernels against the oracle, on seeded inputs whose row pitches satisfy
the 16-byte rule of TMA, over every operand majorness, tile width, tail and batch form the kernel claims."""
import ml_dtypes
import numpy as np
import pytest

from conftest import case_seed
from oracle import qbmm_oracle

pytestmark = pytest.mark.gpu

E4M3, E5M2 = ml_dtypes.float8_e4m3fn, ml_dtypes.float8_e5m2


def _run(aclnn, x1, x2, s1, s2, bias, t1, t2, group, out_name, expect_kernel, bn=None):
    import os

    from gpu_util import desc, out_tensor, out_to_np
    import torch

    m = x1.shape[-1] if t1 else x1.shape[-2]
    n = x2.shape[-2] if t2 else x2.shape[-1]
    batch = tuple(x1.shape[:-2]) if x1.ndim > 2 else (tuple(x2.shape[:-2]) if x2.ndim > 2 else ())
    out = out_tensor(batch + (m, n), out_name)
    if bn:
        os.environ["OPSNN_QMM_BN"] = str(bn)
    try:
        aclnn.quant_matmul_v5(desc(aclnn, x1), desc(aclnn, x2), desc(aclnn, s1), desc(aclnn, s2),
                              aclnn.Tensor(out.shape, out_name, out), desc(aclnn, bias), t1, t2, group)
    finally:
        os.environ.pop("OPSNN_QMM_BN", None)
    torch.cuda.synchronize()
    assert aclnn.last_kernel_name() == expect_kernel, aclnn.last_kernel_name()
    assert aclnn.lib().opsnn_qmm_umma_status(1) == 0
    return out_to_np(out)


INT8_CASES = [
    # m, k, n, t1, t2, bn, per-token, bias kind, out
    (128, 256, 512, False, False, None, True, "i32", "bfloat16"),
    (300, 400, 384, False, False, 128, True, None, "bfloat16"),      # tails in m and k, mn-major B
    (300, 400, 384, False, False, 256, True, "f32", "float16"),
    (130, 1040, 208, False, True, 32, True, "i32", "bfloat16"),      # k-major B, narrow tiles
    (130, 1040, 208, False, True, 64, False, None, "bfloat16"),
    (130, 1040, 208, False, True, 256, True, "bf16", "bfloat16"),
    (272, 528, 400, True, False, 128, True, None, "float16"),        # mn-major A (x1 stored (k,m)), mn-major B
    (272, 528, 400, True, True, 64, True, "i32", "bfloat16"),        # mn-major A, k-major B
    (64, 4096, 1024, False, False, None, False, "i32", "int32"),     # int32 accumulator out
    (1, 128, 16, False, True, None, True, None, "bfloat16"),
    (300, 400, 384, False, False, 64, True, "i32", "bfloat16"),      # n-major B in the 64-byte swizzle
    (130, 528, 208, False, False, 32, True, "f32", "float16"),       # n-major B in the 32-byte swizzle, n tail
    (272, 528, 400, True, False, 32, False, None, "bfloat16"),       # both operands stored along m / n
    (128, 4096, 1024, False, False, None, True, "i32", "bfloat16"),  # few tiles: the host picks a narrow tile by itself
    (2200, 256, 304, False, False, 128, True, "i32", "bfloat16"),    # 18 tile rows: a band of 16 and a ragged band of 2
]


@pytest.mark.parametrize("case", INT8_CASES, ids=[str(c) for c in INT8_CASES])
def test_int8_dequant_bit_exact(aclnn, case):
    m, k, n, t1, t2, bn, pertoken, bias_kind, out_name = case
    rng = np.random.default_rng(case_seed(case))
    x1 = rng.integers(-127, 128, (k, m) if t1 else (m, k), dtype=np.int8)
    x2 = rng.integers(-127, 128, (n, k) if t2 else (k, n), dtype=np.int8)
    s2 = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    s1 = rng.uniform(1e-3, 1e-2, m).astype(np.float32) if (pertoken and out_name != "int32") else None
    bias = {None: None, "i32": rng.integers(-1000, 1001, n).astype(np.int32), "f32": rng.uniform(-1, 1, n).astype(np.float32),
            "bf16": rng.uniform(-1, 1, n).astype(np.float32).astype(ml_dtypes.bfloat16)}[bias_kind]
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, bias, t1, t2, 0, out_name)
    got = _run(aclnn, x1, x2, s1, s2, bias, t1, t2, 0, out_name, "qmm_umma_deq", bn)
    assert np.array_equal(np.asarray(got).view(np.uint8), np.asarray(want).view(np.uint8)), \
        "%d of %d elements differ" % ((np.asarray(got).astype(np.float64) != np.asarray(want).astype(np.float64)).sum(), got.size)


def test_int8_batched_and_broadcast(aclnn):
    rng = np.random.default_rng(77)
    x1 = rng.integers(-127, 128, (3, 160, 256), dtype=np.int8)
    x2 = rng.integers(-127, 128, (256, 320), dtype=np.int8)  # broadcast over the batch
    s2 = rng.uniform(1e-3, 1e-2, 320).astype(np.float32)
    want = qbmm_oracle.quant_matmul_v5(x1, x2, None, s2, None, False, False, 0, "bfloat16")
    got = _run(aclnn, x1, x2, None, s2, None, False, False, 0, "bfloat16", "qmm_umma_deq")
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    x2b = rng.integers(-127, 128, (3, 320, 256), dtype=np.int8)
    want = qbmm_oracle.quant_matmul_v5(x1, x2b, None, s2, None, False, True, 0, "bfloat16")
    got = _run(aclnn, x1, x2b, None, s2, None, False, True, 0, "bfloat16", "qmm_umma_deq")
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def _fp8(rng, shape, dt):
    return rng.standard_normal(shape).astype(np.float32).astype(dt)


PB_CASES = [
    # m, k, n, t1, t2, group_m, bn, da, db, out
    (256, 512, 512, False, False, 1, 256, E4M3, E4M3, "bfloat16"),
    (200, 400, 304, False, False, 1, 128, E4M3, E4M3, "bfloat16"),    # tails everywhere (pitches still 16-byte multiples)
    (200, 400, 304, False, True, 128, 256, E4M3, E5M2, "float16"),    # B-B, k-major B
    (208, 400, 304, True, False, 128, 128, E5M2, E4M3, "float32"),    # x1 stored (k,m)
    (208, 400, 304, True, True, 1, 256, E4M3, E4M3, "bfloat16"),
]


@pytest.mark.parametrize("case", PB_CASES, ids=[str(c[:7]) for c in PB_CASES])
def test_fp8_perblock(aclnn, case):
    from gpu_util import check_close

    m, k, n, t1, t2, gm, bn, da, db, out_name = case
    rng = np.random.default_rng(case_seed(case[:7]))
    x1 = _fp8(rng, (k, m) if t1 else (m, k), da)
    x2 = _fp8(rng, (n, k) if t2 else (k, n), db)
    kb, mg, ng = -(-k // 128), -(-m // gm), -(-n // 128)
    s1 = rng.uniform(0.5, 2, (kb, mg) if t1 else (mg, kb)).astype(np.float32)
    s2 = rng.uniform(0.5, 2, (ng, kb) if t2 else (kb, ng)).astype(np.float32)
    group = (gm << 32) | (128 << 16) | 128
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, None, t1, t2, group, out_name)
    ref32 = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, None, t1, t2, group, "float32")
    got = _run(aclnn, x1, x2, s1, s2, None, t1, t2, group, out_name, "qmm_umma_perblock", bn)
    check_close(got, want, ref32, out_name)

I8PB_CASES = [
    # m, k, n, t1, t2, bn, bias, out
    (256, 512, 512, False, False, 128, None, "bfloat16"),
    (200, 400, 304, False, False, 256, "f32", "bfloat16"),   # tails everywhere
    (200, 400, 304, False, True, 128, "bf16", "bfloat16"),   # k-major B, scales (n/128, k/128)
    (208, 400, 304, True, False, 128, "i32", "bfloat16"),    # x1 stored (k,m), scales (k/128, m)
    (144, 1040, 208, True, True, 256, "f32", "float16"),
]


@pytest.mark.parametrize("case", I8PB_CASES, ids=[str(c) for c in I8PB_CASES])
def test_int8_perblock_bit_exact(aclnn, case):
    """int8 with 1 x 128 / 128 x 128 fp32 scales: each 128-k partial is an exact int32, converted, multiplied by
    s1 * s2 and added with separate roundings like the reference's golden, so the result is compared bit for bit."""
    m, k, n, t1, t2, bn, bias_kind, out_name = case
    rng = np.random.default_rng(case_seed(case))
    x1 = rng.integers(-127, 128, (k, m) if t1 else (m, k), dtype=np.int8)
    x2 = rng.integers(-127, 128, (n, k) if t2 else (k, n), dtype=np.int8)
    kb, ng = -(-k // 128), -(-n // 128)
    s1 = rng.uniform(1e-3, 1e-2, (kb, m) if t1 else (m, kb)).astype(np.float32)
    s2 = rng.uniform(1e-2, 1e-1, (ng, kb) if t2 else (kb, ng)).astype(np.float32)
    bias = {None: None, "f32": rng.standard_normal(n).astype(np.float32), "i32": rng.integers(-5, 6, n).astype(np.int32),
            "bf16": rng.standard_normal(n).astype(ml_dtypes.bfloat16)}[bias_kind]
    group = (1 << 32) | (128 << 16) | 128
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, bias, t1, t2, group, out_name)
    got = _run(aclnn, x1, x2, s1, s2, bias, t1, t2, group, out_name, "qmm_umma_perblock", bn)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))



def test_fp8_dequant_doublescale(aclnn):
    from gpu_util import check_close

    rng = np.random.default_rng(5)
    x1, x2 = _fp8(rng, (144, 256), E4M3), _fp8(rng, (256, 208), E4M3)
    s1 = rng.uniform(0.5, 2, 1).astype(np.float32)
    s2 = rng.uniform(0.5, 2, 208).astype(np.float32)
    bias = rng.uniform(-1, 1, 208).astype(np.float32)
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, bias, False, False, 0, "bfloat16")
    ref32 = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, bias, False, False, 0, "float32")
    got = _run(aclnn, x1, x2, s1, s2, bias, False, False, 0, "bfloat16", "qmm_umma_deq")
    check_close(got, want, ref32, "bfloat16")


PAIR_CASES = [
    # m, k, n, t1, t2, per-token, bias kind, out
    (256, 256, 256, False, True, True, "i32", "bfloat16"),
    (512, 1024, 768, False, False, True, None, "bfloat16"),        # n-major B, each CTA loads its own 128 columns
    (300, 400, 400, False, False, True, "f32", "float16"),         # tails in m (odd CTA partly / wholly past m), k and n
    (640, 528, 336, True, True, True, "i32", "bfloat16"),          # x1 stored (k,m)
    (257, 2048, 272, False, True, False, "bf16", "bfloat16"),      # one row in the second CTA's half
    (2500, 256, 528, False, True, True, "i32", "bfloat16"),        # 10 pair-tile rows: a band of 8 and a ragged band of 2
]


@pytest.mark.parametrize("case", PAIR_CASES, ids=[str(c) for c in PAIR_CASES])
def test_int8_dequant_cta_pairs_bit_exact(aclnn, case, monkeypatch):
    """The cta_group::2 kernel (two CTAs of a cluster share a 256 x 256 tile), forced for shapes the host tile selection
    would give to the single-CTA kernel, against the oracle: bit for bit."""
    m, k, n, t1, t2, pertoken, bias_kind, out_name = case
    monkeypatch.setenv("OPSNN_QMM_PAIR", "1")
    rng = np.random.default_rng(case_seed(case))
    x1 = rng.integers(-127, 128, (k, m) if t1 else (m, k), dtype=np.int8)
    x2 = rng.integers(-127, 128, (n, k) if t2 else (k, n), dtype=np.int8)
    s2 = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    s1 = rng.uniform(1e-3, 1e-2, m).astype(np.float32) if pertoken else None
    bias = {None: None, "i32": rng.integers(-1000, 1001, n).astype(np.int32), "f32": rng.uniform(-1, 1, n).astype(np.float32),
            "bf16": rng.uniform(-1, 1, n).astype(np.float32).astype(ml_dtypes.bfloat16)}[bias_kind]
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, bias, t1, t2, 0, out_name)
    got = _run(aclnn, x1, x2, s1, s2, bias, t1, t2, 0, out_name, "qmm_umma_pair_deq")
    assert np.array_equal(np.asarray(got).view(np.uint8), np.asarray(want).view(np.uint8))


def test_cta_pairs_batched_fp8_and_auto_selection(aclnn, monkeypatch):
    from gpu_util import check_close

    # large enough for the host tile selection to pick pairs by itself: 3 x 1024 x 1024 -> 48 pair tiles... needs >= 74
    rng = np.random.default_rng(9)
    x1 = rng.integers(-127, 128, (5, 1024, 512), dtype=np.int8)
    x2 = rng.integers(-127, 128, (5, 1024, 512), dtype=np.int8)  # stored (n,k)
    s2 = rng.uniform(1e-3, 1e-2, 1024).astype(np.float32)
    want = qbmm_oracle.quant_matmul_v5(x1, x2, None, s2, None, False, True, 0, "bfloat16")
    got = _run(aclnn, x1, x2, None, s2, None, False, True, 0, "bfloat16", "qmm_umma_pair_deq")  # 5 * 4 * 4 = 80 tiles
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    # fp8 per-tensor/-channel dequant on pairs
    monkeypatch.setenv("OPSNN_QMM_PAIR", "1")
    a1, a2 = _fp8(rng, (384, 512), E4M3), _fp8(rng, (512, 320), E5M2)
    sc2 = rng.uniform(0.5, 2, 320).astype(np.float32)
    sc1 = rng.uniform(0.5, 2, 384).astype(np.float32)
    want = qbmm_oracle.quant_matmul_v5(a1, a2, sc1, sc2, None, False, False, 0, "bfloat16")
    ref32 = qbmm_oracle.quant_matmul_v5(a1, a2, sc1, sc2, None, False, False, 0, "float32")
    got = _run(aclnn, a1, a2, sc1, sc2, None, False, False, 0, "bfloat16", "qmm_umma_pair_deq")
    check_close(got, want, ref32, "bfloat16")


def test_older_entry_points_v4_v3_match_v5(aclnn):
    """aclnnQuantMatmulV4 / V3 run the same plan and kernel as V5: bit-identical output."""
    import torch

    from gpu_util import desc, out_tensor, out_to_np

    rng = np.random.default_rng(31)
    m, k, n = 192, 512, 320
    x1 = rng.integers(-127, 128, (m, k), dtype=np.int8)
    x2 = rng.integers(-127, 128, (k, n), dtype=np.int8)
    s2 = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    s1 = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    bias = rng.integers(-1000, 1001, n).astype(np.int32)
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, bias, False, False, 0, "bfloat16")
    out = out_tensor((m, n), "bfloat16")
    aclnn.quant_matmul_v4(desc(aclnn, x1), desc(aclnn, x2), desc(aclnn, s2), aclnn.Tensor(out.shape, "bfloat16", out),
                          pertoken_scale=desc(aclnn, s1), bias=desc(aclnn, bias))
    torch.cuda.synchronize()
    assert aclnn.last_kernel_name() == "qmm_umma_deq"
    assert np.array_equal(out_to_np(out).view(np.uint16), want.view(np.uint16))
    want3 = qbmm_oracle.quant_matmul_v5(x1, x2, None, s2, bias, False, False, 0, "bfloat16")
    out3 = out_tensor((m, n), "bfloat16")
    aclnn.quant_matmul_v4(desc(aclnn, x1), desc(aclnn, x2), desc(aclnn, s2), aclnn.Tensor(out3.shape, "bfloat16", out3),
                          bias=desc(aclnn, bias), api="v3")
    torch.cuda.synchronize()
    assert np.array_equal(out_to_np(out3).view(np.uint16), want3.view(np.uint16))


PAIR_PB_CASES = [
    # m, k, n, t1, t2, group_m, int8, bias, out
    (512, 512, 256, False, True, 1, False, None, "bfloat16"),       # k-major B as stored
    (512, 512, 256, False, False, 1, False, None, "bfloat16"),      # x2 stored (k,n): transposed into workspace first
    (300, 400, 304, False, False, 128, False, None, "float16"),     # tails in m, n, k; B-B
    (272, 528, 400, True, True, 1, False, None, "float32"),         # x1 stored (k,m)
    (512, 1024, 384, False, False, 1, True, "f32", "bfloat16"),     # int8: bit-exact
    (304, 400, 304, True, True, 1, True, "i32", "bfloat16"),
    (2500, 256, 272, False, False, 1, True, None, "bfloat16"),      # 10 pair-tile rows: a band of 8 and a ragged band of 2
]


@pytest.mark.parametrize("tile_n", ["128", "256"])
@pytest.mark.parametrize("case", PAIR_PB_CASES, ids=[str(c) for c in PAIR_PB_CASES])
def test_perblock_cta_pairs(aclnn, case, tile_n, monkeypatch):
    """The per-block kernels on CTA pairs (256 x 128 tiles with four TMEM buffers, or 256 x 256 tiles with two and the register
    file re-divided between the warp roles): same promotion arithmetic as the single-CTA kernel; the int8 form stays
    bit-identical to the reference."""
    from gpu_util import check_close

    m, k, n, t1, t2, gm, is_int, bias_kind, out_name = case
    rng = np.random.default_rng(case_seed(case))
    kb, mg, ng = -(-k // 128), -(-m // gm), -(-n // 128)
    if is_int:
        x1 = rng.integers(-127, 128, (k, m) if t1 else (m, k), dtype=np.int8)
        x2 = rng.integers(-127, 128, (n, k) if t2 else (k, n), dtype=np.int8)
        s1 = rng.uniform(1e-3, 1e-2, (kb, mg) if t1 else (mg, kb)).astype(np.float32)
        s2 = rng.uniform(1e-2, 1e-1, (ng, kb) if t2 else (kb, ng)).astype(np.float32)
    else:
        x1 = _fp8(rng, (k, m) if t1 else (m, k), E4M3)
        x2 = _fp8(rng, (n, k) if t2 else (k, n), E4M3)
        s1 = rng.uniform(0.5, 2, (kb, mg) if t1 else (mg, kb)).astype(np.float32)
        s2 = rng.uniform(0.5, 2, (ng, kb) if t2 else (kb, ng)).astype(np.float32)
    bias = {None: None, "f32": rng.standard_normal(n).astype(np.float32), "i32": rng.integers(-5, 6, n).astype(np.int32)}[bias_kind]
    group = (gm << 32) | (128 << 16) | 128
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, bias, t1, t2, group, out_name)
    monkeypatch.setenv("OPSNN_QMM_PAIR", "1")
    monkeypatch.setenv("OPSNN_QMM_PB_BN", tile_n)
    got = _run(aclnn, x1, x2, s1, s2, bias, t1, t2, group, out_name, "qmm_umma_pair_perblock")
    if is_int:
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    else:
        ref32 = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, None, t1, t2, group, "float32")
        check_close(got, want, ref32, out_name)


KSPLIT_CASES = [
    # m, k, n, t1, t2, ksplit, per-token, bias, out
    (128, 4096, 512, False, False, 4, True, "i32", "bfloat16"),
    (100, 1040, 208, False, True, 2, True, "f32", "float16"),      # k tail: the last split is shorter
    (130, 2048, 300, False, True, 3, False, None, "bfloat16"),     # two m tiles, uneven splits
    (64, 4096, 1024, False, False, 8, False, "i32", "int32"),      # raw int32 accumulator out
    (128, 2048, 256, True, False, 5, True, None, "bfloat16"),      # x1 stored (k,m)
]


@pytest.mark.parametrize("case", KSPLIT_CASES, ids=[str(c) for c in KSPLIT_CASES])
def test_int8_split_k_bit_exact(aclnn, case, monkeypatch):
    """Few output tiles: the k range is split over several CTAs, partial int32 tiles meet in the workspace and the CTA that
    completes the tile's arrival count sums them and runs the epilogue. Integer partial sums: still bit-identical."""
    m, k, n, t1, t2, ks, per_token, bias_kind, out_name = case
    rng = np.random.default_rng(case_seed(case))
    x1 = rng.integers(-127, 128, (k, m) if t1 else (m, k), dtype=np.int8)
    x2 = rng.integers(-127, 128, (n, k) if t2 else (k, n), dtype=np.int8)
    s2 = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    s1 = rng.uniform(1e-3, 1e-2, m).astype(np.float32) if per_token else None
    bias = {None: None, "i32": rng.integers(-1000, 1001, n).astype(np.int32), "f32": rng.standard_normal(n).astype(np.float32)}[bias_kind]
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, bias, t1, t2, 0, out_name)
    monkeypatch.setenv("OPSNN_QMM_KSPLIT", str(ks))
    for _ in range(2):  # the second call finds the first call's counters in the workspace: the nonce tells them apart
        got = _run(aclnn, x1, x2, s1, s2, bias, t1, t2, 0, out_name, "qmm_umma_deq_splitk")
        assert np.array_equal(np.asarray(got).view(np.uint8), np.asarray(want).view(np.uint8))


def test_fp8_split_k(aclnn, monkeypatch):
    from gpu_util import check_close

    rng = np.random.default_rng(77)
    m, k, n = 96, 3072, 384
    x1, x2 = _fp8(rng, (m, k), E4M3), _fp8(rng, (n, k), E5M2)
    s1 = rng.uniform(0.5, 2, m).astype(np.float32)
    s2 = rng.uniform(0.5, 2, n).astype(np.float32)
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, None, False, True, 0, "bfloat16")
    ref32 = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, None, False, True, 0, "float32")
    monkeypatch.setenv("OPSNN_QMM_KSPLIT", "4")
    got = _run(aclnn, x1, x2, s1, s2, None, False, True, 0, "bfloat16", "qmm_umma_deq_splitk")
    check_close(got, want, ref32, "bfloat16")


def test_perblock_cta_pairs_batched(aclnn, monkeypatch):
    """Batched per-block operands on the CTA-pair kernel: per-batch scales, x2 stored (k,n)."""
    from gpu_util import check_close

    rng = np.random.default_rng(4242)
    b, m, k, n = 3, 272, 384, 256
    x1, x2 = _fp8(rng, (b, m, k), E4M3), _fp8(rng, (b, k, n), E4M3)
    s1 = rng.uniform(0.5, 2, (b, m, k // 128)).astype(np.float32)
    s2 = rng.uniform(0.5, 2, (b, k // 128, n // 128)).astype(np.float32)
    group = (1 << 32) | (128 << 16) | 128
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, None, False, False, group, "bfloat16")
    ref32 = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, None, False, False, group, "float32")
    monkeypatch.setenv("OPSNN_QMM_PAIR", "1")
    got = _run(aclnn, x1, x2, s1, s2, None, False, False, group, "bfloat16", "qmm_umma_pair_perblock")
    check_close(got, want, ref32, "bfloat16")


def test_tensor_core_wait_that_runs_out_reaches_the_caller(aclnn, monkeypatch):
    """Every wait in the tcgen05 kernels is bounded. A test-only switch makes the copy producer stop after the eighth k-block of
    each tile with the poll limit cut to thousands, so the MMA warp's wait for the ninth runs out while nothing is in flight.
    The kernel must come back by itself (all roles leave, TMEM is freed), the error word must be set, the NEXT aclnn call must
    be refused with ACLNN_ERR_RUNTIME_ERROR (the word is mirrored to the host), and after opsnn_qmm_umma_status(1) everything
    works again. Nothing faults, traps or hangs: the wait simply gives up."""
    import torch

    from gpu_util import DEV, out_to_np

    rng = np.random.default_rng(11)
    m, k, n = 256, 4096, 512
    x1 = rng.integers(-127, 128, (m, k), dtype=np.int8)
    x2 = rng.integers(-127, 128, (k, n), dtype=np.int8)
    s1 = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    s2 = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    t = lambda a: aclnn.from_torch(torch.from_numpy(a).to(DEV))  # noqa: E731
    d = [t(x1), t(x2), t(s1), t(s2)]
    L = aclnn.lib()
    assert L.opsnn_qmm_umma_status(1) == 0

    def run():
        out = torch.full((m, n), -7777.0, dtype=torch.bfloat16, device=DEV)
        aclnn.quant_matmul_v5(d[0], d[1], d[2], d[3], aclnn.from_torch(out))
        torch.cuda.synchronize()
        return out

    monkeypatch.setenv("OPSNN_QMM_PAIR", "0")  # the single-CTA kernel carries the test switch
    monkeypatch.setenv("OPSNN_TEST_UMMA_STALL_KBLOCK", "8")
    monkeypatch.setenv("OPSNN_TEST_UMMA_POLL_LIMIT", "20000")
    run()
    assert aclnn.last_kernel_name() == "qmm_umma_deq"
    monkeypatch.delenv("OPSNN_TEST_UMMA_STALL_KBLOCK")
    monkeypatch.delenv("OPSNN_TEST_UMMA_POLL_LIMIT")
    with pytest.raises(aclnn.AclnnError) as err:  # refused before anything is enqueued
        run()
    assert err.value.status == aclnn.ACLNN_ERR_RUNTIME_ERROR and "bounded wait" in str(err.value)
    code = L.opsnn_qmm_umma_status(1)  # read and clear; also restores the poll limit
    assert code != 0 and (code >> 8) in (2, 3), hex(code)  # the MMA issuer or an epilogue warp gave up first
    out = run()
    assert L.opsnn_qmm_umma_status(1) == 0
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, None, out_dtype="bfloat16")
    assert np.array_equal(out_to_np(out).view(np.uint16), want.view(np.uint16))
