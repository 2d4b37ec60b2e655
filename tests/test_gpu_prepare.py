"""GPU: prepare-once weights (include/opsnn_b200_prepare.h). A registered x2 must give the unprepared call's output bit for bit, with
the per-call layout kernels gone from the launch list; a call on other tensors, or after the release, runs as before."""
import ml_dtypes
import numpy as np
import pytest

from conftest import case_seed
from oracle import qbmm_oracle

pytestmark = pytest.mark.gpu

E4M3, E2M1, E8M0 = ml_dtypes.float8_e4m3fn, ml_dtypes.float4_e2m1fn, ml_dtypes.float8_e8m0fnu
GROUP_MX = (1 << 32) | (1 << 16) | 32

CASES = [
    # dtype, batch, m, k, n, x2 stored (n,k)?
    (E4M3, (), 512, 1024, 1344, False),    # MXFP8, weight stored (k,n): moved k-contiguous once, scale atoms once
    (E4M3, (2,), 300, 512, 672, False),    # batched, ragged m
    (E4M3, (), 256, 512, 896, True),       # already (n,k): only the scale atoms are prepared
    (E2M1, (), 512, 1024, 1344, False),    # MXFP4 stored (k,n): the transposition the tensor core needs, once
    (E2M1, (2,), 256, 512, 448, True),
]


@pytest.mark.parametrize("case", CASES, ids=[str((c[0].__name__,) + c[1:]) for c in CASES])
def test_prepared_equals_unprepared(aclnn, case):
    import torch

    from gpu_util import desc, out_tensor, out_to_np

    dt, batch, m, k, n, t2 = case
    rng = np.random.default_rng(case_seed(str(case)))
    kq = -(-k // 64)
    x1 = (rng.standard_normal(batch + (m, k)).astype(np.float32) * (2.0 if dt == E2M1 else 1.0)).astype(dt)
    x2 = (rng.standard_normal(batch + ((n, k) if t2 else (k, n))).astype(np.float32) * (2.0 if dt == E2M1 else 1.0)).astype(dt)
    s1 = np.exp2(rng.integers(-3, 4, batch + (m, kq, 2)).astype(np.float32)).astype(E8M0)
    s2 = np.exp2(rng.integers(-3, 4, batch + ((n, kq, 2) if t2 else (kq, n, 2))).astype(np.float32)).astype(E8M0)
    bias = rng.uniform(-2, 2, n).astype(np.float32)
    d_x1, d_x2, d_s1, d_s2, d_bias = (desc(aclnn, a) for a in (x1, x2, s1, s2, bias))

    def run():
        out = out_tensor(batch + (m, n), "bfloat16")
        before = aclnn.launch_count()
        aclnn.quant_matmul_v5(d_x1, d_x2, d_s1, d_s2, aclnn.Tensor(out.shape, "bfloat16", out), d_bias, False, t2, GROUP_MX)
        torch.cuda.synchronize()
        return out_to_np(out).view(np.uint16), aclnn.launch_count() - before, aclnn.last_kernel_name()

    plain, launches_plain, kern = run()
    assert kern.startswith("qmm_umma"), kern
    storage = aclnn.prepare_x2(d_x2, d_s2, t2, GROUP_MX, m_hint=m)
    assert storage is not None
    torch.cuda.synchronize()
    prepared, launches_prepared, kern2 = run()
    assert kern2 == kern
    assert np.array_equal(prepared, plain)
    # x2Scale's relayout is gone, and with it the weight move where there was one
    moved = (not t2) and (dt == E2M1)
    assert launches_prepared == launches_plain - 1 - (1 if moved else 0), (launches_plain, launches_prepared)
    # against the oracle as well
    want = qbmm_oracle.compute_mx(x1, x2, s1, s2, bias, False, t2, "float32") if not batch else np.stack(
        [qbmm_oracle.compute_mx(x1[i], x2[i], s1[i], s2[i], bias, False, t2, "float32") for i in range(batch[0])])
    got = prepared.view(ml_dtypes.bfloat16).astype(np.float64)
    rms = np.sqrt(np.mean(want.astype(np.float64) ** 2))
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 0.05 * rms)) <= 1e-2
    # a different m selects its own plan and still agrees with its unprepared self
    aclnn.release_x2(d_x2)
    again, launches_again, _ = run()
    assert np.array_equal(again, plain) and launches_again == launches_plain
    del storage


def test_nothing_to_prepare_for_int8(aclnn):
    import torch

    from gpu_util import DEV

    x2 = aclnn.from_torch(torch.zeros((256, 512), dtype=torch.int8, device=DEV))
    s2 = aclnn.from_torch(torch.ones((512,), dtype=torch.float32, device=DEV))
    assert aclnn.prepare_x2(x2, s2, False, 0, m_hint=128) is None


WQ_CASES = [
    # weight bits, x dtype, m, k, n, group, offset
    (4, "bfloat16", 64, 1024, 1024, 128, True),
    (4, "float16", 300, 2048, 768, 128, False),     # ragged m
    (8, "bfloat16", 128, 1024, 512, 0, True),       # int8 weight, per-channel
]


@pytest.mark.parametrize("case", WQ_CASES, ids=[str(c) for c in WQ_CASES])
def test_prepared_prefill_weight_equals_unprepared(aclnn, case):
    """aclnnWeightQuantBatchMatmulV2 beyond the decode range dequantises the whole weight per call; with the weight registered
    through opsnnWeightQuantPrepare the call asks for no workspace, launches only the matmul and gives the same bits; m <= 16
    keeps streaming the packed weight; after the release everything is as before."""
    import torch

    from gpu_util import DEV
    from oracle import wqbmm_oracle

    bits, xdt, m, k, n, g, has_off = case
    rng = np.random.default_rng(case_seed(str(case)))
    nd = ml_dtypes.bfloat16 if xdt == "bfloat16" else np.float16
    td = torch.bfloat16 if xdt == "bfloat16" else torch.float16
    dev16 = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16).copy()).view(td).to(DEV)  # noqa: E731
    x = rng.standard_normal((m, k)).astype(np.float32).astype(nd)
    groups = k // g if g else 1
    sc = rng.uniform(0.005, 0.02, (groups, n)).astype(np.float32).astype(nd)
    of = rng.uniform(-1, 1, (groups, n)).astype(np.float32).astype(nd) if has_off else None
    if bits == 4:
        w = rng.integers(-8, 8, (k, n)).astype(np.int8)
        tw = torch.from_numpy(wqbmm_oracle.pack_int4_words(w).copy()).to(DEV)
    else:
        w = rng.integers(-128, 128, (k, n)).astype(np.int8)
        tw = torch.from_numpy(w.copy()).to(DEV)
    tx, ts = dev16(x), dev16(sc if g else sc[0])
    to = dev16(of if g else of[0]) if has_off else None
    d_x, d_w, d_s = aclnn.from_torch(tx), aclnn.from_torch(tw), aclnn.from_torch(ts)
    d_o = aclnn.from_torch(to) if has_off else None

    def run(rows):
        y = torch.full((rows, n), -7777.0, dtype=td, device=DEV)
        before = aclnn.launch_count()
        ws = aclnn.weight_quant_batch_matmul(aclnn.from_torch(tx[:rows]), d_w, d_s, aclnn.from_torch(y), d_o, None, g)
        torch.cuda.synchronize()
        return y.view(torch.int16).cpu().numpy().copy(), aclnn.launch_count() - before, ws, aclnn.last_kernel_name()

    plain, launches_plain, ws_plain, name_plain = run(m)
    small_plain = run(16)
    assert ws_plain >= k * n * 2 and launches_plain >= 2
    storage = aclnn.prepare_weight(d_w, d_s, d_o, g, xdt)
    assert storage is not None and storage.numel() >= k * n * 2
    try:
        prepared, launches_prep, ws_prep, name_prep = run(m)
        assert np.array_equal(prepared, plain)
        assert ws_prep == 0 and launches_prep == launches_plain - 1 and name_prep == name_plain
        small_prep = run(16)
        assert np.array_equal(small_prep[0], small_plain[0]) and small_prep[3] == small_plain[3]  # m <= 16: unchanged path
    finally:
        aclnn.release_weight(d_w)
    again = run(m)
    assert np.array_equal(again[0], plain) and again[1] == launches_plain and again[2] == ws_plain
    want = wqbmm_oracle.weight_quant_batch_matmul(x, w, sc, of, None, g).astype(np.float64)
    got = torch.from_numpy(plain).view(td).float().numpy().astype(np.float64)
    rms = np.sqrt(np.mean(want ** 2))
    tol = 2.0 ** -7 if xdt == "bfloat16" else 2.0 ** -9
    assert np.all(np.abs(got - want) <= tol * np.maximum(np.abs(want), 0.05 * rms) * 1.01)
