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
