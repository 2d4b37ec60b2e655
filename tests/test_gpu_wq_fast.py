"""GPU parity of the high-performance precision mode (innerPrecise = 1 of aclnnWeightQuantBatchMatmulV3) of the W4A16
decode path. The reference documents this mode as faster "with some loss of accuracy" and gives it no separate golden
(weight_quant_batch_matmul_v2/docs/aclnnWeightQuantBatchMatmulV3.md:389), so the yardstick is the stated tolerance
against the fp32 dequantised product x @ ((w + offset) * scale) with NO intermediate rounding: max relative error
<= 1e-2 (bf16) / 5e-3 (fp16); the kernel in fact stays within about one output ulp of it."""
import numpy as np
import pytest

from conftest import load_golden
from oracle import wqbmm_oracle

pytestmark = pytest.mark.gpu

FAST_FIXTURES = ["wq_bf16_s4_group128_offset_m16", "wq_bf16_s4_group160_m1_fbias", "wq_fp16_s4_group64_bias_m8",
                 "wq_fp16_s4_channel_offset_bias"]


def _unrounded(a, meta):
    return wqbmm_oracle.fp32_dequant_product(a["x"], a["w"], a["scale"], a.get("offset"), a.get("bias"), meta["group_size"])


@pytest.mark.parametrize("name", FAST_FIXTURES)
def test_fast_mode_fixture(aclnn, name):
    from gpu_util import np_name, run_wq_fixture

    a, meta = load_golden(name)
    got = run_wq_fixture(aclnn, a, meta, kernel=0, api="v3", inner_precise=1).astype(np.float64)
    assert aclnn.last_kernel_name() == "wqbmm_decode_fast", name
    ref = np.asarray(_unrounded(a, meta), dtype=np.float64)
    bf16 = np_name(a["out"]) == "bfloat16"
    rms = np.sqrt(np.mean(ref ** 2))
    den = np.maximum(np.abs(ref), 0.05 * rms)
    rel = np.max(np.abs(got - ref) / den)
    assert rel <= (1e-2 if bf16 else 5e-3), (name, rel)
    # one rounding of the output (bf16: 2^-9 of the value, fp16: 2^-12) plus the fp32 cancellation of the B * sum(x) term (B = 136 /
    # 1032), whose size depends on where the k ranges of the CTAs fall: within two output ulps for fp16
    assert rel <= (2.0 ** -8 if bf16 else 2.0 ** -9) * 1.05, (name, rel)
    # and it is at least as close to the unrounded product as the default mode's golden is
    gold = a["out"].astype(np.float64)
    assert np.max(np.abs(got - ref) / den) <= np.max(np.abs(gold - ref) / den) + 1e-12


def test_default_mode_is_unchanged_by_the_flag_being_zero(aclnn):
    from gpu_util import run_wq_fixture

    a, meta = load_golden("wq_bf16_s4_group128_offset_m16")
    y0 = run_wq_fixture(aclnn, a, meta, kernel=0, api="v3", inner_precise=0)
    assert aclnn.last_kernel_name() == "wqbmm_decode"
    y2 = run_wq_fixture(aclnn, a, meta, kernel=0, api="v2")
    assert np.array_equal(y0.view(np.uint16), y2.view(np.uint16))


def test_fast_mode_c2_shape_properties(aclnn):
    """Full benchmark shape (m16 k8192 n28672 g128) in the high-performance mode: run-to-run determinism, exact zero rows,
    exact linearity under x2, row independence, and 512 sampled columns against the unrounded fp32 dequantised product."""
    import torch

    from gpu_util import DEV, out_to_np

    m, k, n, g = 16, 8192, 28672, 128
    gen = torch.Generator(device=DEV).manual_seed(1002)
    x = torch.randn((m, k), generator=gen, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    x[5].zero_()
    w = torch.randint(-8, 8, (k, n), generator=gen, device=DEV, dtype=torch.int32)
    words = torch.zeros((k, n // 8), dtype=torch.int32, device=DEV)
    for j in range(8):
        words |= (w[:, j::8] & 0xF) << (4 * j)
    scale = (torch.rand((k // g, n), generator=gen, device=DEV) * 0.015 + 0.005).to(torch.bfloat16)
    offset = (torch.rand((k // g, n), generator=gen, device=DEV) * 2 - 1).to(torch.bfloat16)

    def run(xx):
        y = torch.full((xx.shape[0], n), -7777.0, dtype=torch.bfloat16, device=DEV)
        aclnn.weight_quant_batch_matmul(aclnn.from_torch(xx), aclnn.from_torch(words), aclnn.from_torch(scale),
                                        aclnn.from_torch(y), aclnn.from_torch(offset), None, g, inner_precise=1)
        torch.cuda.synchronize()
        assert aclnn.last_kernel_name() == "wqbmm_decode_fast"
        return y

    y1 = run(x)
    assert torch.equal(y1, run(x))
    assert not bool((y1 == -7777.0).any())
    assert bool((y1[5] == 0).all())
    assert torch.equal(run(x * 2).float(), y1.float() * 2)
    assert torch.equal(run(x[3:4].contiguous())[0], y1[3])
    cols = np.sort(np.random.default_rng(3).choice(n, 512, replace=False))
    ct = torch.from_numpy(cols).to(DEV)
    wn = w[:, ct].cpu().numpy().astype(np.int8)
    ref = np.asarray(wqbmm_oracle.fp32_dequant_product(out_to_np(x), wn, out_to_np(scale[:, ct].contiguous()),
                                                       out_to_np(offset[:, ct].contiguous()), None, g), dtype=np.float64)
    got = out_to_np(y1[:, ct].contiguous()).astype(np.float64)
    rms = np.sqrt(np.mean(ref ** 2))
    rel = np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 0.05 * rms))
    assert rel <= 2.0 ** -8 * 1.05, rel


@pytest.mark.parametrize("inner_precise", [0, 1])
def test_cluster_combine_matches_workspace_combine(aclnn, monkeypatch, inner_precise):
    """The k-splits of a strip launched as one thread-block cluster (fragments summed over distributed shared memory, no
    global scratch) give bit for bit what the workspace combination gives: same split boundaries, same summation order."""
    from gpu_util import run_wq_fixture

    a, meta = load_golden("wq_bf16_s4_group128_offset_m16")
    monkeypatch.setenv("OPSNN_WQ_DECODE_SPLITS", "2")
    y_ws = run_wq_fixture(aclnn, a, meta, kernel=0, api="v3", inner_precise=inner_precise)
    monkeypatch.setenv("OPSNN_WQ_DECODE_CLUSTER", "1")
    y_cl = run_wq_fixture(aclnn, a, meta, kernel=0, api="v3", inner_precise=inner_precise)
    assert aclnn.last_kernel_name() == ("wqbmm_decode_fast" if inner_precise else "wqbmm_decode")
    assert np.array_equal(y_ws.view(np.uint16), y_cl.view(np.uint16))
