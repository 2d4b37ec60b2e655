"""The torch-tensor entry points (signatures of torch_npu.npu_quant_matmul / npu_weight_quant_batchmatmul) against the oracle."""
import ml_dtypes
import numpy as np
import pytest

from oracle import qbmm_oracle, wqbmm_oracle

pytestmark = pytest.mark.gpu


def _bf16_np(t):
    import torch

    return t.view(torch.int16).cpu().numpy().view(ml_dtypes.bfloat16)


def test_npu_quant_matmul_int8_per_token_and_transposed_weight(pkg):
    import torch

    rng = np.random.default_rng(5)
    m, k, n = 130, 1040, 208
    x1 = rng.integers(-127, 128, (m, k), dtype=np.int8)
    x2 = rng.integers(-127, 128, (n, k), dtype=np.int8)  # stored (n, k), handed over as a .t() view
    s1 = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    s2 = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    bias = rng.integers(-1000, 1001, n).astype(np.int32)
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, bias, False, True, 0, "bfloat16")
    dev = "cuda:0"
    y = pkg.torch_api.npu_quant_matmul(torch.from_numpy(x1).to(dev), torch.from_numpy(x2).to(dev).t(), torch.from_numpy(s2).to(dev),
                                       pertoken_scale=torch.from_numpy(s1).to(dev), bias=torch.from_numpy(bias).to(dev),
                                       output_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    assert y.shape == (m, n) and y.dtype == torch.bfloat16
    assert np.array_equal(_bf16_np(y).view(np.uint16), want.view(np.uint16))


def test_npu_quant_matmul_fp8_per_block_group_sizes(pkg):
    import torch

    from gpu_util import check_close

    rng = np.random.default_rng(6)
    m, k, n = 256, 512, 384
    x1 = rng.standard_normal((m, k)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
    x2 = rng.standard_normal((k, n)).astype(np.float32).astype(ml_dtypes.float8_e4m3fn)
    s1 = rng.uniform(0.5, 2, (m, k // 128)).astype(np.float32)
    s2 = rng.uniform(0.5, 2, (k // 128, n // 128)).astype(np.float32)
    group = (1 << 32) | (128 << 16) | 128
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, None, False, False, group, "bfloat16")
    ref32 = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, None, False, False, group, "float32")
    dev = "cuda:0"
    f8 = lambda a: torch.from_numpy(a.view(np.uint8)).to(dev).view(torch.float8_e4m3fn)  # noqa: E731
    y = pkg.torch_api.npu_quant_matmul(f8(x1), f8(x2), torch.from_numpy(s2).to(dev), pertoken_scale=torch.from_numpy(s1).to(dev),
                                       output_dtype=torch.bfloat16, group_sizes=[1, 128, 128])
    torch.cuda.synchronize()
    check_close(_bf16_np(y), want, ref32, "bfloat16")


@pytest.mark.parametrize("m", [4, 64])
def test_npu_weight_quant_batchmatmul_int4_words(pkg, m):
    import torch

    rng = np.random.default_rng(7 + m)
    k, n, g = 512, 256, 128
    x = rng.standard_normal((m, k)).astype(ml_dtypes.bfloat16)
    w = rng.integers(-8, 8, (k, n)).astype(np.int8)
    scale = rng.uniform(0.005, 0.02, (k // g, n)).astype(ml_dtypes.bfloat16)
    offset = rng.uniform(-1, 1, (k // g, n)).astype(ml_dtypes.bfloat16)
    want = wqbmm_oracle.weight_quant_batch_matmul(x, w, scale, offset, None, g).astype(np.float64)
    dev = "cuda:0"
    bf = lambda a: torch.from_numpy(a.view(np.int16).copy()).to(dev).view(torch.bfloat16)  # noqa: E731
    words = torch.from_numpy(wqbmm_oracle.pack_int4_words(w).copy()).to(dev)
    y = pkg.torch_api.npu_weight_quant_batchmatmul(bf(x), words, bf(scale), bf(offset), antiquant_group_size=g)
    torch.cuda.synchronize()
    assert y.shape == (m, n) and y.dtype == torch.bfloat16
    got = _bf16_np(y).astype(np.float64)
    assert np.all(np.abs(got - want) <= 2 * 2.0 ** -7 * np.maximum(np.abs(want), 0.05 * np.sqrt(np.mean(want ** 2))) * 1.01)
