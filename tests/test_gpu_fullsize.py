"""GPU parity of the tensor-core configurations at their full benchmark sizes, through the C ABI.

c3 (fp8 per-block 4096 x 7168 x 18432), c4 (MXFP4, 8 batches of 8192^3) and c5 (dynamic MX quant + MXFP8, 32 batches of
2048 x 4096 x 14336 with bias) are too large for the numpy oracle as a whole, so scattered rows x scattered columns of the
output (always including the first and last row and column block, and the first and last batch) are checked against it:
max relative error <= 1e-2 against the fp32 product, plus no element left unwritten anywhere. Full-size-only behaviour is what
this covers: banded tile order over thousands of tiles, batch strides of gigabytes, the scale-atom workspace, the persistent
schedule. Inputs follow the quantisation recipes the configurations name (amax/448 block scales; floor(log2 amax) - emax e8m0).
The workload builders are the benchmark's own (bench.py), so the benchmark and these tests exercise the same calls."""
import argparse
import importlib.util
import os

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("opsnn_bench", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _args(workload):
    return argparse.Namespace(steps=3, warmup=3, no_cpu_baseline=True, workload=workload, batch=0, comm=None)


def test_c3_fp8_perblock_full_size(aclnn, bench):
    import torch

    dev = torch.device("cuda", 0)
    res = bench.run_c3(torch, dev, aclnn, _args("c3"), bench.measured_peaks(), 0, 1, None)
    assert res["kernel"] == "qmm_umma_pair_perblock", res["kernel"]  # the CTA-pair tensor-core kernel, not the coverage one
    par = res["parity"]
    assert par["checked_elems"] >= 128 * 1024 and not par["unwritten_elems"]
    assert par["max_rel_err"] <= 1e-2 and par["ok"], par


def test_c4_mxfp4_full_size_first_and_last_batch(aclnn, bench):
    import torch

    dev = torch.device("cuda", 0)
    res = bench.run_mx(torch, dev, aclnn, _args("c4"), bench.measured_peaks(), 0, 1, None, "c4")
    assert res["kernel"] == ["qmm_umma_pair_mxfp4"], res["kernel"]
    par = res["parity"]
    assert par["checked_elems"] >= 2 * 64 * 256 and not par["unwritten_elems"]
    assert par["max_rel_err"] <= 1e-2 and par["ok"], par


def test_c5_quantiser_then_mxfp8_full_size_both_bias_dtypes(aclnn, bench):
    """The chain the configuration names: bf16 activations with 0.1 % outliers x50 -> aclnnDynamicMxQuant -> MXFP8 matmul + bias.
    The quantised operand must equal the quantiser oracle bit for bit on the sampled rows; the output is checked with the fp32
    bias the reference takes (quant_matmul_checker.cpp:1685-1687) and with the bf16 bias this library accepts as an extension."""
    import torch

    dev = torch.device("cuda", 0)
    res = bench.run_mx(torch, dev, aclnn, _args("c5"), bench.measured_peaks(), 0, 1, None, "c5")
    assert res["kernel"] == ["mx_quant_stream", "qmm_umma_pair_mxfp8"], res["kernel"]
    par = res["parity"]
    # fp32 bias, bf16 bias, and once more after the weight was registered with opsnnQuantMatmulPrepareX2
    assert [c["bias"] for c in par["cases"]] == ["float32", "bfloat16", "prepared x2, float32"]
    assert all(c["quantiser_bit_exact"] for c in par["cases"]), par
    assert par["max_rel_err"] <= 1e-2 and not par["unwritten_elems"] and par["ok"], par
