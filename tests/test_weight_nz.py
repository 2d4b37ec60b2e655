"""aclnnWeightQuantBatchMatmulNz: the FRACTAL_NZ layout helper against the reference's nz_to_nd (fixtures), the entry point's
argument rules on CPU, and on the GPU the same result as the row-major call."""
import numpy as np
import pytest

from conftest import case_seed, golden_names, load_golden
from oracle import wqbmm_oracle

ACL_FORMAT_FRACTAL_NZ = 29


@pytest.mark.parametrize("name", golden_names("nz_layout_"))
def test_nz_layout_matches_reference(name):
    a, meta = load_golden(name)
    k, n, k0, n0 = meta["k"], meta["n"], meta["k0"], meta["n0"]
    assert np.array_equal(wqbmm_oracle.nz_to_nd(a["nz"], (k, n)), a["nd"])
    assert np.array_equal(wqbmm_oracle.nz_to_nd(wqbmm_oracle.nd_to_nz(a["nd"], k0, n0), (k, n)), a["nd"])


def test_nz_entry_argument_rules(aclnn):
    T = aclnn.Tensor
    x, y = T((8, 64), "bfloat16"), T((8, 128), "bfloat16")
    sc = T((128,), "bfloat16")
    w_nz = T((64, 128), "int8", fmt=ACL_FORMAT_FRACTAL_NZ, storage_shape=(4, 4, 16, 32))
    st, ws, ex = aclnn.weight_quant_batch_matmul_get_workspace_size(x, w_nz, sc, None, None, None, None, 0, y, inner_precise="nz")
    assert st == 0 and ws >= 64 * 128, (st, ws, aclnn.last_error())
    aclnn.destroy_executor(ex)
    # a row-major weight is refused by this entry point, a fractal one by the V2 entry point
    st, _, _ = aclnn.weight_quant_batch_matmul_get_workspace_size(x, T((64, 128), "int8"), sc, None, None, None, None, 0, y,
                                                                  inner_precise="nz")
    assert st == 161002
    st, _, _ = aclnn.weight_quant_batch_matmul_get_workspace_size(x, w_nz, sc, None, None, None, None, 0, y)
    assert st == 161002
    # storage dims that do not tile the view
    bad = T((64, 128), "int8", fmt=ACL_FORMAT_FRACTAL_NZ, storage_shape=(4, 3, 16, 32))
    st, _, _ = aclnn.weight_quant_batch_matmul_get_workspace_size(x, bad, sc, None, None, None, None, 0, y, inner_precise="nz")
    assert st == 161002


@pytest.mark.gpu
@pytest.mark.parametrize("case", [(8, 512, 256, 128, True, 16, 64), (40, 200, 136, 0, False, 16, 32), (300, 1024, 640, 128, True, 16, 64)],
                         ids=["int4-decode", "int8-tails", "int4-prefill"])
def test_nz_weight_gives_the_row_major_result(aclnn, case):
    import ml_dtypes
    import torch

    from gpu_util import desc, out_tensor, out_to_np

    m, k, n, g, int4, k0, n0 = case
    rng = np.random.default_rng(case_seed(case))
    x = rng.standard_normal((m, k)).astype(ml_dtypes.bfloat16)
    w = (rng.integers(-8, 8, (k, n)) if int4 else rng.integers(-127, 128, (k, n))).astype(np.int8)
    sshape = (k // g, n) if g else (n,)
    scale = rng.uniform(0.005, 0.02, sshape).astype(ml_dtypes.bfloat16)
    offset = rng.uniform(-1, 1, sshape).astype(ml_dtypes.bfloat16)
    want = wqbmm_oracle.weight_quant_batch_matmul(x, w, scale, offset, None, g).astype(np.float64)
    nz = wqbmm_oracle.nd_to_nz(w, k0, n0)  # [n1, k1, k0, n0], one value per element
    if int4:
        nib = nz.astype(np.uint8) & 0xF
        store = torch.from_numpy((nib[..., 0::2] | (nib[..., 1::2] << 4)).copy()).cuda()
        d_w = aclnn.Tensor((k, n), "int4", store, fmt=ACL_FORMAT_FRACTAL_NZ, storage_shape=nz.shape)
    else:
        store = torch.from_numpy(nz.copy()).cuda()
        d_w = aclnn.Tensor((k, n), "int8", store, fmt=ACL_FORMAT_FRACTAL_NZ, storage_shape=nz.shape)
    y = out_tensor((m, n), "bfloat16")
    aclnn.weight_quant_batch_matmul(desc(aclnn, x), d_w, desc(aclnn, scale), aclnn.Tensor((m, n), "bfloat16", y), desc(aclnn, offset),
                                    None, g, inner_precise="nz")
    torch.cuda.synchronize()
    got = out_to_np(y).astype(np.float64)
    rms = np.sqrt(np.mean(want ** 2))
    assert np.all(np.abs(got - want) <= 2 * 2.0 ** -7 * np.maximum(np.abs(want), 0.05 * rms) * 1.01)


def test_quant_matmul_weight_nz_argument_rules(aclnn):
    """aclnnQuantMatmulWeightNz (aclnn_quant_matmul_weight_nz.h:41-55 of the reference): x2 must be FRACTAL_NZ with storage dims that
    tile its view; the reported workspace includes the row-major copy."""
    T = aclnn.Tensor
    x1, out = T((32, 64), "int8"), T((32, 128), "bfloat16")
    s2 = T((128,), "float32")
    x2_nz = T((64, 128), "int8", fmt=ACL_FORMAT_FRACTAL_NZ, storage_shape=(4, 4, 16, 32))
    st, ws, ex = aclnn.quant_matmul_v5_get_workspace_size(x1, x2_nz, None, s2, None, None, None, None, None, False, False, 0, out,
                                                          weight_nz=True)
    assert st == 0 and ws >= 64 * 128, (st, ws, aclnn.last_error())
    aclnn.destroy_executor(ex)
    st, _, _ = aclnn.quant_matmul_v5_get_workspace_size(x1, T((64, 128), "int8"), None, s2, None, None, None, None, None, False, False, 0,
                                                        out, weight_nz=True)
    assert st == 161002  # row-major x2 is refused by this entry point ...
    st, _, _ = aclnn.quant_matmul_v5_get_workspace_size(x1, x2_nz, None, s2, None, None, None, None, None, False, False, 0, out)
    assert st == 161002  # ... and a fractal one by aclnnQuantMatmulV5
    bad = T((64, 128), "int8", fmt=ACL_FORMAT_FRACTAL_NZ, storage_shape=(4, 3, 16, 32))
    st, _, _ = aclnn.quant_matmul_v5_get_workspace_size(x1, bad, None, s2, None, None, None, None, None, False, False, 0, out, weight_nz=True)
    assert st == 161002


@pytest.mark.gpu
@pytest.mark.parametrize("case", [(128, 512, 256, False, 16, 32), (96, 200, 176, False, 16, 32), (64, 256, 320, True, 16, 32)],
                         ids=["aligned", "ragged", "x2_stored_nk"])
def test_quant_matmul_weight_nz_gives_the_nd_result(aclnn, case):
    """int8 per-token x per-channel: the FRACTAL_NZ call equals the ND call bit for bit (and the oracle)."""
    import torch

    from gpu_util import DEV, out_to_np
    from oracle import qbmm_oracle

    m, k, n, tb, r0, c0 = case
    rng = np.random.default_rng(case_seed(case))
    x1 = rng.integers(-127, 128, (m, k), dtype=np.int8)
    x2 = rng.integers(-127, 128, (n, k) if tb else (k, n), dtype=np.int8)  # the stored 2-D matrix
    s1 = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    s2 = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    bias = rng.integers(-1000, 1001, n).astype(np.int32)
    want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, bias, transpose_x2=tb, out_dtype="bfloat16")
    nz = wqbmm_oracle.nd_to_nz(x2, r0, c0)
    t = lambda a: aclnn.from_torch(torch.from_numpy(np.ascontiguousarray(a)).to(DEV))  # noqa: E731
    d_nz = aclnn.Tensor(x2.shape, "int8", torch.from_numpy(nz.copy()).to(DEV), fmt=ACL_FORMAT_FRACTAL_NZ, storage_shape=nz.shape)
    outs = []
    for nzcall in (False, True):
        out = torch.full((m, n), -7777.0, dtype=torch.bfloat16, device=DEV)
        aclnn.quant_matmul_v5(t(x1), d_nz if nzcall else t(x2), t(s1), t(s2), aclnn.from_torch(out), t(bias), False, tb, 0, weight_nz=nzcall)
        torch.cuda.synchronize()
        outs.append(out_to_np(out).view(np.uint16))
    assert np.array_equal(outs[0], want.view(np.uint16))
    assert np.array_equal(outs[1], outs[0])
