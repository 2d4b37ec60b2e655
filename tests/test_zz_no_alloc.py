"""GPU: opsnn_wqbmm_decode_static_launch (scratch inside the library's device image, no allocation at the call) against
opsnn_wqbmm_launch with caller workspace, through the kernel-level C ABI. Collected last on purpose: the static scratch
is shared by all calls on the device, so this file also shows that it works after everything else has run."""
import ctypes

import numpy as np
import pytest

from oracle import wqbmm_oracle

pytestmark = pytest.mark.gpu

M, K, N, G = 16, 2048, 5120, 128  # 10 strips of 512 columns -> k is split across CTAs, so the scratch is really used


def _problem(torch, seed):
    rng = np.random.default_rng(seed)
    w_int = rng.integers(-8, 8, size=(K, N), dtype=np.int8)
    words = wqbmm_oracle.pack_int4_words(w_int)  # (K, N/8) int32, low nibble first
    d = "cuda:0"
    t = {
        "x": torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(d).to(torch.bfloat16),
        "w": torch.from_numpy(words).to(d),
        "scale": torch.from_numpy(rng.uniform(0.005, 0.02, (K // G, N)).astype(np.float32)).to(d).to(torch.bfloat16),
        "offset": torch.from_numpy(rng.integers(-3, 4, (K // G, N)).astype(np.float32)).to(d).to(torch.bfloat16),
    }
    return t


def _params(aclnn, t, y, workspace=None):
    p = aclnn.WqbmmParams()
    p.x_dtype, p.w_dtype, p.bias_dtype, p.trans_w = aclnn.ACL_BF16, aclnn.ACL_INT4, -1, 0
    p.m, p.n, p.k = M, N, K
    p.x, p.x_ld = t["x"].data_ptr(), K
    p.w, p.w_ld = t["w"].data_ptr(), N
    p.scale, p.offset = t["scale"].data_ptr(), t["offset"].data_ptr()
    p.group_size, p.scale_sg, p.scale_sn = G, N, 1
    p.bias = None
    p.y, p.y_ld = y.data_ptr(), N
    if workspace is not None:
        p.workspace, p.workspace_size = workspace.data_ptr(), workspace.numel()
    return p


def test_static_scratch_matches_workspace_entry_point_twice(aclnn, monkeypatch):
    import torch

    # The static-scratch entry point runs the register-prefetch decode kernel. opsnn_wqbmm_launch picks between that kernel
    # and the shared-memory-ring one (same arithmetic, different k-split boundaries, so fp32 sums may differ in the last
    # bit); the switch below makes it take the same kernel, so the comparison can be bit for bit.
    monkeypatch.setenv("OPSNN_WQ_DECODE_LEGACY", "1")
    L = aclnn.lib()
    for call, seed in enumerate((11, 12)):  # two calls in a row, different data: the scratch is reused as it was left
        t = _problem(torch, seed)
        y_ws = torch.empty((M, N), dtype=torch.bfloat16, device="cuda:0")
        y_st = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda:0")
        probe = _params(aclnn, t, y_ws)
        assert L.opsnn_wqbmm_select_kernel(ctypes.byref(probe)) == 2
        ws = torch.empty(int(L.opsnn_wqbmm_workspace_size(ctypes.byref(probe), 2)), dtype=torch.uint8, device="cuda:0")
        p_ws = _params(aclnn, t, y_ws, ws)
        assert L.opsnn_wqbmm_launch(ctypes.byref(p_ws), 2, None) == 0
        assert aclnn.last_kernel_name() == "wqbmm_decode"
        torch.cuda.synchronize()

        free_before = torch.cuda.mem_get_info()[0] if call == 1 else None  # after the first call's one-time set-up
        p_st = _params(aclnn, t, y_st)
        assert L.opsnn_wqbmm_decode_static_launch(ctypes.byref(p_st), None) == 0, aclnn.last_error()
        assert aclnn.last_kernel_name() == "wqbmm_decode_static"
        torch.cuda.synchronize()
        if free_before is not None:
            assert torch.cuda.mem_get_info()[0] == free_before  # the call took no device memory

        a = y_ws.view(torch.int16).cpu().numpy()
        b = y_st.view(torch.int16).cpu().numpy()
        assert np.array_equal(a, b), "call %d: %d elements differ" % (call, int((a != b).sum()))
        # and both are right: sampled columns against the numpy oracle (<= 1 bf16 ulp, summation order only)
        cols = np.arange(0, N, 37)
        w_int = wqbmm_oracle.unpack_int4_words(t["w"].cpu().numpy())[:, cols]
        f32 = lambda v: v.float().cpu().numpy()
        import ml_dtypes
        bf = ml_dtypes.bfloat16
        want = wqbmm_oracle.weight_quant_batch_matmul(f32(t["x"]).astype(bf), w_int, f32(t["scale"])[:, cols].astype(bf),
                                                      f32(t["offset"])[:, cols].astype(bf), None, G).astype(np.float64)
        got = f32(y_st)[:, cols].astype(np.float64)
        rms = np.sqrt(np.mean(want ** 2))
        assert np.all(np.abs(got - want) <= 2.0 ** -7 * np.maximum(np.abs(want), 0.05 * rms) * 1.01)


def test_static_scratch_rejects_sizes_beyond_its_limit(aclnn):
    import torch

    L = aclnn.lib()
    t = _problem(torch, 13)
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda:0")
    p = _params(aclnn, t, y)
    p.n = 304 * 512 + 8  # one column group past what the scratch covers; rejected before anything is read
    p.w_ld = p.y_ld = p.scale_sg = p.n
    before = aclnn.launch_count()
    assert L.opsnn_wqbmm_decode_static_launch(ctypes.byref(p), None) != 0
    assert "exceeds" in aclnn.last_error()
    assert aclnn.launch_count() == before
    p2 = _params(aclnn, t, y)
    p2.m = 17  # outside the decode kernel's range
    assert L.opsnn_wqbmm_decode_static_launch(ctypes.byref(p2), None) != 0
    assert "range" in aclnn.last_error()
    assert aclnn.launch_count() == before
    p3 = _params(aclnn, t, y)
    p3.k = 0  # no k-step at all: the kernel's prefetch would read weight rows that do not exist
    assert L.opsnn_wqbmm_decode_static_launch(ctypes.byref(p3), None) != 0
    assert aclnn.launch_count() == before
