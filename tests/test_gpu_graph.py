"""GPU: the aclnn calls are plain stream work (no allocation, no synchronisation, no host read-back in phase 2), so a serving
loop can capture them into a CUDA graph and replay it. Checked here for the streaming decode kernels - both ways of combining
the k-splits: the workspace form carries a launch nonce in its arguments, which a replay repeats, so the kernel has to leave the
tags clean - and for the one-call MX form (activation quantiser + block-scaled matmul). A replay must give the bits of the eager
call, also after the captured input buffers got new contents."""
import numpy as np
import pytest

from oracle import wqbmm_oracle

pytestmark = pytest.mark.gpu


def _capture(torch, fn):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()  # warm-up on the capture stream: one-time function attributes, cached occupancy answers
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("cluster", ["0", "1"], ids=["workspace combine", "cluster combine"])
def test_decode_calls_replay_from_a_graph(aclnn, monkeypatch, cluster, bits):
    import torch

    from gpu_util import DEV

    monkeypatch.setenv("OPSNN_WQ_DECODE_CLUSTER", cluster)
    m, k, n, g = 16, 4096, 4096, 128
    gen = torch.Generator(device=DEV).manual_seed(77 + bits)
    x = torch.randn((m, k), generator=gen, device=DEV).to(torch.bfloat16)
    x_new = torch.randn((m, k), generator=gen, device=DEV).to(torch.bfloat16)
    if bits == 4:
        w = torch.randint(-2 ** 31, 2 ** 31 - 1, (k, n // 8), generator=gen, device=DEV, dtype=torch.int32)
    else:
        w = torch.randint(-128, 128, (k, n), generator=gen, device=DEV, dtype=torch.int8)
    sc = (torch.rand((k // g, n), generator=gen, device=DEV) * 0.01 + 0.005).to(torch.bfloat16)
    of = (torch.rand((k // g, n), generator=gen, device=DEV) * 2 - 1).to(torch.bfloat16)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    d = [aclnn.from_torch(t) for t in (x, w, sc, y, of)]
    ws = aclnn.weight_quant_batch_matmul(d[0], d[1], d[2], d[3], d[4], None, g)
    workspace = torch.empty(max(ws, 1), dtype=torch.uint8, device=DEV)

    def call():
        aclnn.weight_quant_batch_matmul(d[0], d[1], d[2], d[3], d[4], None, g, workspace=workspace)

    def eager(xv):
        x.copy_(xv)
        y.fill_(-7777.0)
        call()
        torch.cuda.synchronize()
        return y.clone()

    x0 = x.clone()
    want0, want1 = eager(x0), eager(x_new)
    assert aclnn.last_kernel_name() == ("wqbmm_decode" if bits == 4 else "wqbmm_decode8")
    assert aclnn.last_decode_plan()[2] == int(cluster)
    assert not torch.equal(want0, want1)
    x.copy_(x0)

    def three_calls():  # several launches per graph: each keeps the nonce it was captured with
        for _ in range(3):
            call()

    graph = _capture(torch, three_calls)
    for xv, want in ((x0, want0), (x_new, want1), (x0, want0)):
        x.copy_(xv)
        y.fill_(-7777.0)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, want)
    assert aclnn.lib().opsnn_wqbmm_decode_status(1) == 0


def test_mx_one_call_form_replays_from_a_graph(aclnn):
    """bf16 activations quantised on the fly + MXFP8 matmul (two kernels and a scale re-layout per call) inside a graph."""
    import ml_dtypes
    import torch

    from gpu_util import DEV, desc

    from oracle import mx_quant_oracle

    m, k, n = 256, 512, 448
    rng = np.random.default_rng(11)
    x1 = rng.standard_normal((m, k)).astype(np.float32).astype(ml_dtypes.bfloat16)
    wq, ws_ = mx_quant_oracle.dynamic_mx_quant(rng.standard_normal((n, k)).astype(np.float32).astype(ml_dtypes.bfloat16), "float8_e4m3fn")
    ws_ = ws_.view(ml_dtypes.float8_e8m0fnu)
    group_mx = (1 << 32) | (1 << 16) | 32
    tx = torch.from_numpy(x1.view(np.int16).copy()).view(torch.bfloat16).to(DEV)
    tx_new = (tx.float() * 1.5 + 0.25).to(torch.bfloat16)
    d_x = aclnn.from_torch(tx)
    d_w, d_ws = desc(aclnn, wq), desc(aclnn, ws_)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    d_out = aclnn.from_torch(out)
    ws_bytes = aclnn.quant_matmul_v5(d_x, d_w, None, d_ws, d_out, None, False, True, group_mx)
    workspace = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=DEV)

    def call():
        aclnn.quant_matmul_v5(d_x, d_w, None, d_ws, d_out, None, False, True, group_mx, workspace=workspace)

    def eager(xv):
        tx.copy_(xv)
        out.fill_(-7777.0)
        call()
        torch.cuda.synchronize()
        return out.clone()

    x0 = tx.clone()
    want0, want1 = eager(x0), eager(tx_new)
    assert not torch.equal(want0, want1)
    tx.copy_(x0)
    graph = _capture(torch, call)
    for xv, want in ((x0, want0), (tx_new, want1)):
        tx.copy_(xv)
        out.fill_(-7777.0)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want)
    assert aclnn.lib().opsnn_qmm_umma_status(1) == 0
