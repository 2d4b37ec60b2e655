"""GPU parity: aclnnWeightQuantBatchMatmulV2/V3 and aclnnDynamicMxQuant through the C ABI."""
import numpy as np
import pytest

from conftest import case_seed, golden_names, load_golden
from oracle import mx_quant_oracle, wqbmm_oracle

pytestmark = pytest.mark.gpu


def _ref64(a, meta):
    """fp32 dequantised product: x @ w' with w' the dequantised weight (the reference's two roundings in x's dtype),
    accumulated in float64 - the yardstick of the stated tolerance."""
    t = meta["transpose_weight"]
    w = a["w"].T if t else a["w"]
    sc = a["scale"].T if (t and a["scale"].ndim == 2) else a["scale"]
    of = a.get("offset")
    if of is not None and t and of.ndim == 2:
        of = of.T
    wd = wqbmm_oracle.dequant_weight(w, sc, of, meta["group_size"], a["x"].dtype.type).astype(np.float64)
    out = a["x"].astype(np.float64) @ wd
    if a.get("bias") is not None:
        out = out + a["bias"].astype(np.float64)
    return out


@pytest.mark.parametrize("kernel", [1, 0], ids=["generic", "auto"])
@pytest.mark.parametrize("name", golden_names("wq_"))
def test_fixture(aclnn, name, kernel):
    from gpu_util import check_close, np_name, run_wq_fixture

    a, meta = load_golden(name)
    got = run_wq_fixture(aclnn, a, meta, kernel=kernel)
    check_close(got, a["out"], _ref64(a, meta), np_name(a["out"]), floor_rms=0.05)


def test_decode_kernel_is_selected_and_matches_golden_tightly(aclnn):
    """The small-m int4 fixtures must run on the streaming decode kernel, and since it reproduces the reference's two
    roundings per weight its output may differ from the golden only by fp32 summation order: <= 1 ulp of the output
    dtype, on a small fraction of elements."""
    from gpu_util import np_name, run_wq_fixture

    for name in ("wq_bf16_s4_group128_offset_m16", "wq_bf16_s4_group160_m1_fbias", "wq_fp16_s4_group64_bias_m8",
                 "wq_fp16_s4_channel_offset_bias"):
        a, meta = load_golden(name)
        got = run_wq_fixture(aclnn, a, meta, kernel=0, api="v3")
        assert aclnn.last_kernel_name() == "wqbmm_decode", name
        g = got.astype(np.float64)
        w = a["out"].astype(np.float64)
        ulp = 2.0 ** -7 if np_name(a["out"]) == "bfloat16" else 2.0 ** -10
        rms = np.sqrt(np.mean(w ** 2))
        assert np.all(np.abs(g - w) <= ulp * np.maximum(np.abs(w), 0.05 * rms) * 1.01), name
        assert np.mean(g != w) < 0.05, name


def test_decode_c2_shape_properties(aclnn):
    """Full benchmark shape (m16 k8192 n28672 g128): checked through size-independent properties and a sampled oracle.
      * linearity in x: f(2x) == 2 f(x) bit for bit (powers of two commute with every rounding here);
      * zero rows of x give exactly-zero rows of y; rows are independent (row i of a 16-row call == the 1-row call);
      * 512 sampled output columns against the numpy oracle."""
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
                                        aclnn.from_torch(y), aclnn.from_torch(offset), None, g)
        torch.cuda.synchronize()
        assert aclnn.last_kernel_name() == "wqbmm_decode"
        return y

    y1 = run(x)
    y1b = run(x)
    assert torch.equal(y1, y1b), "two identical calls must agree bit for bit (the cross-CTA sum has a fixed order)"
    assert not bool((y1 == -7777.0).any())
    assert bool((y1[5] == 0).all())
    y2 = run(x * 2)
    assert torch.equal(y2.float(), y1.float() * 2)
    y_row = run(x[3:4].contiguous())
    assert torch.equal(y_row[0], y1[3])
    cols = np.sort(np.random.default_rng(3).choice(n, 512, replace=False))
    ct = torch.from_numpy(cols).to(DEV)
    wn = w[:, ct].cpu().numpy().astype(np.int8)
    want = wqbmm_oracle.weight_quant_batch_matmul(out_to_np(x), wn, out_to_np(scale[:, ct].contiguous()),
                                                  out_to_np(offset[:, ct].contiguous()), None, g)
    got = out_to_np(y1[:, ct].contiguous())
    gw, ww = got.astype(np.float64), want.astype(np.float64)
    rms = np.sqrt(np.mean(ww ** 2))
    assert np.all(np.abs(gw - ww) <= 2.0 ** -7 * np.maximum(np.abs(ww), 0.05 * rms) * 1.01)


@pytest.mark.parametrize("name", golden_names("mxq_"))
def test_dynamic_mx_quant_fixture(aclnn, name):
    import torch

    from gpu_util import DEV, desc

    a, meta = load_golden(name)
    x = a["x"]
    dst = meta["dst"]
    ybytes = x.shape[:-1] + ((x.shape[-1] // 2,) if dst == "float4_e2m1" else (x.shape[-1],))
    y = torch.full(ybytes, 0xAA, dtype=torch.uint8, device=DEV)
    s = torch.full(a["scale"].shape, 0xAA, dtype=torch.uint8, device=DEV)
    aclnn.dynamic_mx_quant(desc(aclnn, x), aclnn.Tensor(x.shape, dst, y), aclnn.Tensor(a["scale"].shape, "float8_e8m0", s), dst,
                           axis=meta.get("axis", -1), round_mode=meta.get("round_mode", "rint").encode(), scale_alg=meta.get("scale_alg", 0))
    torch.cuda.synchronize()
    want_y = a["y"].view(np.uint8)
    if dst == "float4_e2m1":
        want_y = (want_y[..., 0::2] & 0xF) | ((want_y[..., 1::2] & 0xF) << 4)
    assert np.array_equal(s.cpu().numpy(), a["scale"].view(np.uint8)), "e8m0 scales differ"
    assert np.array_equal(y.cpu().numpy(), want_y), "quantised elements differ"


PREFILL_CASES = [
    # m, k, n, group, int4, transposed weight, packed int32 words, offset, bias, x dtype
    (17, 512, 256, 128, True, False, True, True, None, "bfloat16"),
    (300, 1024, 640, 128, True, False, True, True, "x", "bfloat16"),      # tails in m and n tiles
    (256, 1000, 512, 0, True, False, False, True, "x", "float16"),        # per-channel, k not a multiple of 64
    (130, 768, 264, 64, True, True, False, False, None, "bfloat16"),      # weight stored (n,k)
    (64, 512, 384, 64, False, False, False, True, "x", "float16"),        # int8 weight
    (512, 2048, 2048, 128, True, False, True, True, None, "bfloat16"),    # CTA-pair tiles
    (64, 512, 384, 0, False, True, False, True, "x", "bfloat16"),          # int8 weight stored (n,k), per-channel
    (40, 1024, 520, 128, True, True, True, True, None, "float16"),         # int4 words stored (n, k/8), groups
]


@pytest.mark.parametrize("case", PREFILL_CASES, ids=[str(c) for c in PREFILL_CASES])
def test_prefill_dequant_then_tensor_core_matmul(aclnn, case):
    """m beyond the decode range: the weight is dequantised with the reference's two roundings into workspace and multiplied
    by the tcgen05 bf16/fp16 kernel, so the output differs from the golden only by fp32 summation order."""
    import ml_dtypes

    from gpu_util import np_name, run_wq_fixture

    m, k, n, group, int4, tw, words, has_off, bias_kind, xname = case
    xdt = ml_dtypes.bfloat16 if xname == "bfloat16" else np.float16
    rng = np.random.default_rng(case_seed(case))
    x = rng.standard_normal((m, k)).astype(xdt)
    w = rng.integers(-8, 8, (k, n)).astype(np.int8) if int4 else rng.integers(-127, 128, (k, n)).astype(np.int8)
    sshape = (-(-k // group), n) if group else (n,)
    scale = rng.uniform(0.005, 0.02, sshape).astype(xdt)
    offset = rng.uniform(-1, 1, sshape).astype(xdt) if has_off else None
    bias = {None: None, "x": rng.standard_normal(n).astype(xdt), "f32": rng.standard_normal(n).astype(np.float32)}[bias_kind]
    want = wqbmm_oracle.weight_quant_batch_matmul(x, w, scale, offset, bias, group)
    a = dict(x=x, w=w.T.copy() if tw else w, scale=scale.T.copy() if (tw and scale.ndim == 2) else scale,
             offset=None if offset is None else (offset.T.copy() if (tw and offset.ndim == 2) else offset), bias=bias, out=want)
    meta = dict(transpose_weight=tw, w_is_int4=int4, packed_int32=words, group_size=group)
    got = run_wq_fixture(aclnn, a, meta, kernel=0)
    assert aclnn.last_kernel_name() in ("qmm_umma_deq", "qmm_umma_pair_deq"), aclnn.last_kernel_name()
    assert aclnn.lib().opsnn_qmm_umma_status(1) == 0
    g, wv = got.astype(np.float64), want.astype(np.float64)
    ulp = 2.0 ** -7 if np_name(want) == "bfloat16" else 2.0 ** -10
    rms = np.sqrt(np.mean(wv ** 2))
    assert np.all(np.abs(g - wv) <= 2 * ulp * np.maximum(np.abs(wv), 0.05 * rms) * 1.01)
    assert np.mean(g != wv) < 0.1


@pytest.mark.parametrize("m,inner_precise,n", [(40, 0, 16384), (33, 1, 16384), (32, 0, 4096)])
def test_decode_kernel_in_chunks_of_16_rows(aclnn, m, inner_precise, n):
    """16 < m <= 48 against a large weight: one launch of the streaming decode kernel per 16 rows of x (two launches from 2^24
    weights on, three from 3 x 2^24)."""
    import ml_dtypes

    from gpu_util import run_wq_fixture

    k, g = 4096, 128
    rng = np.random.default_rng(100 + m)
    x = rng.standard_normal((m, k)).astype(ml_dtypes.bfloat16)
    w = rng.integers(-8, 8, (k, n)).astype(np.int8)
    scale = rng.uniform(0.005, 0.02, (k // g, n)).astype(ml_dtypes.bfloat16)
    offset = rng.uniform(-1, 1, (k // g, n)).astype(ml_dtypes.bfloat16)
    want = wqbmm_oracle.weight_quant_batch_matmul(x, w, scale, offset, None, g)
    a = dict(x=x, w=w, scale=scale, offset=offset, bias=None, out=want)
    meta = dict(transpose_weight=False, w_is_int4=True, packed_int32=True, group_size=g)
    got = run_wq_fixture(aclnn, a, meta, kernel=0, api="v3", inner_precise=inner_precise)
    assert aclnn.last_kernel_name() in ("wqbmm_decode", "wqbmm_decode_fast"), aclnn.last_kernel_name()
    gv = got.astype(np.float64)
    if inner_precise == 0:  # the reference's two roundings per weight: one output ulp from the golden
        wv = want.astype(np.float64)
        tol = 2.0 ** -7
    else:  # high-performance mode: measured against the unrounded fp32 product, as the API documents it
        wv = np.asarray(wqbmm_oracle.fp32_dequant_product(x, w, scale, offset, None, g), dtype=np.float64)
        tol = 2.0 ** -8 * 1.05
    rms = np.sqrt(np.mean(wv ** 2))
    assert np.all(np.abs(gv - wv) <= tol * np.maximum(np.abs(wv), 0.05 * rms) * 1.01)


@pytest.mark.parametrize("cluster", ["0", "1"], ids=["workspace combine", "cluster combine"])
def test_decode_wait_that_runs_out_is_reported_and_the_next_call_is_fine(aclnn, monkeypatch, cluster):
    """Every wait in the bulk-copy decode kernel is bounded. Here the producer is told (test-only switch) to stop issuing copies
    after the eighth stage of each CTA's range, with a poll limit of a few thousand, so the consumers' wait for the ninth stage
    runs out while nothing is in flight: the kernel must come back by itself, leave its error word at 1 (a stage never
    arrived), and the next, ordinary call must work. Nothing faults, traps or hangs: the wait simply gives up. Both ways of
    combining the k-splits are covered: with the splits launched as a cluster, the CTAs that gave up still join the cluster's
    barriers and mark their fragments invalid, so nobody waits for them and nobody writes."""
    import torch

    from gpu_util import DEV, out_to_np

    m, k, n, g = 16, 8192, 4096, 128
    rng = np.random.default_rng(5)
    import ml_dtypes
    x = rng.standard_normal((m, k)).astype(np.float32).astype(ml_dtypes.bfloat16)
    w = rng.integers(-8, 8, (k, n)).astype(np.int8)
    sc = rng.uniform(0.005, 0.02, (k // g, n)).astype(np.float32).astype(ml_dtypes.bfloat16)
    of = rng.uniform(-1, 1, (k // g, n)).astype(np.float32).astype(ml_dtypes.bfloat16)
    bf = lambda a: torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(DEV)  # noqa: E731
    tx, tw, ts, to = bf(x), torch.from_numpy(wqbmm_oracle.pack_int4_words(w).copy()).to(DEV), bf(sc), bf(of)
    L = aclnn.lib()
    assert L.opsnn_wqbmm_decode_status(1) == 0

    def run():
        y = torch.full((m, n), -7777.0, dtype=torch.bfloat16, device=DEV)
        aclnn.weight_quant_batch_matmul(aclnn.from_torch(tx), aclnn.from_torch(tw), aclnn.from_torch(ts), aclnn.from_torch(y),
                                        aclnn.from_torch(to), None, g)
        torch.cuda.synchronize()
        return y

    monkeypatch.setenv("OPSNN_WQ_DECODE_SPLITS", "2")           # 64 stages per CTA
    monkeypatch.setenv("OPSNN_WQ_DECODE_CLUSTER", cluster)
    monkeypatch.setenv("OPSNN_TEST_DECODE_STALL_STAGE", "8")
    monkeypatch.setenv("OPSNN_TEST_DECODE_POLL_LIMIT", "3000")
    y_bad = run()
    assert aclnn.last_kernel_name() == "wqbmm_decode"
    assert L.opsnn_wqbmm_decode_status(1) == 1                   # reported, and cleared (which also restores the poll limit)
    assert bool((y_bad == -7777.0).all())                        # a kernel that gave up writes nothing
    monkeypatch.delenv("OPSNN_TEST_DECODE_STALL_STAGE")
    monkeypatch.delenv("OPSNN_TEST_DECODE_POLL_LIMIT")
    y = run()
    assert L.opsnn_wqbmm_decode_status(1) == 0
    want = wqbmm_oracle.weight_quant_batch_matmul(x, w, sc, of, None, g).astype(np.float64)
    got = out_to_np(y).astype(np.float64)
    rms = np.sqrt(np.mean(want ** 2))
    assert np.all(np.abs(got - want) <= 2.0 ** -7 * np.maximum(np.abs(want), 0.05 * rms) * 1.01)


COMBINE_CASES = [
    # weight bits, x dtype, m, k, n, group, bias, inner_precise, k-splits
    (4, "bfloat16", 16, 8192, 3584, 128, False, None, 16),   # a 1/8 column shard of the benchmark's decode shape
    (4, "bfloat16", 16, 8192, 3584, 128, False, 1, 16),
    (4, "float16", 7, 4096, 1296, 128, True, None, 5),       # ragged last strip, m < 16, bias, a split count that does not divide the fragments
    (4, "bfloat16", 16, 2048, 512, 64, False, None, 3),
    (8, "bfloat16", 16, 8192, 2048, 0, True, None, 16),
    (8, "float16", 3, 4096, 1040, 128, False, None, 7),
]


@pytest.mark.parametrize("case", COMBINE_CASES, ids=[str(c) for c in COMBINE_CASES])
def test_cluster_combine_equals_workspace_combine(aclnn, monkeypatch, case):
    """The k-splits of a strip are summed either by the last CTA to arrive, from fragments in the workspace, or - launched as one
    thread-block cluster - over distributed shared memory, each CTA a slice of the strip. Both add the fragments in CTA order,
    so for the same split count the outputs must be identical bit for bit; the oracle bounds them as in the other tests."""
    import ml_dtypes
    import torch

    from gpu_util import DEV, out_to_np

    bits, xdt, m, k, n, g, with_bias, ip, splits = case
    rng = np.random.default_rng(m * 131 + n)
    nd = ml_dtypes.bfloat16 if xdt == "bfloat16" else np.float16
    td = torch.bfloat16 if xdt == "bfloat16" else torch.float16
    dev16 = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16).copy()).view(td).to(DEV)  # noqa: E731
    x = rng.standard_normal((m, k)).astype(np.float32).astype(nd)
    groups = k // g if g else 1
    sc = rng.uniform(0.005, 0.02, (groups, n)).astype(np.float32).astype(nd)
    of = rng.uniform(-1, 1, (groups, n)).astype(np.float32).astype(nd)
    bias = rng.standard_normal(n).astype(np.float32).astype(nd) if with_bias else None
    if bits == 4:
        w = rng.integers(-8, 8, (k, n)).astype(np.int8)
        tw = torch.from_numpy(wqbmm_oracle.pack_int4_words(w).copy()).to(DEV)
    else:
        w = rng.integers(-128, 128, (k, n)).astype(np.int8)
        tw = torch.from_numpy(w.copy()).to(DEV)
    tx, ts, to = dev16(x), dev16(sc if g else sc[0]), dev16(of if g else of[0])
    tb = dev16(bias) if with_bias else None
    monkeypatch.setenv("OPSNN_WQ_DECODE_SPLITS", str(splits))
    outs = []
    for cluster in ("0", "1"):
        monkeypatch.setenv("OPSNN_WQ_DECODE_CLUSTER", cluster)
        y = torch.full((m, n), -7777.0, dtype=td, device=DEV)
        aclnn.weight_quant_batch_matmul(aclnn.from_torch(tx), aclnn.from_torch(tw), aclnn.from_torch(ts), aclnn.from_torch(y),
                                        aclnn.from_torch(to), aclnn.from_torch(tb) if tb is not None else None, g, inner_precise=ip)
        torch.cuda.synchronize()
        assert aclnn.last_kernel_name() in ("wqbmm_decode", "wqbmm_decode_fast", "wqbmm_decode8")
        outs.append(y.view(torch.int16).cpu().numpy().copy())
        last = y
    assert aclnn.lib().opsnn_wqbmm_decode_status(1) == 0
    assert np.array_equal(outs[0], outs[1])
    if ip:  # the high-performance mode is measured against the unrounded product, as the API documents it
        want = np.asarray(wqbmm_oracle.fp32_dequant_product(x, w, sc, of, bias, g), dtype=np.float64)
        tol = 2.0 ** -8 * 1.05
    else:
        want = wqbmm_oracle.weight_quant_batch_matmul(x, w, sc, of, bias, g).astype(np.float64)
        tol = 2.0 ** -7 if xdt == "bfloat16" else 2.0 ** -9
    got = out_to_np(last).astype(np.float64)
    rms = np.sqrt(np.mean(want ** 2))
    assert np.all(np.abs(got - want) <= tol * np.maximum(np.abs(want), 0.05 * rms) * 1.01)


def test_narrow_output_is_planned_as_clusters(aclnn):
    """A 1/8 column shard of the benchmark's decode shape (what one of eight GPUs gets): the k-ranges of a strip run as one
    thread-block cluster of as many CTAs as the device keeps resident for all seven strips at once. The full width (56 strips
    of 5 k-ranges, two CTAs per SM) runs as clusters too when the device keeps all 56 resident under the load-balancing
    policy, which a B200 does; a width whose cluster size does not pack (48 strips of 6) keeps the workspace combination."""
    import torch

    from gpu_util import DEV

    def plan(n):
        m, k, g = 16, 8192, 128
        gen = torch.Generator(device=DEV).manual_seed(n)
        x = torch.randn((m, k), generator=gen, device=DEV).to(torch.bfloat16)
        w = torch.randint(-2 ** 31, 2 ** 31 - 1, (k, n // 8), generator=gen, device=DEV, dtype=torch.int32)
        sc = (torch.rand((k // g, n), generator=gen, device=DEV) * 0.01 + 0.005).to(torch.bfloat16)
        y = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
        aclnn.weight_quant_batch_matmul(aclnn.from_torch(x), aclnn.from_torch(w), aclnn.from_torch(sc), aclnn.from_torch(y), None, None, g)
        torch.cuda.synchronize()
        assert aclnn.last_kernel_name() == "wqbmm_decode"
        return aclnn.last_decode_plan()

    strips, splits, cluster = plan(3584)
    assert strips == 7 and (cluster & 1) == 1 and 2 <= splits <= 16
    strips, splits, cluster = plan(28672)
    assert strips == 56 and splits == 5 and cluster == 1
    strips, splits, cluster = plan(24576)
    assert strips == 48 and splits == 6 and cluster == 0


W4_NK_CASES = [
    # x dtype, m, k, n, group, offset, bias, packed as int32 words
    ("bfloat16", 16, 4096, 1024, 128, True, False, True),      # the benchmark's form with the weight stored (n,k)
    ("float16", 16, 2048, 768, 256, True, True, False),        # two stages per group, fp16, int4 dtype
    ("bfloat16", 5, 4096, 1048, 0, False, True, True),         # per-channel, ragged last strip, m < 16
    ("float16", 1, 8192, 512, 128, False, False, True),        # m = 1, no offset
    ("bfloat16", 13, 4128, 2056, 0, True, False, False),       # k not a multiple of the 128-row stage (the second x box runs out)
    ("bfloat16", 16, 16384, 64, 128, True, False, True),       # fewer columns than one copy box has rows
]


@pytest.mark.parametrize("case", W4_NK_CASES, ids=[str(c) for c in W4_NK_CASES])
def test_w4a16_weight_stored_nk_streaming_kernel(aclnn, case):
    """INT4 weights stored (n,k) - the transposed view of the API, k contiguous, scales stored (n, groups) - at m <= 16 run on the
    (n,k) form of the bulk-copy decode kernel with the golden's two roundings per weight (wqbmmv2_kernel_golden.py:242-297): only the
    fp32 summation order differs, <= 1 ulp of the output dtype."""
    import ml_dtypes

    from gpu_util import run_wq_fixture

    xdt, m, k, n, group, has_off, has_bias, words = case
    rng = np.random.default_rng(case_seed(case))
    np_dt = ml_dtypes.bfloat16 if xdt == "bfloat16" else np.float16
    x = rng.standard_normal((m, k)).astype(np.float32).astype(np_dt)
    w = rng.integers(-8, 8, (k, n)).astype(np.int8)
    groups = k // group if group else 1
    sc = rng.uniform(0.005, 0.02, (groups, n)).astype(np.float32).astype(np_dt)
    of = rng.uniform(-2, 2, (groups, n)).astype(np.float32).astype(np_dt) if has_off else None
    bias = rng.uniform(-1, 1, n).astype(np.float32).astype(np_dt) if has_bias else None
    want = wqbmm_oracle.weight_quant_batch_matmul(x, w, sc, of, bias, group)
    # the fixture runner takes the stored (transposed) arrays
    a = dict(x=x, w=np.ascontiguousarray(w.T), scale=np.ascontiguousarray(sc.T) if group else sc[0],
             offset=None if of is None else (np.ascontiguousarray(of.T) if group else of[0]), bias=bias, out=want)
    meta = dict(transpose_weight=True, w_is_int4=True, packed_int32=words, group_size=group)
    got = run_wq_fixture(aclnn, a, meta, kernel=0)
    assert aclnn.last_kernel_name() == "wqbmm_decode", aclnn.last_kernel_name()
    assert aclnn.lib().opsnn_wqbmm_decode_status(1) == 0
    gv, wv = got.astype(np.float64), want.astype(np.float64)
    assert not np.any(gv == -7777.0)
    ulp = 2.0 ** -7 if xdt == "bfloat16" else 2.0 ** -10
    rms = np.sqrt(np.mean(wv ** 2))
    assert np.all(np.abs(gv - wv) <= ulp * np.maximum(np.abs(wv), 0.05 * rms) * 1.01)


F8_CASES = [
    # x dtype, m, k, n, group, bias, NaN encodings planted, weight (and per-group scale) stored transposed
    ("bfloat16", 16, 2048, 1024, 0, False, False, False),     # per-channel
    ("float16", 16, 2048, 768, 128, False, False, False),     # per-group, fp16
    ("bfloat16", 5, 4096, 1040, 0, True, True, False),        # ragged last strip, m < 16, bias, NaN weights
    ("float16", 1, 8192, 512, 64, True, True, False),         # one group per stage, m = 1
    ("float16", 16, 2048, 1024, 0, False, False, True),       # weight stored (n,k)
    ("bfloat16", 16, 2048, 768, 128, False, True, True),
    ("float16", 5, 4096, 1040, 0, True, True, True),
]


def _f8_tensor(aclnn, codes, trans=False):
    import torch

    from gpu_util import DEV

    if trans:  # stored (n,k), described as the (k,n) view
        stored = torch.from_numpy(np.ascontiguousarray(codes.T)).to(DEV)
        return aclnn.Tensor(codes.shape, "float8_e4m3fn", stored, strides=(1, codes.shape[0]))
    return aclnn.Tensor(codes.shape, "float8_e4m3fn", torch.from_numpy(codes.copy()).to(DEV))


def _dev16_t(aclnn, a):
    """A 2-D 16-bit array stored transposed, described as the view of its own shape."""
    return aclnn.from_torch(_torch16(np.ascontiguousarray(a.T)).t())


def _torch16(a):
    import ml_dtypes
    import torch

    from gpu_util import DEV

    if a.dtype == np.dtype(ml_dtypes.bfloat16):
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(DEV)
    return torch.from_numpy(a.copy()).to(DEV)


def _dev16(aclnn, a):
    return None if a is None else aclnn.from_torch(_torch16(a))


@pytest.mark.parametrize("case", F8_CASES, ids=[str(c) for c in F8_CASES])
def test_a16f8_small_m_streaming_kernel(aclnn, case):
    """FLOAT8_E4M3FN weights at m <= 16 run on the 8-bit streaming kernel. Every byte code occurs (subnormals, both zeros, +-448);
    the dequantised weight rn(w * scale) is the golden's (wqbmmv2_kernel_golden.py:199-297), so only the fp32 summation order
    differs: <= 1 ulp of the output dtype. Where NaN encodings (0x7f, 0xff) are planted, exactly the columns that hold one are NaN."""
    import ml_dtypes
    import torch

    from gpu_util import DEV, out_to_np

    xdt, m, k, n, group, has_bias, plant, trans = case
    rng = np.random.default_rng(case_seed(case))
    np_dt = ml_dtypes.bfloat16 if xdt == "bfloat16" else np.float16
    x = rng.standard_normal((m, k)).astype(np.float32).astype(np_dt)
    codes = rng.integers(0, 256, (k, n)).astype(np.uint8)
    codes[(codes & 0x7F) == 0x7F] ^= 0x01                # no NaN by chance (0x7f -> 0x7e = 448)
    nan_cols = []
    if plant:
        nan_cols = [0, 1, 17, 510, 511, n - 1, n - 16]
        for i, c in enumerate(nan_cols):
            codes[(i * 997 + 3) % k, c] = 0x7F if i % 2 == 0 else 0xFF
        codes[k - 1, 2] = 0xFF
        nan_cols.append(2)
    w = codes.view(ml_dtypes.float8_e4m3fn)
    groups = k // group if group else 1
    sc = rng.uniform(0.002, 0.01, (groups, n)).astype(np.float32).astype(np_dt)
    bias = rng.uniform(-1, 1, n).astype(np.float32).astype(np_dt) if has_bias else None

    y = torch.full((m, n), -7777.0, dtype=torch.bfloat16 if xdt == "bfloat16" else torch.float16, device=DEV)
    d_sc = (_dev16_t(aclnn, sc) if trans else _dev16(aclnn, sc)) if group else _dev16(aclnn, sc[0])
    aclnn.weight_quant_batch_matmul(_dev16(aclnn, x), _f8_tensor(aclnn, codes, trans), d_sc, aclnn.from_torch(y), None, _dev16(aclnn, bias), group)
    torch.cuda.synchronize()
    assert aclnn.last_kernel_name() == "wqbmm_decode8", aclnn.last_kernel_name()
    with np.errstate(invalid="ignore"):
        want = wqbmm_oracle.weight_quant_batch_matmul(x, w, sc, None, bias, group).astype(np.float64)
    got = out_to_np(y).astype(np.float64)
    assert not np.any(got == -7777.0)
    is_nan = np.zeros(n, dtype=bool)
    is_nan[nan_cols] = True
    assert np.array_equal(np.isnan(want), np.broadcast_to(is_nan, want.shape))
    assert np.array_equal(np.isnan(got), np.isnan(want)), "NaN columns differ"
    ok = ~np.isnan(want)
    ulp = 2.0 ** -7 if xdt == "bfloat16" else 2.0 ** -10
    rms = np.sqrt(np.mean(want[ok] ** 2))
    assert np.all(np.abs(got[ok] - want[ok]) <= ulp * np.maximum(np.abs(want[ok]), 0.05 * rms) * 1.01)


@pytest.mark.parametrize("trans", [False, True], ids=["(k,n)", "(n,k)"])
@pytest.mark.parametrize("xdt", ["bfloat16", "float16"])
def test_a16f8_dequantisation_is_bit_exact(aclnn, xdt, trans):
    """With one-hot rows of x the product is the dequantised weight row itself (every other term is a zero), so the streaming kernel's
    e4m3 -> 16-bit conversion and its single rounding of w * scale are compared bit for bit with the oracle, for every finite byte
    code in every selected row (subnormals and both zeros included) and for scales that push products into the 16-bit type's
    subnormal range."""
    import ml_dtypes
    import torch

    from gpu_util import DEV, out_to_np

    m, k, n, group = 16, 2048, 1024, 128
    rng = np.random.default_rng(41 if xdt == "bfloat16" else 43)
    np_dt = ml_dtypes.bfloat16 if xdt == "bfloat16" else np.float16
    rows = rng.choice(k, m, replace=False)
    x = np.zeros((m, k), dtype=np_dt)
    x[np.arange(m), rows] = 1
    codes = ((np.arange(k)[:, None] * 7 + np.arange(n)[None, :] * 13) % 256).astype(np.uint8)   # every code in every row
    codes[(codes & 0x7F) == 0x7F] ^= 0x01
    w = codes.view(ml_dtypes.float8_e4m3fn)
    tiny = 2.0 ** -120 if xdt == "bfloat16" else 2.0 ** -14
    sc = rng.uniform(0.002, 0.01, (k // group, n)).astype(np.float32)
    sc[:, 0::5] *= -1
    sc[:, 1::7] = tiny * rng.uniform(1, 2, sc[:, 1::7].shape)        # products in the subnormal range of the 16-bit type
    sc = sc.astype(np_dt)
    y = torch.full((m, n), -7777.0, dtype=torch.bfloat16 if xdt == "bfloat16" else torch.float16, device=DEV)
    aclnn.weight_quant_batch_matmul(_dev16(aclnn, x), _f8_tensor(aclnn, codes, trans), _dev16_t(aclnn, sc) if trans else _dev16(aclnn, sc),
                                    aclnn.from_torch(y), None, None, group)
    torch.cuda.synchronize()
    assert aclnn.last_kernel_name() == "wqbmm_decode8", aclnn.last_kernel_name()
    want = wqbmm_oracle.weight_quant_batch_matmul(x, w, sc, None, None, group)
    got = out_to_np(y)
    assert np.array_equal(got.astype(np.float32), want.astype(np.float32))
    assert np.count_nonzero(want.astype(np.float32)) > m * n // 2


CHUNK8_CASES = [
    # weight kind, stored (n,k), m
    ("int8", False, 40),
    ("e4m3", True, 33),
    ("int4", True, 48),
]


@pytest.mark.parametrize("case", CHUNK8_CASES, ids=[str(c) for c in CHUNK8_CASES])
def test_8bit_and_nk_decode_kernels_in_chunks_of_16_rows(aclnn, case):
    """16 < m <= 48 against a large weight: the 8-bit streaming kernels and the (n,k) int4 kernel run once per 16 rows of x, like the
    (k,n) int4 kernel; same <= 1 ulp criterion as a single launch."""
    import ml_dtypes
    import torch

    from gpu_util import DEV, out_to_np, run_wq_fixture

    kind, trans, m = case
    k, n, g = 4096, 16384, 128
    rng = np.random.default_rng(case_seed(case))
    x = rng.standard_normal((m, k)).astype(np.float32).astype(ml_dtypes.bfloat16)
    sc = rng.uniform(0.005, 0.02, (k // g, n)).astype(np.float32).astype(ml_dtypes.bfloat16)
    if kind == "int4":
        w = rng.integers(-8, 8, (k, n)).astype(np.int8)
        of = rng.uniform(-1, 1, (k // g, n)).astype(np.float32).astype(ml_dtypes.bfloat16)
        want = wqbmm_oracle.weight_quant_batch_matmul(x, w, sc, of, None, g)
        a = dict(x=x, w=np.ascontiguousarray(w.T), scale=np.ascontiguousarray(sc.T), offset=np.ascontiguousarray(of.T), bias=None, out=want)
        got = run_wq_fixture(aclnn, a, dict(transpose_weight=True, w_is_int4=True, packed_int32=True, group_size=g), kernel=0)
        assert aclnn.last_kernel_name() == "wqbmm_decode", aclnn.last_kernel_name()
    else:
        y = torch.full((m, n), -7777.0, dtype=torch.bfloat16, device=DEV)
        d_sc = _dev16_t(aclnn, sc) if trans else _dev16(aclnn, sc)
        if kind == "int8":
            w = rng.integers(-128, 128, (k, n)).astype(np.int8)
            d_w = aclnn.from_torch(torch.from_numpy(np.ascontiguousarray(w.T)).to(DEV).t() if trans else torch.from_numpy(w).to(DEV))
        else:
            codes = rng.integers(0, 256, (k, n)).astype(np.uint8)
            codes[(codes & 0x7F) == 0x7F] ^= 0x01
            w = codes.view(ml_dtypes.float8_e4m3fn)
            d_w = _f8_tensor(aclnn, codes, trans)
        want = wqbmm_oracle.weight_quant_batch_matmul(x, w, sc, None, None, g)
        aclnn.weight_quant_batch_matmul(_dev16(aclnn, x), d_w, d_sc, aclnn.from_torch(y), None, None, g)
        torch.cuda.synchronize()
        assert aclnn.last_kernel_name() == "wqbmm_decode8", aclnn.last_kernel_name()
        got = out_to_np(y)
    gv, wv = got.astype(np.float64), want.astype(np.float64)
    assert not np.any(gv == -7777.0)
    rms = np.sqrt(np.mean(wv ** 2))
    assert np.all(np.abs(gv - wv) <= 2.0 ** -7 * np.maximum(np.abs(wv), 0.05 * rms) * 1.01)


W8_CASES = [
    # x dtype, m, k, n, group, offset, bias, weight (and per-group scale / offset) stored transposed
    ("bfloat16", 16, 2048, 1024, 0, False, False, False),     # per-channel, symmetric: the common W8A16 form
    ("bfloat16", 5, 4096, 1040, 0, True, True, False),        # ragged last strip, fewer than 16 rows, offset + bias
    ("float16", 16, 2048, 768, 128, True, False, False),      # per-group (two stages per group), fp16
    ("bfloat16", 1, 8192, 512, 64, False, True, False),       # one group per stage, m = 1
    ("bfloat16", 16, 2048, 1024, 0, False, False, True),      # weight stored (n,k), k contiguous
    ("float16", 5, 4096, 1040, 0, True, True, True),
    ("bfloat16", 16, 2048, 768, 128, True, False, True),      # scales stored (n, groups)
    ("float16", 1, 8192, 512, 64, False, True, True),
    ("bfloat16", 13, 4112, 2064, 0, True, False, True),       # k not a multiple of the 64-row stage, ragged strip
    ("float16", 16, 16384, 64, 0, False, False, True),        # fewer columns than one copy box has rows
]


@pytest.mark.parametrize("case", W8_CASES, ids=[str(c) for c in W8_CASES])
def test_w8a16_small_m_streaming_kernel(aclnn, case):
    """INT8 weights at m <= 16 run on their own streaming kernel (the reference's n-first regime,
    weight_quant_batch_matmul_v2/op_kernel/arch35/n_first/*); it reproduces the golden's two roundings per weight, so only the
    fp32 summation order differs: <= 1 ulp of the output dtype."""
    import ml_dtypes
    import torch

    from gpu_util import DEV, out_to_np

    xdt, m, k, n, group, has_off, has_bias, trans = case
    rng = np.random.default_rng(case_seed(case))
    np_dt = ml_dtypes.bfloat16 if xdt == "bfloat16" else np.float16
    x = rng.standard_normal((m, k)).astype(np.float32).astype(np_dt)
    w = rng.integers(-128, 128, (k, n)).astype(np.int8)
    groups = k // group if group else 1
    sc = rng.uniform(0.002, 0.01, (groups, n)).astype(np.float32).astype(np_dt)
    of = rng.uniform(-3, 3, (groups, n)).astype(np.float32).astype(np_dt) if has_off else None
    bias = rng.uniform(-1, 1, n).astype(np.float32).astype(np_dt) if has_bias else None

    def dev(a):
        return None if a is None else aclnn.from_torch(_torch16(a))

    def dev_t(a):  # stored transposed, described as the (rows, cols) view the API takes
        return None if a is None else aclnn.from_torch(_torch16(np.ascontiguousarray(a.T)).t())

    y = torch.full((m, n), -7777.0, dtype=torch.bfloat16 if xdt == "bfloat16" else torch.float16, device=DEV)
    if trans:
        aclnn.weight_quant_batch_matmul(dev(x), dev_t(w), dev_t(sc) if group else dev(sc[0]), aclnn.from_torch(y),
                                        (dev_t(of) if group else dev(of[0])) if of is not None else None, dev(bias), group)
    else:
        aclnn.weight_quant_batch_matmul(dev(x), dev(w), dev(sc if group else sc[0]), aclnn.from_torch(y), dev(of if (group or of is None) else of[0]),
                                        dev(bias), group)
    torch.cuda.synchronize()
    assert aclnn.last_kernel_name() == "wqbmm_decode8", aclnn.last_kernel_name()
    want = wqbmm_oracle.weight_quant_batch_matmul(x, w, sc, of, bias, group).astype(np.float64)
    got = out_to_np(y).astype(np.float64)
    assert not np.any(got == -7777.0)
    ulp = 2.0 ** -7 if xdt == "bfloat16" else 2.0 ** -10
    rms = np.sqrt(np.mean(want ** 2))
    assert np.all(np.abs(got - want) <= ulp * np.maximum(np.abs(want), 0.05 * rms) * 1.01)
