"""GPU parity on seeded random shapes: the per-block kernel on CTA pairs and the weight-only paths, against the oracle.

The fixtures pin chosen shapes; these cases walk ragged m, k tails inside a 128-k block, n that is not a multiple of
the tile, every transpose combination and every weight layout, with the shape drawn from a fixed seed so that a failure
names a reproducible case."""
import ml_dtypes
import numpy as np
import pytest

from oracle import qbmm_oracle, wqbmm_oracle

pytestmark = pytest.mark.gpu

E4M3 = ml_dtypes.float8_e4m3fn


def _perblock_case(rng):
    m = int(rng.integers(1, 700))
    k = int(rng.integers(1, 9)) * 128 + int(rng.choice([0, 16, 64, 112]))
    n = int(rng.integers(1, 40)) * 16
    t1, t2 = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
    is_int = bool(rng.integers(0, 2))
    gm = 1 if is_int else int(rng.choice([1, 128]))
    if t1:
        m = (m + 15) // 16 * 16  # x1 stored (k, m): the row pitch must be a multiple of 16 bytes for the tensor-core path
    kb, mg, ng = -(-k // 128), -(-m // gm), -(-n // 128)
    if is_int:
        x1 = rng.integers(-127, 128, (k, m) if t1 else (m, k), dtype=np.int8)
        x2 = rng.integers(-127, 128, (n, k) if t2 else (k, n), dtype=np.int8)
        s1 = rng.uniform(1e-3, 1e-2, (kb, mg) if t1 else (mg, kb)).astype(np.float32)
        s2 = rng.uniform(1e-2, 1e-1, (ng, kb) if t2 else (kb, ng)).astype(np.float32)
    else:
        x1 = rng.standard_normal((k, m) if t1 else (m, k)).astype(np.float32).astype(E4M3)
        x2 = rng.standard_normal((n, k) if t2 else (k, n)).astype(np.float32).astype(E4M3)
        s1 = rng.uniform(0.5, 2, (kb, mg) if t1 else (mg, kb)).astype(np.float32)
        s2 = rng.uniform(0.5, 2, (ng, kb) if t2 else (kb, ng)).astype(np.float32)
    return m, k, n, t1, t2, is_int, gm, x1, x2, s1, s2


@pytest.mark.parametrize("tile_n", ["128", "256"])
@pytest.mark.parametrize("seed", [1, 2, 4])
def test_perblock_pair_random_shapes(aclnn, seed, tile_n, monkeypatch):
    """int8 per-block results are bit-exact (integer partial sums promoted exactly, fp32 operations in the reference's
    order); fp8 per-block within the stated bf16 tolerance of the fp32 result."""
    from gpu_util import check_close, desc, out_tensor, out_to_np
    import torch

    monkeypatch.setenv("OPSNN_QMM_PAIR", "1")
    monkeypatch.setenv("OPSNN_QMM_PB_BN", tile_n)
    rng = np.random.default_rng(seed)
    for _ in range(10):
        m, k, n, t1, t2, is_int, gm, x1, x2, s1, s2 = _perblock_case(rng)
        tag = f"seed={seed} m={m} k={k} n={n} t1={t1} t2={t2} int8={is_int} gm={gm}"
        group = (gm << 32) | (128 << 16) | 128
        want = qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, None, t1, t2, group, "bfloat16")
        out = out_tensor((m, n), "bfloat16")
        aclnn.quant_matmul_v5(desc(aclnn, x1), desc(aclnn, x2), desc(aclnn, s1), desc(aclnn, s2),
                              aclnn.Tensor(out.shape, "bfloat16", out), None, t1, t2, group)
        torch.cuda.synchronize()
        assert aclnn.lib().opsnn_qmm_umma_status(1) == 0, tag
        assert aclnn.last_kernel_name() in ("qmm_umma_pair_perblock", "qmm_umma_perblock"), tag
        got = out_to_np(out)
        if is_int:
            assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), tag
        else:
            check_close(got, want, qbmm_oracle.quant_matmul_v5(x1, x2, s1, s2, None, t1, t2, group, "float32"), "bfloat16")


@pytest.mark.parametrize("seed", [1, 2, 4])
def test_weight_only_random_shapes(aclnn, seed):
    """Every weight layout (int8 / int4 bytes / int4 in int32 words, stored (k,n) or (n,k)), per-channel and per-group,
    with and without offset, m from 1 to 300 so that the decode, chunked-decode and dequantise-then-matmul paths are all
    drawn: within 2 ulp of the output dtype of the oracle (the paths differ from it only in fp32 summation order and, for
    the matmul path, in rounding the dequantised weight once more to 16 bits, which is exact here)."""
    from gpu_util import run_wq_fixture

    rng = np.random.default_rng(seed)
    for _ in range(10):
        m = int(rng.integers(1, 300))
        k = int(rng.integers(2, 20)) * 64
        n = int(rng.integers(1, 60)) * 8
        int4, tw = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        g = int(rng.choice([0, 32, 64, 128]))
        if g and (k % g or g >= k):
            g = 64
        words = int4 and not tw and bool(rng.integers(0, 2))
        xdt = ml_dtypes.bfloat16 if rng.integers(0, 2) else np.float16
        x = rng.standard_normal((m, k)).astype(xdt)
        w = (rng.integers(-8, 8, (k, n)) if int4 else rng.integers(-127, 128, (k, n))).astype(np.int8)
        sshape = (k // g, n) if g else (n,)
        scale = rng.uniform(0.005, 0.02, sshape).astype(xdt)
        offset = rng.uniform(-1, 1, sshape).astype(xdt) if rng.integers(0, 2) else None
        tag = f"seed={seed} m={m} k={k} n={n} int4={int4} tw={tw} g={g} words={words} {np.dtype(xdt).name} off={offset is not None}"
        want = wqbmm_oracle.weight_quant_batch_matmul(x, w, scale, offset, None, g)

        def stored(a):
            return a.T.copy() if (tw and a is not None and a.ndim == 2) else a

        a = dict(x=x, w=stored(w), scale=stored(scale), offset=stored(offset), bias=None, out=want)
        meta = dict(transpose_weight=tw, w_is_int4=int4, packed_int32=words, group_size=g)
        got = run_wq_fixture(aclnn, a, meta, kernel=0).astype(np.float64)
        assert aclnn.lib().opsnn_qmm_umma_status(1) == 0, tag
        wv = want.astype(np.float64)
        ulp = 2.0 ** -7 if xdt is ml_dtypes.bfloat16 else 2.0 ** -10
        rms = np.sqrt(np.mean(wv ** 2)) + 1e-30
        assert np.all(np.abs(got - wv) <= 2 * ulp * np.maximum(np.abs(wv), 0.05 * rms) * 1.01), tag


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_streaming_decode_kernels_random_shapes(aclnn, seed):
    """Weights large enough (k n >= 2^20) for the streaming decode kernels at m <= 16, every kind they take - INT4 in int32 words,
    INT8, FLOAT8_E4M3FN, each stored (k,n) or (n,k) with the scales stored the same way - ragged strips, k that is not a multiple of
    a stage, per-channel and per-group scales, offsets, bias: within 1 ulp of the output dtype of the oracle (fp32 summation order
    is the only difference), and most draws must really have run on a streaming kernel."""
    import torch

    from gpu_util import desc, out_tensor, out_to_np

    rng = np.random.default_rng(seed)
    streamed = 0
    draws = 12
    for _ in range(draws):
        kind = str(rng.choice(["int4", "int8", "e4m3"]))
        tw = bool(rng.integers(0, 2))
        m = int(rng.integers(1, 17))
        k = int(rng.integers(32, 130)) * 32
        n = int(rng.integers(max(1, (1 << 20) // k // 16 + 1), 160)) * 16
        g = int(rng.choice([0, 128, 256]))
        if g and (k % g or g >= k):
            g = 0
        xdt = ml_dtypes.bfloat16 if rng.integers(0, 2) else np.float16
        x = rng.standard_normal((m, k)).astype(np.float32).astype(xdt)
        sshape = (k // g, n) if g else (n,)
        scale = rng.uniform(0.005, 0.02, sshape).astype(np.float32).astype(xdt)
        offset = rng.uniform(-1, 1, sshape).astype(np.float32).astype(xdt) if (kind != "e4m3" and rng.integers(0, 2)) else None
        bias = rng.uniform(-1, 1, n).astype(np.float32).astype(xdt) if rng.integers(0, 2) else None
        if kind == "int4":
            w = rng.integers(-8, 8, (k, n)).astype(np.int8)
            words = wqbmm_oracle.pack_int4_words(w.T.copy() if tw else w)  # packed along the stored inner axis
            d_w = desc(aclnn, words, strides=(1, words.shape[1]), shape=(words.shape[1], words.shape[0])) if tw else desc(aclnn, words)
        elif kind == "int8":
            w = rng.integers(-128, 128, (k, n)).astype(np.int8)
            d_w = desc(aclnn, w.T.copy(), strides=(1, k), shape=(k, n)) if tw else desc(aclnn, w)
        else:
            codes = rng.integers(0, 256, (k, n)).astype(np.uint8)
            codes[(codes & 0x7F) == 0x7F] ^= 0x01
            w = codes.view(ml_dtypes.float8_e4m3fn)
            d_w = desc(aclnn, w.T.copy(), strides=(1, k), shape=(k, n)) if tw else desc(aclnn, w)

        def sdesc(a):
            if a is None:
                return None
            if tw and a.ndim == 2:  # stored (n, groups), described as (groups, n)
                return desc(aclnn, a.T.copy(), strides=(1, a.shape[0]), shape=a.shape)
            return desc(aclnn, a)

        tag = f"seed={seed} {kind} tw={tw} m={m} k={k} n={n} g={g} {np.dtype(xdt).name} off={offset is not None} bias={bias is not None}"
        want = wqbmm_oracle.weight_quant_batch_matmul(x, w, scale, offset, bias, g)
        name = "bfloat16" if xdt is ml_dtypes.bfloat16 else "float16"
        out = out_tensor((m, n), name)
        aclnn.weight_quant_batch_matmul(desc(aclnn, x), d_w, sdesc(scale), aclnn.Tensor((m, n), name, out), sdesc(offset), desc(aclnn, bias), g)
        torch.cuda.synchronize()
        streamed += aclnn.last_kernel_name() in ("wqbmm_decode", "wqbmm_decode8")
        assert aclnn.lib().opsnn_wqbmm_decode_status(1) == 0, tag
        got, wv = out_to_np(out).astype(np.float64), want.astype(np.float64)
        assert not np.any(got == -7777.0), tag
        ulp = 2.0 ** -7 if xdt is ml_dtypes.bfloat16 else 2.0 ** -10
        rms = np.sqrt(np.mean(wv ** 2)) + 1e-30
        assert np.all(np.abs(got - wv) <= ulp * np.maximum(np.abs(wv), 0.05 * rms) * 1.01), tag
    assert streamed >= draws * 2 // 3, streamed
