"""CPU: the oracle (oracle/*.py, oracle/c) against the committed outputs of the reference's own goldens."""
import numpy as np
import pytest

from conftest import golden_names, load_golden
from oracle import mx_quant_oracle, qbmm_oracle, wqbmm_oracle


def _close(got, want, dtype_name):
    """Float outputs: the fixtures were produced with this machine's BLAS; another CPU may sum in another order, so allow
    one unit in the last place of the output dtype on a few elements. Integer outputs: exact."""
    g = np.asarray(got).astype(np.float64)
    w = np.asarray(want).astype(np.float64)
    if dtype_name in ("int32", "int8"):
        return np.array_equal(g, w)
    ulp = {"bfloat16": 2.0 ** -7, "float16": 2.0 ** -10, "float32": 2.0 ** -18}[dtype_name]
    fin = np.isfinite(w)
    ok = np.abs(g - w)[fin] <= ulp * np.maximum(np.abs(w[fin]), 1e-30) * 1.01 + 1e-30
    return ok.mean() > 0.995 and np.array_equal(np.isfinite(g), fin)


@pytest.mark.parametrize("name", golden_names("qmm_"))
def test_qmm_oracle_matches_reference_golden(name):
    a, meta = load_golden(name)
    u64 = meta["dtypes"].get("x2_scale") == "uint64"
    bias = a.get("bias")
    if bias is not None and "y_scale" in meta["dtypes"] or (bias is not None and bias.ndim == 2):
        bias = bias.reshape(-1)  # the A8W4 modes take bias as (1, n)
    got = qbmm_oracle.quant_matmul_v5(a["x1"], a["x2"], a.get("x1_scale"), a["x2_scale"], bias,
                                      meta["transpose_x1"], meta["transpose_x2"],
                                      _full_group(meta, a), meta["out_dtype"], x2_scale_is_u64=u64, y_scale=a.get("y_scale"),
                                      x2_offset=a.get("x2_offset"))
    assert got.shape == a["out"].shape
    assert _close(got, a["out"], meta["out_dtype"])


def _full_group(meta, a):
    return meta["group_size"]


@pytest.mark.parametrize("name", golden_names("wq_"))
def test_wq_oracle_matches_reference_golden(name):
    a, meta = load_golden(name)
    t = meta["transpose_weight"]
    w = a["w"].T if t else a["w"]
    sc = a["scale"].T if (t and a["scale"].ndim == 2) else a["scale"]
    of = a.get("offset")
    if of is not None and t and of.ndim == 2:
        of = of.T
    got = wqbmm_oracle.weight_quant_batch_matmul(a["x"], w, sc, of, a.get("bias"), meta["group_size"])
    assert _close(got, a["out"], meta["dtypes"]["out"])


@pytest.mark.parametrize("name", golden_names("mxq_"))
def test_mx_quant_oracle_matches_reference_golden(name):
    a, meta = load_golden(name)
    y, s = mx_quant_oracle.dynamic_mx_quant(a["x"], meta["dst"], axis=meta.get("axis", -1), scale_alg=meta.get("scale_alg", 0),
                                            round_mode=meta.get("round_mode", "rint"))
    assert np.array_equal(y.view(np.uint8), a["y"].view(np.uint8))
    assert np.array_equal(s, a["scale"].view(np.uint8))


def test_int4_pack_roundtrip():
    rng = np.random.default_rng(5)
    v = rng.integers(-8, 8, (7, 64)).astype(np.int8)
    p = wqbmm_oracle.pack_int4_words(v)
    assert p.shape == (7, 8) and p.dtype == np.int32
    assert np.array_equal(wqbmm_oracle.unpack_int4_words(p), v)
    # element j of a word sits at bits [4j, 4j+4) (matmul_quant_util.py:228-273 of the reference)
    one = np.zeros((1, 8), np.int8)
    one[0, 3] = -3
    assert int(wqbmm_oracle.pack_int4_words(one)[0, 0]) == ((-3) & 0xF) << 12


def test_faithful_dequant_is_within_tolerance_of_fp32_product():
    """The reference's double-rounded dequant sits well inside the stated 1e-2 bound of an fp32 dequantised product."""
    a, meta = load_golden("wq_bf16_s4_group128_offset_m16")
    ref = wqbmm_oracle.fp32_dequant_product(a["x"], a["w"], a["scale"], a["offset"], None, meta["group_size"])
    got = a["out"].astype(np.float64)
    rms = np.sqrt(np.mean(ref ** 2))
    assert np.max(np.abs(got - ref) / (np.abs(ref) + rms)) < 1e-2
