"""The plain-C oracle (oracle/c) against the golden fixtures generated from the reference's own goldens."""
import numpy as np

from conftest import load_golden
from oracle import c_oracle, wqbmm_oracle


def test_c_int8_kc_is_bit_identical_to_reference_golden():
    a, meta = load_golden("qmm_kc_int8_bf16")
    out, acc = c_oracle.qmm_int8_kc(a["x1"], a["x2"], a["x2_scale"], a.get("x1_scale"), a.get("bias"), threads=4, want_acc=True)
    assert np.array_equal(acc, a["x1"].astype(np.int32) @ a["x2"].astype(np.int32))
    assert np.array_equal(out, a["out"].view(np.uint16))
    one = c_oracle.qmm_int8_kc(a["x1"], a["x2"], a["x2_scale"], a.get("x1_scale"), a.get("bias"), threads=1)
    assert np.array_equal(one, out)  # threading does not change results


def test_c_w4a16_group_matches_reference_golden_within_summation_order():
    a, meta = load_golden("wq_bf16_s4_group128_offset_m16")
    w = a["w"]
    words = wqbmm_oracle.pack_int4_words(w)
    y = c_oracle.wq_w4a16_group(a["x"].view(np.uint16), words, a["scale"].view(np.uint16), a["offset"].view(np.uint16),
                                meta["group_size"], threads=3)
    got = (y.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    want = a["out"].astype(np.float64)
    rms = np.sqrt(np.mean(want ** 2))
    # same dequantised weights bit for bit; only the fp32 summation order differs from numpy's BLAS: <= 1 bf16 ulp
    assert np.all(np.abs(got - want) <= 2.0 ** -7 * np.maximum(np.abs(want), 0.05 * rms) * 1.01)
    assert np.mean(y != a["out"].view(np.uint16)) < 0.05
    part = c_oracle.wq_w4a16_group(a["x"].view(np.uint16), words, a["scale"].view(np.uint16), a["offset"].view(np.uint16),
                                   meta["group_size"], col_begin=8, col_end=24, threads=2)
    assert np.array_equal(part[:, 8:24], y[:, 8:24]) and not part[:, 24:].any() and not part[:, :8].any()
