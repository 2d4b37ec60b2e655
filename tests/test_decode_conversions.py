"""CPU: the bit-level conversions the streaming decode kernels use, restated in numpy and checked over every input code.

The kernels (ops-nn_b200/csrc/cuda/wqbmm_decode_tma.cu, wqbmm_decode8_tma.cu) turn packed weights into bf16 / fp16 pairs with
logic operations and exact 16-bit arithmetic instead of conversion instructions. Each identity below is what one of those
sequences relies on; the GPU tests check the kernels against the oracle, this file checks the identities themselves so that a
reader can see (and a change to a constant must keep) why the sequences are exact."""
import ml_dtypes
import numpy as np
import pytest

BF16 = ml_dtypes.bfloat16


def _as16(bits, dt):
    return np.asarray(bits, dtype=np.uint16).view(dt).astype(np.float64)


def test_int4_magic_number_is_exact():
    """(nibble ^ 8) | magic reads as B + w with B = 136 (bf16) / 1032 (fp16) for the two's-complement nibble of w in [-8, 7]."""
    w = np.arange(-8, 8)
    nib = (w & 0xF).astype(np.uint16)
    assert np.array_equal(_as16((nib ^ 8) | 0x4300, BF16), 136.0 + w)
    assert np.array_equal(_as16((nib ^ 8) | 0x6400, np.float16), 1032.0 + w)


def test_int8_conversion_is_exact():
    """bf16: ((b & 0x7f) | 0x4300) - ((b & 0x80) | 0x4300) = w; fp16: (((b ^ 0x80) & 0xff) | 0x6400) - 1152 = w, both subtractions
    exact in the 16-bit type."""
    w = np.arange(-128, 128)
    b = (w & 0xFF).astype(np.uint16)
    lo, hi = _as16((b & 0x7F) | 0x4300, BF16), _as16((b & 0x80) | 0x4300, BF16)
    assert np.array_equal((lo - hi).astype(BF16).astype(np.float64), w)
    f = _as16(((b ^ 0x80) & 0xFF) | 0x6400, np.float16)
    assert np.array_equal((f - 1152.0).astype(np.float16).astype(np.float64), w)


@pytest.mark.parametrize("dt,shift,rebias", [(BF16, 4, 2.0 ** 120), (np.float16, 7, 2.0 ** 8)])
def test_e4m3_conversion_is_exact_for_every_finite_code(dt, shift, rebias):
    """The seven magnitude bits moved under the sign of the 16-bit type read as w / rebias - normals, subnormals and both zeros -
    and the product with rebias is exactly representable, so one multiplication restores w."""
    codes = np.arange(256, dtype=np.uint16)
    finite = (codes & 0x7F) != 0x7F
    bits = ((codes & 0x7F) << shift) | ((codes & 0x80) << 8)
    got = _as16(bits, dt) * rebias
    want = codes.astype(np.uint8).view(ml_dtypes.float8_e4m3fn).astype(np.float64)
    assert np.array_equal(got[finite], want[finite])
    assert np.array_equal(got[finite].astype(dt).astype(np.float64), got[finite])                   # representable: the multiply is exact
    assert np.array_equal(np.signbit(got[finite]), np.signbit(want[finite]))                        # -0 stays -0
    assert np.all(np.abs(got[~finite]) == 480.0) and not np.any(np.abs(want[finite]) == 480.0)      # what the NaN test guards against
    assert np.all(np.isnan(want[~finite]))


def test_e4m3_nan_detector_flags_exactly_the_nan_bytes():
    """((x & 0x7f7f7f7f) + 0x01010101) & 0x80808080 has bit 7 of a byte set iff that byte is 0x7f or 0xff; no carry crosses bytes."""
    rng = np.random.default_rng(0)
    by = rng.integers(0, 256, (4096, 4)).astype(np.uint8)
    by[::7, 1] = 0x7F
    by[::11, 3] = 0xFF
    by[::13, 0] = 0xFE
    x = by.view("<u4")[:, 0].astype(np.uint64)
    flags = (((x & 0x7F7F7F7F) + 0x01010101) & 0x80808080).astype(np.uint32)
    got = np.stack([(flags >> (8 * i + 7)) & 1 for i in range(4)], axis=1).astype(bool)
    assert np.array_equal(got, (by & 0x7F) == 0x7F)


def test_permuted_k_order_of_the_nk_kernels_pairs_a_and_b_consistently():
    """The (n,k) kernels feed an m16n8k16 MMA with B registers (k0, k2 | k1, k3) of a lane's four bytes (int8) or (n0, n4 | n1, n5)
    and (n2, n6 | n3, n7) of its eight nibbles (int4), and build the A fragment from x[row][same k] in the same positions: every k of a
    16- / 32-row step is used exactly once and meets its own x element."""
    # int8: lane q owns k = 4q .. 4q+3; MMA slot (reg, half) of lane q multiplies A slot (reg, half) of lane q
    used = []
    for q in range(4):
        b_regs = [(4 * q + 0, 4 * q + 2), (4 * q + 1, 4 * q + 3)]   # deq(r), deq(r >> 8)
        a_regs = [(4 * q + 0, 4 * q + 2), (4 * q + 1, 4 * q + 3)]   # prmt(lo, hi, 0x5410), prmt(lo, hi, 0x7632)
        assert a_regs == b_regs
        used += [k for pair in b_regs for k in pair]
    assert sorted(used) == list(range(16))
    # int4: lane q owns k = 8q .. 8q+7 of a 32-row step; two MMAs
    used = []
    for q in range(4):
        base = 8 * q
        b_lo = [(base + 0, base + 4), (base + 1, base + 5)]       # deq(r), deq(r >> 4)
        b_hi = [(base + 2, base + 6), (base + 3, base + 7)]       # deq(r >> 8), deq(r >> 12)
        x_regs = [(base + 0, base + 1), (base + 2, base + 3), (base + 4, base + 5), (base + 6, base + 7)]  # one 16-byte load
        lo16 = lambda a, c: (x_regs[a][0], x_regs[c][0])  # noqa: E731  prmt 0x5410: low halves
        hi16 = lambda a, c: (x_regs[a][1], x_regs[c][1])  # noqa: E731  prmt 0x7632: high halves
        assert [lo16(0, 2), hi16(0, 2)] == b_lo
        assert [lo16(1, 3), hi16(1, 3)] == b_hi
        used += [k for pair in b_lo + b_hi for k in pair]
    assert sorted(used) == list(range(32))
