"""CPU: opsnn_wqbmm_select_kernel on parameter blocks with stand-in addresses (nothing is launched, no device is touched): which
weight-only calls go to the streaming decode kernels, which are run in chunks of 16 rows, which take dequantise-then-matmul."""
import ctypes

import pytest

GENERIC, DECODE, DECODE_FAST, PREFILL = 1, 2, 3, 4


def _probe(aclnn, m, k, n, g=128, w_dtype=None, trans=False, inner_precise=0, scale_dtype=None, offset=True):
    p = aclnn.WqbmmParams()
    p.x_dtype, p.bias_dtype, p.trans_w = aclnn.ACL_BF16, -1, 1 if trans else 0
    p.w_dtype = aclnn.ACL_INT4 if w_dtype is None else w_dtype
    p.m, p.n, p.k = m, n, k
    p.x, p.x_ld = 4096, k
    p.w, p.w_ld = 8192, (k if trans else n)
    p.scale, p.offset = 12288, (16384 if offset else None)
    groups = k // g if g else 1
    p.group_size, p.scale_sg, p.scale_sn = g, ((1 if trans else n) if g else 0), (groups if trans else 1)
    if scale_dtype is not None:
        p.scale_dtype = scale_dtype
    p.bias = None
    p.y, p.y_ld = 20480, n
    p.inner_precise = inner_precise
    return p


@pytest.fixture(scope="module")
def aclnn():
    from conftest import load_package

    return load_package().aclnn


def _sel(aclnn, *a, **kw):
    return aclnn.lib().opsnn_wqbmm_select_kernel(ctypes.byref(_probe(aclnn, *a, **kw)))


def test_small_m_int4_runs_on_the_decode_kernels(aclnn):
    assert _sel(aclnn, 16, 4096, 4096) == DECODE
    assert _sel(aclnn, 1, 8192, 28672) == DECODE
    assert _sel(aclnn, 16, 8192, 28672, inner_precise=1) == DECODE_FAST
    assert _sel(aclnn, 64, 8192, 28672) == PREFILL


def test_chunks_of_16_rows_start_where_they_were_measured_to_pay(aclnn):
    """Two launches (m <= 32) from 2^24 weights on, three (m <= 48) from 3 x 2^24; below that, and beyond 48 rows, dequantise-then-
    matmul."""
    assert _sel(aclnn, 32, 4096, 4096) == DECODE            # 2^24
    assert _sel(aclnn, 32, 4096, 2048) == PREFILL           # 2^23
    assert _sel(aclnn, 17, 4096, 4096) == DECODE
    assert _sel(aclnn, 48, 4096, 4096) == PREFILL           # three launches: not yet
    assert _sel(aclnn, 48, 4096, 12288) == DECODE           # 3 x 2^24
    assert _sel(aclnn, 33, 4096, 14336) == DECODE
    assert _sel(aclnn, 49, 8192, 28672) == PREFILL
    assert _sel(aclnn, 40, 8192, 28672, inner_precise=1) == DECODE_FAST


def test_eight_bit_weights_take_the_streaming_kernel_from_2_20_weights_on(aclnn):
    for wd in (aclnn.ACL_INT8, aclnn.ACL_FLOAT8_E4M3FN):
        off = wd == aclnn.ACL_INT8  # fp8 weights take no offset
        for trans in (False, True):
            assert _sel(aclnn, 16, 2048, 1024, g=0, w_dtype=wd, trans=trans, offset=off) == DECODE
            assert _sel(aclnn, 16, 1024, 512, g=0, w_dtype=wd, trans=trans, offset=off) != DECODE
            assert _sel(aclnn, 32, 4096, 4096, g=0, w_dtype=wd, trans=trans, offset=off) == DECODE   # in chunks
    assert _sel(aclnn, 16, 2048, 1024, g=0, w_dtype=aclnn.ACL_FLOAT8_E4M3FN) != DECODE   # an offset with fp8 weights: not this kernel
    assert _sel(aclnn, 16, 2048, 1024, g=32, w_dtype=aclnn.ACL_INT8) != DECODE   # groups must be whole 64-row stages


def test_e8m0_scales_never_reach_the_decode_kernels(aclnn):
    assert _sel(aclnn, 16, 4096, 4096, g=32, scale_dtype=aclnn.ACL_FLOAT8_E8M0) not in (DECODE, DECODE_FAST)
    assert _sel(aclnn, 16, 4096, 4096, g=0, w_dtype=aclnn.ACL_INT8, scale_dtype=aclnn.ACL_FLOAT8_E8M0) not in (DECODE, DECODE_FAST)
