"""Generates the golden fixtures in this folder by running the REFERENCE's own numpy goldens on seeded inputs.

Run where a checkout of hicann/ops-nn is available ($OPSNN_REFERENCE_ROOT, or a `reference` folder next to this repository):

    python tests/golden/make_golden.py

Each fixture `<case>.npz` holds the inputs, the reference golden's output and a JSON `meta` record (dtypes, attributes).
Low-precision arrays are stored as their raw bytes (one element per byte for fp8/e8m0, one code per byte for fp4/int4).
Shapes, dtypes, transposes and value ranges are those of the reference's system-test rows
(matmul/*/tests/st/arch35/ttk_*.csv; the CSVs carry no data, inputs there are drawn unseeded), scaled down where a row
would make the fixture large. While generating, every case is also run through `oracle/` and must match the reference
output bit for bit on this machine; that is what pins the oracle.
"""
import json
import os
import sys

import ml_dtypes
import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import mx_quant_oracle, qbmm_oracle, ref_loader, wqbmm_oracle  # noqa: E402

BF16 = ml_dtypes.bfloat16
E4M3 = ml_dtypes.float8_e4m3fn
E5M2 = ml_dtypes.float8_e5m2
E2M1 = ml_dtypes.float4_e2m1fn
E8M0 = ml_dtypes.float8_e8m0fnu
INT4 = ml_dtypes.int4

NAMES = {np.dtype(BF16): "bfloat16", np.dtype(E4M3): "float8_e4m3fn", np.dtype(E5M2): "float8_e5m2",
         np.dtype(E2M1): "float4_e2m1", np.dtype(E8M0): "float8_e8m0", np.dtype(INT4): "int4"}
ACL = {"float32": 0, "float16": 1, "int8": 2, "int32": 3, "bfloat16": 27, "float8_e5m2": 35, "float8_e4m3fn": 36}


def dname(a):
    return NAMES.get(a.dtype, a.dtype.name)


def raw(a):
    """Array -> storable array + dtype name."""
    n = dname(a)
    if n in ("bfloat16",):
        return a.view(np.uint16), n
    if n in ("float8_e4m3fn", "float8_e5m2", "float8_e8m0", "float4_e2m1"):
        return a.view(np.uint8), n
    if n == "int4":
        return a.astype(np.int8), n
    return a, n


def save(name, arrays, meta):
    out = {}
    meta = dict(meta)
    meta["dtypes"] = {}
    for k, v in arrays.items():
        if v is None:
            continue
        r, n = raw(np.ascontiguousarray(v))
        out[k] = r
        meta["dtypes"][k] = n
    out["meta"] = np.frombuffer(json.dumps(meta, sort_keys=True).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: (v.shape, meta["dtypes"][k]) for k, v in arrays.items() if v is not None})


def bits_equal(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.shape == b.shape and a.dtype == b.dtype and a.tobytes() == b.tobytes()


def q_fp8(rng, shape, dt, scale=1.0):
    return (rng.standard_normal(shape).astype(np.float32) * scale).astype(dt)


def q_fp4(rng, shape):
    return (rng.standard_normal(shape).astype(np.float32) * 2.0).astype(E2M1)


def e8m0(rng, shape, lo=-3, hi=3):
    return np.exp2(rng.integers(lo, hi + 1, shape).astype(np.float32)).astype(E8M0)


# ------------------------------------------------------------------------------------------------------------
def qmm_case(G, name, seed, x1, x2, x1s, x2s, bias, t1, t2, group, out, note, x2s_u64=None, check_oracle=True,
             api_group=None, per_tile=False, offset=None):
    """x2s_u64: the packed uint64 tensor handed to the API when the scale is the fixpipe-packed form.
    per_tile: int8 per-block, computed by the V4 golden's compute_per_tile (2-D operands only)."""
    ref = G["qbmmv3"]
    kw = dict(dtype=ACL.get(out, 0), transpose_x1=t1, transpose_x2=t2, group_size=group, output_dtypes=[out])
    a = x1.T if t1 and x1.ndim == 2 else x1
    b = x2.T if t2 and x2.ndim == 2 else x2
    m = x1.shape[-1] if t1 else x1.shape[-2]
    n = x2.shape[-2] if t2 else x2.shape[-1]
    batched = x1.ndim > 2 or x2.ndim > 2
    if per_tile:
        y = G["qbmmv4"].compute_per_tile(x1, x2, x1s, x2s, bias, t1, t2, group, out)
    elif batched:
        nb = max(x1.shape[0] if x1.ndim > 2 else 1, x2.shape[0] if x2.ndim > 2 else 1)
        outs = []
        for i in range(nb):  # the reference golden cannot take 4-D mx scales: call it per batch
            pick = lambda t, core: t if (t is None or t.ndim <= core) else t[i if t.shape[0] > 1 else 0]
            mx = x2s.dtype == np.dtype(E8M0)
            pb = (not mx) and x1s is not None and x1s.ndim > 1
            sc_core = 3 if mx else (2 if pb else 1)
            outs.append(ref.qbmmv3_kernel_compute(pick(x1, 2), pick(x2, 2), pick(x2s, sc_core), None,
                                                  bias if bias is None or bias.ndim == 1 else bias[i, 0],
                                                  pick(x1s, sc_core), output_shapes=[(m, n)], **kw)[0])
        y = np.stack(outs)
    else:
        if x2s_u64 is not None:
            y = ref.QuantBatchMatmulV3TestSpec.golden(x1, x2, x2s_u64, offset, bias, x1s, output_shapes=[(m, n)],
                                                      scale_dtype="uint64", **kw)[0]
        else:
            y = ref.qbmmv3_kernel_compute(x1, x2, x2s, None, bias, x1s, output_shapes=[(m, n)], **kw)[0]
    if check_oracle:
        yo = qbmm_oracle.quant_matmul_v5(x1, x2, x1s, x2s_u64 if x2s_u64 is not None else x2s, bias, t1, t2, group, out,
                                         x2_scale_is_u64=x2s_u64 is not None, x2_offset=offset)
        assert bits_equal(y, yo), "oracle != reference for " + name
    save("qmm_" + name, dict(x1=x1, x2=x2, x1_scale=x1s, x2_scale=x2s_u64 if x2s_u64 is not None else x2s, bias=bias, out=y,
                             x2_offset=offset),
         dict(op="quant_matmul_v5", transpose_x1=t1, transpose_x2=t2, group_size=group if api_group is None else api_group,
              out_dtype=out, seed=seed, note=note))


def a8w4_case(G, name, seed, x1, x2, x1s, x2s, ys, bias, out, note):
    """fp8 x fp4 through the V4 golden's entry (mx when the scales are e8m0, T-CG when x2Scale is bf16/fp16 + yScale);
    x2 is stored (n,k) (transposeX2 = true), groupSizeK 32, as the API demands for these modes."""
    y = G["qbmmv4"].qbmmv4_kernel_compute(x1, x2, bias, x1s, x2s, ys, transpose_x1=False, transpose_x2=True, group_size=32,
                                          output_dtypes=[out])
    y = y[0] if isinstance(y, (list, tuple)) else y
    yo = qbmm_oracle.quant_matmul_v5(x1, x2, x1s, x2s, None if bias is None else bias.reshape(-1), False, True, 32, out,
                                     y_scale=ys)
    assert bits_equal(y, yo), "oracle != reference for " + name
    save("qmm_" + name, dict(x1=x1, x2=x2, x1_scale=x1s, x2_scale=x2s, y_scale=ys, bias=bias, out=y),
         dict(op="quant_matmul_v5", transpose_x1=False, transpose_x2=True, group_size=32, out_dtype=out, seed=seed, note=note))


def gen_qmm(G):
    i8 = lambda rng, shape: rng.integers(-127, 128, shape, dtype=np.int8)
    f32 = lambda rng, shape, lo=1e-3, hi=1e-2: rng.uniform(lo, hi, shape).astype(np.float32)

    rng = np.random.default_rng(11)
    qmm_case(G, "kc_int8_bf16", 11, i8(rng, (128, 256)), i8(rng, (256, 512)), f32(rng, (128,)), f32(rng, (512,)),
             rng.integers(-1000, 1001, (512,)).astype(np.int32), False, False, 0, "bfloat16",
             "ttk_aclnn_quant_batch_matmul_v5_st.csv v3_kc_int8_fp32 shape, int32 bias, bf16 out")
    rng = np.random.default_rng(12)
    qmm_case(G, "kc_int8_fp16_transA", 12, i8(rng, (811, 131)), i8(rng, (811, 160)), f32(rng, (131,)), f32(rng, (160,)),
             None, True, False, 0, "float16", "ttk_kernel_quant_batch_matmul_v3_st.csv qbmm_KC_case0001")
    rng = np.random.default_rng(13)
    qmm_case(G, "kc_int8_bf16scale_transB", 13, i8(rng, (679, 149)), i8(rng, (238, 149)), f32(rng, (679,)),
             f32(rng, (238,)).astype(BF16), None, False, True, 0, "bfloat16", "qbmm_KC_case0003 (bf16 channel scale)")
    rng = np.random.default_rng(14)
    qmm_case(G, "kc_int8_fbias", 14, i8(rng, (332, 348)), i8(rng, (304, 348)), f32(rng, (332,)), f32(rng, (304,)),
             rng.uniform(-1, 1, (304,)).astype(np.float32), False, True, 0, "bfloat16",
             "qbmm_KC_case0014 scaled down: float bias after dequant")
    rng = np.random.default_rng(15)
    qmm_case(G, "tc_int8_bf16scale_transA", 15, i8(rng, (257, 447)), i8(rng, (257, 941)), None,
             f32(rng, (941,)).astype(BF16), None, True, False, 0, "bfloat16", "qbmm_TC_case0005")
    rng = np.random.default_rng(16)
    qmm_case(G, "tt_int8_bf16scale_transA", 16, i8(rng, (691, 272)), i8(rng, (691, 592)), None,
             f32(rng, (1,)).astype(BF16), None, True, False, 0, "bfloat16", "qbmm_TT_case0005 (19-bit scale truncation)")
    rng = np.random.default_rng(17)
    qmm_case(G, "tt_int8_fbias_longk", 17, i8(rng, (44, 8192)), i8(rng, (8192, 144)), None, f32(rng, (1,)),
             rng.uniform(-1, 1, (144,)).astype(np.float32), False, False, 0, "bfloat16",
             "qbmm_streamk_tt_int8_fp32_fp32_bias_nd")
    rng = np.random.default_rng(18)
    sc = rng.uniform(-1e-2, 1e-2, (16,)).astype(np.float32)
    u64 = (np.ascontiguousarray(sc).view(np.uint32) & np.uint32(0xFFFFE000)).astype(np.uint64)
    qmm_case(G, "tc_int8_u64scale_fp16", 18, i8(rng, (16, 32)), i8(rng, (32, 16)), None, None,
             rng.integers(-1000, 1001, (16,)).astype(np.int32), False, False, 0, "float16",
             "test_aclnn_quant_matmul_v5_api.csv A8W8FP16_perchannel: fixpipe-packed uint64 scale", x2s_u64=u64)
    rng = np.random.default_rng(19)
    qmm_case(G, "tc_int8_int32out", 19, i8(rng, (100, 200)), i8(rng, (200, 72)), None, f32(rng, (72,)),
             rng.integers(-1000, 1001, (72,)).astype(np.int32), False, False, 0, "int32", "int32 accumulator + bias out")
    # fp8 per-block
    rng = np.random.default_rng(20)
    qmm_case(G, "gb_fp8_bf16", 20, q_fp8(rng, (200, 384), E4M3), q_fp8(rng, (384, 300), E4M3), f32(rng, (200, 3), .5, 2),
             f32(rng, (3, 3), .5, 2), None, False, False, (1 << 32) | (128 << 16) | 128, "bfloat16",
             "G-B per-block, tails in m and n")
    rng = np.random.default_rng(21)
    qmm_case(G, "bb_fp8_fp16_transB", 21, q_fp8(rng, (300, 283), E4M3), q_fp8(rng, (261, 283), E5M2),
             f32(rng, (3, 3), .5, 2), f32(rng, (3, 3), .5, 2), None, False, True, (128 << 32) | (128 << 16) | 128, "float16",
             "qbmm_BB_case scaled down: B-B, e4m3 x e5m2, tails in every dim, x2 stored (n,k)")
    rng = np.random.default_rng(22)
    qmm_case(G, "bb_fp8_fp16_transA", 22, q_fp8(rng, (283, 300), E5M2), q_fp8(rng, (283, 261), E4M3),
             f32(rng, (3, 3), .5, 2), f32(rng, (3, 3), .5, 2), None, True, False, (128 << 32) | (128 << 16) | 128, "float16",
             "B-B with x1 stored (k,m): scales are stored (k/128, m/128)")
    # int8 per-block (the V4 golden's PER_TILE mode)
    gb = (1 << 32) | (128 << 16) | 128
    rng = np.random.default_rng(40)
    qmm_case(G, "pt_int8_bf16", 40, i8(rng, (200, 384)), i8(rng, (384, 300)), f32(rng, (200, 3), 1e-3, 1e-2),
             f32(rng, (3, 3), 1e-2, 1e-1), None, False, False, gb, "bfloat16", "int8 G-B per-block, tails in m and n",
             per_tile=True)
    rng = np.random.default_rng(41)
    qmm_case(G, "pt_int8_bf16_bias_transB", 41, i8(rng, (77, 300)), i8(rng, (261, 300)), f32(rng, (77, 3), 1e-3, 1e-2),
             f32(rng, (3, 3), 1e-2, 1e-1), rng.standard_normal(261).astype(np.float32), False, True, gb, "bfloat16",
             "int8 G-B per-block, x2 stored (n,k) with scales (n/128,k/128), k tail, fp32 bias", per_tile=True)
    rng = np.random.default_rng(42)
    qmm_case(G, "pt_int8_fp16_big", 42, i8(rng, (384, 1024)), i8(rng, (512, 1024)), f32(rng, (384, 8), 1e-3, 1e-2),
             f32(rng, (4, 8), 1e-2, 1e-1), None, False, True, gb, "float16", "int8 G-B per-block, whole tiles",
             per_tile=True)
    # int4 x int4 (per-token x per-channel and per-tensor with a packed scale): same integer arithmetic as int8
    i4 = lambda rng, shape: rng.integers(-8, 8, shape).astype(np.int8).astype(INT4)
    rng = np.random.default_rng(70)
    qmm_case(G, "kc_int4_bf16_transB", 70, i4(rng, (77, 512)), i4(rng, (200, 512)), f32(rng, (77,)), f32(rng, (200,)),
             rng.integers(-100, 101, 200).astype(np.int32), False, True, 0, "bfloat16",
             "int4 x int4 per-token x per-channel, x2 stored (n,k), int32 bias")
    rng = np.random.default_rng(71)
    qmm_case(G, "kc_int4_fp16", 71, i4(rng, (130, 256)), i4(rng, (256, 320)), f32(rng, (130,)), f32(rng, (320,)), None, False, False,
             0, "float16", "int4 x int4, x2 stored (k,n): packed along n")
    # int4 x int4 asymmetric per-group (the V4 golden's INT4_ASYMMETRICAL mode): k % 1024 == 0, n % 256 == 0, x2 stored (n,k)
    rng = np.random.default_rng(72)
    m, k, n = 50, 1024, 256
    x1, x2 = i4(rng, (m, k)), i4(rng, (n, k))
    x1s = f32(rng, (m, 1))
    x2s = f32(rng, (k // 256, n), 1e-2, 1e-1)
    x2o = rng.uniform(-4, 4, (k // 256, n)).astype(np.float16)
    y = G["qbmmv4"].compute_int4_asymmetrical(x1, x2, x1s, x2s, x2o, False, True, "bfloat16")
    yo = qbmm_oracle.quant_matmul_v5(x1, x2, x1s, x2s, None, False, True, 256, "bfloat16", x2_offset=x2o)
    assert bits_equal(y, yo), "oracle != reference for kg_int4_asym"
    save("qmm_kg_int4_asym_bf16", dict(x1=x1, x2=x2, x1_scale=x1s, x2_scale=x2s, x2_offset=x2o, out=y),
         dict(op="quant_matmul_v5", transpose_x1=False, transpose_x2=True, group_size=256, out_dtype="bfloat16", seed=72,
              note="INT4 x INT4 per-group asymmetric: x1Scale (m,1), x2Scale / x2Offset (k/256, n)"))
    # int8 requantised output: uint64 scale = fp32 scale | 1 << 46 | s9 offset << 37 (matmul_quant_util.py:146-155)
    import matmul_quant_util as mqu  # on sys.path once the goldens are loaded
    rng = np.random.default_rng(60)
    sc = rng.uniform(2e-5, 6e-4, 300).astype(np.float32) * rng.choice([-1, 1], 300).astype(np.float32)
    qmm_case(G, "tc_int8_requant", 60, i8(rng, (77, 512)), i8(rng, (512, 300)), None, None,
             rng.integers(-20000, 20001, 300).astype(np.int32), False, False, 0, "int8",
             "int8 output, per-channel packed scale, int32 bias, no offset", x2s_u64=mqu.pack_u64_scale(sc))
    rng = np.random.default_rng(61)
    sc = rng.uniform(2e-5, 6e-5, 208).astype(np.float32)
    off = rng.uniform(-60, 60, 208).astype(np.float32)
    qmm_case(G, "tc_int8_requant_offset_transB", 61, i8(rng, (130, 1040)), i8(rng, (208, 1040)), None, None, None, False, True,
             0, "int8", "int8 output with the 9-bit offset packed into the scale, x2 stored (n,k)",
             x2s_u64=mqu.pack_u64_scale(sc, off), offset=off)
    # A8W4: fp8 x fp4 (the V4 golden's MX and T_CG modes)
    def u64_scale(rng, n, lo, hi):
        sc = rng.uniform(lo, hi, (1, n)).astype(np.float32)
        return (np.ascontiguousarray(sc).view(np.uint32) & np.uint32(0xFFFFE000)).astype(np.uint64)

    rng = np.random.default_rng(50)
    a8w4_case(G, "a8w4_mx_bf16", 50, q_fp8(rng, (96, 256), E4M3), q_fp4(rng, (200, 256)), e8m0(rng, (96, 4, 2)),
              e8m0(rng, (200, 4, 2)), None, None, "bfloat16", "MxA8W4: e4m3 x e2m1, e8m0 scales per 32, tails in m and n")
    rng = np.random.default_rng(51)
    a8w4_case(G, "a8w4_mx_fp16_bias", 51, q_fp8(rng, (16, 128), E4M3), q_fp4(rng, (128, 128)), e8m0(rng, (16, 2, 2), -2, 2),
              e8m0(rng, (128, 2, 2), -2, 2), None, rng.standard_normal((1, 128)).astype(np.float16), "float16",
              "test_aclnn_quant_matmul_v5_api.csv MxA8W4_Bias_fp16: bias (1,n) in the output dtype")
    rng = np.random.default_rng(52)
    a8w4_case(G, "a8w4_tcg_fp16", 52, q_fp8(rng, (16, 64), E4M3), q_fp4(rng, (16, 64)), None,
              rng.uniform(0.25, 4, (16, 2)).astype(BF16), u64_scale(rng, 16, 0.01, 0.1), None, "float16",
              "test_aclnn_quant_matmul_v5_api.csv A8W4F_TCG_fp16_ok: bf16 group scale (n, k/32), uint64 yScale (1,n)")
    rng = np.random.default_rng(53)
    a8w4_case(G, "a8w4_tcg_bf16_f16scale", 53, q_fp8(rng, (150, 512), E4M3), q_fp4(rng, (272, 512)), None,
              rng.uniform(0.05, 8, (272, 16)).astype(np.float16), u64_scale(rng, 272, 0.01, 0.1), None, "bfloat16",
              "T-CG with an fp16 group scale, tails in m and n")
    # fp8 double scale / per-tensor
    rng = np.random.default_rng(23)
    qmm_case(G, "tt_fp8_doublescale_fp16", 23, q_fp8(rng, (48, 96), E4M3), q_fp8(rng, (96, 80), E4M3), f32(rng, (1,), .5, 2),
             f32(rng, (1,), .5, 2), None, False, False, 0, "float16", "T-T double scale: merged scale keeps 19 bits")
    rng = np.random.default_rng(24)
    qmm_case(G, "tc_fp8_doublescale_fbias", 24, q_fp8(rng, (48, 96), E5M2), q_fp8(rng, (96, 80), E5M2),
             f32(rng, (1,), .5, 2), f32(rng, (80,), .5, 2), rng.uniform(-1, 1, (80,)).astype(np.float32), False, False, 0,
             "bfloat16", "api csv FP8E5M2..dynamic_tc_bias_float")
    # mx
    rng = np.random.default_rng(25)
    qmm_case(G, "mxfp8_bias_bf16", 25, q_fp8(rng, (64, 256), E4M3), q_fp8(rng, (256, 96), E4M3), e8m0(rng, (64, 4, 2)),
             e8m0(rng, (4, 96, 2)), rng.uniform(-1, 1, (96,)).astype(np.float32), False, False, (1 << 32) | (1 << 16) | 32,
             "bfloat16", "mx fp8, x2 stored (k,n)")
    rng = np.random.default_rng(26)
    qmm_case(G, "mxfp8_transB_oddgroups", 26, q_fp8(rng, (70, 160), E4M3), q_fp8(rng, (90, 160), E5M2), e8m0(rng, (70, 3, 2)),
             e8m0(rng, (90, 3, 2)), None, False, True, (1 << 32) | (1 << 16) | 32, "float16",
             "k=160: 5 groups, the 6th scale is padding (groupSize must be explicit: 160 is not divisible by 6)")
    rng = np.random.default_rng(27)
    qmm_case(G, "mxfp4_transB_fp32", 27, q_fp4(rng, (197, 960)), q_fp4(rng, (154, 960)), e8m0(rng, (197, 15, 2)),
             e8m0(rng, (154, 15, 2)), None, False, True, (1 << 32) | (1 << 16) | 32, "float32",
             "qbmm_MXFP4_case0001 (n scaled down): k=960 = 30 groups")
    rng = np.random.default_rng(28)
    qmm_case(G, "mxfp4_bf16", 28, q_fp4(rng, (33, 128)), q_fp4(rng, (128, 72)), e8m0(rng, (33, 2, 2)), e8m0(rng, (2, 72, 2)),
             None, False, False, 0, "bfloat16", "mx fp4 with x2 stored (k,n); groupSize 0 is inferred as [1,1,32]")
    rng = np.random.default_rng(29)
    qmm_case(G, "mxfp8_batched_bias", 29, q_fp8(rng, (3, 40, 128), E4M3), q_fp8(rng, (3, 128, 56), E4M3),
             e8m0(rng, (3, 40, 2, 2)), e8m0(rng, (3, 2, 56, 2)), rng.uniform(-1, 1, (56,)).astype(np.float32), False, False,
             (1 << 32) | (1 << 16) | 32, "bfloat16", "batched mx (the reference golden is called per batch)")


# ------------------------------------------------------------------------------------------------------------
def wq_case(G, name, seed, x, w, scale, offset, bias, group, trans_w, note, packed=False):
    """w: integer values as stored ((k,n), or (n,k) when trans_w); scale/offset as stored (transposed with the weight)."""
    ref = G["wqbmmv2"]
    out_name = "bfloat16" if x.dtype == np.dtype(BF16) else "float16"
    wfloat = w.dtype != np.int8
    wt = w if wfloat else (w.astype(INT4) if np.abs(w).max() <= 8 and packed is not None and name.find("s8") < 0 else w)
    y = ref.wqbmm_kernel_compute(x, wt, scale, offset, None, None, bias, transpose_x=False, transpose_weight=trans_w,
                                 antiquant_group_size=group, output_dtypes=[out_name])[0]
    wk = w.T if trans_w else w
    sk = scale.T if (trans_w and scale.ndim == 2) else scale
    ok = None if offset is None else (offset.T if (trans_w and offset.ndim == 2) else offset)
    yo = wqbmm_oracle.weight_quant_batch_matmul(x, wk, sk, ok, bias, group)
    assert bits_equal(y, yo), "oracle != reference for " + name
    save("wq_" + name, dict(x=x, w=w, scale=scale, offset=offset, bias=bias, out=y),
         dict(op="weight_quant_batch_matmul_v2", group_size=group, transpose_weight=trans_w, seed=seed, note=note,
              w_is_int4=bool(name.find("s8") < 0) and not wfloat, packed_int32=bool(packed), w_float=bool(wfloat)))


def gen_wq(G):
    def xs(rng, shape, dt):
        return rng.standard_normal(shape).astype(np.float32).astype(dt)

    def sc(rng, shape, dt, lo=0.005, hi=0.02):
        return rng.uniform(lo, hi, shape).astype(np.float32).astype(dt)

    i4 = lambda rng, shape: rng.integers(-8, 8, shape).astype(np.int8)
    rng = np.random.default_rng(41)
    wq_case(G, "bf16_s4_group128_offset_m16", 41, xs(rng, (16, 512), BF16), i4(rng, (512, 256)), sc(rng, (4, 256), BF16),
            sc(rng, (4, 256), BF16, -1, 1), None, 128, False, "the decode benchmark configuration, scaled down", packed=True)
    rng = np.random.default_rng(42)
    wq_case(G, "bf16_s4_group160_m1_fbias", 42, xs(rng, (1, 384), BF16), i4(rng, (384, 576)), sc(rng, (3, 576), BF16), None,
            rng.uniform(-1, 1, (576,)).astype(np.float32), 160, False,
            "ttk_kernel_weight_quant_batch_matmul_v2_st.csv rdv_F16S4_g_nd_small_data_range (n scaled down)", packed=True)
    rng = np.random.default_rng(43)
    wq_case(G, "fp16_s8_group64_offset", 43, xs(rng, (30, 256), np.float16), rng.integers(-128, 128, (256, 512)).astype(np.int8),
            sc(rng, (4, 512), np.float16), sc(rng, (4, 512), np.float16, -1, 1), None, 64, False,
            "rdv_F16S8_g_nd_not_align (n scaled down)")
    rng = np.random.default_rng(44)
    wq_case(G, "fp16_s4_channel_offset_bias", 44, xs(rng, (4, 64), np.float16), i4(rng, (64, 384)), sc(rng, (384,), np.float16),
            sc(rng, (384,), np.float16, -1, 1), xs(rng, (384,), np.float16), 0, False, "rdv_F16S4_c_nd_normal family")
    rng = np.random.default_rng(45)
    wq_case(G, "fp16_s4_channel_transW", 45, xs(rng, (4, 64), np.float16), i4(rng, (272, 64)), sc(rng, (272,), np.float16),
            None, None, 0, True, "rdv_F16S4_c_nd_normal_02: weight stored (n,k)")
    rng = np.random.default_rng(46)
    wq_case(G, "bf16_s4_channel_offset_bias_m40", 46, xs(rng, (40, 640), BF16), i4(rng, (640, 768)), sc(rng, (768,), BF16),
            sc(rng, (768,), BF16, -1, 1), xs(rng, (768,), BF16), 0, False,
            "ttk_aclnn..basic_st.csv st_v2_bf16_s4_perchannel_offset_bias (m scaled down), int32-packed weight", packed=True)
    rng = np.random.default_rng(47)
    wq_case(G, "bf16_s8_tensor", 47, xs(rng, (9, 96), BF16), rng.integers(-128, 128, (96, 40)).astype(np.int8),
            sc(rng, (1,), BF16), None, None, 0, False, "per-tensor scale")
    rng = np.random.default_rng(48)
    wq_case(G, "fp16_s4_group64_bias_m8", 48, xs(rng, (8, 768), np.float16), i4(rng, (768, 576)), sc(rng, (12, 576), np.float16),
            None, xs(rng, (576,), np.float16), 64, False, "st_v2_fp16_s4_pergroup_bias (m scaled down)", packed=True)


    # fp8 / fp4 weights (A16F8, A16MXF4): same two roundings; mx = e8m0 scale per 32 rows, row count padded to even
    rng = np.random.default_rng(49)
    wq_case(G, "bf16_f8e4m3_channel_m20", 49, xs(rng, (20, 256), BF16), q_fp8(rng, (256, 320), E4M3), sc(rng, (320,), BF16),
            None, None, 0, False, "A16F8 per-channel (the API takes no offset with fp8 weights)")
    rng = np.random.default_rng(50)
    wq_case(G, "fp16_f8e4m3_group64_m4", 50, xs(rng, (4, 192), np.float16), q_fp8(rng, (192, 136), E4M3), sc(rng, (3, 136), np.float16),
            None, xs(rng, (136,), np.float16), 64, False, "A16F8 per-group, bias")
    rng = np.random.default_rng(51)
    wq_case(G, "bf16_mxfp4_m40", 51, xs(rng, (40, 192), BF16), q_fp4(rng, (192, 128)), e8m0(rng, (6, 128), -4, 1), None, None, 32, False,
            "A16MXF4: e2m1 weight, e8m0 scale per 32 rows (the golden itself only takes k that is a multiple of 64)")
    rng = np.random.default_rng(52)
    wq_case(G, "fp16_mxfp4_m3", 52, xs(rng, (3, 128), np.float16), q_fp4(rng, (128, 72)), e8m0(rng, (4, 72), -4, 1), None, None, 32, False,
            "A16MXF4 with fp16 activations")


# ------------------------------------------------------------------------------------------------------------
def gen_mxq(G):
    ref = G["mxquant"]
    cases = [("bf16_e4m3", 61, (16, 256), BF16, "float8_e4m3fn", 36, -1), ("bf16_e4m3_tail", 62, (5, 100), BF16, "float8_e4m3fn", 36, -1),
             ("fp16_e5m2", 63, (7, 192), np.float16, "float8_e5m2", 35, -1), ("bf16_e2m1", 64, (8, 128), BF16, "float4_e2m1", 40, -1),
             ("bf16_e4m3_outliers_3d", 65, (2, 6, 160), BF16, "float8_e4m3fn", 36, -1),
             # blocks along the second-to-last axis: what a (k, n) weight needs; scales come out as (k/64, n, 2)
             ("bf16_e4m3_axis0", 66, (256, 48), BF16, "float8_e4m3fn", 36, 0), ("fp16_e5m2_axis1_tail_3d", 67, (3, 100, 20), np.float16, "float8_e5m2", 35, -2),
             ("bf16_e2m1_axis0", 68, (96, 64), BF16, "float4_e2m1", 40, -2),
             # the other shared-exponent rule (scaleAlg 1, fp8) and the other fp4 rounding modes
             ("bf16_e4m3_alg1", 69, (9, 160), BF16, "float8_e4m3fn", 36, -1), ("fp16_e5m2_alg1", 70, (6, 96), np.float16, "float8_e5m2", 35, -1),
             ("bf16_e2m1_round", 71, (8, 128), BF16, "float4_e2m1", 40, -1), ("fp16_e2m1_floor", 72, (8, 128), np.float16, "float4_e2m1", 40, -1)]
    for name, seed, shape, dt, dst, code, axis in cases:
        alg = 1 if name.endswith("alg1") else 0
        rmode = "round" if name.endswith("round") else ("floor" if name.endswith("floor") else "rint")
        rng = np.random.default_rng(seed)
        x = rng.standard_normal(shape).astype(np.float32)
        if "outliers" in name:
            mask = rng.random(shape) < 0.01
            x = np.where(mask, x * 50, x)
            x[0, 0, :32] = 0.0  # an all-zero block
        x = x.astype(dt)
        y, scale = ref.dynamic_mx_quant_golden(x, axis=axis, round_mode=rmode, dst_type=code, blocksize=32, scale_alg=alg,
                                               output_dtypes=[dst, "float8_e8m0"])
        yo, so = mx_quant_oracle.dynamic_mx_quant(x, dst, axis=axis, scale_alg=alg, round_mode=rmode)
        assert bits_equal(np.asarray(y).view(np.uint8), yo.view(np.uint8)), "oracle != reference (y) for " + name
        assert bits_equal(np.asarray(scale).view(np.uint8), so), "oracle != reference (scale) for " + name
        save("mxq_" + name, dict(x=x, y=np.asarray(y), scale=np.asarray(scale)),
             dict(op="dynamic_mx_quant", dst=dst, axis=axis, scale_alg=alg, round_mode=rmode, seed=seed,
                  note="quant/dynamic_mx_quant golden"))


def gen_nz(G):
    """FRACTAL_NZ storage -> (k, n) by the reference's nz_to_nd (matmul_golden_util.py:76-114), on random storage contents
    (padding included), for the layout helper the aclnnWeightQuantBatchMatmulNz tests build their inputs with."""
    import matmul_golden_util as mgu  # on sys.path once the goldens are loaded

    rng = np.random.default_rng(80)
    for i, (k, n, k0, n0) in enumerate([(50, 70, 16, 32), (64, 128, 16, 64), (33, 40, 16, 8)]):
        nz = rng.integers(-128, 128, (-(-n // n0), -(-k // k0), k0, n0)).astype(np.int8)
        nd = mgu.nz_to_nd(nz, (k, n))
        assert bits_equal(nd, wqbmm_oracle.nz_to_nd(nz, (k, n)))
        assert bits_equal(mgu.nz_to_nd(wqbmm_oracle.nd_to_nz(nd, k0, n0), (k, n)), nd)
        save("nz_layout_%d" % i, dict(nz=nz, nd=nd), dict(op="nz_to_nd", k=k, n=n, k0=k0, n0=n0, seed=80))


if __name__ == "__main__":
    assert ref_loader.available(), "reference tree not found"
    G = ref_loader.goldens()
    gen_qmm(G)
    gen_wq(G)
    gen_mxq(G)
    gen_nz(G)
