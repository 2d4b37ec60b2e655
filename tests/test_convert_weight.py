"""aclnnConvertWeightToINT4Pack: argument rules on CPU (matmul/convert_weight_to_int4_pack/op_host/op_api/
aclnn_convert_weight_to_int4_pack.cpp:155-316 of the reference) and the packing kernel against the numpy restatement."""
import numpy as np
import pytest

from conftest import case_seed

from oracle import wqbmm_oracle


def test_argument_rules(aclnn):
    T = aclnn.Tensor
    cases = [
        (T((64, 128), "int32"), T((64, 16), "int32"), 0),
        (T((64, 128), "int32"), T((64, 128), "int4"), 0),
        (T((2, 64, 128), "int32"), T((2, 64, 16), "int32"), 0),
        (T((64, 128), "float32"), T((64, 128), "float4_e2m1"), 0),
        (T((64, 128), "float32"), T((64, 16), "float32"), 0),
        (T((64, 128), "int32"), T((64, 128), "float4_e2m1"), 161002),   # dtype pair
        (T((64, 128), "float16"), T((64, 16), "int32"), 161002),        # weight dtype
        (T((64, 100), "int32"), T((64, 12), "int32"), 161002),          # last dim not a multiple of 8
        (T((64, 127), "int32"), T((64, 127), "int4"), 161002),          # odd last dim
        (T((64, 128), "int32"), T((64, 15), "int32"), 161002),          # shape mismatch
        (T((128,), "int32"), T((16,), "int32"), 161002),                # rank
        (T((0, 128), "int32"), T((0, 16), "int32"), 161002),            # empty
    ]
    for w, p, want in cases:
        st, ws, ex = aclnn.convert_weight_to_int4_pack_get_workspace_size(w, p)
        assert st == want, (w.shape, p.shape, st, aclnn.last_error())
        if st == 0:
            assert ws == 0
            aclnn.destroy_executor(ex)
    st, _, _ = aclnn.convert_weight_to_int4_pack_get_workspace_size(None, T((64, 16), "int32"))
    assert st == 161001


def test_oracle_packing_matches_the_word_layout_the_matmul_reads():
    """Packing (k, n) int32 nibble values gives exactly the int32 words aclnnWeightQuantBatchMatmulV2 takes
    (element j of a word at bits 4j, matmul_quant_util.py:228-273 of the reference)."""
    rng = np.random.default_rng(3)
    w = rng.integers(-8, 8, (32, 64)).astype(np.int32)
    packed = wqbmm_oracle.convert_weight_to_b4_pack(w)
    assert np.array_equal(packed.view(np.int32), wqbmm_oracle.pack_int4_words(w.astype(np.int8)))
    assert np.array_equal(wqbmm_oracle.unpack_int4_words(packed.view(np.int32)), w.astype(np.int8))


@pytest.mark.gpu
@pytest.mark.parametrize("shape,src,dst", [((256, 512), "int32", "int32"), ((3, 40, 72), "int32", "int4"),
                                           ((130, 264), "float32", "float4_e2m1"), ((64, 128), "float32", "float32"),
                                           ((5, 6), "int32", "int4")])
def test_pack_kernel_matches_oracle(aclnn, shape, src, dst):
    import torch

    rng = np.random.default_rng(case_seed((shape, src, dst)))
    if src == "int32":
        w = rng.integers(-8, 8, shape).astype(np.int32)
        w[..., ::7] |= rng.integers(0, 1 << 20, w[..., ::7].shape).astype(np.int32) << 4  # bits above the nibble are ignored
    else:
        vals = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], dtype=np.float32)
        w = (vals[rng.integers(0, 8, shape)] * rng.choice([-1, 1], shape)).astype(np.float32)
        w.flat[::11] = 0.3  # not an e2m1 value: packs as code 0
    want = wqbmm_oracle.convert_weight_to_b4_pack(w)
    tw = torch.from_numpy(w).cuda()
    out = torch.full(want.shape, 0x5A, dtype=torch.uint8, device="cuda")
    pshape = shape if dst in ("int4", "float4_e2m1") else shape[:-1] + (shape[-1] // 8,)
    aclnn.convert_weight_to_int4_pack(aclnn.from_torch(tw), aclnn.Tensor(pshape, dst, out))
    torch.cuda.synchronize()
    assert aclnn.last_kernel_name() == "pack_b4"
    assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.gpu
def test_packed_weight_feeds_the_weight_quant_matmul(aclnn):
    """The reference's flow: quantised weight carried in int32 -> aclnnConvertWeightToINT4Pack -> aclnnWeightQuantBatchMatmulV2."""
    import ml_dtypes
    import torch

    from gpu_util import desc, out_tensor, out_to_np

    rng = np.random.default_rng(9)
    m, k, n, g = 8, 512, 256, 128
    x = rng.standard_normal((m, k)).astype(ml_dtypes.bfloat16)
    w = rng.integers(-8, 8, (k, n)).astype(np.int32)
    scale = rng.uniform(0.005, 0.02, (k // g, n)).astype(ml_dtypes.bfloat16)
    offset = rng.uniform(-1, 1, (k // g, n)).astype(ml_dtypes.bfloat16)
    want = wqbmm_oracle.weight_quant_batch_matmul(x, w.astype(np.int8), scale, offset, None, g)
    tw = torch.from_numpy(w).cuda()
    packed = torch.empty((k, n // 8), dtype=torch.int32, device="cuda")
    aclnn.convert_weight_to_int4_pack(aclnn.from_torch(tw), aclnn.from_torch(packed))
    y = out_tensor((m, n), "bfloat16")
    aclnn.weight_quant_batch_matmul(desc(aclnn, x), aclnn.from_torch(packed), desc(aclnn, scale), aclnn.Tensor((m, n), "bfloat16", y),
                                    desc(aclnn, offset), None, g)
    torch.cuda.synchronize()
    got = out_to_np(y).astype(np.float64)
    wv = want.astype(np.float64)
    assert np.all(np.abs(got - wv) <= 2.0 ** -7 * np.maximum(np.abs(wv), 0.05 * np.sqrt(np.mean(wv ** 2))) * 1.01)
