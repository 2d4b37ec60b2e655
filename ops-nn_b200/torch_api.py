"""torch-tensor entry points with the signatures of the torch-npu plugin functions that sit on top of these operators in the
reference's stack (`torch_npu.npu_quant_matmul`, `torch_npu.npu_weight_quant_batchmatmul`; call forms as exercised by
matmul/weight_quant_batch_matmul_v2/tests/assets/wqbmmv2_e2e_golden.py:196-275 of the reference). They take CUDA tensors,
allocate the output and the workspace with torch, and run the aclnn two-phase call on the current stream. Transposed weights
are passed the torch way, as `.t()` views: the library reads the strides, nothing is copied."""
from . import aclnn as _aclnn


def _torch():
    import torch

    return torch


def npu_quant_matmul(x1, x2, scale, *, offset=None, pertoken_scale=None, bias=None, output_dtype=None, group_sizes=None,
                     x1_dtype=None, x2_dtype=None, scale_dtype=None, pertoken_scale_dtype=None):
    """aclnnQuantMatmulV5 behind the torch-npu signature. x1 (.., m, k), x2 (.., k, n) (or a transposed view of (n, k));
    `scale` is x2's scale (per-tensor/-channel, per-block, or e8m0), `pertoken_scale` x1's; `group_sizes` = [gm, gn, gk].
    `x1_dtype` / `x2_dtype` / `scale_dtype` / `pertoken_scale_dtype` name the element type of tensors torch cannot type itself
    (e.g. "float4_e2m1" over uint8 storage, "float8_e8m0" scales); the logical last dim of a 4-bit tensor is twice its
    storage. output_dtype defaults to torch.int8 like the plugin (requantised output needs a packed int64 scale)."""
    torch = _torch()
    out_dtype = output_dtype if output_dtype is not None else torch.int8

    def describe(t, name):
        if t is None:
            return None
        if name in ("float4_e2m1", "int4"):
            shape = tuple(t.shape[:-1]) + (t.shape[-1] * 2,)
            strides = tuple(s * 2 for s in t.stride()[:-1]) + (1,)
            if t.dim() >= 2 and t.stride(-1) != 1:  # transposed view of packed storage: the packed axis is the second to last
                shape = tuple(t.shape[:-2]) + (t.shape[-2] * 2, t.shape[-1])
                strides = tuple(s * 2 for s in t.stride()[:-2]) + (1, t.stride(-1) * 2)
            return _aclnn.from_torch(t, name, shape, strides)
        return _aclnn.from_torch(t, name) if name is not None else _aclnn.from_torch(t)

    d_x1, d_x2 = describe(x1, x1_dtype), describe(x2, x2_dtype)
    m = d_x1.shape[-2]
    n = d_x2.shape[-1]
    batch = tuple(x1.shape[:-2]) if x1.dim() > 2 else (tuple(x2.shape[:-2]) if x2.dim() > 2 else ())
    out = torch.empty(batch + (m, n), dtype=out_dtype, device=x1.device)
    group = 0
    if group_sizes is not None:
        gm, gn, gk = (list(group_sizes) + [0, 0, 0])[:3]
        group = (int(gm) << 32) | (int(gn) << 16) | int(gk)
    _aclnn.quant_matmul_v5(d_x1, d_x2, describe(pertoken_scale, pertoken_scale_dtype), describe(scale, scale_dtype),
                           _aclnn.from_torch(out), _aclnn.from_torch(bias), False, False, group, x2_offset=_aclnn.from_torch(offset))
    return out


def npu_weight_quant_batchmatmul(x, weight, antiquant_scale, antiquant_offset=None, quant_scale=None, quant_offset=None,
                                 bias=None, antiquant_group_size=0, inner_precise=0, weight_dtype=None):
    """aclnnWeightQuantBatchMatmulV3 behind the torch-npu signature. x (m, k) bf16/fp16; weight (k, n) int8, or int32 words of
    eight int4 values (k, n / 8), or a `.t()` view of the (n, k) storage; scale/offset (n,), (1, n) or (k / group, n).
    quant_scale / quant_offset (int8 output) are not implemented and must be None."""
    torch = _torch()
    if quant_scale is not None or quant_offset is not None:
        raise NotImplementedError("quant_scale / quant_offset (int8 output) are not implemented")
    d_w = _aclnn.from_torch(weight, weight_dtype) if weight_dtype is not None else _aclnn.from_torch(weight)
    n = weight.shape[-1] * (8 if weight.dtype == torch.int32 and weight.stride(-1) == 1 else 1)
    y = torch.empty((x.shape[0], n), dtype=x.dtype, device=x.device)
    _aclnn.weight_quant_batch_matmul(_aclnn.from_torch(x), d_w, _aclnn.from_torch(antiquant_scale), _aclnn.from_torch(y),
                                     _aclnn.from_torch(antiquant_offset), _aclnn.from_torch(bias), int(antiquant_group_size),
                                     inner_precise=int(inner_precise))
    return y
