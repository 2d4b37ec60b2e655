"""ctypes bindings of the aclnn entry points exported by libopsnn_b200.so, plus torch-tensor conveniences.

Mirrors the reference's operator interface (names, argument order and meaning, status codes):
  aclnnQuantMatmulV5[GetWorkspaceSize]            matmul/quant_batch_matmul_v4/op_host/op_api/aclnn_quant_matmul_v5.h:43-60
  aclnnWeightQuantBatchMatmulV2/V3[GetWorkspaceSize]  matmul/weight_quant_batch_matmul_v2/op_host/op_api/*.h
  aclnnDynamicMxQuant[GetWorkspaceSize]           quant/dynamic_mx_quant/docs/aclnnDynamicMxQuant.md:76-95
  aclnnConvertWeightToINT4Pack[GetWorkspaceSize]  matmul/convert_weight_to_int4_pack/op_host/op_api/aclnn_convert_weight_to_int4_pack.h:30-45

There is no CPU or PyTorch fallback: if the shared library is missing, loading fails; if no CUDA device is present,
phase 2 fails with ACLNN_ERR_RUNTIME_ERROR.
"""
import ctypes
import os
from ctypes import POINTER, byref, c_bool, c_char_p, c_int, c_int32, c_int64, c_uint64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libopsnn_b200.so")

ACLNN_SUCCESS = 0
ACLNN_ERR_PARAM_NULLPTR = 161001
ACLNN_ERR_PARAM_INVALID = 161002
ACLNN_ERR_RUNTIME_ERROR = 361001
ACLNN_ERR_INNER_FIND_KERNEL_ERROR = 561003

STATUS_NAMES = {0: "ACLNN_SUCCESS", 161001: "ACLNN_ERR_PARAM_NULLPTR", 161002: "ACLNN_ERR_PARAM_INVALID",
                361001: "ACLNN_ERR_RUNTIME_ERROR", 561003: "ACLNN_ERR_INNER_FIND_KERNEL_ERROR"}

# aclDataType
ACL_FLOAT, ACL_FLOAT16, ACL_INT8, ACL_INT32, ACL_UINT8, ACL_INT64, ACL_UINT64 = 0, 1, 2, 3, 4, 9, 10
ACL_BF16, ACL_INT4, ACL_HIFLOAT8, ACL_FLOAT8_E5M2, ACL_FLOAT8_E4M3FN, ACL_FLOAT8_E8M0 = 27, 29, 34, 35, 36, 37
ACL_FLOAT4_E2M1, ACL_FLOAT4_E1M2 = 40, 41
DTYPE_BY_NAME = {"float32": 0, "float16": 1, "int8": 2, "int32": 3, "uint8": 4, "int64": 9, "uint64": 10, "bfloat16": 27,
                 "int4": 29, "hifloat8": 34, "float8_e5m2": 35, "float8_e4m3fn": 36, "float8_e8m0": 37,
                 "float4_e2m1": 40, "float4_e1m2": 41}
for _k, _v in list(DTYPE_BY_NAME.items()):
    DTYPE_BY_NAME["ACL_" + {"float32": "FLOAT", "bfloat16": "BF16"}.get(_k, _k.upper())] = _v
DTYPE_BITS = {0: 32, 1: 16, 2: 8, 3: 32, 4: 8, 9: 64, 10: 64, 27: 16, 29: 4, 34: 8, 35: 8, 36: 8, 37: 8, 40: 4, 41: 4}
ACL_FORMAT_ND, ACL_FORMAT_FRACTAL_NZ = 2, 29



class WqbmmParams(ctypes.Structure):
    """OpsnnWqbmmParams of include/opsnn_b200_kernels.h (the kernel-level C ABI below the aclnn layer)."""
    _fields_ = [("x_dtype", c_int32), ("w_dtype", c_int32), ("bias_dtype", c_int32), ("trans_w", c_int32),
                ("m", c_int64), ("n", c_int64), ("k", c_int64),
                ("x", c_void_p), ("x_ld", c_int64), ("w", c_void_p), ("w_ld", c_int64),
                ("scale", c_void_p), ("offset", c_void_p), ("group_size", c_int64), ("scale_sg", c_int64),
                ("scale_sn", c_int64), ("bias", c_void_p), ("y", c_void_p), ("y_ld", c_int64),
                ("workspace", c_void_p), ("workspace_size", c_uint64), ("inner_precise", c_int32),
                ("nz_k0", c_int32), ("nz_n0", c_int32), ("scale_dtype", c_int32), ("prep_w", c_void_p)]


_lib = None


def lib():
    """Loads the shared library (once). Raises if it has not been built: there is nothing to fall back to."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError("libopsnn_b200.so is not built (%s); run `python ops-nn_b200/build.py`" % LIB_PATH)
    L = ctypes.CDLL(LIB_PATH)
    P64 = POINTER(c_int64)
    L.aclCreateTensor.restype = c_void_p
    L.aclCreateTensor.argtypes = [P64, c_uint64, c_int, P64, c_int64, c_int, P64, c_uint64, c_void_p]
    L.aclDestroyTensor.argtypes = [c_void_p]
    L.aclDestroyAclOpExecutor.argtypes = [c_void_p]
    L.aclGetRecentErrMsg.restype = c_char_p
    T = c_void_p
    L.aclnnQuantMatmulV5GetWorkspaceSize.argtypes = [T, T, T, T, T, T, T, T, T, c_bool, c_bool, c_int64, T,
                                                      POINTER(c_uint64), POINTER(c_void_p)]
    L.aclnnQuantMatmulWeightNzGetWorkspaceSize.argtypes = L.aclnnQuantMatmulV5GetWorkspaceSize.argtypes
    L.aclnnWeightQuantBatchMatmulV2GetWorkspaceSize.argtypes = [T, T, T, T, T, T, T, c_int, T, POINTER(c_uint64),
                                                                 POINTER(c_void_p)]
    L.aclnnWeightQuantBatchMatmulV3GetWorkspaceSize.argtypes = [T, T, T, T, T, T, T, c_int, c_int, T, POINTER(c_uint64),
                                                                 POINTER(c_void_p)]
    L.aclnnWeightQuantBatchMatmulNzGetWorkspaceSize.argtypes = [T, T, T, T, T, T, T, c_int, T, POINTER(c_uint64),
                                                                 POINTER(c_void_p)]
    L.aclnnDynamicMxQuantGetWorkspaceSize.argtypes = [T, c_int64, c_char_p, c_int64, c_int64, c_int64, T, T,
                                                       POINTER(c_uint64), POINTER(c_void_p)]
    L.aclnnConvertWeightToINT4PackGetWorkspaceSize.argtypes = [T, T, POINTER(c_uint64), POINTER(c_void_p)]
    L.aclnnQuantMatmulV4GetWorkspaceSize.argtypes = [T, T, T, T, T, T, c_bool, c_bool, T, POINTER(c_uint64), POINTER(c_void_p)]
    L.aclnnQuantMatmulV3GetWorkspaceSize.argtypes = [T, T, T, T, T, c_bool, c_bool, T, POINTER(c_uint64), POINTER(c_void_p)]
    for name in ("aclnnQuantMatmulV5", "aclnnQuantMatmulWeightNz", "aclnnQuantMatmulV4", "aclnnQuantMatmulV3", "aclnnWeightQuantBatchMatmulV2",
                 "aclnnWeightQuantBatchMatmulV3", "aclnnWeightQuantBatchMatmulNz", "aclnnDynamicMxQuant",
                 "aclnnConvertWeightToINT4Pack"):
        getattr(L, name).argtypes = [c_void_p, c_uint64, c_void_p, c_void_p]
        getattr(L, name).restype = c_int32
        getattr(L, name + "GetWorkspaceSize").restype = c_int32
    L.opsnn_launch_count.restype = c_uint64
    L.opsnn_qmm_umma_status.restype = ctypes.c_uint32
    L.opsnn_qmm_umma_status.argtypes = [c_int32]
    L.opsnn_wqbmm_decode_status.restype = ctypes.c_uint32
    L.opsnn_wqbmm_decode_status.argtypes = [c_int32]
    L.opsnn_wqbmm_decode_last_plan.restype = None
    L.opsnn_wqbmm_decode_last_plan.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    L.opsnn_last_kernel_name.restype = c_char_p
    for name in ("opsnn_wqbmm_launch", "opsnn_wqbmm_decode_static_launch"):
        getattr(L, name).restype = c_int32
    L.opsnn_wqbmm_launch.argtypes = [POINTER(WqbmmParams), c_int32, c_void_p]
    L.opsnn_wqbmm_decode_static_launch.argtypes = [POINTER(WqbmmParams), c_void_p]
    L.opsnn_wqbmm_workspace_size.restype = c_uint64
    L.opsnn_wqbmm_workspace_size.argtypes = [POINTER(WqbmmParams), c_int32]
    L.opsnn_wqbmm_select_kernel.restype = c_int32
    L.opsnn_wqbmm_select_kernel.argtypes = [POINTER(WqbmmParams)]
    L.opsnnQuantMatmulPrepareX2GetStorageSize.argtypes = [T, T, c_bool, c_int64, c_int64, POINTER(c_uint64)]
    L.opsnnQuantMatmulPrepareX2.argtypes = [T, T, c_bool, c_int64, c_int64, c_void_p, c_uint64, c_void_p]
    L.opsnnQuantMatmulReleaseX2.argtypes = [T]
    L.opsnnWeightQuantPrepareGetStorageSize.argtypes = [T, T, T, c_int32, c_int32, POINTER(c_uint64)]
    L.opsnnWeightQuantPrepare.argtypes = [T, T, T, c_int32, c_int32, c_void_p, c_uint64, c_void_p]
    L.opsnnWeightQuantRelease.argtypes = [T]
    for name in ("opsnnQuantMatmulPrepareX2GetStorageSize", "opsnnQuantMatmulPrepareX2", "opsnnQuantMatmulReleaseX2",
                 "opsnnWeightQuantPrepareGetStorageSize", "opsnnWeightQuantPrepare", "opsnnWeightQuantRelease"):
        getattr(L, name).restype = c_int32
    L.opsnn_probe_umma.argtypes = [c_int32, c_int32, POINTER(ctypes.c_double)]
    L.opsnn_probe_mix.argtypes = [c_int32, POINTER(ctypes.c_double)]
    L.opsnn_probe_tmem_read.argtypes = [c_int32, c_int32, POINTER(ctypes.c_double)]
    L.opsnn_probe_umma.restype = L.opsnn_probe_mix.restype = L.opsnn_probe_tmem_read.restype = c_int32
    I64, I32, U64, VP = c_int64, c_int32, c_uint64, c_void_p
    L.opsnn_shard_range.restype = None
    L.opsnn_shard_range.argtypes = [I64, I32, I32, I64, POINTER(I64), POINTER(I64)]
    L.opsnn_comm_unique_id.argtypes = [VP]
    L.opsnn_comm_init.argtypes = [VP, I32, I32, POINTER(VP)]
    L.opsnn_comm_destroy.argtypes = [VP]
    L.opsnn_gather_columns_workspace.restype = U64
    L.opsnn_gather_columns_workspace.argtypes = [I32, I64, I64, I64, I32]
    L.opsnn_gather_columns.argtypes = [VP, VP, I64, I64, I64, I64, I32, VP, VP, U64, VP]
    L.opsnn_gather_batch.argtypes = [VP, VP, I64, U64, VP, VP]
    L.opsnn_comm_symmetric_alloc.argtypes = [VP, U64, POINTER(VP), POINTER(VP)]
    L.opsnn_comm_symmetric_free.argtypes = [VP, VP]
    L.opsnn_comm_bind_columns.argtypes = [VP, VP, VP, I64, I64]
    L.opsnn_comm_unbind.argtypes = [VP]
    L.opsnn_comm_arrive_and_wait.argtypes = [VP, VP]
    L.opsnn_comm_allgather_columns.argtypes = [VP, VP, I64, I64, VP, I64, I64, I32, VP]
    L.opsnn_comm_allgather_columns.restype = c_int32
    L.opsnn_comm_status.argtypes = [VP, I32]
    L.opsnn_comm_status.restype = ctypes.c_uint32
    for name in ("opsnn_comm_symmetric_alloc", "opsnn_comm_symmetric_free", "opsnn_comm_bind_columns", "opsnn_comm_unbind",
                 "opsnn_comm_arrive_and_wait"):
        getattr(L, name).restype = c_int32
    for name in ("opsnn_comm_unique_id", "opsnn_comm_init", "opsnn_comm_destroy", "opsnn_gather_columns", "opsnn_gather_batch"):
        getattr(L, name).restype = c_int32
    _lib = L
    return L


def last_error():
    return lib().aclGetRecentErrMsg().decode()


def launch_count():
    return int(lib().opsnn_launch_count())


def last_kernel_name():
    return lib().opsnn_last_kernel_name().decode()


def last_decode_plan():
    """(strips, k-ranges per strip, 1 if the k-ranges ran as one thread-block cluster) of this thread's last streaming decode launch."""
    v = (c_int32 * 3)()
    base = ctypes.addressof(v)
    lib().opsnn_wqbmm_decode_last_plan(base, base + 4, base + 8)
    return int(v[0]), int(v[1]), int(v[2])


class AclnnError(RuntimeError):
    def __init__(self, api, status):
        self.status = status
        super().__init__("%s returned %s (%d): %s" % (api, STATUS_NAMES.get(status, "?"), status, last_error()))


class Tensor:
    """An aclTensor descriptor. `data` is a device address (int) or a torch tensor whose storage backs the view."""

    def __init__(self, shape, dtype, data=0, strides=None, offset=0, fmt=ACL_FORMAT_ND, storage_shape=None):
        self.shape = tuple(int(s) for s in shape)
        self.dtype = DTYPE_BY_NAME[dtype] if isinstance(dtype, str) else int(dtype)
        self._keep = data
        ptr = data if isinstance(data, int) else (data.data_ptr() if data is not None else 0)
        n = len(self.shape)
        dims = (c_int64 * max(n, 1))(*self.shape)
        st = None if strides is None else (c_int64 * max(n, 1))(*[int(s) for s in strides])
        sshape = self.shape if storage_shape is None else tuple(storage_shape)
        sd = (c_int64 * max(len(sshape), 1))(*sshape)
        self.handle = lib().aclCreateTensor(dims, n, self.dtype, st, int(offset), int(fmt), sd, len(sshape), c_void_p(ptr))
        if not self.handle:
            raise ValueError("aclCreateTensor rejected the arguments")

    def __del__(self):
        try:
            if getattr(self, "handle", None):
                lib().aclDestroyTensor(c_void_p(self.handle))
                self.handle = None
        except Exception:
            pass


def _h(t):
    return None if t is None else c_void_p(t.handle)


def _torch_dtype_code(t):
    import torch

    m = {torch.float32: ACL_FLOAT, torch.float16: ACL_FLOAT16, torch.bfloat16: ACL_BF16, torch.int8: ACL_INT8,
         torch.int32: ACL_INT32, torch.uint8: ACL_UINT8, torch.int64: ACL_INT64}
    for name, code in (("float8_e4m3fn", ACL_FLOAT8_E4M3FN), ("float8_e5m2", ACL_FLOAT8_E5M2), ("uint64", ACL_UINT64)):
        if hasattr(torch, name):
            m[getattr(torch, name)] = code
    return m[t.dtype]


def from_torch(t, dtype=None, shape=None, strides=None):
    """Descriptor over a torch tensor's memory. `dtype`/`shape` override the torch view for types torch lacks
    (e.g. a uint8 tensor of packed fp4 described as ACL_FLOAT4_E2M1 with twice the inner extent)."""
    if t is None:
        return None
    code = _torch_dtype_code(t) if dtype is None else (DTYPE_BY_NAME[dtype] if isinstance(dtype, str) else dtype)
    if shape is None:
        shape, strides = tuple(t.shape), tuple(t.stride())
    return Tensor(shape, code, t, strides)


def _stream():
    import torch

    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _workspace(nbytes, like):
    import torch

    if nbytes == 0:
        return None, c_void_p(0)
    ws = torch.empty(int(nbytes), dtype=torch.uint8, device=like.device)
    return ws, c_void_p(ws.data_ptr())


# ---- phase-1-only helpers (return the raw status; used by the argument-validation tests) -----------------------

def quant_matmul_v5_get_workspace_size(x1, x2, x1_scale, x2_scale, y_scale, x1_offset, x2_offset, y_offset, bias,
                                       transpose_x1, transpose_x2, group_size, out, weight_nz=False):
    ws, ex = c_uint64(0), c_void_p(0)
    fn = lib().aclnnQuantMatmulWeightNzGetWorkspaceSize if weight_nz else lib().aclnnQuantMatmulV5GetWorkspaceSize
    st = fn(_h(x1), _h(x2), _h(x1_scale), _h(x2_scale), _h(y_scale), _h(x1_offset),
                                                  _h(x2_offset), _h(y_offset), _h(bias), bool(transpose_x1),
                                                  bool(transpose_x2), int(group_size), _h(out), byref(ws), byref(ex))
    return st, ws.value, ex


def quant_matmul_v4(x1, x2, scale, out, offset=None, pertoken_scale=None, bias=None, transpose_x1=False, transpose_x2=False,
                    api="v4"):
    """Runs aclnnQuantMatmulV4 (or V3 with api="v3": no per-token scale) on the current torch CUDA stream: the older entry
    points of the same operator, argument order (scale, offset, pertokenScale, bias)."""
    ws, ex = c_uint64(0), c_void_p(0)
    L = lib()
    if api == "v3":
        st = L.aclnnQuantMatmulV3GetWorkspaceSize(_h(x1), _h(x2), _h(scale), _h(offset), _h(bias), bool(transpose_x1),
                                                  bool(transpose_x2), _h(out), byref(ws), byref(ex))
        name, run = "aclnnQuantMatmulV3", L.aclnnQuantMatmulV3
    else:
        st = L.aclnnQuantMatmulV4GetWorkspaceSize(_h(x1), _h(x2), _h(scale), _h(offset), _h(pertoken_scale), _h(bias),
                                                  bool(transpose_x1), bool(transpose_x2), _h(out), byref(ws), byref(ex))
        name, run = "aclnnQuantMatmulV4", L.aclnnQuantMatmulV4
    if st != ACLNN_SUCCESS:
        raise AclnnError(name + "GetWorkspaceSize", st)
    keep, wp = _workspace(ws.value, out._keep)
    st = run(wp, c_uint64(ws.value), ex, _stream())
    if st != ACLNN_SUCCESS:
        raise AclnnError(name, st)
    return ws.value


def weight_quant_batch_matmul_get_workspace_size(x, weight, antiquant_scale, antiquant_offset, quant_scale, quant_offset,
                                                 bias, antiquant_group_size, y, inner_precise=None):
    ws, ex = c_uint64(0), c_void_p(0)
    L = lib()
    if inner_precise == "nz":
        st = L.aclnnWeightQuantBatchMatmulNzGetWorkspaceSize(_h(x), _h(weight), _h(antiquant_scale), _h(antiquant_offset),
                                                             _h(quant_scale), _h(quant_offset), _h(bias),
                                                             int(antiquant_group_size), _h(y), byref(ws), byref(ex))
    elif inner_precise is None:
        st = L.aclnnWeightQuantBatchMatmulV2GetWorkspaceSize(_h(x), _h(weight), _h(antiquant_scale), _h(antiquant_offset),
                                                             _h(quant_scale), _h(quant_offset), _h(bias),
                                                             int(antiquant_group_size), _h(y), byref(ws), byref(ex))
    else:
        st = L.aclnnWeightQuantBatchMatmulV3GetWorkspaceSize(_h(x), _h(weight), _h(antiquant_scale), _h(antiquant_offset),
                                                             _h(quant_scale), _h(quant_offset), _h(bias),
                                                             int(antiquant_group_size), int(inner_precise), _h(y),
                                                             byref(ws), byref(ex))
    return st, ws.value, ex


def destroy_executor(ex):
    if ex is not None and ex.value:
        lib().aclDestroyAclOpExecutor(ex)


# ---- both phases on device tensors -------------------------------------------------------------------------------

def quant_matmul_v5(x1, x2, x1_scale, x2_scale, out, bias=None, transpose_x1=False, transpose_x2=False, group_size=0,
                    x2_offset=None, workspace=None, y_scale=None, weight_nz=False):
    """Runs aclnnQuantMatmulV5 (aclnnQuantMatmulWeightNz with weight_nz: x2 described as FRACTAL_NZ) on the current torch CUDA
    stream. Arguments are `Tensor` descriptors over device memory; `out` is written in place. Returns the workspace size used."""
    st, ws_size, ex = quant_matmul_v5_get_workspace_size(x1, x2, x1_scale, x2_scale, y_scale, None, x2_offset, None, bias,
                                                         transpose_x1, transpose_x2, group_size, out, weight_nz)
    if st != ACLNN_SUCCESS:
        raise AclnnError("aclnnQuantMatmul%sGetWorkspaceSize" % ("WeightNz" if weight_nz else "V5"), st)
    if workspace is not None and workspace.numel() >= ws_size:
        keep, wp = workspace, c_void_p(workspace.data_ptr())
    else:
        keep, wp = _workspace(ws_size, out._keep)
    run = lib().aclnnQuantMatmulWeightNz if weight_nz else lib().aclnnQuantMatmulV5
    st = run(wp, c_uint64(ws_size if keep is None else keep.numel()), ex, _stream())
    if st != ACLNN_SUCCESS:
        raise AclnnError("aclnnQuantMatmul%s" % ("WeightNz" if weight_nz else "V5"), st)
    return ws_size


def weight_quant_batch_matmul(x, weight, antiquant_scale, y, antiquant_offset=None, bias=None, antiquant_group_size=0,
                              inner_precise=None, workspace=None):
    """Runs aclnnWeightQuantBatchMatmulV2 (V3 when `inner_precise` is 0 / 1, the Nz entry point when it is "nz") on the current
    torch CUDA stream."""
    st, ws_size, ex = weight_quant_batch_matmul_get_workspace_size(x, weight, antiquant_scale, antiquant_offset, None, None,
                                                                   bias, antiquant_group_size, y, inner_precise)
    api = "aclnnWeightQuantBatchMatmulNz" if inner_precise == "nz" else (
        "aclnnWeightQuantBatchMatmulV2" if inner_precise is None else "aclnnWeightQuantBatchMatmulV3")
    if st != ACLNN_SUCCESS:
        raise AclnnError(api + "GetWorkspaceSize", st)
    if workspace is not None and workspace.numel() >= ws_size:
        keep, wp = workspace, c_void_p(workspace.data_ptr())
    else:
        keep, wp = _workspace(ws_size, y._keep)
    st = getattr(lib(), api)(wp, c_uint64(ws_size if keep is None else keep.numel()), ex, _stream())
    if st != ACLNN_SUCCESS:
        raise AclnnError(api, st)
    return ws_size


def convert_weight_to_int4_pack_get_workspace_size(weight, weight_int4_pack):
    ws, ex = c_uint64(0), c_void_p(0)
    st = lib().aclnnConvertWeightToINT4PackGetWorkspaceSize(_h(weight), _h(weight_int4_pack), byref(ws), byref(ex))
    return st, ws.value, ex


def convert_weight_to_int4_pack(weight, weight_int4_pack):
    """Runs aclnnConvertWeightToINT4Pack on the current torch CUDA stream: one 4-bit value per 32-bit element of `weight`
    -> two per byte in `weight_int4_pack`."""
    st, _, ex = convert_weight_to_int4_pack_get_workspace_size(weight, weight_int4_pack)
    if st != ACLNN_SUCCESS:
        raise AclnnError("aclnnConvertWeightToINT4PackGetWorkspaceSize", st)
    st = lib().aclnnConvertWeightToINT4Pack(c_void_p(0), c_uint64(0), ex, _stream())
    if st != ACLNN_SUCCESS:
        raise AclnnError("aclnnConvertWeightToINT4Pack", st)


def dynamic_mx_quant(x, y_out, mxscale_out, dst_type, axis=-1, round_mode=b"rint", blocksize=32, scale_alg=0):
    ws, ex = c_uint64(0), c_void_p(0)
    code = DTYPE_BY_NAME[dst_type] if isinstance(dst_type, str) else dst_type
    st = lib().aclnnDynamicMxQuantGetWorkspaceSize(_h(x), int(axis), round_mode, int(code), int(blocksize), int(scale_alg),
                                                   _h(y_out), _h(mxscale_out), byref(ws), byref(ex))
    if st != ACLNN_SUCCESS:
        raise AclnnError("aclnnDynamicMxQuantGetWorkspaceSize", st)
    st = lib().aclnnDynamicMxQuant(c_void_p(0), c_uint64(0), ex, _stream())
    if st != ACLNN_SUCCESS:
        raise AclnnError("aclnnDynamicMxQuant", st)


# ---- prepare-once weights (include/opsnn_b200_prepare.h) ----------------------------------------------------------

def prepare_x2(x2, x2_scale, transpose_x2=False, group_size=0, m_hint=128):
    """opsnnQuantMatmulPrepareX2 on the current torch CUDA stream. Returns the storage tensor (uint8, device) that now backs the
    registration and must be kept alive by the caller, or None when the mode has nothing to prepare."""
    import torch

    need = c_uint64(0)
    st = lib().opsnnQuantMatmulPrepareX2GetStorageSize(_h(x2), _h(x2_scale), bool(transpose_x2), int(group_size), int(m_hint), byref(need))
    if st != ACLNN_SUCCESS:
        raise AclnnError("opsnnQuantMatmulPrepareX2GetStorageSize", st)
    if need.value == 0:
        return None
    storage = torch.empty(int(need.value), dtype=torch.uint8, device=x2._keep.device)
    st = lib().opsnnQuantMatmulPrepareX2(_h(x2), _h(x2_scale), bool(transpose_x2), int(group_size), int(m_hint),
                                         c_void_p(storage.data_ptr()), c_uint64(need.value), _stream())
    if st != ACLNN_SUCCESS:
        raise AclnnError("opsnnQuantMatmulPrepareX2", st)
    return storage


def release_x2(x2):
    st = lib().opsnnQuantMatmulReleaseX2(_h(x2))
    if st != ACLNN_SUCCESS:
        raise AclnnError("opsnnQuantMatmulReleaseX2", st)


def prepare_weight(weight, antiquant_scale, antiquant_offset=None, antiquant_group_size=0, x_dtype="bfloat16"):
    """opsnnWeightQuantPrepare on the current torch CUDA stream: the weight dequantised once for the prefill path (m > 16). Returns
    the storage tensor the caller must keep alive, or None when this weight has no prefill path."""
    import torch

    code = DTYPE_BY_NAME[x_dtype] if isinstance(x_dtype, str) else x_dtype
    need = c_uint64(0)
    st = lib().opsnnWeightQuantPrepareGetStorageSize(_h(weight), _h(antiquant_scale), _h(antiquant_offset), int(antiquant_group_size),
                                                     int(code), byref(need))
    if st != ACLNN_SUCCESS:
        raise AclnnError("opsnnWeightQuantPrepareGetStorageSize", st)
    if need.value == 0:
        return None
    storage = torch.empty(int(need.value), dtype=torch.uint8, device=weight._keep.device)
    st = lib().opsnnWeightQuantPrepare(_h(weight), _h(antiquant_scale), _h(antiquant_offset), int(antiquant_group_size), int(code),
                                       c_void_p(storage.data_ptr()), c_uint64(need.value), _stream())
    if st != ACLNN_SUCCESS:
        raise AclnnError("opsnnWeightQuantPrepare", st)
    return storage


def release_weight(weight):
    st = lib().opsnnWeightQuantRelease(_h(weight))
    if st != ACLNN_SUCCESS:
        raise AclnnError("opsnnWeightQuantRelease", st)


# ---- multi-GPU helpers (include/opsnn_b200_shard.h) --------------------------------------------------------------

def shard_range(total, world, rank, multiple=1):
    """opsnn_shard_range: [begin, end) of `rank`'s share (the C mirror of shard.split_range)."""
    b, e = c_int64(0), c_int64(0)
    lib().opsnn_shard_range(int(total), int(world), int(rank), int(multiple), byref(b), byref(e))
    return b.value, e.value


class Comm:
    """The library's own NCCL communicator (opsnn_comm_*): created once per process from an initialised torch.distributed group,
    which is only used to hand rank 0's 128-byte NCCL id to the other ranks."""

    def __init__(self, world, rank, device, broadcast=None):
        import torch

        self.world, self.rank, self.device = int(world), int(rank), device
        idbuf = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            raw = (ctypes.c_ubyte * 128)()
            rc = lib().opsnn_comm_unique_id(raw)
            if rc != 0:
                raise RuntimeError("opsnn_comm_unique_id failed (%d): %s" % (rc, last_error()))
            idbuf = torch.tensor(list(raw), dtype=torch.uint8)
        if world > 1:
            if broadcast is None:
                import torch.distributed as dist

                t = idbuf.to(device) if dist.get_backend() == "nccl" else idbuf
                dist.broadcast(t, src=0)
                idbuf = t.cpu()
            else:
                idbuf = broadcast(idbuf)
        raw = (ctypes.c_ubyte * 128)(*[int(v) for v in idbuf.tolist()])
        h = c_void_p(0)
        rc = lib().opsnn_comm_init(raw, self.world, self.rank, byref(h))
        if rc != 0:
            raise RuntimeError("opsnn_comm_init failed (%d): %s" % (rc, last_error()))
        self.handle = h
        self._ws = None

    def gather_columns(self, y_local, n_total, multiple=8, out=None):
        """Every rank receives the (m, n_total) output from the ranks' (m, width) column shards; enqueued on the current stream."""
        import torch

        m = y_local.shape[0]
        eb = y_local.element_size()
        need = lib().opsnn_gather_columns_workspace(self.world, m, int(n_total), int(multiple), eb)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(int(need), dtype=torch.uint8, device=y_local.device)
        if out is None:
            out = torch.empty((m, int(n_total)), dtype=y_local.dtype, device=y_local.device)
        rc = lib().opsnn_gather_columns(self.handle, c_void_p(y_local.data_ptr()), int(y_local.stride(0)), m, int(n_total), int(multiple), eb,
                                        c_void_p(out.data_ptr()), c_void_p(self._ws.data_ptr()), c_uint64(self._ws.numel()), _stream())
        if rc != 0:
            raise RuntimeError("opsnn_gather_columns failed (%d): %s" % (rc, last_error()))
        return out

    def gather_batch(self, y_local, batch_total, out=None):
        """Every rank receives the (batch_total, ...) output from equal contiguous batch shards; enqueued on the current stream."""
        import torch

        per = y_local[0].numel() * y_local.element_size()
        if out is None:
            out = torch.empty((int(batch_total),) + tuple(y_local.shape[1:]), dtype=y_local.dtype, device=y_local.device)
        rc = lib().opsnn_gather_batch(self.handle, c_void_p(y_local.data_ptr()), int(batch_total), c_uint64(per), c_void_p(out.data_ptr()), _stream())
        if rc != 0:
            raise RuntimeError("opsnn_gather_batch failed (%d): %s" % (rc, last_error()))
        return out

    # ---- the gather folded into the decode kernels' epilogue (opsnn_comm_symmetric_alloc / bind_columns / arrive_and_wait) ----

    def symmetric_empty(self, shape, dtype):
        """Collective. A zeroed tensor of `shape` on every rank, in memory every rank has mapped: a torch view of this rank's block."""
        import torch

        class _Raw:  # zero-copy view of library-owned device memory
            def __init__(self, ptr, nbytes):
                self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}

        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        local = c_void_p(0)
        rc = lib().opsnn_comm_symmetric_alloc(self.handle, c_uint64(max(nbytes, 16)), byref(local), None)
        if rc != 0:
            raise RuntimeError("opsnn_comm_symmetric_alloc failed (%d): %s" % (rc, last_error()))
        with torch.cuda.device(self.device):
            flat = torch.as_tensor(_Raw(local.value, nbytes), device=self.device)
        return flat.view(dtype).view(*[int(d) for d in shape])

    def bind_columns(self, y_local, y_full, multiple=8):
        """From now on decode calls whose output is `y_local` (this rank's column shard) also store it into every rank's `y_full`
        (from symmetric_empty); follow each such call with arrive_and_wait()."""
        rc = lib().opsnn_comm_bind_columns(self.handle, c_void_p(y_local.data_ptr()), c_void_p(y_full.data_ptr()), int(y_full.shape[-1]), int(multiple))
        if rc != 0:
            raise RuntimeError("opsnn_comm_bind_columns failed (%d): %s" % (rc, last_error()))

    def unbind(self, y_local):
        lib().opsnn_comm_unbind(c_void_p(y_local.data_ptr()))

    def arrive_and_wait(self):
        """Collective, on the current stream: afterwards every rank's stores into the bound outputs are complete."""
        rc = lib().opsnn_comm_arrive_and_wait(self.handle, _stream())
        if rc != 0:
            raise RuntimeError("opsnn_comm_arrive_and_wait failed (%d): %s" % (rc, last_error()))

    def allgather_columns_peer(self, y_local, y_full, multiple=8):
        """Collective, on the current stream: one kernel copies this rank's column shard into every rank's `y_full` (from
        symmetric_empty) with peer stores and waits for the other ranks' shards to have arrived."""
        rc = lib().opsnn_comm_allgather_columns(self.handle, c_void_p(y_local.data_ptr()), int(y_local.stride(0)), int(y_local.shape[0]),
                                                c_void_p(y_full.data_ptr()), int(y_full.shape[-1]), int(multiple), y_local.element_size(), _stream())
        if rc != 0:
            raise RuntimeError("opsnn_comm_allgather_columns failed (%d): %s" % (rc, last_error()))

    def status(self, reset=True):
        """0, or 1 when a wait for the other ranks ran out (synchronises the device)."""
        return int(lib().opsnn_comm_status(self.handle, 1 if reset else 0))

    def close(self):
        if getattr(self, "handle", None) is not None and self.handle.value:
            lib().opsnn_comm_destroy(self.handle)
            self.handle = c_void_p(0)
