"""CPU: the shared library loads without a GPU and exports every function the public headers declare."""
import ctypes
import os
import re

from conftest import ROOT


def _declared_functions():
    names = set()
    inc = os.path.join(ROOT, "include")
    for dp, _, fs in os.walk(inc):
        for f in fs:
            if not f.endswith(".h"):
                continue
            src = open(os.path.join(dp, f)).read()
            src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
            for m in re.finditer(r"(?:ACLNN_API|OPSNN_API|OPSNN_SHARD_API)\s+[\w\s\*]+?\b(\w+)\s*\(", src):
                names.add(m.group(1))
    return sorted(names)


def test_every_declared_symbol_is_exported(aclnn):
    L = aclnn.lib()
    names = _declared_functions()
    assert len(names) >= 20, names
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_headers_are_plain_c():
    """The boundary is a C ABI: the headers must compile as C (no torch or C++ types in any signature)."""
    import subprocess
    import tempfile

    inc = os.path.join(ROOT, "include")
    hdrs = ["aclnn_compat/acl_base.h", "aclnnop/aclnn_quant_matmul_v5.h", "aclnnop/aclnn_weight_quant_batch_matmul_v2.h",
            "aclnnop/aclnn_weight_quant_batch_matmul_v3.h", "aclnnop/aclnn_dynamic_mx_quant.h", "aclnnop/aclnn_quant_matmul_v4.h",
            "aclnnop/aclnn_convert_weight_to_int4_pack.h", "aclnnop/aclnn_quant_matmul_weight_nz.h", "opsnn_b200_kernels.h", "opsnn_b200_shard.h", "opsnn_b200_prepare.h"]
    with tempfile.TemporaryDirectory() as td:
        src = os.path.join(td, "t.c")
        with open(src, "w") as fh:
            fh.write("".join('#include "%s"\n' % h for h in hdrs) + "int main(void){return 0;}\n")
        subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-fsyntax-only", "-I", inc, src], check=True)


def test_tensor_descriptor_roundtrip(aclnn):
    t = aclnn.Tensor((3, 4, 5), "bfloat16")
    assert t.handle
    L = aclnn.lib()
    assert L.aclDestroyTensor(ctypes.c_void_p(t.handle)) == 0
    t.handle = None
    assert aclnn.Tensor((0, 5), "int8").handle  # empty tensors are legal descriptors
