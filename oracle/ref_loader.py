"""Imports the reference's own numpy goldens from a checkout of hicann/ops-nn (never copied into this repository).

Only `tests/golden/make_golden.py` uses this, on a machine that has the reference tree ($OPSNN_REFERENCE_ROOT, or a
`reference` folder next to this repository). The goldens import `en_dtypes`, which is not installable here; a shim module maps the two dtypes
the hot path needs onto ml_dtypes (float4_e2m1 -> float4_e2m1fn, float8_e8m0 -> float8_e8m0fnu).

Test infrastructure only (see oracle/__init__.py).
"""
import importlib.util
import os
import sys
import types

import ml_dtypes
import numpy as np

REF = os.environ.get("OPSNN_REFERENCE_ROOT",
                     os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))


def available():
    return os.path.isdir(os.path.join(REF, "matmul", "quant_batch_matmul_v3", "tests", "assets"))


def _install_shim():
    if "en_dtypes" in sys.modules:
        return
    m = types.ModuleType("en_dtypes")
    m.float4_e2m1 = ml_dtypes.float4_e2m1fn
    m.float8_e8m0 = ml_dtypes.float8_e8m0fnu

    class _Missing:  # dtypes with no implementation available here; unused by the hot path
        pass

    m.float4_e1m2 = type("float4_e1m2", (_Missing,), {})
    m.hifloat8 = type("hifloat8", (_Missing,), {})
    sys.modules["en_dtypes"] = m


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


_cache = {}


def goldens():
    """Returns a dict of the reference golden modules: qbmmv3, qbmmv4 (kernel goldens), wqbmmv2, mxquant."""
    if _cache:
        return _cache
    _install_shim()
    for d in ("matmul/common/tests/st/arch35", "matmul/quant_batch_matmul_v3/tests/assets",
              "matmul/quant_batch_matmul_v4/tests/assets", "matmul/weight_quant_batch_matmul_v2/tests/assets"):
        p = os.path.join(REF, d)
        if p not in sys.path:
            sys.path.insert(0, p)
    import matmul_golden_util  # noqa: E402

    matmul_golden_util._DTYPE_TO_STR[np.dtype(ml_dtypes.float4_e2m1fn)] = "float4_e2m1"
    matmul_golden_util._DTYPE_TO_STR[np.dtype(ml_dtypes.float8_e8m0fnu)] = "float8_e8m0"
    import qbmmv3_kernel_golden  # noqa: E402
    import qbmmv4_kernel_golden  # noqa: E402
    import wqbmmv2_kernel_golden  # noqa: E402

    _cache["util"] = matmul_golden_util
    _cache["qbmmv3"] = qbmmv3_kernel_golden
    _cache["qbmmv4"] = qbmmv4_kernel_golden
    _cache["wqbmmv2"] = wqbmmv2_kernel_golden
    _cache["mxquant"] = _load(os.path.join(REF, "quant/dynamic_mx_quant/tests/assets/golden.py"), "ref_dynamic_mx_quant_golden")
    return _cache
