import importlib.util
import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_package():
    """Imports the `ops-nn_b200` folder as module `ops_nn_b200` and makes sure the shared library is built."""
    if "ops_nn_b200" in sys.modules:
        return sys.modules["ops_nn_b200"]
    pkg_dir = os.path.join(ROOT, "ops-nn_b200")
    spec = importlib.util.spec_from_file_location("ops_nn_b200", os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ops_nn_b200"] = mod
    if not os.path.exists(os.path.join(pkg_dir, "lib", "libopsnn_b200.so")):
        bspec = importlib.util.spec_from_file_location("opsnn_build", os.path.join(pkg_dir, "build.py"))
        b = importlib.util.module_from_spec(bspec)
        bspec.loader.exec_module(b)
        b.build()
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def aclnn(pkg):
    return pkg.aclnn


@pytest.fixture(autouse=True)
def _device_status_words(request):
    """After every GPU test: no kernel of the library may have given up a bounded wait. A give-up leaves the output
    undefined, so without this check it could pass as (or hide behind) a parity mismatch."""
    yield
    if request.node.get_closest_marker("gpu") is None or "ops_nn_b200" not in sys.modules:
        return
    L = sys.modules["ops_nn_b200"].aclnn.lib()
    umma = L.opsnn_qmm_umma_status(1)
    decode = L.opsnn_wqbmm_decode_status(1)
    assert umma == 0, "a tensor-core kernel gave up a bounded wait: status 0x%x" % umma
    assert decode == 0, "the streaming decode kernel gave up a bounded wait: status %d" % decode


def golden_names(prefix):
    return sorted(f[:-4] for f in os.listdir(GOLDEN) if f.startswith(prefix) and f.endswith(".npz"))


def load_golden(name):
    """Returns (arrays as numpy with ml_dtypes views restored, meta dict)."""
    import ml_dtypes

    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    meta = json.loads(bytes(z["meta"]).decode())
    views = {"bfloat16": ml_dtypes.bfloat16, "float8_e4m3fn": ml_dtypes.float8_e4m3fn, "float8_e5m2": ml_dtypes.float8_e5m2,
             "float8_e8m0": ml_dtypes.float8_e8m0fnu, "float4_e2m1": ml_dtypes.float4_e2m1fn}
    out = {}
    for k, dt in meta["dtypes"].items():
        a = z[k]
        if dt == "int4" and name.startswith("qmm_"):
            out[k] = a.astype(ml_dtypes.int4)  # stored one value per byte
        else:
            out[k] = a.view(views[dt]) if dt in views else a
    return out, meta


def case_seed(case):
    """Seed for a parametrised case's random inputs: the same in every process (the built-in hash of a string is salted
    per interpreter run, which would make a failure unrepeatable)."""
    import zlib

    return zlib.crc32(repr(case).encode()) & 0x7FFFFFFF
