"""ops-nn_b200: B200 (sm_100a) implementation of hicann/ops-nn's quantized-matmul path behind its aclnn C API.

The product is the shared library `lib/libopsnn_b200.so` (C++ host code + CUDA kernels; headers in `include/`).
This Python package is a thin ctypes mirror of the same entry points for tests, benchmarks and PyTorch users:

    aclnn   - 1:1 bindings of the aclnn two-phase functions plus helpers that run both phases on torch tensors
    shard   - N / batch sharding of one call over the GPUs of a box (one process per GPU)

The folder name contains a hyphen; import it with `importlib` (see `load_package()` in `__graft_entry__.py`) under the
module name `ops_nn_b200`.
"""
from . import aclnn  # noqa: F401
from . import shard  # noqa: F401
from . import torch_api  # noqa: F401
