"""CPU oracle: a restatement of the reference's golden arithmetic for the quantized-matmul hot path.

TEST INFRASTRUCTURE ONLY. Nothing in the product (the `ops-nn_b200` package or its shared library) imports, links or
executes anything in this folder; only `tests/`, `__graft_entry__.smoke()` and `bench.py`'s CPU-baseline legs do, and
only as the checker. Parity is pinned: `tests/golden/make_golden.py` ran the reference's own numpy goldens (imported
from the reference tree through `oracle/ref_loader.py`) on seeded inputs and stored inputs + outputs as fixtures;
`tests/test_oracle.py` checks every function here against those fixtures.
"""
