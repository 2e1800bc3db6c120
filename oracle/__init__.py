"""TEST INFRASTRUCTURE -- not part of the product.

ctypes loaders for the CPU oracle (oracle/_build/libth_oracle.so, the restatement of TH's CPU
results in th_oracle.cpp) and, where it was built, for the library compiled from cutorch's own
headers (oracle/_ref/libref_check.so).  Only tests/, __graft_entry__.smoke() and the CPU
baseline legs of bench.py import this package.
"""
from .loader import Oracle, RefCheck, build_oracle, oracle_path, ref_path  # noqa: F401
