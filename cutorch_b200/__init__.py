"""cutorch_b200 -- B200-native apply / reduce core behind cutorch's THC C API.

The product is the shared library ``cutorch_b200/lib/libthcb200.so`` (C ABI declared in
``include/thcb200.h`` and ``include/THC/THC.h``).  This package only loads it through ctypes
and mirrors cutorch's tensor-method interface on top of the ``THCuda*Tensor_*`` symbols so that
tests and benchmarks call the library the way cutorch's Lua layer does.
"""
from ._lib import load_library, library_path, LibraryMissing  # noqa: F401
