"""The C-ABI library loads without a GPU and exports every symbol the headers declare; the
THC structs keep the field order cutorch's FFI mirrors (FFI.lua:11-81)."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import pytest

from cutorch_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent
CREALS = ["CudaByte", "CudaChar", "CudaShort", "CudaInt", "CudaLong", "CudaHalf", "Cuda", "CudaDouble"]


def exported():
    out = subprocess.run(["nm", "-D", "--defined-only", str(_lib.library_path())], capture_output=True, text=True, check=True)
    return {ln.split()[-1] for ln in out.stdout.splitlines() if ln.strip()}


def test_descriptor_abi_symbols_are_exported():
    text = (ROOT / "include" / "thcb200.h").read_text()
    names = set(re.findall(r"\b(thcb200_[a-z0-9_]+)\s*\(", text))
    assert len(names) >= 15
    missing = names - exported()
    assert not missing, missing


def test_thc_api_symbols_are_exported():
    api = (ROOT / "include" / "THC" / "THCTypeAPI.h").read_text()
    syms = exported()
    missing = []
    # split the per-type header into its conditional blocks
    floating_only = set()
    signed_or_fp = set()
    block = None
    for ln in api.splitlines():
        if ln.startswith("#if THC_T_FLOATING || THC_T_SIGNED"):
            block = "sf"
        elif ln.startswith("#if THC_T_FLOATING"):
            block = "f"
        elif ln.startswith("#endif"):
            block = None
        for m in re.finditer(r"THC(Tensor|Storage)_\((\w+)\)", ln):
            if "THC_API" not in ln and not ln.strip().startswith("THC_API"):
                continue
            key = (m.group(1), m.group(2))
            if block == "f":
                floating_only.add(key)
            elif block == "sf":
                signed_or_fp.add(key)
    for ln in api.splitlines():
        if not ln.startswith("THC_API"):
            continue
        m = re.search(r"THC(Tensor|Storage)_\((\w+)\)", ln)
        if not m:
            continue
        kind, name = m.groups()
        for creal in CREALS:
            fp = creal in ("CudaHalf", "Cuda", "CudaDouble")
            if (kind, name) in floating_only and not fp:
                continue
            if (kind, name) in signed_or_fp and creal in ("CudaByte", "CudaChar"):
                continue
            sym = f"TH{creal}{kind}_{name}"
            if sym not in syms:
                missing.append(sym)
    assert not missing, missing[:20]
    for name in ("THCState_alloc", "THCudaInit", "THCState_getCurrentStream", "THCudaByteTensor_logicalall",
                 "THCudaByteTensor_logicalany", "THLongStorage_newWithSize", "THC_float2half"):
        assert name in syms


def test_cpu_gpu_copy_entry_points():
    """The copies between CPU and GPU tensors: THCTensor_(copy<Type>) is covered by the header walk
    above; the names that start with the CPU tensor's type (lib/THC/generic/THCTensorCopy.h:26-39)
    are listed here."""
    syms = exported()
    names = ["Byte", "Char", "Short", "Int", "Long", "Half", "Float", "Double"]
    missing = [f"TH{cpu}Tensor_copyCuda{real}" for cpu in names for real in names if f"TH{cpu}Tensor_copyCuda{real}" not in syms]
    missing += [f"TH{real}Tensor_{n}" for real in names for n in ("copyCuda", "copyAsyncCuda") if f"TH{real}Tensor_{n}" not in syms]
    assert not missing, missing[:10]
    assert "thcb200_copy_from_host" in syms and "thcb200_copy_to_host" in syms


def test_configs_minimum_entry_points():
    syms = exported()
    need = ["THCudaTensor_cadd", "THCudaTensor_sumall", "THCudaTensor_addcmul", "THCudaTensor_copy", "THCudaTensor_sum",
            "THCudaTensor_max", "THCudaTensor_cmul", "THCudaTensor_add", "THCudaHalfTensor_sigmoid", "THCudaHalfTensor_mean",
            "THCudaHalfTensor_norm", "THCudaHalfTensor_sum", "THCudaHalfTensor_div", "THCudaHalfTensor_pow",
            "THCudaIntTensor_cmul", "THCudaIntTensor_sumall", "THCudaDoubleTensor_sumall"]
    assert not [s for s in need if s not in syms]


def test_struct_layout_matches_cutorch(tmp_path):
    """Field offsets of THCStorage / THCTensor as a C compiler sees them through THC.h."""
    src = tmp_path / "layout.c"
    src.write_text(r'''
#include <stdio.h>
#include <stddef.h>
#include "THC/THC.h"
int main(void) {
  printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu\n", offsetof(THCudaStorage, data), offsetof(THCudaStorage, size),
         offsetof(THCudaStorage, refcount), offsetof(THCudaStorage, flag), offsetof(THCudaStorage, allocator),
         offsetof(THCudaStorage, allocatorContext), offsetof(THCudaStorage, view), offsetof(THCudaStorage, device),
         sizeof(THCudaStorage));
  printf("%zu %zu %zu %zu %zu %zu %zu %zu\n", offsetof(THCudaTensor, size), offsetof(THCudaTensor, stride),
         offsetof(THCudaTensor, nDimension), offsetof(THCudaTensor, storage), offsetof(THCudaTensor, storageOffset),
         offsetof(THCudaTensor, refcount), offsetof(THCudaTensor, flag), sizeof(THCudaTensor));
  printf("%zu %zu\n", sizeof(half), sizeof(THCudaHalfTensor));
  return 0;
}
''')
    exe = tmp_path / "layout"
    r = subprocess.run(["gcc", "-I", str(ROOT / "include"), "-I", "/usr/local/cuda/include", str(src), "-o", str(exe)],
                       capture_output=True, text=True)
    if r.returncode != 0:
        pytest.fail(r.stderr[-2000:])
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split("\n")
    assert out[0].split() == ["0", "8", "16", "20", "24", "32", "40", "48", "56"]
    assert out[1].split() == ["0", "8", "16", "24", "32", "40", "44", "48"]
    assert out[2].split() == ["2", "48"]


def test_host_layout_predicates():
    lib = _lib.load_library()
    d = lambda sizes, strides: C.byref(_lib.make_desc(4096, _lib.F32, sizes, strides))  # the pointer is never dereferenced
    assert lib.thcb200_overlapping(d([3, 4], [4, 1])) == 0
    assert lib.thcb200_overlapping(d([3, 4], [0, 1])) == 1          # expanded dim
    assert lib.thcb200_overlapping(d([3, 4], [1, 3])) == 0          # transposed, dense
    assert lib.thcb200_overlapping(d([3, 4], [2, 1])) == 1          # rows overlap
    assert lib.thcb200_overlapping(d([3, 4], [8, 2])) == 0          # holes
    assert lib.thcb200_overlapping(d([1, 1], [0, 0])) == 0
    assert lib.thcb200_can_use_32bit(d([1 << 20, 1 << 10], [1 << 10, 1])) == 1
    assert lib.thcb200_can_use_32bit(d([1 << 22, 1 << 10], [1 << 10, 1])) == 0   # 2^32 elements
    assert lib.thcb200_can_use_32bit(d([4, 4], [1 << 31, 1])) == 0                # offsets beyond 32 bits


def test_library_reports_missing_cuda_cleanly():
    """Without a GPU a context cannot be created: the call fails with a CUDA status, nothing
    falls back to a CPU path."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = _lib.load_library()
    ctx = C.c_void_p()
    rc = lib.thcb200_ctx_create(C.byref(ctx), 0)
    assert rc == -4 and lib.thcb200_last_error()


def test_view_extent_and_the_check_against_an_allocation():
    """The host-side bound check that stands in for cutorch's device-side asserts
    (lib/THC/THCTensorInfo.cuh:228-278): the smallest and largest offset a view reaches, as
    canUse32BitIndexMath sums them (lib/THC/THCTensorTypeUtils.cu:220-245), against what the
    caller says the allocation holds."""
    lib = _lib.load_library()
    P = C.POINTER
    lib.thcb200_view_extent.argtypes = [P(_lib.TensorDesc), P(C.c_int64), P(C.c_int64)]
    lib.thcb200_check_extent.argtypes = [P(_lib.TensorDesc), C.c_int64, C.c_int64]
    lo, hi = C.c_int64(7), C.c_int64(7)
    cases = [(((4, 5), (5, 1)), 0, 19), (((4, 5), (1, 4)), 0, 19), (((3, 4), (8, 2)), 0, 22), (((10,), (0,)), 0, 0),
             (((3, 4), (-4, 1)), -8, 3), (((2, 3, 4), (100, -10, 3)), -20, 109)]
    for (sizes, strides), wlo, whi in cases:
        d = _lib.make_desc(0x1000, 6, sizes, strides)
        assert lib.thcb200_view_extent(C.byref(d), C.byref(lo), C.byref(hi)) == 1
        assert (lo.value, hi.value) == (wlo, whi), (sizes, strides)
        assert lib.thcb200_check_extent(C.byref(d), -wlo, whi) == 0
        assert lib.thcb200_check_extent(C.byref(d), -wlo, whi - 1) == (-3 if whi > 0 else 0) or whi == 0
        if wlo < 0:
            assert lib.thcb200_check_extent(C.byref(d), -wlo - 1, whi) == -3
            assert b"reaches offsets" in lib.thcb200_last_error()
    empty = _lib.make_desc(0x1000, 6, (3, 0), (1, 1))
    assert lib.thcb200_view_extent(C.byref(empty), C.byref(lo), C.byref(hi)) == 0
    assert lib.thcb200_check_extent(C.byref(empty), 0, 0) == 0
