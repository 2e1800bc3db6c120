"""Generates the golden fixtures of tests/golden/ from cutorch's own code.

Needs oracle/_ref/libref_check.so, i.e. a checkout of cutorch where oracle/Makefile's REF points
(make -C oracle REF=<cutorch tree>).
The fixtures travel with the repository so that the checks also run where the reference tree is
absent:
  collapse_dims.json  TensorInfo::collapseDims outputs (lib/THC/THCTensorInfo.cuh:74-224) and
                      IndexToOffset samples (:228-278) for the baseline configs' views and for
                      seeded random views (holes, transposes, size-1 dims, excluded dims)
  functors.json       outputs of the pointwise functor bodies (lib/THC/THCTensorMathPointwise.cuh,
                      lib/THC/THCNumerics.cuh) on fixed inputs, as hex bit patterns

  compare_masked.json outputs of the comparison functors into Byte and into the operands' type
                      (lib/THC/THCTensorMathCompare.cuh, THCTensorMathCompareT.cuh) and of the Byte-masked
                      fill / copy / select functors (lib/THC/THCTensorMasked.cuh) on fixed inputs
  thc_prototypes.json the C prototypes of lib/THC/generic/*.h (and the two non-generic Byte entry
                      points), normalised to one line each, per header

    python tests/golden/make_golden.py
"""
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from oracle import RefCheck  # noqa: E402


def random_view(r):
    nd = int(r.integers(1, 7))
    sizes = [int(r.choice([1, 1, 2, 3, 4, 5, 7])) for _ in range(nd)]
    # start from a contiguous layout of a (possibly padded) parent, then permute / slice
    parent = [s + int(r.integers(0, 3)) * int(r.integers(0, 2)) for s in sizes]
    strides, run = [0] * nd, 1
    for d in reversed(range(nd)):
        strides[d] = run
        run *= parent[d]
    if nd > 1 and r.random() < 0.5:
        a, b = (int(v) for v in r.choice(nd, 2, replace=False))
        sizes[a], sizes[b] = sizes[b], sizes[a]
        strides[a], strides[b] = strides[b], strides[a]
    if r.random() < 0.3:
        d = int(r.integers(0, nd))
        strides[d] *= 2
    return sizes, strides


def main():
    ref = RefCheck()
    r = np.random.default_rng(20240607)
    cases = []
    fixed = [
        ([64, 256, 56, 56], [802816, 3136, 56, 1], -1),
        ([64, 256, 56, 56], [1605632, 6272, 112, 2], -1),
        ([64, 256, 56, 56], [802816, 1, 256, 14336], -1),
        ([32768, 1], [8192, 1], -1),
        ([1, 8192], [8192, 1], -1),
        ([32768, 8192], [8192, 1], 1),
        ([32768, 8192], [8192, 1], 0),
        ([4, 1, 3, 5], [30, 15, 5, 1], 2),
        ([1, 1, 1], [1, 1, 1], -1),
        ([5], [3], -1),
    ]
    for sizes, strides, ex in fixed:
        cases.append((sizes, strides, ex))
    for _ in range(300):
        sizes, strides = random_view(r)
        ex = -1 if r.random() < 0.6 else int(r.integers(0, len(sizes)))
        if all(s == 1 for s in sizes):
            ex = -1  # the reference asserts on an excluded dim of an all-ones view
        cases.append((sizes, strides, ex))
    out = []
    for sizes, strides, ex in cases:
        cs, ct, ret = ref.collapse_dims(sizes, strides, ex)
        n = int(np.prod(sizes))
        samples = sorted({0, n - 1, n // 2, n // 3, (n * 2) // 3})
        offs = [[int(i), int(ref.index_to_offset(sizes, strides, int(i)))] for i in samples]
        out.append({"sizes": sizes, "strides": strides, "exclude": ex, "out_sizes": cs, "out_strides": ct, "ret": ret,
                    "offsets": offs})
    (HERE / "collapse_dims.json").write_text(json.dumps(out, separators=(",", ":")))

    # functor outputs
    fx = {}
    n = 64
    rr = np.random.default_rng(7)
    for dt in (np.float32, np.float64):
        a = rr.uniform(-3, 3, n).astype(dt)
        b = rr.uniform(-3, 3, n).astype(dt)
        b[b == 0] = 1
        c = rr.uniform(0.5, 3, n).astype(dt)
        pos = np.abs(a) + 0.25
        unit = (a / 3).astype(dt)
        table = {
            "SIGMOID": ([a], 0, 0), "SIGN": ([a], 0, 0), "ADD": ([a, b], 0, 0), "CADD": ([a, b], 2.5, 0), "SUB": ([a, b], 0, 0),
            "MUL": ([a, b], 0, 0), "DIV": ([a, b], 0, 0), "CPOW": ([pos, b], 0, 0), "CREMAINDER": ([a, b], 0, 0),
            "CFMOD": ([a, b], 0, 0), "CLAMP": ([a], -1.0, 1.5), "LERP": ([a, b], 0.3, 0), "CMAX": ([a, b], 0, 0),
            "CMIN": ([a, b], 0, 0), "MAX_S": ([a], 0.5, 0), "MIN_S": ([a], 0.5, 0), "ADDCMUL": ([a, b, c], 0.5, 0),
            "ADDCDIV": ([a, b, c], 0.5, 0), "POW": ([pos], 2.7, 0), "TPOW": ([a], 1.5, 0),
            "LOG": ([pos], 0, 0), "LGAMMA": ([pos], 0, 0), "LOG1P": ([pos], 0, 0), "EXP": ([a], 0, 0), "COS": ([a], 0, 0),
            "SIN": ([a], 0, 0), "SQRT": ([pos], 0, 0), "RSQRT": ([pos], 0, 0), "CEIL": ([a], 0, 0), "FLOOR": ([a], 0, 0),
            "TRUNC": ([a], 0, 0), "ACOS": ([unit], 0, 0), "COSH": ([a], 0, 0), "ASIN": ([unit], 0, 0), "SINH": ([a], 0, 0),
            "TAN": ([unit], 0, 0), "ATAN": ([a], 0, 0), "TANH": ([a], 0, 0), "ROUND": ([a], 0, 0), "FRAC": ([a], 0, 0),
            "CINV": ([pos], 0, 0), "NEG": ([a], 0, 0), "ABS": ([a], 0, 0),
        }
        for name, (ins, s0, s1) in table.items():
            res = ref.apply(name, np.zeros(n, dt), ins, s0, s1)
            fx[f"{np.dtype(dt).name}.{name}"] = {"inputs": [x.tobytes().hex() for x in ins], "s0": s0, "s1": s1,
                                               "out": res.tobytes().hex()}
    for dt in (np.uint8, np.int8, np.int16, np.int32, np.int64):
        info = np.iinfo(dt)
        a = rr.integers(max(info.min, -100), min(info.max, 100) + 1, n).astype(dt)
        b = rr.integers(max(info.min, -9), 10, n).astype(dt)
        b[b == 0] = 3
        c = rr.integers(1, 7, n).astype(dt)
        sh = rr.integers(0, 4, n).astype(dt)
        nonneg = np.abs(a.astype(np.int64)).astype(dt) if info.min < 0 else a
        table = {
            "SIGN": ([a], 0, 0), "ADD": ([a, b], 0, 0), "CADD": ([a, b], 3, 0), "SUB": ([a, b], 0, 0), "MUL": ([a, b], 0, 0),
            "DIV": ([a, b], 0, 0), "CREMAINDER": ([a, b], 0, 0), "CFMOD": ([a, b], 0, 0), "CLAMP": ([a], 2, 40),
            "CMAX": ([a, b], 0, 0), "CMIN": ([a, b], 0, 0), "MAX_S": ([a], 5, 0), "MIN_S": ([a], 5, 0),
            "ADDCMUL": ([a, b, c], 2, 0), "ADDCDIV": ([a, b, c], 2, 0), "CLSHIFT": ([nonneg, sh], 0, 0),
            "CRSHIFT": ([nonneg, sh], 0, 0), "CBITAND": ([a, b], 0, 0), "CBITOR": ([a, b], 0, 0), "CBITXOR": ([a, b], 0, 0),
        }
        for name, (ins, s0, s1) in table.items():
            res = ref.apply(name, np.zeros(n, dt), ins, s0, s1)
            fx[f"{np.dtype(dt).name}.{name}"] = {"inputs": [x.tobytes().hex() for x in ins], "s0": s0, "s1": s1,
                                               "out": res.tobytes().hex()}
    (HERE / "functors.json").write_text(json.dumps(fx, separators=(",", ":")))
    print(f"wrote {len(out)} collapse cases and {len(fx)} functor vectors")

    # comparison and mask functors
    cm = {}
    n = 96
    rc = np.random.default_rng(11)
    for dt in (np.uint8, np.int8, np.int16, np.int32, np.int64, np.float32, np.float64):
        if np.dtype(dt).kind == "f":
            a = rc.integers(-3, 4, n).astype(dt)
            b = rc.integers(-3, 4, n).astype(dt)
            a[5], b[9], a[20], b[20] = np.nan, np.nan, np.nan, np.nan      # comparisons with NaN are false, ne is true
            a[7], b[7] = 0.0, -0.0
        else:
            lo = 0 if np.dtype(dt).kind == "u" else -3
            a = rc.integers(lo, 4, n).astype(dt)
            b = rc.integers(lo, 4, n).astype(dt)
        mask = (rc.uniform(size=n) < 0.45).astype(np.uint8)
        mask[rc.integers(0, n, 5)] = 7          # any non-zero byte is "set"
        packed = rc.integers(10, 100, int((mask != 0).sum())).astype(dt)
        key = np.dtype(dt).name
        entry = {"a": a.tobytes().hex(), "b": b.tobytes().hex(), "mask": mask.tobytes().hex(), "packed": packed.tobytes().hex(),
                 "scalar": 1, "fill": 9}
        for name in ("lt", "gt", "le", "ge", "eq", "ne"):
            entry[name + "Tensor"] = ref.compare(name, a, b).tobytes().hex()
            entry[name + "Value"] = ref.compare(name, a, 1).tobytes().hex()
            entry[name + "TensorT"] = ref.compare(name, a, b, same_type=True).tobytes().hex()
            entry[name + "ValueT"] = ref.compare(name, a, 1, same_type=True).tobytes().hex()
        entry["maskedFill"] = ref.masked("fill", a, mask, value=9).tobytes().hex()
        entry["maskedCopy"] = ref.masked("copy", a, mask, other=packed).tobytes().hex()
        entry["maskedSelect"] = ref.masked("select", a, mask).tobytes().hex()
        cm[key] = entry
    (HERE / "compare_masked.json").write_text(json.dumps(cm, separators=(",", ":")))
    print(f"wrote comparison and mask vectors for {len(cm)} element types")

    write_prototypes()


PROTOTYPE_HEADERS = ["generic/THCTensorMathPointwise.h", "generic/THCTensorMathPairwise.h", "generic/THCTensorMathReduce.h",
                     "generic/THCTensorMathCompare.h", "generic/THCTensorMathCompareT.h", "generic/THCTensorMathScan.h",
                     "generic/THCTensorMath.h", "generic/THCTensorCopy.h", "generic/THCTensorMasked.h",
                     "generic/THCTensorIndex.h", "generic/THCTensorScatterGather.h"]


def normalise_prototype(text: str) -> str:
    """One prototype as a canonical string: comments and THC_API dropped, whitespace collapsed,
    no space around punctuation, parameter names kept (they are part of what a reader diffs)."""
    import re
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    text = text.replace("THC_API", " ")
    text = re.sub(r"\s+", " ", text).strip()
    text = re.sub(r"\s*([(),*])\s*", r"\1", text)
    return text


def prototypes_of(text: str):
    """The THC_API declarations of a header, each normalised, in file order."""
    import re
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    return [normalise_prototype(m.group(0)) for m in re.finditer(r"THC_API[^;]*;", text)]


def write_prototypes():
    from oracle.loader import cutorch_tree
    tree = cutorch_tree()
    if not tree:
        print("no cutorch tree: thc_prototypes.json left as it is")
        return
    out = {}
    for h in PROTOTYPE_HEADERS:
        out[h] = prototypes_of((Path(tree) / "lib" / "THC" / h).read_text())
    (HERE / "thc_prototypes.json").write_text(json.dumps(out, indent=0))
    print(f"wrote {sum(len(v) for v in out.values())} prototypes from {len(out)} headers")


if __name__ == "__main__":
    main()
