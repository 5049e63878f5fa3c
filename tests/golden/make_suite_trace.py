"""Records every call the REFERENCE's own test-suite makes into its native module and stores the calls
as known-answer cases: tests/golden/reference_suite_trace.npz.

    make -C oracle ref
    python tests/golden/make_suite_trace.py --ref <reference checkout>

The reference's Python package is imported as in make_golden.py (symlinks to its .py files beside its
native module built into oracle/_ref, CPU path).  Each compute function of its ``_C`` module is wrapped
by a recorder, then the reference's test files are run in place, in this process, by pytest.  What is
written: for every distinct call the function name, the arguments (views as dtype / shape / strides /
offset over the bytes of their storage; scalars, axis lists, dtypes as they are) and the result the
reference's CPU kernels returned (the bytes of the result storage; for in-place and scatter calls the
destination storage after the call).  None of the reference's code or test text is stored, only these
numeric inputs and outputs.  The replay (tests/test_gpu_reference_trace.py) feeds the same arguments to
this library on the device and compares, so the shapes, strides, dtypes and values are the ones the
reference's authors chose for their tests, not ones chosen here.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(HERE))

MAX_STORAGE_ELEMENTS = 1 << 16
# the finite-difference gradient checks repeat one call shape thousands of times with one element
# perturbed (through an in-place add on a one-element view at a moving offset): keep this many value
# sets per distinct (function, dtypes, shapes, strides, scalars)
MAX_PER_SIGNATURE = 3

VIEW_FUNCS = ["add", "subtract", "multiply", "divide", "pw_equal", "pw_greater", "pw_greater_eq", "equals", "matmul",
              "exp", "log", "pow", "sqrt", "tanh", "sigmoid", "neg", "relu", "sum", "max", "min", "argmax", "argmin",
              "add_inplace", "sub_inplace", "mul_inplace", "div_inplace", "copy_inplace", "cast", "copy_view",
              "clone_contiguous_view_from", "scatter_to_axes", "gather_from_axes"]
MUTATES_FIRST = {"add_inplace", "sub_inplace", "mul_inplace", "div_inplace", "copy_inplace"}
NP_KIND = {"Bool": np.bool_, "Int32": np.int32, "Int64": np.int64, "Float32": np.float32, "Float64": np.float64}


class Recorder:
    def __init__(self, C):
        self.C = C
        self.blob = bytearray()
        self.blob_index: dict[str, tuple[int, int]] = {}
        self.pending_bytes: dict[str, bytes] = {}
        self.calls: list[dict] = []
        self.seen: set[bytes] = set()
        self.skipped = 0
        self.capped = 0
        self.per_signature: dict[bytes, int] = {}

    # ---- serialisation
    def _bytes(self, storage) -> dict:
        arr = np.frombuffer(memoryview(storage), dtype=NP_KIND[storage.dtype.name]) if storage.size else np.zeros(0, NP_KIND[storage.dtype.name])
        raw = arr.tobytes()
        key = hashlib.sha1(raw).hexdigest()
        self.pending_bytes[key] = raw
        return {"dtype": storage.dtype.name, "size": int(storage.size), "blob": key}

    def finish(self):
        """Lay out the bytes the kept calls refer to; replace content hashes by [offset, length]."""
        def walk(node):
            if isinstance(node, dict):
                if isinstance(node.get("blob"), str):
                    key = node["blob"]
                    if key not in self.blob_index:
                        raw = self.pending_bytes[key]
                        self.blob_index[key] = (len(self.blob), len(raw))
                        self.blob += raw
                    node["blob"] = list(self.blob_index[key])
                for v in node.values():
                    walk(v)
            elif isinstance(node, list):
                for v in node:
                    walk(v)
        for call in self.calls:
            walk(call)

    def _arg(self, a):
        C = self.C
        if isinstance(a, C.TensorView):
            if a.storage.device != C.Device.Cpu or a.storage.size > MAX_STORAGE_ELEMENTS:
                raise OverflowError
            return {"view": self._bytes(a.storage), "shape": [int(s) for s in a.shape], "strides": [int(s) for s in a.strides],
                    "offset": int(a.offset)}
        if isinstance(a, C.Storage):
            if a.device != C.Device.Cpu or a.size > MAX_STORAGE_ELEMENTS:
                raise OverflowError
            return {"storage": self._bytes(a)}
        if isinstance(a, C.Dtype):
            return {"dtype_arg": a.name}
        if isinstance(a, bool):
            return {"bool": a}
        if isinstance(a, int):
            return {"int": a}
        if isinstance(a, float):
            return {"float": repr(a)}
        if isinstance(a, (list, tuple)):
            return {"list": [self._arg(x) for x in a]}
        raise TypeError(type(a))

    def wrap(self, name, fn):
        C = self.C

        def recorded(*args, **kwargs):
            try:
                call = {"fn": name, "args": [self._arg(a) for a in args], "kwargs": {k: self._arg(v) for k, v in kwargs.items()}}
            except (OverflowError, TypeError):
                self.skipped += 1
                return fn(*args, **kwargs)
            try:
                result = fn(*args, **kwargs)
            except Exception as e:  # the error class is part of the contract (RuntimeError / ValueError / TypeError)
                call["raises"] = type(e).__name__
                self._keep(call)
                raise
            if name in MUTATES_FIRST:
                call["after"] = self._bytes(args[0].storage)
            elif name in ("copy_view", "scatter_to_axes"):
                call["after"] = self._bytes(kwargs["out"].storage)
            elif isinstance(result, C.Storage):
                if result.size > MAX_STORAGE_ELEMENTS:
                    self.skipped += 1
                    return result
                call["result"] = self._bytes(result)
            elif isinstance(result, bool):
                call["result_bool"] = result
            self._keep(call)
            return result

        return recorded

    @staticmethod
    def _signature(node):
        """The call with the storage contents taken out."""
        if isinstance(node, dict):
            return {k: Recorder._signature(v) for k, v in node.items()
                    if k not in ("blob", "after", "result", "result_bool", "offset")}
        if isinstance(node, list):
            return [Recorder._signature(v) for v in node]
        return node

    def _keep(self, call):
        key = hashlib.sha1(json.dumps(call, sort_keys=True).encode()).digest()
        if key in self.seen:
            return
        self.seen.add(key)
        sig = hashlib.sha1(json.dumps(self._signature(call), sort_keys=True).encode()).digest()
        n = self.per_signature.get(sig, 0)
        if n >= MAX_PER_SIGNATURE:
            self.capped += 1
            return
        self.per_signature[sig] = n + 1
        self.calls.append(call)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("NT_REFERENCE", str(REPO.parent / "reference")))
    args = ap.parse_args()
    ref = Path(args.ref)
    from make_golden import import_reference

    nt = import_reference(ref)
    C = nt._C
    rec = Recorder(C)
    for name in VIEW_FUNCS:
        setattr(C, name, rec.wrap(name, getattr(C, name)))
    import pytest

    files = ["tests/test_ops/test_tensor_core.py", "tests/test_ops/test_tensor_core_ops.py", "tests/test_factories.py",
             "tests/test_ops/test_tensor_binary_ops.py", "tests/test_ops/test_tensor_unary_ops.py",
             "tests/test_ops/test_tensor_reduction_ops.py", "tests/test_ops/test_tensor_inplace_ops.py", "tests/test_autograd.py"]
    rc = pytest.main(["-q", "-p", "no:cacheprovider", "-x", *[str(ref / f) for f in files]])
    if rc != 0:
        raise SystemExit(f"the reference's own tests did not pass here (pytest exit code {rc})")
    rec.finish()
    manifest = json.dumps(rec.calls).encode()
    out = HERE / "reference_suite_trace.npz"
    np.savez_compressed(out, blob=np.frombuffer(bytes(rec.blob), dtype=np.uint8), manifest=np.frombuffer(manifest, dtype=np.uint8))
    by_fn: dict[str, int] = {}
    for c in rec.calls:
        by_fn[c["fn"]] = by_fn.get(c["fn"], 0) + 1
    print(f"{len(rec.calls)} calls kept ({rec.capped} beyond {MAX_PER_SIGNATURE} value sets per signature, {rec.skipped} too large), "
          f"{len(rec.blob) / 1024:.0f} KiB of storage bytes, file {out.stat().st_size / 1024:.0f} KiB")
    print(json.dumps(by_fn, sort_keys=True))


if __name__ == "__main__":
    main()
