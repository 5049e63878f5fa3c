"""Replay of the reference's own test-suite at the native-module boundary.

tests/golden/reference_suite_trace.npz holds every distinct call the reference's tests make into its
``_C`` module on the CPU path (recorded by tests/golden/make_suite_trace.py from the reference itself):
function, views (dtype / shape / strides / offset over the storage bytes), scalars, axis lists -- and
what the reference's kernels returned.  Here each call is issued to this library with the same arguments
on the device, through the C ABI, and the result compared:

  bit-exact   add, subtract, multiply, divide, neg, relu, sqrt, comparisons, equals, max, min, argmax,
              argmin, in-place ops, copies, index-array gather / scatter, cast, integer pow / sum / matmul
  <= 2 ulp    exp, log, tanh, sigmoid, pow in Float32 (<= 4 ulp of a double in Float64)
  sum         |diff| <= 1e-5 * sum|x| (Float32), 1e-13 * sum|x| (Float64)
  matmul      |diff| <= 1e-4 * (|A||B|)_ij (Float32, the default 3xTF32 mode), 1e-13 (Float64)
  errors      a call the reference rejects must be rejected here with the same exception class

The shapes (0-d to 5-d), strides (0, negative, transposed), offsets and dtypes are the ones the
reference's authors chose for their tests.  Without a GPU only the file itself is checked.
"""

import builtins
import json
from pathlib import Path

import numpy as np
import pytest

from tests.util import ulp_distance

REPO = Path(__file__).resolve().parent.parent
TRACE = REPO / "tests" / "golden" / "reference_suite_trace.npz"
NP_KIND = {"Bool": np.bool_, "Int32": np.int32, "Int64": np.int64, "Float32": np.float32, "Float64": np.float64}
EXACT = {"add", "subtract", "multiply", "divide", "neg", "relu", "sqrt", "pw_equal", "pw_greater", "pw_greater_eq", "max",
         "min", "argmax", "argmin", "add_inplace", "sub_inplace", "mul_inplace", "div_inplace", "copy_inplace", "copy_view",
         "clone_contiguous_view_from", "gather_from_axes", "scatter_to_axes", "cast"}
ULP = {"exp", "log", "tanh", "sigmoid", "pow"}


def load_trace():
    z = np.load(TRACE)
    return json.loads(bytes(z["manifest"]).decode()), z["blob"]


def test_trace_file_is_complete():
    """No GPU needed: the file loads, is of the recorded size, and every function it names exists here."""
    import nanotorch_b200 as nt

    calls, blob = load_trace()
    assert len(calls) >= 1000 and len(blob) > 500_000
    names = {c["fn"] for c in calls}
    assert len(names) == 32 and all(hasattr(nt._C, n) for n in names)
    assert sum("raises" in c for c in calls) >= 10


class Replayer:
    def __init__(self, nt, blob):
        self.nt, self._C, self.blob = nt, nt._C, blob
        self.dt = {"Bool": nt.bool_, "Int32": nt.int32, "Int64": nt.int64, "Float32": nt.float32, "Float64": nt.float64}

    def host(self, spec) -> np.ndarray:
        off, n = spec["blob"]
        return np.frombuffer(self.blob[off:off + n].tobytes(), dtype=NP_KIND[spec["dtype"]])

    def storage(self, spec):
        a = self.host(spec)
        s = self._C.Storage.allocate(spec["size"], self.dt[spec["dtype"]], self.nt.Device.Cuda)
        if a.size:
            s.upload(a.ctypes.data, a.nbytes)
        return s

    def download(self, storage, dtype_name) -> np.ndarray:
        out = np.empty(storage.size, NP_KIND[dtype_name])
        if out.size:
            storage.download(out.ctypes.data, out.nbytes)
        return out

    def arg(self, a, keep):
        if "view" in a:
            s = self.storage(a["view"])
            keep.append((s, a))
            return self._C.TensorView(s, tuple(a["shape"]), tuple(a["strides"]), a["offset"])
        if "storage" in a:
            s = self.storage(a["storage"])
            keep.append((s, a))
            return s
        if "dtype_arg" in a:
            return self.dt[a["dtype_arg"]]
        if "bool" in a:
            return a["bool"]
        if "int" in a:
            return a["int"]
        if "float" in a:
            return float(a["float"])
        return [self.arg(x, keep) for x in a["list"]]

    def np_view(self, a) -> np.ndarray:
        base = self.host(a["view"])
        if not a["shape"]:
            return base[a["offset"]].reshape(())
        return np.lib.stride_tricks.as_strided(base[a["offset"]:], shape=a["shape"],
                                               strides=[s * base.itemsize for s in a["strides"]])


def same_bits(got, want):
    if got.dtype.kind == "f":
        u = f"u{got.itemsize}"
        return bool(((got.view(u) == want.view(u)) | (np.isnan(got) & np.isnan(want))).all())
    return bool(np.array_equal(got, want))


@pytest.mark.gpu
def test_replay_on_the_device(nt):
    calls, blob = load_trace()
    r = Replayer(nt, blob)
    _C = nt._C
    failures, worst_ulp, counts = [], {}, {}
    for i, call in enumerate(calls):
        fn = call["fn"]
        keep: list = []
        args = [r.arg(a, keep) for a in call["args"]]
        kwargs = {k: r.arg(v, keep) for k, v in call["kwargs"].items()}
        counts[fn] = counts.get(fn, 0) + 1
        if "raises" in call:
            try:
                getattr(_C, fn)(*args, **kwargs)
                failures.append(f"#{i} {fn}: the reference raises {call['raises']}, nothing raised here")
            except getattr(builtins, call["raises"]):
                pass
            except Exception as e:  # noqa: BLE001
                failures.append(f"#{i} {fn}: the reference raises {call['raises']}, got {type(e).__name__}: {e}")
            continue
        try:
            result = getattr(_C, fn)(*args, **kwargs)
        except Exception as e:  # noqa: BLE001
            failures.append(f"#{i} {fn}: {type(e).__name__}: {e}")
            continue
        if "result_bool" in call:
            if bool(result) != call["result_bool"]:
                failures.append(f"#{i} {fn}: {result} != {call['result_bool']}")
            continue
        if "after" in call:
            target = keep[0][0] if fn not in ("copy_view", "scatter_to_axes") else kwargs["out"].storage
            want = r.host(call["after"])
            got = r.download(target, call["after"]["dtype"])
        else:
            want = r.host(call["result"])
            if result.dtype.name != call["result"]["dtype"] or result.size != call["result"]["size"]:
                failures.append(f"#{i} {fn}: result is {result.dtype.name}[{result.size}], the reference's "
                                f"{call['result']['dtype']}[{call['result']['size']}]")
                continue
            got = r.download(result, call["result"]["dtype"])
        is_float = want.dtype.kind == "f"
        if fn in EXACT or not is_float:
            ok = same_bits(got, want)
        elif fn in ULP:
            ok = not (np.isnan(got) ^ np.isnan(want)).any()
            if ok and want.size:
                if want.dtype == np.float32:
                    d = int(ulp_distance(got, want).max())
                    limit = 2
                else:
                    fin = np.isfinite(want) & np.isfinite(got)
                    ok = bool(np.array_equal(got[~fin], want[~fin]) or (np.isnan(got[~fin]) == np.isnan(want[~fin])).all())
                    d = int((np.abs(got[fin] - want[fin]) / np.spacing(np.abs(want[fin]))).max()) if fin.any() else 0
                    limit = 4
                worst_ulp[(fn, want.dtype.name)] = max(worst_ulp.get((fn, want.dtype.name), 0), d)
                ok = ok and d <= limit
        elif fn == "sum":
            x = r.np_view(call["args"][0]).astype(np.float64)
            scale = np.abs(x).sum() + 1e-300
            rel = 1e-5 if want.dtype == np.float32 else 1e-13
            with np.errstate(all="ignore"):
                ok = bool(((np.abs(got.astype(np.float64) - want) <= rel * scale) | (got == want) | (np.isnan(got) & np.isnan(want))).all())
        elif fn == "matmul":
            a, b = r.np_view(call["args"][0]).astype(np.float64), r.np_view(call["args"][1]).astype(np.float64)
            with np.errstate(all="ignore"):
                bound = (np.abs(a) @ np.abs(b)).reshape(-1) + 1e-300
                rel = 1e-4 if want.dtype == np.float32 else 1e-13
                ok = bool(((np.abs(got.astype(np.float64) - want) <= rel * bound) | (got == want) | (np.isnan(got) & np.isnan(want))).all())
        else:
            ok = False
        if not ok:
            bad = np.flatnonzero(~((got == want) | (np.isnan(got.astype(np.float64)) & np.isnan(want.astype(np.float64)))))
            j = int(bad[0]) if bad.size else -1
            failures.append(f"#{i} {fn} {call['args'][:1]}: {bad.size} of {want.size} elements differ, first at {j}: "
                            f"got {got[j] if j >= 0 else ''} want {want[j] if j >= 0 else ''}")
    _C.cuda_sync()
    print(f"replayed {len(calls)} calls of {len(counts)} functions; worst ulp distances {worst_ulp}")
    assert not failures, f"{len(failures)} of {len(calls)} calls differ:\n" + "\n".join(failures[:40])
