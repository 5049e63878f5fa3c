"""The reference's OWN test files, run against this package's host layer.

Where a checkout of the reference is present (NT_REFERENCE, or the default location the golden
generator uses), its test files are executed in a subprocess, in place (nothing is copied), with
``nanotorch`` aliased to ``nanotorch_b200``.  They build Cpu tensors; this library computes on the device
only.  Two runs:

1. On libnt_b200.so.  Every test that reaches a kernel must fail with the library's "requires Cuda"
   RuntimeError -- and with nothing else: view bookkeeping, index plans, shape and dtype rules, factories,
   error classes and messages behave as the reference's tests expect wherever no kernel is needed.
2. With the reference's own native module (oracle/_ref, Cpu path) substituted for ``nanotorch_b200._C``
   (tests/ref_backend.py).  Now the kernels exist, and the whole Python layer of this package -- Tensor,
   the autograd op classes and their composed backward chains, nn, index-array getitem/setitem -- has to
   pass every one of those tests, the autograd tests included: the reference's finite-difference
   gradcheck of every op class on random strided float64 inputs of up to five dimensions (its ``op_spec``
   tooling is loaded from the checkout and each op's declared input specification is attached to this
   package's class of the same name; only the 100-fold repetition marked slow there is left out).

3. The other way round: the reference's own Python package on this library's ``_C`` shim.

4. On a GPU (``-m gpu``): the reference's CUDA-parametrised tests, live on libnt_b200.so.

Skipped without a checkout."""

import os
import subprocess
import sys
import xml.etree.ElementTree as ET
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
REFERENCE = Path(os.environ.get("NT_REFERENCE", str(REPO.parent / "reference")))  # a checkout beside this repository

ALIAS = '''
import sys
{prologue}
import nanotorch_b200 as _nt
from nanotorch_b200 import _C, nn, autograd, cuda
core = sys.modules["nanotorch_b200.tensor"]  # the package attribute `tensor` is the factory function
for _k in dir(_nt):
    if not _k.startswith("__"):
        globals()[_k] = getattr(_nt, _k)
for _name, _mod in (("_C", _C), ("nn", nn), ("autograd", autograd), ("cuda", cuda), ("core", core),
                    ("_data_type", _nt), ("factories", _nt)):
    sys.modules["nanotorch." + _name] = _mod
# the reference's test helpers, loaded from where they lie
import importlib.util as _ilu
_spec = _ilu.spec_from_file_location("nanotorch.autograd.ops_spec", r"{ops_spec}")
_mod = _ilu.module_from_spec(_spec)
sys.modules["nanotorch.autograd.ops_spec"] = _mod
_spec.loader.exec_module(_mod)
autograd.ops_spec = _mod
# the input specification each op class of the reference declares for that tooling (`op_spec = (...)`),
# read from the reference's sources where they lie and attached to this package's class of the same name
import ast as _ast
for _file in ("ops_binary", "ops_unary", "ops_reduction", "ops_special"):
    _tree = _ast.parse(open(r"{autograd_dir}/" + _file + ".py").read())
    for _cls in (_n for _n in _tree.body if isinstance(_n, _ast.ClassDef)):
        for _stmt in _cls.body:
            if isinstance(_stmt, _ast.Assign) and getattr(_stmt.targets[0], "id", None) == "op_spec" and hasattr(autograd, _cls.name):
                _expr = compile(_ast.Expression(_stmt.value), _file, "eval")
                setattr(getattr(autograd, _cls.name), "op_spec", eval(_expr, {{"sp": _mod}}))
'''
SWAP_BACKEND = 'import tests.ref_backend as _rb\nsys.modules["nanotorch_b200._C"] = _rb'

OP_FILES = ["tests/test_ops/test_tensor_core.py", "tests/test_ops/test_tensor_core_ops.py", "tests/test_factories.py",
            "tests/test_ops/test_tensor_binary_ops.py", "tests/test_ops/test_tensor_unary_ops.py",
            "tests/test_ops/test_tensor_reduction_ops.py", "tests/test_ops/test_tensor_inplace_ops.py"]

pytestmark = pytest.mark.skipif(not (REFERENCE / "tests").is_dir(), reason="no checkout of the reference here")


def _run(tmp_path, prologue, files, extra=()):
    """(passed, [(test id, failure text)]) of the reference's test files under the alias."""
    pytest.importorskip("torch")  # the reference's tests compare against it
    pkg = tmp_path / "alias" / "nanotorch"
    pkg.mkdir(parents=True)
    ops_spec = REFERENCE / "src" / "nanotorch" / "autograd" / "ops_spec.py"
    (pkg / "__init__.py").write_text(ALIAS.format(prologue=prologue, ops_spec=ops_spec, autograd_dir=ops_spec.parent))
    os.symlink(REFERENCE / "src" / "nanotorch" / "testing.py", pkg / "testing.py")
    report = tmp_path / "report.xml"
    env = dict(os.environ, PYTHONPATH=f"{tmp_path / 'alias'}{os.pathsep}{REPO}")
    proc = subprocess.run([sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", f"--junitxml={report}", *extra,
                           *[str(REFERENCE / f) for f in files]], cwd=tmp_path, env=env, capture_output=True, text=True)
    assert report.exists(), proc.stdout[-2000:] + proc.stderr[-2000:]
    passed, failed = 0, []
    for case in ET.parse(report).getroot().iter("testcase"):
        if case.find("skipped") is not None:
            continue
        problems = list(case.findall("failure")) + list(case.findall("error"))
        if not problems:
            passed += 1
        else:
            text = " ".join((p.get("message") or "") + (p.text or "") for p in problems)
            failed.append((f"{case.get('classname')}::{case.get('name')}", text))
    return passed, failed


def test_on_the_device_library_only_kernel_calls_fail(tmp_path):
    passed, failed = _run(tmp_path, "", OP_FILES)
    other = [f"{name}: {text[:300]}" for name, text in failed if "requires Cuda" not in text]
    assert not other, "host-layer behaviour differs from the reference's tests:\n" + "\n".join(other[:20])
    assert passed >= 400 and failed, (passed, len(failed))


def test_on_the_reference_cpu_backend_everything_passes(tmp_path):
    from oracle import oracle as O

    if not O.ref_available():
        pytest.skip("oracle/_ref is not built")
    passed, failed = _run(tmp_path, SWAP_BACKEND, OP_FILES + ["tests/test_autograd.py"], extra=("-k", "not test_ops_specs_extensive"))
    assert not failed, "\n".join(f"{name}: {text[:300]}" for name, text in failed[:20])
    assert passed >= 1230, passed


def test_the_references_python_layer_runs_on_this_librarys_shim(tmp_path):
    """The other direction (the ctypes shim dropped in as ``nanotorch/_C.py``): the reference's OWN Python package, its files
    linked in place, with ``nanotorch/_C.py`` forwarding to ``nanotorch_b200._C`` instead of the pybind11
    module.  Its tests build Cpu tensors, so whatever reaches a kernel fails with "requires Cuda"; nothing
    else may fail -- Dtype/Device enum behaviour, Storage's buffer protocol, from_iterable, TensorView,
    the factories and the error classes are what the reference's Python layer expects of ``_C``."""
    pytest.importorskip("torch")
    src = REFERENCE / "src" / "nanotorch"
    pkg = tmp_path / "refpy" / "nanotorch"
    for path in src.rglob("*.py"):
        dst = pkg / path.relative_to(src)
        dst.parent.mkdir(parents=True, exist_ok=True)
        os.symlink(path, dst)
    (pkg / "_C.py").write_text("from nanotorch_b200._C import *  # noqa: F401,F403\n"
                               "from nanotorch_b200._C import Device, Dtype, Storage, TensorView  # noqa: F401\n")
    report = tmp_path / "report.xml"
    env = dict(os.environ, PYTHONPATH=f"{tmp_path / 'refpy'}{os.pathsep}{REPO}")
    files = OP_FILES + ["tests/test_autograd.py"]
    proc = subprocess.run([sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", f"--junitxml={report}",
                           *[str(REFERENCE / f) for f in files]], cwd=tmp_path, env=env, capture_output=True, text=True)
    assert report.exists(), proc.stdout[-2000:] + proc.stderr[-2000:]
    passed, other = 0, []
    for case in ET.parse(report).getroot().iter("testcase"):
        if case.find("skipped") is not None:
            continue
        problems = list(case.findall("failure")) + list(case.findall("error"))
        text = " ".join((p.get("message") or "") + (p.text or "") for p in problems)
        if not problems:
            passed += 1
        elif "requires Cuda" not in text:
            other.append(f"{case.get('classname')}::{case.get('name')}: {text[:300]}")
    assert not other, "\n".join(other[:20])
    assert passed >= 400, passed


@pytest.mark.gpu
def test_on_a_gpu_the_cuda_parametrised_tests_pass(tmp_path):
    """The reference's CUDA-parametrised tests against libnt_b200.so on a device.

    Most of the reference's tests take a ``device`` fixture with a "cpu" and a "cuda" parameter
    (tests/conftest.py:5-20), and the "cuda" half is skipped where no device is present.  Here, on a GPU,
    through the same in-place alias, that half runs on this library -- Python layer and kernels together:
    the CPU-vs-CUDA differential tests of every unary op (tests/test_ops/test_tensor_unary_ops.py:92-142),
    the random batched products (tests/test_ops/test_tensor_binary_ops.py:344-357), reductions over
    views, in-place semantics, the autograd known answers.  Every test that ran with the "cuda" parameter
    must pass.  Tests that build Cpu tensors reach no kernel here (this library computes on the device
    only): those may fail with the "requires Cuda" error and with nothing else.  Needs a checkout of the
    reference (NT_REFERENCE): skipped where there is none."""
    import nanotorch_b200 as nt

    if not nt.is_available():
        pytest.skip("no CUDA device")
    passed, failed = _run(tmp_path, "", OP_FILES + ["tests/test_autograd.py"], extra=("-k", "not test_ops_specs_extensive"))
    is_cuda = lambda name: "[cuda" in name or "-cuda" in name  # noqa: E731
    unexplained = [(n, t) for n, t in failed if "requires Cuda" not in t]
    cases = [c for c in ET.parse(tmp_path / "report.xml").getroot().iter("testcase") if c.find("skipped") is None]
    cuda_ran = [c for c in cases if is_cuda(c.get("name") or "")]
    cuda_passed = [c for c in cuda_ran if not (list(c.findall("failure")) + list(c.findall("error")))]
    cuda_on_cpu_tensors = [n for n, t in failed if is_cuda(n) and "requires Cuda" in t]
    print(f"reference suite on the device: {len(cases)} tests ran, {passed} passed; cuda-parametrised: {len(cuda_ran)} ran, "
          f"{len(cuda_passed)} passed, {len(cuda_on_cpu_tensors)} build Cpu tensors whatever the parameter and stop at "
          f"'requires Cuda'; {len(unexplained)} failures not explained by 'requires Cuda'")
    for n, t in unexplained:
        print("UNEXPLAINED", n, "::", " ".join(t.split())[:600])
    assert not unexplained, f"{len(unexplained)} failures, first: " + "\n".join(f"{n}: {t[:400]}" for n, t in unexplained[:10])
    assert len(cuda_passed) >= 350, len(cuda_passed)


GOLDEN_RUN = r'''
import sys
import numpy as np
import tests.ref_backend as rb
sys.modules["nanotorch_b200._C"] = rb
import nanotorch_b200 as nt
import nanotorch_b200.nn as nn

g = np.load(sys.argv[1])
bits = lambda a: np.asarray(a, dtype=np.float32).view(np.uint32)
T = lambda a, grad=False: nt.Tensor.from_numpy(np.asarray(a, dtype=np.float32), "cpu", requires_grad=grad)

# configuration 1: 784 -> 256 -> 10, ReLU, 100 SGD steps on one batch
nt.manual_seed(0)
model = nn.Sequential(nn.Linear(784, 256, device="cpu"), nn.ReLU(), nn.Linear(256, 10, device="cpu"))
X = T(np.random.default_rng(1).standard_normal((256, 784)))
Y = T(np.random.default_rng(2).standard_normal((256, 10)))
opt = nn.GradientDescent(model.parameters(), lr=0.01)
losses = []
for _ in range(100):
    loss = nt.mean((model(X) - Y) ** 2)
    opt.zero_grad(); loss.backward(); opt.step()
    losses.append(loss.item())
assert np.array_equal(bits(losses), bits(g["mlp1/losses"])), "loss curve"
assert np.array_equal(bits(model.parameters()[2].numpy()), bits(g["mlp1/W2_final"])), "final W2"
assert np.array_equal(bits(model.parameters()[1].numpy()), bits(g["mlp1/b1_final"])), "final b1"

# every binary op x layout and every unary op: forward and backward through this package's autograd
a, G = g["ew/in/a"], g["ew/in/G"]
for name, fn in dict(add=lambda x, y: x + y, sub=lambda x, y: x - y, mul=lambda x, y: x * y, div=lambda x, y: x / y).items():
    for layout in ("contig", "bcast", "transposed"):
        src = {"contig": "d" if name == "div" else "b", "bcast": "dv" if name == "div" else "v",
               "transposed": "dt" if name == "div" else "bt"}[layout]
        x, y = T(a, True), T(g["ew/in/" + src], True)
        res = fn(x, y.T if layout == "transposed" else y)
        (res * T(G)).sum().backward()
        for got, key in ((res, "out"), (x.grad, "gx"), (y.grad, "gy")):
            assert np.array_equal(bits(got.numpy()), bits(g[f"ew/{name}/{layout}/{key}"])), (name, layout, key)
unary = {"exp": ("n", lambda t: t.exp()), "neg": ("n", lambda t: -t), "relu": ("n", nt.relu), "tanh": ("n", nt.tanh),
         "sigmoid": ("n", nt.sigmoid), "log": ("p", lambda t: t.log()), "sqrt": ("p", nt.sqrt),
         "pow2": ("a", lambda t: t ** 2.0), "pow3.7": ("p", lambda t: t ** 3.7), "powm1": ("p", lambda t: t ** -1.0)}
for name, (src, fn) in unary.items():
    x = T(g["ew/in/" + src], True)
    res = fn(x)
    (res * T(G)).sum().backward()
    assert np.array_equal(bits(res.numpy()), bits(g[f"ew/{name}/out"])), name
    assert np.array_equal(bits(x.grad.numpy()), bits(g[f"ew/{name}/gx"])), name + " backward"
# reductions with backward
xr = g["red/in/x"]
for axes in [(0,), (1,), (2,), (0, 2), (1, 2), (0, 1, 2), None]:
    for keepdim in (False, True):
        for name in ("sum", "mean", "max", "min"):
            t = T(xr, True)
            res = getattr(t, name)(axes, keepdim)
            key = f"red/{name}/{'all' if axes is None else ''.join(map(str, axes))}/{int(keepdim)}"
            assert np.array_equal(bits(res.numpy()), bits(g[key + "/out"])), key
            res.sum().backward()
            assert np.array_equal(bits(t.grad.numpy()), bits(g[key + "/gx"])), key + " backward"
print("golden-ok")
'''


def test_golden_fixtures_through_this_packages_python_layer_on_the_reference_cpu_backend(tmp_path):
    """The fixtures were produced by the reference's Python layer on its native module; this package's
    Python layer on that same native module must reproduce them bit for bit -- the 100-step loss curve of
    configuration 1 with its final parameters, and forward + backward of every op.  What differs between
    the two runs is only the host code: op classes, backward chains, unbroadcast, the optimizer."""
    from oracle import oracle as O

    if not O.ref_available():
        pytest.skip("oracle/_ref is not built")
    script = tmp_path / "golden_run.py"
    script.write_text(GOLDEN_RUN)
    env = dict(os.environ, PYTHONPATH=str(REPO))
    proc = subprocess.run([sys.executable, str(script), str(REPO / "tests" / "golden" / "reference_cpu.npz")],
                          cwd=tmp_path, env=env, capture_output=True, text=True)
    assert proc.returncode == 0 and "golden-ok" in proc.stdout, proc.stdout[-1500:] + proc.stderr[-3000:]
