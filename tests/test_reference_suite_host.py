"""The reference's OWN test files, run against this package's host layer.

Where a checkout of the reference is present (NT_REFERENCE, or the default location the golden
generator uses), its tests of the Tensor object, of the op wrappers and of the factories are executed
in a subprocess with ``nanotorch`` aliased to ``nanotorch_b200``.  Those tests build Cpu tensors; this
library computes on the device only, so every test that reaches a kernel must fail with the library's
"requires Cuda" RuntimeError -- and with nothing else: view bookkeeping, indexing plans, shape and
dtype rules, factories, error classes and messages all have to behave as the reference's tests expect.
Nothing of the reference is copied: the files are run where they lie.  Skipped without a checkout."""

import os
import subprocess
import sys
import xml.etree.ElementTree as ET
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
REFERENCE = Path(os.environ.get("NT_REFERENCE", "/root/reference"))

ALIAS = '''
import sys
import nanotorch_b200 as _nt
from nanotorch_b200 import _C, nn, autograd, cuda, tensor as core
for _k in dir(_nt):
    if not _k.startswith("__"):
        globals()[_k] = getattr(_nt, _k)
for _name, _mod in (("_C", _C), ("nn", nn), ("autograd", autograd), ("cuda", cuda), ("core", core)):
    sys.modules["nanotorch." + _name] = _mod
'''

FILES = ["tests/test_ops/test_tensor_core.py", "tests/test_ops/test_tensor_core_ops.py", "tests/test_factories.py",
         "tests/test_ops/test_tensor_binary_ops.py", "tests/test_ops/test_tensor_unary_ops.py",
         "tests/test_ops/test_tensor_reduction_ops.py", "tests/test_ops/test_tensor_inplace_ops.py"]


@pytest.mark.skipif(not (REFERENCE / "tests").is_dir(), reason="no checkout of the reference here")
def test_reference_tests_only_fail_where_a_kernel_is_needed(tmp_path):
    pytest.importorskip("torch")  # the reference's tests compare against it
    pkg = tmp_path / "alias" / "nanotorch"
    pkg.mkdir(parents=True)
    (pkg / "__init__.py").write_text(ALIAS)
    os.symlink(REFERENCE / "src" / "nanotorch" / "testing.py", pkg / "testing.py")  # the reference's test helper
    report = tmp_path / "report.xml"
    env = dict(os.environ, PYTHONPATH=f"{tmp_path / 'alias'}{os.pathsep}{REPO}")
    proc = subprocess.run([sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", f"--junitxml={report}",
                           *[str(REFERENCE / f) for f in FILES]], cwd=tmp_path, env=env, capture_output=True, text=True)
    assert report.exists(), proc.stdout[-2000:] + proc.stderr[-2000:]
    passed, device_only, other = 0, 0, []
    for case in ET.parse(report).getroot().iter("testcase"):
        problems = list(case.findall("failure")) + list(case.findall("error"))
        if case.find("skipped") is not None:
            continue
        if not problems:
            passed += 1
            continue
        text = " ".join((p.get("message") or "") + (p.text or "") for p in problems)
        if "requires Cuda" in text:
            device_only += 1
        else:
            other.append(f"{case.get('classname')}::{case.get('name')}: {text[:300]}")
    assert not other, "host-layer behaviour differs from the reference's tests:\n" + "\n".join(other[:20])
    assert passed >= 400 and device_only > 0, (passed, device_only)
