"""The branch-light tanh the GPU kernels use (nanotorch_b200/csrc/tanh_exact.h) is compiled here for
the host and must equal the host libm's tanhf -- what the reference's CPU path calls
(src/cpp/ops/unary_ops.cu:106) -- bit for bit over a sweep of the whole float range.  The header
only uses IEEE +,-,*,/ and integer operations, so the device build returns the same bits."""

import subprocess
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent

SRC = r"""
#include <math.h>
#include <stdio.h>
#include "tanh_exact.h"
int main(void) {
  long bad = 0, n = 0;
  for (uint64_t u = 0; u < 0x100000000ull; u += 211) {
    float x = nt_u2f((uint32_t)u);
    float a = tanhf(x), b = nt_tanh_f32(x);
    if (nt_f2u(a) != nt_f2u(b) && !(isnan(a) && isnan(b))) {
      if (bad < 5) printf("x=%a libm=%a restated=%a\n", x, a, b);
      bad++;
    }
    n++;
  }
  /* every float in [-4, 4] around the N(0,1) bulk at a finer stride */
  for (uint32_t u = 0; u <= 0x40800000u; u += 13) {
    for (int s = 0; s < 2; ++s) {
      float x = nt_u2f(u | ((uint32_t)s << 31));
      if (nt_f2u(tanhf(x)) != nt_f2u(nt_tanh_f32(x))) bad++;
      n++;
    }
  }
  printf("checked=%ld mismatches=%ld\n", n, bad);
  return bad != 0;
}
"""


def test_restated_tanh_is_bit_exact_with_host_libm(tmp_path):
    src = tmp_path / "tanh_check.c"
    src.write_text(SRC)
    exe = tmp_path / "tanh_check"
    subprocess.run(["gcc", "-O2", "-fno-fast-math", "-ffp-contract=off", f"-I{REPO / 'nanotorch_b200' / 'csrc'}",
                    "-o", str(exe), str(src), "-lm"], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    sys.stdout.write(out.stdout)
    assert out.returncode == 0, out.stdout
    assert "mismatches=0" in out.stdout
