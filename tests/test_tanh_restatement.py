"""The branch-light tanh the GPU kernels use (nanotorch_b200/csrc/tanh_exact.h) is compiled here for
the host and must equal the host libm's tanhf -- what the reference's CPU path calls
(src/cpp/ops/unary_ops.cu:106) -- bit for bit over a sweep of the whole float range.  The header
only uses IEEE +,-,*,/ and integer operations, so the device build returns the same bits."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent

# The two default-mode checks below walk the float range with a stride (about 10^8 arguments, seconds).
# NT_EXHAUSTIVE=1 in the environment makes them visit every one of the 2^32 arguments (OpenMP, about a
# minute on 8 cores); both pass in that form: tanh worst case 2 ulp from the host libm and always
# correctly rounded, sigmoid worst case 2 ulp from the reference's expression.
EXHAUSTIVE = os.environ.get("NT_EXHAUSTIVE") == "1"


def _build_and_run(tmp_path, name, source, stride):
    src = tmp_path / f"{name}.c"
    src.write_text(source)
    exe = tmp_path / name
    subprocess.run(["gcc", "-O2", "-fopenmp", "-fno-fast-math", "-ffp-contract=off", f"-DSTRIDE={1 if EXHAUSTIVE else stride}",
                    f"-I{REPO / 'nanotorch_b200' / 'csrc'}", "-o", str(exe), str(src), "-lm"], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    sys.stdout.write(out.stdout)
    return out

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


FAST_SRC = r"""
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include "cr_math.h"
static float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static long key(float f) { int32_t i; memcpy(&i, &f, 4); return i < 0 ? -(long)(i & 0x7fffffff) : i; }
int main(void) {
  long n = 0, over2 = 0, not_cr = 0, libm_vs_cr_max = 0;
#pragma omp parallel for schedule(dynamic, 1 << 16) reduction(+ : n, over2, not_cr) reduction(max : libm_vs_cr_max)
  for (uint64_t u = 0; u < 0x100000000ull; u += STRIDE) {
    float x = u2f((uint32_t)u);
    if (isnan(x)) continue;
    float libm = tanhf(x), fast = nt_tanh_fast_f32(x), cr = (float)tanh((double)x);
    if (labs(key(libm) - key(fast)) > 2) over2++;
    if (key(fast) != key(cr)) not_cr++;
    long d = labs(key(libm) - key(cr));
    if (d > libm_vs_cr_max) libm_vs_cr_max = d;
    n++;
  }
  printf("checked=%ld over_2ulp=%ld differs_from_correctly_rounded=%ld libm_vs_cr_max=%ld\n", n, over2, not_cr, libm_vs_cr_max);
  return (over2 != 0) || (not_cr != 0);
}
"""


def test_default_tanh_is_correctly_rounded_and_within_2ulp_of_host_libm(tmp_path):
    """cr_math.h (the default mode): equal to float(tanh(double(x))) for every argument of the sweep,
    hence within 2 ulp of the host libm, whose own distance to the correctly rounded value is at most 2."""
    out = _build_and_run(tmp_path, "tanh_fast_check", FAST_SRC, 41)
    assert out.returncode == 0, out.stdout
    assert "over_2ulp=0" in out.stdout and "differs_from_correctly_rounded=0" in out.stdout


SIGMOID_SRC = r"""
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include "sigmoid_f32.h"
static float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static long key(float f) { int32_t i; memcpy(&i, &f, 4); return i < 0 ? -(long)(i & 0x7fffffff) : i; }
int main(void) {
  long n = 0, over2 = 0, worst = 0;
#pragma omp parallel for schedule(dynamic, 1 << 16) reduction(+ : n, over2) reduction(max : worst)
  for (uint64_t u = 0; u < 0x100000000ull; u += STRIDE) {
    float x = u2f((uint32_t)u);
    if (isnan(x)) continue;
    float ref = 1.0f / (1.0f + expf(-x));   /* the reference's functor on the host libm */
    float got = nt_sigmoid_f32(x);
    long d = labs(key(ref) - key(got));
    if (d > worst) worst = d;
    if (d > 2) over2++;
    n++;
  }
  printf("checked=%ld over_2ulp=%ld worst=%ld\n", n, over2, worst);
  return over2 != 0;
}
"""


def test_sigmoid_within_2ulp_of_the_reference_expression_on_host_libm(tmp_path):
    out = _build_and_run(tmp_path, "sigmoid_check", SIGMOID_SRC, 53)
    assert out.returncode == 0, out.stdout


def test_sigmoid_table_is_what_its_generator_prints():
    """The 64 {hi, lo} pairs of 2^(j/64) in sigmoid_f32.h are the output of gen_exp2f_table.py, and hi + lo
    reproduces 2^(j/64) to better than 2^-45."""
    import re
    from fractions import Fraction

    csrc = REPO / "nanotorch_b200" / "csrc"
    printed = subprocess.run([sys.executable, str(csrc / "gen_exp2f_table.py")], capture_output=True, text=True, check=True).stdout
    rows = [l.strip() for l in printed.splitlines() if l.strip().startswith("{")]
    assert len(rows) == 64
    header = (csrc / "sigmoid_f32.h").read_text()
    for row in rows:
        assert row in header, row
    for j, row in enumerate(rows):
        hi, lo = (float.fromhex(t.rstrip("f")) for t in re.findall(r"-?0x[0-9a-f.]+p[+-]\d+f", row))
        exact = 2.0 ** (j / 64.0)                       # a double: 2^-53 relative
        assert abs((Fraction(hi) + Fraction(lo)) - Fraction(exact)) < Fraction(2) ** -44
