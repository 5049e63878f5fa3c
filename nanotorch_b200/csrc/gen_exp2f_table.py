"""Prints the table of sigmoid_f32.h: 2^(j/64), j = 0..63, as hi + lo of two floats (hi the nearest float,
lo the nearest float of the rest), and the Cody-Waite pieces of ln2/64.  50-digit decimal arithmetic.

    python nanotorch_b200/csrc/gen_exp2f_table.py
"""
from decimal import Decimal, getcontext

import numpy as np

getcontext().prec = 60


def f32(d: Decimal) -> np.float32:
    return np.float32(float(d))


def hexf(x: np.float32) -> str:
    return float(x).hex() + "f"


LN2 = Decimal(2).ln()
rows = []
for j in range(64):
    v = Decimal(2) ** (Decimal(j) / Decimal(64))
    hi = f32(v)
    lo = f32(v - Decimal(float(hi)))
    rows.append(f"  {{{hexf(hi)}, {hexf(lo)}}},")
print("\n".join(rows))
c = LN2 / 64
c1 = np.float32(1419.0 / 131072.0)  # the leading 11 bits of ln2/64: n * c1 - x is exact for |n| < 2^14
c2 = f32(c - Decimal(float(c1)))
c3 = f32(c - Decimal(float(c1)) - Decimal(float(c2)))
print("C1", hexf(c1), "C2", hexf(c2), "C3", hexf(c3), "64/ln2", hexf(f32(Decimal(64) / LN2)))
