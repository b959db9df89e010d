"""The int8 quantiser of the oracle against an exact-rational evaluation of its
definition (the reference has no quantisation, so this definition is the pin)."""
from fractions import Fraction

import numpy as np
import torch

from oracle import attention_oracle as oracle


def _rne_to_format(fr, mant_bits, emin, emax_val):
    """Round a non-negative Fraction to the nearest value of a binary float format (ties to even)."""
    if fr == 0:
        return Fraction(0)
    import math
    e = math.floor(math.log2(fr))
    while Fraction(2) ** e > fr:
        e -= 1
    while Fraction(2) ** (e + 1) <= fr:
        e += 1
    e = max(e, emin)
    ulp = Fraction(2) ** (e - mant_bits)
    qn = fr / ulp
    lo = qn.numerator // qn.denominator
    rem = qn - lo
    if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and lo % 2 == 1):
        lo += 1
    val = lo * ulp
    return val if val <= emax_val else None  # None = overflow to inf


def _exact_codes(row):
    xs = [Fraction(float(v)) for v in row]
    amax = max(abs(v) for v in xs)
    q32 = _rne_to_format(amax / 127, 23, -126, Fraction(2) ** 128)       # fp32 division result
    s = _rne_to_format(q32, 10, -14, Fraction(65504))                    # fp16 rounding
    if s is None:
        return [0] * len(xs), float("inf")
    if s == 0:
        return [0] * len(xs), 0.0
    codes = []
    for v in xs:
        sign = -1 if v < 0 else 1
        qf = _rne_to_format(abs(v) / s, 23, -126, Fraction(2) ** 128)     # fp32 division result
        lo = qf.numerator // qf.denominator
        rem = qf - lo
        if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and lo % 2 == 1):
            lo += 1
        codes.append(max(-127, min(127, sign * lo)))
    return codes, float(s)


def test_quantiser_matches_exact_rational_definition():
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(6, 2, 64, generator=g) * 2).to(torch.bfloat16)
    x[0, 0] = 0                      # all-zero row: scale 0, codes 0
    x[1, 1] *= 1e-6                  # subnormal fp16 scale
    x[2, 0, :4] = torch.tensor([0.5, 1.5, 2.5, -2.5]).to(torch.bfloat16) * 127 / 127  # ties
    codes, scales = oracle.quantize_kv_int8(x)
    for t in range(x.shape[0]):
        for h in range(x.shape[1]):
            want, s = _exact_codes(x[t, h].to(torch.float32).tolist())
            assert float(scales[t, h]) == s, (t, h)
            assert codes[t, h].tolist() == want, (t, h)


def test_quantiser_range_and_roundtrip():
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(512, 8, 128, generator=g) * 2).to(torch.bfloat16)
    codes, scales = oracle.quantize_kv_int8(x)
    assert codes.dtype == torch.int8 and scales.dtype == torch.float16
    assert int(codes.min()) >= -127 and int(codes.max()) <= 127
    assert int(codes.abs().amax(-1).min()) >= 126  # the largest element of every row maps to +-127 (or 126 after scale rounding)
    err = (oracle.dequantize_kv_int8(codes, scales) - x.to(torch.float32)).abs().max()
    assert float(err) < 0.06
