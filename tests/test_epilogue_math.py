"""The approximations the 16-bit GEMM epilogues use for GELU and tanh, evaluated on the CPU with the constants read
from the CUDA header.

``gelu_erf_fast`` (``csrc/dfl_common.cuh``) is the rational approximation 7.1.26 of Abramowitz & Stegun for erf,
rewritten as ``max(x, 0) - |x| q(t) exp2(-w^2)``; a mistyped coefficient would stay below the rounding step of an
FP16 output near zero and above it elsewhere, so the constants are pinned here against ``math.erf`` in double
precision (absolute error below 5e-7 over [-12, 12]).  ``tanh_fast`` is ``1 - 2 / (1 + exp2(2 log2(e) x))``.
"""

import math
import re
from pathlib import Path

HEADER = Path(__file__).resolve().parent.parent / "disentangled_flash_b200" / "csrc" / "dfl_common.cuh"


def _body(name: str) -> str:
    text = HEADER.read_text()
    start = text.index(f"float {name}(float x)")
    return text[start:text.index("\n}", start)]


def _constants(body: str) -> list[float]:
    return [float(m) for m in re.findall(r"(-?\d+\.\d+(?:e-?\d+)?)f", body)]


def test_gelu_epilogue_constants():
    c = _constants(_body("gelu_erf_fast"))
    # in source order: sqrt(log2(e)/2), p/sqrt(log2 e), 1.0, a5/2, a4/2, a3/2, a2/2, a1/2, 0.0
    k_w, k_p, one, a5, a4, a3, a2, a1 = c[:8]
    assert one == 1.0
    assert abs(k_w - math.sqrt(math.log2(math.e) / 2)) < 1e-9
    assert abs(k_p - 0.3275911 / math.sqrt(math.log2(math.e))) < 1e-9

    def gelu_fast(x: float) -> float:
        ax = abs(x)
        w = ax * k_w
        t = 1.0 / (k_p * w + 1.0)
        e = 2.0 ** (-w * w)
        q = a5 * t + a4
        q = q * t + a3
        q = q * t + a2
        q = q * t + a1
        return -(ax * (q * t)) * e + max(x, 0.0)

    worst = 0.0
    for i in range(-12000, 12001):
        x = i / 1000.0
        exact = 0.5 * x * (1.0 + math.erf(x / math.sqrt(2.0)))
        worst = max(worst, abs(gelu_fast(x) - exact))
    assert worst < 5e-7, worst


def test_tanh_epilogue_constant():
    c = _constants(_body("tanh_fast"))
    assert abs(c[0] - 2.0 * math.log2(math.e)) < 1e-9
    for i in range(-2000, 2001):
        x = i / 100.0
        approx = 1.0 - 2.0 / (1.0 + 2.0 ** (c[0] * x))
        assert abs(approx - math.tanh(x)) < 1e-12
