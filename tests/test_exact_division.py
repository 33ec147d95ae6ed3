"""CPU: the exact-division sequence every re-quantising CUDA kernel relies on.

The kernels divide thousands of values by one block scale.  Instead of div.rn per element they compute the correctly rounded
reciprocal y = RN(1/b) once and then  q0 = RN(a*y);  r = fma(-b, q0, a);  q = fma(r, y, q0)  (Markstein's correction step),
which must equal the IEEE quotient RN(a/b) bit for bit -- the bit-exactness of every quantised payload rests on it.  The same
sequence, in C with fmaf (oracle/gemm_oracle.c), is compared here with the hardware division on random operands, on operands
shaped like the kernels' (dividends |a| <= amax, divisor amax/127) and on all 2^23 dividend mantissas for divisors that are
hard for reciprocal-based division (mantissas next to a power of two, and next to sqrt(2) where RN(1/b) has its largest
relative error).  The window the kernels use the sequence in is b in [2^-60, 2^60]; outside they fall back to div.rn.
"""
import numpy as np
import pytest


def test_random_operands(oracle):
    rng = np.random.default_rng(0)
    n = 4_000_000
    a = (rng.standard_normal(n) * np.exp2(rng.integers(-40, 40, n))).astype(np.float32)
    b = (rng.uniform(1, 2, n) * np.exp2(rng.integers(-59, 59, n))).astype(np.float32)
    assert oracle.markstein_mismatches(a, b) == 0


def test_quantisation_shaped_operands(oracle):
    """Dividends inside [-amax, amax], divisor = amax/127 (and 127*x / amax, the GEMM epilogue's form)."""
    rng = np.random.default_rng(1)
    n = 4_000_000
    amax = (rng.uniform(1, 2, n) * np.exp2(rng.integers(-30, 20, n))).astype(np.float32)
    x = (rng.uniform(-1, 1, n).astype(np.float32) * amax).astype(np.float32)
    scale = (amax / np.float32(127)).astype(np.float32)
    assert oracle.markstein_mismatches(x, scale) == 0
    assert oracle.markstein_mismatches((np.float32(127) * x).astype(np.float32), amax) == 0
    # the extreme elements themselves: amax / scale and -amax / scale
    assert oracle.markstein_mismatches(amax, scale) == 0 and oracle.markstein_mismatches(-amax, scale) == 0


HARD = [1.0 + 2.0 ** -23, 2.0 - 2.0 ** -23, 1.0 + 2.0 ** -22, 1.4142135, 1.4142137, 1.5, 1.9999995, 1.0000005, 127.0 / 128.0,
        1.0 / 127.0, 3.0, 1.3333334, 1.6666666]


@pytest.mark.parametrize("b", HARD)
def test_every_dividend_mantissa_for_hard_divisors(oracle, b):
    assert oracle.markstein_sweep_mantissas(b, -10) == 0


def test_window_edges(oracle):
    rng = np.random.default_rng(2)
    n = 1_000_000
    a = rng.standard_normal(n).astype(np.float32)
    for e in (-60, 60):
        b = (rng.uniform(1, 2, n) * 2.0 ** e).astype(np.float32) if e < 0 else (rng.uniform(0.5, 1, n) * 2.0 ** e).astype(np.float32)
        scaled = (a * np.float32(2.0 ** (e // 2))).astype(np.float32)
        assert oracle.markstein_mismatches(scaled, b) == 0
