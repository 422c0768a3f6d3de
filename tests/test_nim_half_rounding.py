"""The Nim binding (hippo_leap_b200/nim/backends/b200.nim, floatToHalfRne) converts weights to fp16 with integer
arithmetic; no Nim toolchain exists here, so the same steps are restated below line for line and compared with
numpy's float32 -> float16 conversion (round to nearest even, subnormals kept), which is what the tested Python
mirror and the kernels' __float2half_rn do."""
import numpy as np


def float_to_half_rne(bits: np.ndarray) -> np.ndarray:
    bits = bits.astype(np.uint64)
    sign = (bits >> 16) & 0x8000
    a = bits & 0x7FFFFFFF
    out = np.zeros_like(bits)
    nan = a > 0x7F800000
    inf = (~nan) & (a >= 0x47800000)
    normal = (~nan) & (~inf) & (a >= 0x38800000)
    zero = a < 0x33000000
    sub = (~normal) & (~nan) & (~inf) & (~zero)
    h = (((a >> 23) - 112) << 10) | ((a >> 13) & 0x3FF)
    rem = a & 0x1FFF
    h = h + ((rem > 0x1000) | ((rem == 0x1000) & ((h & 1) == 1)))
    e = a >> 23
    m = (a & 0x7FFFFF) | 0x800000
    shift = np.where(sub, 126 - e, 14).astype(np.uint64)
    r = m >> shift
    rem2 = m & ((np.uint64(1) << shift) - np.uint64(1))
    halfway = np.uint64(1) << (shift - np.uint64(1))
    r = r + ((rem2 > halfway) | ((rem2 == halfway) & ((r & 1) == 1)))
    out = np.where(nan, 0x7E00, out)
    out = np.where(inf, 0x7C00, out)
    out = np.where(normal, h, out)
    out = np.where(sub, r, out)
    return (sign | out).astype(np.uint16)


def test_nim_half_conversion_equals_numpy_round_to_nearest_even():
    g = np.random.Generator(np.random.PCG64(1))
    vals = np.concatenate([
        g.standard_normal(200000).astype(np.float32),
        (g.standard_normal(200000) * 1e-6).astype(np.float32),          # subnormal halves
        (g.standard_normal(50000) * 3e4).astype(np.float32),            # near the overflow threshold
        np.array([0.0, -0.0, 65504.0, 65519.99, 65520.0, 65536.0, 1e9, np.inf, -np.inf, 2.0 ** -24, 2.0 ** -25,
                  1.5 * 2.0 ** -25, 2.0 ** -26, 6.1e-5, 6.103515625e-05, 1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11,
                  1.0 + 2.0 ** -11 + 2.0 ** -20], np.float32),
        g.integers(0, 2 ** 32, 300000, dtype=np.uint64).astype(np.uint32).view(np.float32)])
    vals = vals[~np.isnan(vals)]
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = float_to_half_rne(vals.view(np.uint32))
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, f"{bad.size} mismatches, first: {vals[bad[0]]!r} -> {got[bad[0]]:#06x}, numpy {want[bad[0]]:#06x}"
