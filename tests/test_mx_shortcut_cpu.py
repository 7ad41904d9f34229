"""Proof by enumeration of the MXFP4 single-multiply shortcut of the fused quantise kernel.

The reference divides: code = e2m1_rne(fl(fl(t * c) / s)) with t the unscaled butterfly output,
c = fl32(1/sqrt(g)) and s = fl(2^(e-2) / 0.75) (src/quantization/quantizer.py:162-165, :175-182,
quant_ops.py:57-71 of IST-DASLab/FP-Quant).  The kernel (csrc/quantize.cu, `mx_code_multiplier`)
computes ONE rounded product t * (m * 2^(2-e)) instead, rounded toward zero when c is a power of two
and to nearest otherwise, and converts that to E2M1.  The two can only disagree next to one of the seven
rounding boundaries of the E2M1 grid, so this test walks every fp32 value of t within ULPS ulps of
each boundary's preimage (both signs, all five rotation sizes, a spread of exponents) and demands the
same code from a numpy emulation of the kernel's product and from the oracle's two-step chain.  The
multiplier constants are read from the CUDA source so that the proof cannot drift from the kernel.
"""
import os
import re

import numpy as np
import pytest
import torch

from oracle import fp4

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCE = os.path.join(ROOT, "fp-quant_b200", "csrc", "quantize.cu")
BOUNDARIES = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
ULPS = 20000
HADAMARD_SCALE = {0: 1.0, 16: 0.25, 32: 0.17677669529663687, 64: 0.125, 128: 0.08838834764831845}
POWER_OF_TWO = (0, 16, 64)


def multiplier_bits():
    """{group: fp32 bit pattern of m} from `mx_code_multiplier` in the kernel source."""
    text = open(SOURCE).read()
    body = text[text.index("mx_code_multiplier(int e)"):]
    body = body[: body.index("return pack2")]
    found = {int(g): int(h, 16) for g, h in re.findall(r"GH == (\d+) \? (0x[0-9a-fA-F]+)u", body)}
    last = re.findall(r":\s*(0x[0-9a-fA-F]+)u;", body)
    assert set(found) == {0, 16, 64, 32} and len(last) == 1, "mx_code_multiplier no longer has the expected form"
    found[128] = int(last[0], 16)
    return found


def f32(bits):
    return np.asarray(bits, dtype=np.uint32).view(np.float32)


def product_rn(t, m):
    """fl32(t * m), round to nearest even: the fp64 product of two fp32 numbers is exact."""
    return (t.astype(np.float64) * np.float64(m)).astype(np.float32)


def product_rz(t, m):
    exact = t.astype(np.float64) * np.float64(m)
    r = exact.astype(np.float32)
    too_big = np.abs(r.astype(np.float64)) > np.abs(exact)
    return np.where(too_big, np.nextafter(r, np.float32(0)), r).astype(np.float32)


def e2m1_rne_codes(v):
    """What `cvt.rn.satfinite.e2m1x2.f32` followed by the zero patch yields (ties to the even code)."""
    v = torch.from_numpy(np.ascontiguousarray(v))
    return fp4.e2m1_codes(v.unsqueeze(-1), torch.ones(v.shape[0], 1), 1).squeeze(-1).numpy()


def test_constants_are_the_documented_ones():
    bits = multiplier_bits()
    four_thirds = np.float32(1.0) / np.float32(0.75)
    for g in POWER_OF_TWO:
        assert f32(bits[g]) == np.float32(0.75) * np.float32(HADAMARD_SCALE[g])
    for g in (32, 128):
        assert f32(bits[g]) == np.float32(np.float32(HADAMARD_SCALE[g]) / four_thirds)


@pytest.mark.parametrize("group", [0, 16, 32, 64, 128])
def test_single_product_gives_the_reference_code_near_every_boundary(group):
    m0 = f32(multiplier_bits()[group])
    c = np.float32(HADAMARD_SCALE[group])
    checked = 0
    for e in (-120, -37, -1, 0, 1, 2, 9, 64, 120):            # the kernel takes the shortcut for |e| <= 120
        s = np.float32(2.0 ** (e - 2)) / np.float32(0.75)     # fl(2^(e-2) / 0.75)
        m = np.float32(m0 * np.float32(2.0 ** (2 - e)))       # exact: a power-of-two factor
        assert np.float64(m) == np.float64(m0) * 2.0 ** (2 - e)
        for b in BOUNDARIES:
            centre = np.float32(np.float64(b) * np.float64(s) / np.float64(c))
            base = int(centre.view(np.uint32))
            bits = (base + np.arange(-ULPS, ULPS + 1, dtype=np.int64)).astype(np.uint32)
            t = f32(bits)
            for sign in (1.0, -1.0):
                ts = (t * np.float32(sign)).astype(np.float32)
                shortcut = product_rz(ts, m) if group in POWER_OF_TWO else product_rn(ts, m)
                got = e2m1_rne_codes(shortcut)
                rotated = (ts * c).astype(np.float32)                      # fl(t * c)
                want = fp4.e2m1_codes(torch.from_numpy(rotated).unsqueeze(-1),
                                      torch.full((t.size, 1), float(s)), 1).squeeze(-1).numpy()
                bad = np.nonzero(got != want)[0]
                assert bad.size == 0, (group, e, b, sign, ts[bad[:4]], got[bad[:4]], want[bad[:4]])
                # the band really straddles the boundary: both neighbouring codes occur
                assert len(np.unique(want)) >= 2, (group, e, b)
                checked += t.size
    assert checked == 9 * 7 * 2 * (2 * ULPS + 1)


@pytest.mark.parametrize("group", [0, 16, 32, 64, 128])
def test_single_product_on_random_inputs(group):
    m0 = f32(multiplier_bits()[group])
    c = np.float32(HADAMARD_SCALE[group])
    rng = np.random.default_rng(group)
    for e in (-3, 0, 5):
        s = np.float32(2.0 ** (e - 2)) / np.float32(0.75)
        m = np.float32(m0 * np.float32(2.0 ** (2 - e)))
        # |t * c| up to a little beyond the group maximum 2^(e+1), where the code saturates at 6
        t = (rng.uniform(-1.0, 1.0, 400000) * 2.0 ** (e + 1.2) / float(c)).astype(np.float32)
        shortcut = product_rz(t, m) if group in POWER_OF_TWO else product_rn(t, m)
        got = e2m1_rne_codes(shortcut)
        want = fp4.e2m1_codes(torch.from_numpy((t * c).astype(np.float32)).unsqueeze(-1),
                              torch.full((t.size, 1), float(s)), 1).squeeze(-1).numpy()
        assert np.array_equal(got, want)


def test_division_by_three_in_three_instructions():
    """The NVFP4 scale chain starts with fl(fl(2a) / 12) = fl(a / 3) / 2.  The kernel computes a / 3 as
    q = fl(a r), e = a - 3 q (fused, exact), fl(q + e r) with r = fl(1/3): correctly rounded for every one of
    the 2^23 fp32 mantissas (every step below is exact in fp64 before its single rounding to fp32; the
    exponent does not matter while nothing underflows, which the kernel's range check excludes)."""
    import re

    import numpy as np

    src = open(os.path.join(ROOT, "fp-quant_b200", "csrc", "quantize.cu")).read()
    m = re.search(r"const float r = ([0-9.]+)f;\s*// 0x([0-9a-f]{8})", src)
    assert m, "the reciprocal constant of nv_scale was not found"
    r = np.float32(float(m.group(1)))
    assert r.view(np.uint32) == int(m.group(2), 16) == (np.float32(1.0) / np.float32(3.0)).view(np.uint32)
    for lo in range(1 << 23, 1 << 24, 1 << 21):
        x = np.arange(lo, lo + (1 << 21), dtype=np.int64).astype(np.float64)
        q0 = (x * np.float64(r)).astype(np.float32)
        e64 = x - 3.0 * q0.astype(np.float64)
        e = e64.astype(np.float32)
        assert np.array_equal(e.astype(np.float64), e64)                      # the residual is exact in fp32
        q = (q0.astype(np.float64) + e.astype(np.float64) * np.float64(r)).astype(np.float32)
        assert np.array_equal(q, (x / 3.0).astype(np.float32))
