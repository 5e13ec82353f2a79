"""DSV4-exact numerical mode: the oracle's restatement against the compiled reference
(kernels/cpu/dsv4_fp4_expert.cpp), bit for bit, and against the reference's own known answers."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O

f32p = C.POINTER(C.c_float)
u8p = C.POINTER(C.c_uint8)


def _p(a, t):
    return a.ctypes.data_as(t)


def test_quantize_value_known_answers():
    """E4M3 grid facts (kernels/cuda/backend.cu:212-225): 448 saturates, the subnormal step is 2^-9,
    ties go to even, the sign survives."""
    q = O.port().orc_quantize_e4m3_value
    assert q(1000.0) == 448.0 and q(-1000.0) == -448.0
    assert q(0.001953125) == 0.001953125                  # 2^-9, smallest subnormal
    assert q(0.0009765625) == 0.0                         # half of it: tie to even (0)
    assert q(0.0029296875) == 0.00390625                  # 1.5 * 2^-9: tie to even (2 * 2^-9)
    assert q(1.0625) == 1.0 and q(1.1875) == 1.25         # ties between 1, 1.125, 1.25
    assert q(17.0) == 16.0 and q(19.0) == 20.0            # step 2 in [16, 32)
    assert np.signbit(np.float32(q(-0.0)))


def test_quantize_rows_match_reference_bitwise():
    ref = O.ref()
    if ref is None:
        pytest.skip("compiled reference not built")
    port = O.port()
    rng = np.random.default_rng(7)
    for cols in (128, 384, 4096, 200):
        for scale in (1e-6, 1e-2, 1.0, 37.0, 3e4):
            v = (rng.standard_normal(cols) * scale).astype(np.float32)
            v[::17] = 0.0
            v[5] = np.float32(448.0 * 2.0 ** np.round(np.log2(scale)))      # block maximum on a power-of-two edge
            a, b = v.copy(), v.copy()
            port.orc_quantize_activation_e4m3(_p(a, f32p), cols)
            assert ref.ref_dsv4_quantize(_p(b, f32p), cols) == 0
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), (cols, scale)


@pytest.mark.parametrize("hidden,inter", [(512, 256), (1024, 384)])
def test_expert_matches_reference_bitwise(hidden, inter):
    ref = O.ref()
    if ref is None:
        pytest.skip("compiled reference not built")
    port = O.port()
    rng = np.random.default_rng(hidden + inter)
    w = [rng.integers(0, 256, size=n, dtype=np.uint8) for n in (inter * hidden // 2,) * 3]
    s = [rng.integers(118, 124, size=inter * hidden // 32, dtype=np.uint8) for _ in range(3)]
    for trial in range(3):
        x = (rng.standard_normal(hidden) * (0.5 + trial)).astype(np.float32)
        coef = np.float32(0.37 + 0.2 * trial)
        got = np.empty(hidden, np.float32)
        want = np.empty(hidden, np.float32)
        scratch = np.empty(inter, np.float32)
        rc = port.orc_dsv4_expert(_p(got, f32p), _p(x, f32p), _p(w[0], u8p), _p(s[0], u8p), _p(w[1], u8p),
                                  _p(s[1], u8p), _p(w[2], u8p), _p(s[2], u8p), hidden, inter, float(coef), 10.0,
                                  _p(scratch, f32p))
        assert rc == 0
        for avx in (0, 1):
            assert ref.ref_dsv4_host_expert(_p(want, f32p), _p(x, f32p), _p(w[0], u8p), _p(s[0], u8p),
                                            _p(w[1], u8p), _p(s[1], u8p), _p(w[2], u8p), _p(s[2], u8p), hidden,
                                            inter, float(coef), 10.0, avx) == 0
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (trial, avx)
        assert np.abs(got).max() > 0
