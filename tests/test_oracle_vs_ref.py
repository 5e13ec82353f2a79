"""The plain-C oracle against the reference's own CPU code (compiled unmodified into
oracle/_ref).  Skipped on a machine where that library was never built."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O

f32p, u32p, u8p = O.f32p, O.u32p, O.u8p


def P(a, t):
    return a.ctypes.data_as(t)


def test_scalar_decoders_bit_exact(port, ref):
    for n in range(16):
        assert np.float32(port.orc_e2m1(n, 0)).view(np.uint32) == np.float32(ref.ref_fp4_e2m1(n)).view(np.uint32)
    for b in range(256):
        a, r = np.float32(port.orc_e4m3(b)), np.float32(ref.ref_fp8_e4m3(b))
        assert (np.isnan(a) and np.isnan(r)) or a.view(np.uint32) == r.view(np.uint32)
        assert np.float32(port.orc_e8m0(b, 0)).view(np.uint32) == np.float32(ref.ref_mxfp4_scale(b)).view(np.uint32)
        a, r = np.float32(port.orc_e8m0(b, 1)), np.float32(ref.ref_dsv4_e8m0(b))
        assert (np.isnan(a) and np.isnan(r)) or a == r
    for v in np.random.default_rng(1).normal(0, 4, 2000).astype(np.float32):
        assert port.orc_sigmoid(float(v)) == ref.ref_sigmoid(float(v))
        assert port.orc_silu(float(v)) == ref.ref_silu(float(v))


@pytest.mark.parametrize("name,E,k", [("glm", 256, 8), ("laguna", 256, 10), ("kimi", 896, 16),
                                      ("dsv4", 256, 6), ("glm", 7, 3)])
def test_routers_bit_exact(port, ref, name, E, k):
    rng = np.random.default_rng(hash(name) % 1000 + E)
    T = 64
    logits = rng.normal(0, 1.5, (T, E)).astype(np.float32)
    logits[1, :] = 0.25                      # all-ties row
    logits[2, : E // 2] = logits[2, E // 2: 2 * (E // 2)]   # pairwise ties
    bias = rng.normal(0, 0.2, E).astype(np.float32)
    if name == "glm":
        spec = O.router_spec(E, k, O.SCORE_SIGMOID, True, 1e-20, 2.5)
    elif name == "laguna":
        spec = O.router_spec(E, k, O.SCORE_SIGMOID, True, 0.0, 1.0)
    elif name == "kimi":
        spec = O.router_spec(E, k, O.SCORE_SIGMOID_PLAIN, True, 0.0, 1.0)
    else:
        spec = O.router_spec(E, k, O.SCORE_SQRTSOFTPLUS, True, 0.0, 1.5)
    rc, ids, w = O.route(spec, logits, bias)
    assert rc == 0
    rid = np.empty(k, np.uint32)
    rw = np.empty(k, np.float32)
    for t in range(T):
        row = np.ascontiguousarray(logits[t])
        if name == "glm":
            rc = ref.ref_glm_route(P(row, f32p), P(bias, f32p), E, k, 2.5, P(rid, u32p), P(rw, f32p))
        elif name == "laguna":
            rc = ref.ref_laguna_route(P(row, f32p), P(bias, f32p), E, k, 1, 0.0, P(rid, u32p), P(rw, f32p))
        elif name == "kimi":
            rc = ref.ref_kimi_route(P(row, f32p), P(bias, f32p), E, k, 1.0, P(rid, u32p), P(rw, f32p))
        else:
            rc = ref.ref_dsv4_route(P(row, f32p), P(bias, f32p), E, k, 1.5, P(rid, u32p), P(rw, f32p))
        assert rc == 0
        assert np.array_equal(ids[t], rid), (name, t)
        assert np.array_equal(w[t].view(np.uint32), rw.view(np.uint32)), (name, t)


def test_laguna_softcap_and_unnormalised(port, ref):
    rng = np.random.default_rng(5)
    E, k = 64, 4
    logits = rng.normal(0, 30, (8, E)).astype(np.float32)
    bias = np.zeros(E, np.float32)
    for normalize in (0, 1):
        spec = O.router_spec(E, k, O.SCORE_SIGMOID, bool(normalize), 0.0, 1.0, softcap=20.0)
        rc, ids, w = O.route(spec, logits, bias)
        rid, rw = np.empty(k, np.uint32), np.empty(k, np.float32)
        for t in range(8):
            row = np.ascontiguousarray(logits[t])
            assert ref.ref_laguna_route(P(row, f32p), P(bias, f32p), E, k, normalize, 20.0,
                                        P(rid, u32p), P(rw, f32p)) == 0
            assert np.array_equal(ids[t], rid)
            assert np.array_equal(w[t].view(np.uint32), rw.view(np.uint32))


def _rand_fp4(rng, rows, cols, group):
    packed = rng.integers(0, 256, rows * cols // 2, dtype=np.uint8)
    return packed


def test_nvfp4_matvec_bit_exact(port, ref):
    rng = np.random.default_rng(2)
    rows, cols = 48, 512
    packed = _rand_fp4(rng, rows, cols, 16)
    scales = rng.integers(0, 0x7F, rows * cols // 16, dtype=np.uint8)   # positive finite E4M3
    x = rng.normal(0, 1, cols).astype(np.float32)
    m = O.make_matrix(O.FMT_NVFP4, rows, cols, packed, scales, 203.0)
    got = O.matvec(m, x)
    want = np.empty(rows, np.float32)
    assert ref.ref_laguna_nvfp4_matvec(P(want, f32p), P(x, f32p), P(packed, u8p), P(scales, u8p),
                                       203.0, rows, cols, 0, rows) == 0
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_inkling_multiply_convention_through_the_reciprocal(port, ref):
    """Inkling (ModelOpt) NVFP4 multiplies the block scale by the tensor scale where the layer's format divides
    (src/models/inkling/inkling_ops.cpp:50-56 against src/models/laguna/laguna_ops.cpp:77-91).  The loader header passes
    1 / scale (`invert_global`): bit-identical when the scale is a power of two, otherwise one rounding of the block
    scale apart -- far inside the layer tolerance."""
    rng = np.random.default_rng(12)
    rows, cols = 40, 768
    packed = _rand_fp4(rng, rows, cols, 16)
    scales = rng.integers(0, 0x7F, rows * cols // 16, dtype=np.uint8)
    x = rng.normal(0, 1, cols).astype(np.float32)
    for g, exact in ((0.03125, True), (2.0, True), (0.0123, False), (7.3e-3, False)):
        want = np.empty(rows, np.float32)
        assert ref.ref_inkling_nvfp4_matvec(P(want, f32p), P(x, f32p), P(packed, u8p), P(scales, u8p),
                                            g, rows, cols) == 0
        m = O.make_matrix(O.FMT_NVFP4, rows, cols, packed, scales, float(np.float32(1.0) / np.float32(g)))
        got = O.matvec(m, x)
        if exact:
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        else:
            scale = np.abs(want).max()
            assert np.abs(got - want).max() <= 4e-7 * scale * np.sqrt(cols)


def test_int4_matvec_bit_exact_and_avx2_close(port, ref):
    rng = np.random.default_rng(3)
    rows, cols = 40, 1024
    packed = rng.integers(0, 256, rows * cols // 2, dtype=np.uint8)
    sc = (rng.uniform(0.003, 0.006, rows * cols // 128)).astype(np.float32)
    scales = (sc.view(np.uint32) >> 16).astype(np.uint16)
    x = rng.normal(0, 1, cols).astype(np.float32)
    m = O.make_matrix(O.FMT_INT4, rows, cols, packed, scales.view(np.uint8))
    got = O.matvec(m, x)
    want = np.empty(rows, np.float32)
    assert ref.ref_glm_int4_matvec_scalar(P(want, f32p), P(x, f32p), P(packed, u8p),
                                          P(scales.view(np.uint8), u8p), rows, cols) == 0
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    fast = np.empty(rows, np.float32)
    assert ref.ref_glm_int4_matvec_rows(P(fast, f32p), P(x, f32p), P(packed, u8p),
                                        P(scales.view(np.uint8), u8p), rows, cols, 0, rows) == 0
    assert np.allclose(fast, want, rtol=0, atol=1e-4)     # tests/test_glm_int4.cpp:13-44 bound


def test_mxfp4_matvec_against_both_reference_kernels(port, ref):
    rng = np.random.default_rng(4)
    rows, cols = 64, 2048
    packed = _rand_fp4(rng, rows, cols, 32)
    scales = rng.integers(0x70, 0x80, rows * cols // 32, dtype=np.uint8)
    x = rng.normal(0, 1, cols).astype(np.float32)
    m = O.make_matrix(O.FMT_MXFP4, rows, cols, packed, scales)
    got32 = O.matvec(m, x)
    got64 = O.matvec(m, x, double=True)
    kimi = np.empty(rows, np.float32)
    dsv4 = np.empty(rows, np.float32)
    assert ref.ref_kimi_mxfp4_matvec(P(kimi, f32p), P(x, f32p), P(packed, u8p), P(scales, u8p), rows, cols) == 0
    assert ref.ref_dsv4_fp4_matvec(P(dsv4, f32p), P(x, f32p), P(packed, u8p), P(scales, u8p), rows, cols) == 0
    # double accumulation of exact products: identical after the final rounding
    assert np.array_equal(got64.view(np.uint32), dsv4.view(np.uint32))
    scale = np.abs(dsv4).max()
    assert np.abs(got32 - dsv4).max() <= 2e-6 * scale * np.sqrt(cols)
    assert np.abs(kimi - dsv4).max() <= 2e-6 * scale * np.sqrt(cols)


def test_dequant_rows_match_reference_products(port, ref):
    rng = np.random.default_rng(6)
    rows, cols = 4, 256
    packed = _rand_fp4(rng, rows, cols, 32)
    scales = rng.integers(1, 0xFE, rows * cols // 32, dtype=np.uint8)
    m = O.make_matrix(O.FMT_MXFP4, rows, cols, packed, scales)
    deq = O.dequant(m)
    for r in range(rows):
        for c in range(cols):
            byte = packed[r * cols // 2 + c // 2]
            nib = (byte >> 4) if c & 1 else (byte & 0xF)
            want = np.float32(ref.ref_fp4_e2m1(int(nib))) * np.float32(ref.ref_mxfp4_scale(int(scales[r * cols // 32 + c // 32])))
            assert deq[r, c] == want or (np.isinf(want) and np.isinf(deq[r, c]))


def test_situ_glu_matches_reference_bitwise():
    """kimi_situ_glu, src/models/kimi_k3/kimi_k3_ops.cpp:39-62; closed-form facts from the reference's
    tests/test_kimi_k3_ops.cpp:39-69: zero gate gives zero, large inputs saturate at beta_g * beta_l."""
    import ctypes as C
    ref = O.ref()
    if ref is None:
        pytest.skip("compiled reference not built")
    port = O.port()
    rng = np.random.default_rng(11)
    g = np.concatenate([rng.standard_normal(500) * 3, [0.0, -0.0, 40.0, -40.0, 1e-8]]).astype(np.float32)
    u = np.concatenate([rng.standard_normal(500) * 3, [1.0, 2.0, 40.0, 40.0, -3.0]]).astype(np.float32)
    out = np.empty_like(g)
    f32p = C.POINTER(C.c_float)
    for gb, lb in ((1.0, 1.0), (2.5, 0.75), (7.0, 30.0)):
        assert ref.ref_kimi_situ_glu(out.ctypes.data_as(f32p), g.ctypes.data_as(f32p), u.ctypes.data_as(f32p),
                                     len(g), gb, lb) == 0
        mine = np.array([port.orc_situ_glu(float(a), float(b), gb, lb) for a, b in zip(g, u)], np.float32)
        assert np.array_equal(mine.view(np.uint32), out.view(np.uint32)), (gb, lb)
    assert port.orc_situ_glu(0.0, 5.0, 2.0, 3.0) == 0.0
    assert abs(port.orc_situ_glu(40.0, 40.0, 2.0, 3.0) - 6.0) < 1e-6


def test_hash_route_matches_reference_bitwise():
    """dsv4_route_hash_sqrtsoftplus_f32_into, src/models/dsv4/deepseek_ops.cpp:414-461."""
    import ctypes as C
    ref = O.ref()
    if ref is None:
        pytest.skip("compiled reference not built")
    port = O.port()
    f32p, u32p = C.POINTER(C.c_float), C.POINTER(C.c_uint32)
    rng = np.random.default_rng(3)
    E, k = 256, 6
    spec = O.router_spec(E, k, O.SCORE_SQRTSOFTPLUS, normalize=True, weight_scale=1.5)
    for _ in range(20):
        logits = (rng.standard_normal(E) * 4).astype(np.float32)
        table = rng.choice(E, size=k, replace=False).astype(np.uint32)
        ids_a, w_a = np.empty(k, np.uint32), np.empty(k, np.float32)
        ids_b, w_b = np.empty(k, np.uint32), np.empty(k, np.float32)
        assert port.orc_route_given_row(C.byref(spec), logits.ctypes.data_as(f32p), table.ctypes.data_as(u32p),
                                        ids_a.ctypes.data_as(u32p), w_a.ctypes.data_as(f32p)) == 0
        assert ref.ref_dsv4_route_hash(logits.ctypes.data_as(f32p), table.ctypes.data_as(u32p), E, k, 1.5,
                                       ids_b.ctypes.data_as(u32p), w_b.ctypes.data_as(f32p)) == 0
        assert np.array_equal(ids_a, ids_b) and np.array_equal(w_a.view(np.uint32), w_b.view(np.uint32))
    bad = np.array([0, 1, 2, 3, 4, E], np.uint32)
    assert port.orc_route_given_row(C.byref(spec), logits.ctypes.data_as(f32p), bad.ctypes.data_as(u32p),
                                    ids_a.ctypes.data_as(u32p), w_a.ctypes.data_as(f32p)) == -3


def test_inkling_sink_router_matches_reference():
    """orc_route_sigmoid_sink against the compiled inkling_route_sigmoid_sink (src/models/inkling/inkling_ops.cpp:184-275):
    ids and weights bit for bit, with ties and strongly negative logits (the log-sigmoid branch that must not underflow)."""
    ref = O.ref()
    rng = np.random.default_rng(7)
    E, S, k = 256, 2, 6
    for trial in range(200):
        logits = (rng.standard_normal(E + S) * rng.choice([0.5, 3.0, 30.0])).astype(np.float32)
        if trial % 5 == 0:
            logits[17] = logits[3]                      # an exact tie: the lower index must win
        bias = (rng.standard_normal(E) * 0.1).astype(np.float32)
        if trial % 5 == 0:
            bias[17] = bias[3]
        rc, ids, w = O.route_sigmoid_sink(logits[None, :], bias, E, S, k, np.float32(2.5 * 0.75))
        assert rc == 0
        rids = np.empty(k + S, np.uint32)
        rw = np.empty(k + S, np.float32)
        f32p, u32p = C.POINTER(C.c_float), C.POINTER(C.c_uint32)
        rrc = ref.ref_inkling_route_sink(logits.ctypes.data_as(f32p), bias.ctypes.data_as(f32p), E, S, k,
                                         C.c_float(2.5), C.c_float(0.75), rids.ctypes.data_as(u32p),
                                         rw.ctypes.data_as(f32p))
        assert rrc == 0
        assert np.array_equal(ids[0], rids)
        assert np.array_equal(w[0].view(np.uint32), rw.view(np.uint32)), (trial, w[0], rw)


def test_stable_bf16_hash_matches_reference():
    """orc_stable_bf16_hash against the compiled stable_bf16_hash (src/platform/diagnostics.cpp:84-88), ties, subnormals,
    infinities and NaNs (which the reference truncates instead of rounding) included."""
    ref = O.ref()
    ref.ref_stable_bf16_hash.restype = C.c_uint64
    ref.ref_stable_bf16_hash.argtypes = [C.POINTER(C.c_float), C.c_size_t]
    rng = np.random.default_rng(3)
    v = rng.standard_normal(5000).astype(np.float32)
    special = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1.00390625, 1.01171875, 1e-40, -3e38], np.float32)
    bits = np.array([0x7F800001, 0x7FC00000, 0x3F808000, 0x3F818000], np.uint32).view(np.float32)
    v = np.concatenate([v, special, bits])
    want = int(ref.ref_stable_bf16_hash(v.ctypes.data_as(C.POINTER(C.c_float)), v.size))
    assert O.stable_bf16_hash(v) == want
    assert O.stable_bf16_hash(v[:0]) == 14695981039346656037
