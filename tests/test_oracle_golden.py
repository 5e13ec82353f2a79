"""The CPU oracle against the known-answer vectors the reference keeps in its own tests.

Each case names the reference test it restates (path within the reference project).
"""
import ctypes as C
import struct

import numpy as np
import pytest

from oracle import oracle as O


def bits(f):
    return struct.unpack("<I", struct.pack("<f", f))[0]


def test_e2m1_table_and_positive_zero(port):
    # tests/test_fp4_decode.cpp:56-73
    mags = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for n in range(16):
        want = mags[n & 7] * (-1.0 if n & 8 else 1.0)
        assert port.orc_e2m1(n, 1) == want
    assert bits(port.orc_e2m1(0x8, 1)) == 0            # device decode: +0.0, never -0.0
    assert bits(port.orc_e2m1(0x8, 0)) == 0x80000000   # CPU tables: -0.0
    assert port.orc_e2m1(0x1, 1) == 0.5 and port.orc_e2m1(0x7, 1) == 6.0
    assert port.orc_e2m1(0xF, 1) == -6.0


def test_dsv4_fp4_checkpoint_bytes(port):
    # tests/test_deepseek_ops.cpp:33-51: first 16 packed bytes + first scale of a real
    # checkpoint row; ones in the first 8 columns -> 0.0546875
    enc = np.array([0x8c, 0x54, 0xa2, 0x44, 0xcc, 0x54, 0x6c, 0x55,
                    0x20, 0x2c, 0xe0, 0xea, 0x2d, 0xfd, 0x05, 0x22], np.uint8)
    sc = np.array([0x78], np.uint8)
    m = O.make_matrix(O.FMT_MXFP4, 1, 32, enc, sc)
    x = np.zeros(32, np.float32)
    x[:8] = 1.0
    for dbl in (False, True):
        assert abs(O.matvec(m, x, double=dbl)[0] - 0.0546875) < 1e-7


def test_nvfp4_decode_packing_and_global_scale(port):
    # tests/test_laguna_ops.cpp:57-104
    assert port.orc_e4m3(0x40) == 2.0
    cols = 16
    packed = np.empty(2 * cols // 2, np.uint8)
    packed[:cols // 2] = 0x22
    packed[cols // 2:] = 0x91
    scales = np.array([0x40, 0x40], np.uint8)
    m = O.make_matrix(O.FMT_NVFP4, 2, cols, packed, scales, 4.0)
    y = O.matvec(m, np.ones(cols, np.float32))
    assert y[0] == 16.0 * 0.5 and y[1] == 0.0
    y = O.matvec(m, np.arange(cols, dtype=np.float32))
    assert y[0] == 60.0 and y[1] == -2.0


def test_int4_lsb_first_offset_packing(port):
    # tests/test_compressed_tensors.cpp:70-108
    words = np.zeros(16, np.uint32)
    for w in range(16):
        for lane in range(8):
            value = ((w * 8 + lane) % 16) - 8
            words[w] |= np.uint32(value + 8) << np.uint32(lane * 4)
    scales = np.array([0x00, 0x40], np.uint8)  # BF16 2.0
    m = O.make_matrix(O.FMT_INT4, 1, 128, words.view(np.uint8), scales)
    x = np.arange(1, 129, dtype=np.float32)
    expected = np.float32(0.0)
    for i in range(128):
        expected = np.float32(expected + np.float32(np.float32((i % 16) - 8) * np.float32(2.0)) * x[i])
    assert O.matvec(m, x)[0] == expected


def test_glm_router_bias_ties_scale(port):
    # tests/test_glm_ops.cpp:64-99
    spec = O.router_spec(4, 2, O.SCORE_SIGMOID, True, 1e-20, 2.5)
    rc, ids, w = O.route(spec, np.array([[4.0, 3.0, 2.0, 1.0]], np.float32),
                         np.array([0, 0, 0, 2.0], np.float32))
    assert rc == 0 and list(ids[0]) == [3, 0]
    first, second = port.orc_sigmoid(1.0), port.orc_sigmoid(4.0)
    assert abs(w[0, 0] - first / (first + second) * 2.5) < 1e-6
    assert abs(w[0, 1] - second / (first + second) * 2.5) < 1e-6
    spec = O.router_spec(4, 3, O.SCORE_SIGMOID, True, 1e-20, 2.5)
    rc, ids, w = O.route(spec, np.zeros((1, 4), np.float32), np.zeros(4, np.float32))
    assert list(ids[0]) == [0, 1, 2] and abs(w.sum() - 2.5) < 1e-6


def test_laguna_router(port):
    # tests/test_laguna_ops.cpp:106-139
    spec = O.router_spec(4, 2, O.SCORE_SIGMOID, True)
    rc, ids, w = O.route(spec, np.array([[0, 0, 1.0, -1.0]], np.float32),
                         np.array([1.0, 0, 0, 0], np.float32))
    assert rc == 0 and list(ids[0]) == [0, 2]
    low, high = port.orc_sigmoid(0.0), port.orc_sigmoid(1.0)
    assert abs(w[0, 0] - low / (low + high)) < 1e-6 and abs(w[0, 1] - high / (low + high)) < 1e-6
    rc, ids, w = O.route(spec, np.zeros((1, 4), np.float32), np.zeros(4, np.float32))
    assert list(ids[0]) == [0, 1] and abs(w[0, 0] - 0.5) < 1e-6


def test_kimi_router(port):
    # tests/test_kimi_k3_ops.cpp:121-153
    spec = O.router_spec(4, 2, O.SCORE_SIGMOID_PLAIN, True)
    rc, ids, w = O.route(spec, np.array([[2.0, -2.0, 1.0, -1.0]], np.float32),
                         np.array([0, 5.0, 0, 0], np.float32))
    assert rc == 0 and list(ids[0]) == [1, 0]
    s0, s1 = 1 / (1 + np.exp(-2.0)), 1 / (1 + np.exp(2.0))
    assert abs(w[0, 0] - s1 / (s0 + s1)) < 1e-6 and abs(w[0, 1] - s0 / (s0 + s1)) < 1e-6
    rc, ids, w = O.route(spec, np.full((1, 4), 0.5, np.float32), np.zeros(4, np.float32))
    assert list(ids[0]) == [0, 1]


def test_router_projection_is_row_major(port):
    # tests/test_glm_ops.cpp:89-99: hidden (2,3), rows (1,0),(0,1),(-1,-1) -> expert 1
    def bf(v):
        return np.array([port.orc_f32_to_bf16(float(a)) for a in v], np.uint16)
    x = bf([2.0, 3.0]).reshape(1, 2)
    wg = bf([1, 0, 0, 1, -1, -1]).reshape(3, 2)
    logits = O.router_logits(x, wg)
    assert list(logits[0]) == [2.0, 3.0, -5.0]
    rc, ids, w = O.route(O.router_spec(3, 1, O.SCORE_SIGMOID, True, 1e-20, 2.5), logits,
                         np.zeros(3, np.float32))
    assert ids[0, 0] == 1 and abs(w[0, 0] - 2.5) < 1e-6


def test_group_is_stable_by_expert_then_token_rank(port):
    ids = np.array([[2, 0], [0, 1], [2, 1]], np.uint32)
    counts, offsets, perm = O.group(ids, 4)
    assert list(counts) == [2, 2, 2, 0]
    assert list(offsets) == [0, 2, 4, 6, 6]
    assert list(perm) == [1, 2, 3, 5, 0, 4]
    counts, offsets, perm = O.group(np.zeros((0, 2), np.uint32), 4)   # empty page
    assert list(counts) == [0, 0, 0, 0] and len(perm) == 0


def test_expf_replica_matches_host_libm(port):
    # The CUDA router evaluates this algorithm; it must agree with the libm the reference's
    # routers call.  Sample densely over the range a router logit can take.
    rng = np.random.default_rng(0)
    xs = np.concatenate([rng.uniform(-30, 30, 200000), rng.normal(0, 2, 200000)]).astype(np.float32)
    want = np.exp(xs.astype(np.float32), dtype=np.float32)  # numpy calls libm expf per element
    bad = 0
    for x in xs[:20000]:
        a = port.orc_expf_replica(float(x), 1)
        b = port.orc_expf_replica(float(x), 0)
        bad += a != b
    assert bad == 0   # contraction of the three multiply-adds never changes the float result
    got = np.array([port.orc_expf_replica(float(x), 1) for x in xs[:100000]], np.float32)
    import math
    lib = C.CDLL("libm.so.6")
    lib.expf.restype = C.c_float
    lib.expf.argtypes = [C.c_float]
    ref = np.array([lib.expf(float(x)) for x in xs[:100000]], np.float32)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


def test_log1pf_replica_matches_host_libm(port):
    # sqrt(softplus) router scores: the CUDA router evaluates this restatement of log1pf; it must agree bit for
    # bit with the libm the reference's DSV4 router calls.  Arguments are expf(logit), logit <= 20.
    rng = np.random.default_rng(1)
    logits = np.concatenate([rng.uniform(-40, 20, 150000), rng.normal(0, 3, 150000)]).astype(np.float32)
    xs = np.exp(logits, dtype=np.float32)
    lib = C.CDLL("libm.so.6")
    lib.log1pf.restype = C.c_float
    lib.log1pf.argtypes = [C.c_float]
    got = np.array([port.orc_log1pf_replica(float(x)) for x in xs], np.float32)
    ref = np.array([lib.log1pf(float(x)) for x in xs], np.float32)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
