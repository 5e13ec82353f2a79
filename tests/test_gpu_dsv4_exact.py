"""DSV4-exact numerical mode on the GPU against the oracle (which is pinned bit for bit to the
compiled reference in tests/test_oracle_dsv4.py): every output bit must match."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as O
from strata_b200 import MoeContext, MoeLayer, synth

pytestmark = pytest.mark.gpu
f32p = C.POINTER(C.c_float)
u8p = C.POINTER(C.c_uint8)


def _p(a, t):
    return a.ctypes.data_as(t)


@pytest.fixture(scope="module")
def ctx():
    return MoeContext(0)


@pytest.mark.parametrize("rows,cols", [(3, 128), (5, 4096), (2, 200), (1, 7168), (4, 96)])
def test_quantize_bit_exact(ctx, rows, cols):
    rng = np.random.default_rng(rows * 1000 + cols)
    port = O.port()
    for scale in (1e-5, 3e-3, 1.0, 55.0, 2e4):
        v = (rng.standard_normal((rows, cols)) * scale).astype(np.float32)
        v[:, ::13] = 0.0
        v[0, 1] = np.float32(448.0 * 2.0 ** np.round(np.log2(scale)))     # block maximum on a power-of-two edge
        want = v.copy()
        for r in range(rows):
            port.orc_quantize_activation_e4m3(_p(want[r], f32p), cols)
        got = ctx.quantize_e4m3(torch.from_numpy(v).cuda())
        ctx.synchronize()
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32)), scale


@pytest.mark.parametrize("H,I,E,counts", [(512, 256, 4, [3, 0, 1, 6]), (1024, 384, 3, [1, 5, 2]),
                                          (4096, 2048, 2, [2, 1])])
def test_grouped_experts_bit_exact(ctx, H, I, E, counts):
    cfg = synth.MoeConfig("dsv4x", H=H, I=I, E=E, k=min(2, E), fmt=synth.FMT_MXFP4, T=8, seed=17)
    layer = synth.build_layer(cfg, "cuda")
    ml = MoeLayer(ctx, cfg, max_tokens=16)
    ml.load_synth(layer)
    pairs = sum(counts)
    rng = np.random.default_rng(H + I)
    x = (rng.standard_normal((pairs, H)) * 1.7).astype(np.float32)
    coef = rng.uniform(0.05, 0.9, size=pairs).astype(np.float32)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    y = ml.experts_grouped_dsv4(torch.from_numpy(x).cuda(), torch.from_numpy(offsets).cuda(),
                                torch.from_numpy(coef).cuda(), swiglu_limit=10.0)
    ctx.synchronize()
    got = y.cpu().numpy()
    port = O.port()
    w = {r: [layer.packed[r][e].cpu().numpy().reshape(-1) for e in range(E)] for r in synth.ROLES}
    s = {r: [layer.scales[r][e].cpu().numpy().reshape(-1) for e in range(E)] for r in synth.ROLES}
    scratch = np.empty(I, np.float32)
    pos = 0
    for e, c in enumerate(counts):
        for _ in range(c):
            want = np.empty(H, np.float32)
            rc = port.orc_dsv4_expert(_p(want, f32p), _p(x[pos], f32p), _p(w["gate"][e], u8p), _p(s["gate"][e], u8p),
                                      _p(w["up"][e], u8p), _p(s["up"][e], u8p), _p(w["down"][e], u8p),
                                      _p(s["down"][e], u8p), H, I, float(coef[pos]), 10.0, _p(scratch, f32p))
            assert rc == 0
            assert np.array_equal(got[pos].view(np.uint32), want.view(np.uint32)), (e, pos)
            pos += 1
    assert np.abs(got).max() > 0


def test_rejects_other_formats(ctx):
    from strata_b200 import StrataMoeError
    cfg = synth.MoeConfig("dsv4x_nv", H=256, I=128, E=2, k=1, fmt=synth.FMT_NVFP4, T=2, seed=1)
    layer = synth.build_layer(cfg, "cuda")
    ml = MoeLayer(ctx, cfg, max_tokens=4)
    ml.load_synth(layer)
    with pytest.raises(StrataMoeError):
        ml.experts_grouped_dsv4(torch.zeros(2, 256, device="cuda"), torch.tensor([0, 1, 2], dtype=torch.int32,
                                                                               device="cuda"))
