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


def _bf16_round(a):
    b = a.astype(np.float32).view(np.uint32)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32)


def test_page_through_group_experts_join(ctx):
    """A DSV4 page end to end through the stage calls: route, group, gather the fp32 rows, exact
    experts with the route weights as coefficients, join.  Checked against the oracle's experts and a
    numpy restatement of the join (src/models/dsv4/deepseek_runtime.cpp:5897-5914)."""
    cfg = synth.MoeConfig("dsv4page", H=512, I=256, E=8, k=3, fmt=synth.FMT_MXFP4, T=6, seed=23,
                          score_kind=synth.SCORE_SIGMOID, normalize=True, weight_scale=1.5)
    layer = synth.build_layer(cfg, "cuda")
    ml = MoeLayer(ctx, cfg, max_tokens=cfg.T)
    ml.load_synth(layer)
    T, k, H, I = cfg.T, cfg.k, cfg.H, cfg.I
    ids, w = ml.route(layer.x)
    counts, offsets, perm, inv = ml.group(ids, 0, cfg.E, want_inv=True)
    xf = layer.x.float()
    rows = xf[(perm.long() // k)]
    coef = w.reshape(-1)[perm.long()].contiguous()
    y = ml.experts_grouped_dsv4(rows.contiguous(), offsets, coef, swiglu_limit=10.0)
    rng = np.random.default_rng(5)
    shared = rng.standard_normal((T, H)).astype(np.float32)
    out = ml.combine_dsv4(y, inv, T, torch.from_numpy(shared).cuda())
    ctx.synchronize()
    # oracle
    port = O.port()
    ids_h, w_h, perm_h, inv_h = ids.cpu().numpy(), w.cpu().numpy(), perm.cpu().numpy(), inv.cpu().numpy()
    wt = {r: [layer.packed[r][e].cpu().numpy().reshape(-1) for e in range(cfg.E)] for r in synth.ROLES}
    sc = {r: [layer.scales[r][e].cpu().numpy().reshape(-1) for e in range(cfg.E)] for r in synth.ROLES}
    x_h = xf.cpu().numpy()
    scratch = np.empty(I, np.float32)
    want = np.zeros((T, H), np.float32)
    for t in range(T):
        acc = np.zeros(H, np.float32)
        for r in range(k):
            e = int(ids_h[t, r])
            row = np.empty(H, np.float32)
            xin = np.ascontiguousarray(x_h[t])
            assert port.orc_dsv4_expert(_p(row, f32p), _p(xin, f32p), _p(wt["gate"][e], u8p), _p(sc["gate"][e], u8p),
                                        _p(wt["up"][e], u8p), _p(sc["up"][e], u8p), _p(wt["down"][e], u8p),
                                        _p(sc["down"][e], u8p), H, I, float(w_h[t, r]), 10.0, _p(scratch, f32p)) == 0
            acc = acc + _bf16_round(row)
        want[t] = _bf16_round(acc + _bf16_round(shared[t]))
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
