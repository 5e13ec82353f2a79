"""The dense command (call-compatible with the reference's enqueue_moe / collect_moe) on a GPU:
every listed expert applied to all rows, fp32 host rows in, [expert][row][H] out; protocol errors as
the reference's tests pin them (tests/test_cuda_backend.cpp:1628-1780 of the reference)."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as O
from strata_b200 import MoeContext, MoeLayer, StrataMoeError, synth
from tests import helpers as Hh

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    return MoeContext(0)


def make(ctx, fmt, shared=0):
    cfg = synth.MoeConfig(f"dense{fmt}", H=512, I=256, E=8, k=2, fmt=fmt, T=16, seed=4, I_shared=shared)
    layer = synth.build_layer(cfg, "cuda")
    ml = MoeLayer(ctx, cfg, max_tokens=16, max_pairs=64)
    ml.load_synth(layer)
    return cfg, layer, ml


def oracle_dense(cfg, hidden, experts, coefs):
    arr, keep = Hh.oracle_experts(cfg, experts)
    out = np.empty((len(experts), hidden.shape[0], cfg.H), np.float32)
    a = np.empty(cfg.I, np.float32)
    u = np.empty(cfg.I, np.float32)
    for i, e in enumerate(experts):
        for r in range(hidden.shape[0]):
            x = np.ascontiguousarray(hidden[r])
            rc = O.port().orc_expert_ffn(C.byref(arr[e]), x.ctypes.data_as(O.f32p), float(coefs[i]),
                                         1 if cfg.fmt == synth.FMT_INT4 else 0, 0,
                                         a.ctypes.data_as(O.f32p), u.ctypes.data_as(O.f32p),
                                         out[i, r].ctypes.data_as(O.f32p))
            assert rc == 0
    return out


@pytest.mark.parametrize("fmt", [synth.FMT_MXFP4, synth.FMT_NVFP4, synth.FMT_INT4, synth.FMT_BF16])
def test_dense_command_matches_oracle(ctx, fmt):
    cfg, layer, ml = make(ctx, fmt, shared=128 if fmt == synth.FMT_NVFP4 else 0)
    rng = np.random.default_rng(7)
    rows = 3
    hidden = rng.normal(0, 1, (rows, cfg.H)).astype(np.float32)      # NOT bf16-representable on purpose
    experts = [5, 0, 3]
    coefs = [0.25, 1.5, 0.5] if fmt == synth.FMT_INT4 else [1.0, 1.0, 1.0]
    with_shared = bool(cfg.I_shared)
    ml.enqueue_dense(torch.from_numpy(hidden), experts, coefs, with_shared)
    routed, shared = ml.collect_dense(len(experts), rows, with_shared)
    want = oracle_dense(cfg, hidden, experts, coefs)
    rel, mx = Hh.error_metrics(routed.numpy(), want)
    assert rel <= 2e-4 and mx <= 2.0 ** -6, (rel, mx)
    if with_shared:
        sh, keep = Hh.oracle_shared(cfg)
        a = np.empty(cfg.I_shared, np.float32)
        u = np.empty(cfg.I_shared, np.float32)
        ws = np.empty((rows, cfg.H), np.float32)
        for r in range(rows):
            x = np.ascontiguousarray(hidden[r])
            O.port().orc_expert_ffn(C.byref(sh), x.ctypes.data_as(O.f32p), 1.0, 0, 0, a.ctypes.data_as(O.f32p),
                                    u.ctypes.data_as(O.f32p), ws[r].ctypes.data_as(O.f32p))
        rel, mx = Hh.error_metrics(shared.numpy(), ws)
        assert rel <= 2e-4, rel


def test_dense_protocol(ctx):
    cfg, layer, ml = make(ctx, synth.FMT_MXFP4)
    hidden = torch.randn(2, cfg.H)
    ml.enqueue_dense(hidden, [1], [1.0])
    with pytest.raises(StrataMoeError) as e:          # one command in flight
        ml.enqueue_dense(hidden, [2], [1.0])
    assert e.value.code == -4
    with pytest.raises(StrataMoeError):               # whole-layer call refused meanwhile
        ml.forward(layer.x)
    ml.collect_dense(1, 2)
    with pytest.raises(StrataMoeError):               # nothing left to collect
        ml.collect_dense(1, 2)
    with pytest.raises(StrataMoeError):               # non-INT4 formats take coefficient 1 only
        ml.enqueue_dense(hidden, [1], [0.5])
    with pytest.raises(StrataMoeError):               # expert outside the resident range
        ml.enqueue_dense(hidden, [cfg.E], [1.0])
    with pytest.raises(StrataMoeError) as e:          # a list longer than the resident experts (duplicates)
        ml.enqueue_dense(hidden[:1], [0] * (cfg.E + 1), [1.0] * (cfg.E + 1))
    assert e.value.code == -1
    ml.enqueue_dense(hidden, [1], [1.0])              # workspace reusable after the failures
    ml.collect_dense(1, 2)


def test_forward_rejects_more_pairs_than_the_workspace_holds(ctx):
    cfg = synth.MoeConfig("fewpairs", H=256, I=128, E=4, k=2, fmt=synth.FMT_MXFP4, T=8, seed=4)
    layer = synth.build_layer(cfg, "cuda")
    ml = MoeLayer(ctx, cfg, max_tokens=8, max_pairs=6)     # 8 tokens x top-2 would need 16
    ml.load_synth(layer)
    with pytest.raises(StrataMoeError) as e:
        ml.forward(layer.x)
    assert e.value.code == -1
    out = ml.forward(layer.x[:3])                           # 6 pairs fit
    ctx.synchronize()
    assert torch.isfinite(out).all()


def test_non_finite_result_fails_collect_and_leaves_buffers_untouched(ctx):
    # a reserved 0xFF MXFP4 scale decodes to NaN: collect must fail and not write
    cfg = synth.MoeConfig("nan", H=256, I=128, E=2, k=1, fmt=synth.FMT_MXFP4, T=4, seed=4)
    layer = synth.build_layer(cfg, "cuda")
    layer.scales["gate"][1].fill_(0xFF)
    ml = MoeLayer(ctx, cfg, max_tokens=4, max_pairs=8)
    ml.load_synth(layer)
    hidden = torch.randn(2, cfg.H)
    ml.enqueue_dense(hidden, [1], [1.0])
    routed = torch.full((1, 2, cfg.H), 7.0)
    rc = ml.lib.strata_moe_collect_dense(ml.h, C.c_void_p(routed.data_ptr()), None)
    assert rc == -3
    assert torch.all(routed == 7.0)
    ml.enqueue_dense(hidden, [0], [1.0])              # the layer recovers
    ml.collect_dense(1, 2)
