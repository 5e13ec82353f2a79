"""LatentMoE wrapper (Kimi-K3) on the GPU against the CPU oracle, through the C ABI: routing on the raw hidden
state bit for bit, outputs within the layer bars (the latent and the normalised mixture pass through BF16 on
their way into the tensor-core GEMMs, so the tight bound is that of two BF16 roundings).
ref: kimi_latent_moe_layer, src/models/kimi_k3/kimi_k3_layer.cpp:781-1001."""
import gc

import numpy as np
import pytest
import torch

from strata_b200 import MoeContext, synth
from strata_b200.api import LatentMoe
from tests import helpers as Hh
from oracle import layer_check as Lc

pytestmark = pytest.mark.gpu

REL_L2, MAX_ABS = 1e-2, 2.0 ** -6


@pytest.fixture(scope="module")
def ctx():
    return MoeContext(0)


def run(ctx, cfg, T, sub):
    layer = synth.build_layer(cfg, "cuda", T=T)
    lm = LatentMoe(ctx, cfg, max_tokens=T)
    lm.load_synth(layer)
    out, ids, w = lm.forward(layer.x, want_routing=True)
    ctx.synchronize()
    out2 = lm.forward(layer.x)
    ctx.synchronize()
    assert torch.equal(out, out2)
    ref = Lc.run_oracle_latent(cfg, layer.x.cpu(), token_subset=sub)
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ref["ids"])
    assert np.array_equal(w.cpu().numpy().view(np.uint32), ref["weights"].view(np.uint32))
    rel, mx = Hh.error_metrics(out[torch.as_tensor(np.asarray(sub, np.int64)).cuda()].cpu().numpy(), ref["out"])
    lm.close()
    del layer, lm, out, out2
    gc.collect()
    torch.cuda.empty_cache()
    assert rel <= REL_L2 and mx <= MAX_ABS, (rel, mx)
    assert rel <= 4e-3, rel


@pytest.mark.parametrize("fmt,T", [(synth.FMT_MXFP4, 5), (synth.FMT_NVFP4, 37), (synth.FMT_MXFP4, 300)])
def test_small_latent_layer(ctx, fmt, T):
    cfg = synth.MoeConfig(f"lat{fmt}_{T}", H=256, I=128, E=16, k=4, fmt=fmt, T=T, seed=3, I_shared=256, H_model=512,
                          activation=1, gate_beta=4.0, linear_beta=25.0, score_kind=synth.SCORE_SIGMOID_PLAIN)
    run(ctx, cfg, T, list(range(min(T, 12))))


def test_kimi_shape(ctx):
    run(ctx, synth.CONFIGS["kimi"], 4, [0, 3])
