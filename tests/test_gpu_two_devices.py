"""Two contexts on two GPUs of ONE process, the way the reference backend drives several devices
from one runtime (src/models/glm52/glm_runtime.cpp:1561-1576): the per-device opt-ins of the
kernels (large dynamic shared memory) must hold on every device, not only on the first one used.
Skipped on a box with one GPU."""
import pytest
import torch

from strata_b200 import MoeContext, MoeLayer, synth

pytestmark = pytest.mark.gpu


def test_tensor_core_path_on_a_second_device():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    # 1600 tokens x top-2 over 32 experts: 100 rows per expert (tensor-core tiles) and enough
    # router tiles for the register-blocked projection kernel
    cfg = synth.MoeConfig("twodev", H=512, I=256, E=32, k=2, fmt=synth.FMT_MXFP4, T=1600, seed=5, I_shared=128)
    outs = []
    for dev in (0, 1):
        ctx = MoeContext(dev)
        layer = synth.build_layer(cfg, torch.device("cuda", dev))
        ml = MoeLayer(ctx, cfg, max_tokens=cfg.T)
        ml.load_synth(layer)
        out = ml.forward(layer.x)
        ctx.synchronize()
        outs.append(out.cpu())
        ml.close()
        ctx.close()
    assert torch.isfinite(outs[0]).all()
    assert torch.equal(outs[0], outs[1])
