"""The allocation-free grouping entry point against the regular one (needs a B200).

Who needs it: a host that handed the whole GPU to its own arena at start-up, or that calls from a
section where cudaMalloc's implicit synchronisation is not acceptable, cannot create a layer object
(that allocates workspaces).  strata_moe_group_static takes only caller memory and keeps its scratch
in a fixed device array inside the library.

Checked here, through the C ABI: bit-identical counts / offsets / permutation / inverse to
strata_moe_group on two calls in a row (the second with different sizes, so stale scratch from the
first would show), the size limits, and that it works as the first CUDA call of a fresh process.
This file sorts last on purpose: a failure here cannot hide another test behind `-x`.
"""
import subprocess
import sys
import os

import numpy as np
import pytest
import torch

from strata_b200 import MoeContext, MoeLayer, StrataMoeError, synth
from strata_b200.api import group_static

pytestmark = pytest.mark.gpu


def _ids(T, k, E, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).cuda()


def test_static_group_matches_regular_group_twice():
    ctx = MoeContext(0)
    torch.cuda.set_stream(ctx.stream)
    cfg = synth.MoeConfig("noalloc", H=256, I=128, E=64, k=6, fmt=synth.FMT_MXFP4, T=2000, seed=1)
    ml = MoeLayer(ctx, cfg)
    for call, (T, ebeg, nexp) in enumerate([(2000, 0, 64), (37, 16, 32)]):
        ids = _ids(T, cfg.k, cfg.E, 10 + call)
        want = ml.group(ids, ebeg, nexp, want_inv=True)
        got = group_static(ids, ebeg, nexp, stream=ctx.stream)
        ctx.synchronize()
        n = int(want[1][-1].item())
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1]), call
        assert torch.equal(got[2][:n], want[2][:n]), call
        assert torch.equal(got[3], want[3]), call


def test_static_group_rejects_oversize_with_a_message():
    ids = torch.zeros(8, 2, dtype=torch.int32, device="cuda")
    with pytest.raises(StrataMoeError, match="expert count"):
        group_static(ids, 0, 257)
    big = torch.zeros(65537, 1, dtype=torch.int32, device="cuda")
    with pytest.raises(StrataMoeError, match="too many pairs"):
        group_static(big, 0, 8)


def test_static_group_as_first_call_of_a_fresh_process():
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "import torch, numpy as np\n"
        "from strata_b200.api import group_static\n"
        "ids = torch.tensor([[2, 0], [0, 1], [2, 1]], dtype=torch.int32, device='cuda')\n"
        "c, o, p, i = group_static(ids, 0, 4)\n"
        "torch.cuda.synchronize()\n"
        "assert c.tolist() == [2, 2, 2, 0] and o.tolist() == [0, 2, 4, 6, 6], (c, o)\n"
        "assert p.tolist() == [1, 2, 3, 5, 0, 4], p\n"
        "assert i.tolist() == [4, 0, 1, 2, 5, 3], i\n"
        "print('ok')\n") % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr
