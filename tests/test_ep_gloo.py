"""Expert-parallel exchange logic on CPU: world_size 2 and 4 over gloo, compute by the oracle.
The concatenated rank outputs must equal the single-rank oracle layer bit for bit (same
arithmetic per row, same combine order), which pins the dispatch / regroup / return / combine
index plumbing."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from strata_b200 import synth
from tests import helpers as Hh


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, cfg, T, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["OMP_NUM_THREADS"] = "1"
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from strata_b200.ep import EpMoe, owner_block
    from tests.cpu_ops import OracleOps
    B = owner_block(cfg, world)
    ops = OracleOps(cfg, rank * B, B)
    x = synth.gen_inputs(cfg, T)
    Tl = T // world
    ep = EpMoe(ops, cfg, rank, world)
    out = ep.forward(x[rank * Tl:(rank + 1) * Tl].contiguous())
    ret[rank] = (out.numpy(), ep.last["recv_pairs"])
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,fmt,shared", [(2, synth.FMT_MXFP4, 0), (4, synth.FMT_NVFP4, 128),
                                              (2, synth.FMT_INT4, 0)])
def test_ep_matches_single_rank_oracle(world, fmt, shared):
    cfg = synth.MoeConfig("ep", H=256, I=128, E=8, k=3, fmt=fmt, T=12, seed=5, I_shared=shared,
                          output_scale=2.5 if shared else 1.0, zipf_s=1.1)
    T = 12
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), cfg, T, ret), nprocs=world, join=True)
    got = np.concatenate([ret[r][0] for r in range(world)], 0)
    assert sum(ret[r][1] for r in range(world)) == T * cfg.k      # every pair reached an owner
    ref = Hh.run_oracle(cfg, synth.gen_inputs(cfg, T))
    assert np.array_equal(got.view(np.uint32), ref["out"].view(np.uint32))
