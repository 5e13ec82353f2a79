"""Peer-memory expert parallelism (strata_moe_ep_*) with several ranks stepped by ONE process on
one GPU.  The ranks' windows are ordinary device buffers of the same process, and the stages
run rank after rank (begin on all, dispatch on all, experts on all, finish on all) with a
synchronize in between, so every flag a kernel waits for has already been stored: no kernel ever
waits for another one.  This pins the window layout, the placement arithmetic, the step parity
and the failure paths; tests/test_gpu_ep.py runs the same code as one process per GPU."""
import pytest
import torch

from strata_b200 import MoeContext, MoeLayer, StrataMoeError, synth
from strata_b200.api import EpState, EpWindow

pytestmark = pytest.mark.gpu


class Ranks:
    def __init__(self, cfg, world, T_local, cap, wait_ms=2000, active=None):
        dev = torch.device("cuda", 0)
        self.cfg, self.world = cfg, world
        B = cfg.E // world
        self.ctxs, self.layers, self.wins, self.states = [], [], [], []
        for r in range(world):
            ctx = MoeContext(0)
            part = synth.build_layer(cfg, dev, expert_begin=r * B, expert_end=(r + 1) * B)
            ml = MoeLayer(ctx, cfg, max_tokens=T_local, expert_begin=r * B, expert_count=B,
                          max_pairs=max(cap, T_local * cfg.k))
            ml.load_synth(part)
            self.ctxs.append(ctx)
            self.layers.append(ml)
        nbytes = EpWindow.bytes_needed(self.layers[0], world, cap)
        self.wins = [EpWindow.alloc(c, nbytes) for c in self.ctxs]
        ptrs = [w.ptr for w in self.wins]
        for r in range(world):
            self.states.append(EpState(self.layers[r], r, world, cap, ptrs, wait_ms))
        self.active = list(range(world)) if active is None else active

    def sync(self, check=True):
        errs = []
        for r in self.active:
            try:
                self.ctxs[r].synchronize()
            except StrataMoeError as e:
                errs.append(str(e))
        if check and errs:
            raise AssertionError(errs)
        return errs

    def step(self, xs, check=True):
        for r in self.active:
            self.states[r].begin(xs[r])
        self.sync(check)
        for r in self.active:
            self.states[r].dispatch()
        errs = self.sync(check)
        for r in self.active:
            self.states[r].experts()
        errs += self.sync(check)
        outs = {r: self.states[r].finish() for r in self.active}
        errs += self.sync(check)
        return outs, errs

    def close(self):
        for s in self.states:
            s.close()
        for w in self.wins:
            w.close()
        for ml in self.layers:
            ml.close()
        for c in self.ctxs:
            c.close()


def reference(cfg, x):
    ctx = MoeContext(0)
    full = synth.build_layer(cfg, torch.device("cuda", 0))
    ml = MoeLayer(ctx, cfg, max_tokens=x.shape[0])
    ml.load_synth(full)
    out, aux = ml.forward(x, want_aux=True)
    ctx.synchronize()
    out = out.clone()
    ml.close()
    ctx.close()
    return out, aux


@pytest.mark.parametrize("world,fmt,T_local", [(1, 0, 24), (2, 1, 32), (4, 2, 16), (4, 0, 256), (2, 1, 1), (8, 0, 160), (8, 2, 3)])
def test_peer_steps_match_single_gpu(world, fmt, T_local):
    cfg = synth.MoeConfig("ep_peer", H=512, I=256, E=16, k=4, fmt=fmt, T=T_local * world, seed=21 + fmt,
                          I_shared=128 if fmt == synth.FMT_NVFP4 else 0, zipf_s=1.1)
    T = T_local * world
    ranks = Ranks(cfg, world, T_local, cap=T * cfg.k)
    try:
        for it in range(3):      # three steps: both window parities and a reuse of the first
            x = synth.gen_inputs(cfg, T, seed=100 + it).cuda()
            xs = [x[r * T_local:(r + 1) * T_local].contiguous() for r in range(world)]
            outs, _ = ranks.step(xs)
            got = torch.cat([outs[r] for r in range(world)], 0)
            ref, _ = reference(cfg, x)
            rel = ((got - ref).norm() / ref.norm()).item()
            assert rel <= 2e-3, (it, rel)
    finally:
        ranks.close()


@pytest.mark.parametrize("T_local", [4, 0])
def test_peer_wide_rows_and_a_rank_without_tokens(T_local):
    """Rows wider than the owner-side partial-sum kernel keeps in registers (hidden 9216 > 8192: its recompute
    tail runs), and a step in which rank 1 has no tokens of its own but still serves its experts."""
    cfg = synth.MoeConfig("ep_wide", H=9216, I=128, E=8, k=2, fmt=0, T=8, seed=33)
    world = 2
    T0 = 4
    ranks = Ranks(cfg, world, T0, cap=32)
    try:
        x = synth.gen_inputs(cfg, T0 + T_local, seed=7).cuda()
        xs = [x[:T0].contiguous(), x[T0:].contiguous()]
        for it in range(2):
            outs, _ = ranks.step(xs)
        got = torch.cat([outs[0], outs[1]], 0)
        ref, _ = reference(cfg, x)
        assert got.shape == ref.shape
        rel = ((got - ref).norm() / ref.norm()).item()
        assert rel <= 2e-3, rel
    finally:
        ranks.close()


@pytest.mark.parametrize("world", [2, 8])
def test_peer_full_shape_c3(world):
    """The bench's workload (c3: 16384 tokens, 256 MXFP4 experts, top-8, hidden 7168) over 2 and over 8 ranks stepped
    by one process: every owner runs the tensor-core path on its 131072 / world grouped rows, read through the slot
    table from the token rows it received, and returns one partial sum per received token row.  Both window parities
    must give the same bits."""
    cfg = synth.CONFIGS["c3"]
    T = cfg.T
    T_local = T // world
    ranks = Ranks(cfg, world, T_local, cap=T_local * cfg.k * 3 // 2)
    try:
        x = synth.gen_inputs(cfg, T, seed=5).cuda()
        xs = [x[r * T_local:(r + 1) * T_local].contiguous() for r in range(world)]
        first, _ = ranks.step(xs)
        first = torch.cat([first[r] for r in range(world)], 0).clone()
        second, _ = ranks.step(xs)
        second = torch.cat([second[r] for r in range(world)], 0)
        assert torch.equal(first, second)
        counts = [st.last_counts() for st in ranks.states]
    finally:
        ranks.close()
    ref, aux = reference(cfg, x)
    # a token's row crosses once per owning rank, however many of that rank's experts it selected
    owners = (aux["ids"].long() // (cfg.E // world)).cpu()                       # [T, k]
    visits = torch.zeros(T, world, dtype=torch.bool)
    visits.scatter_(1, owners, True)
    for r in range(world):
        sent, received, pairs = counts[r]
        mine = visits[r * T_local:(r + 1) * T_local]
        assert sent == [int(v) for v in mine.sum(0)]
        assert received == int(visits[:, r].sum())
        assert pairs == int((owners == r).sum())
    assert sum(c[1] for c in counts) < T * min(cfg.k, world)                     # fewer rows than (token, expert) pairs
    rel = ((second - ref).norm() / ref.norm()).item()
    assert rel <= 2e-3, rel
    # per token too: no row may be off by more than f16 rounding of a few partial sums allows
    worst = ((second - ref).norm(dim=1) / ref.norm(dim=1).clamp_min(1e-6)).max().item()
    assert worst <= 1e-2, worst
    # and against the CPU oracle itself on a few tokens of different ranks (the bars of the single-GPU full-shape tests)
    import numpy as np
    from tests import helpers as Hh
    sub = np.asarray([0, T_local - 1, T_local, T - 1])
    want = Hh.run_oracle(cfg, x.cpu(), token_subset=sub)
    rel_o, mx_o = Hh.error_metrics(second[torch.from_numpy(sub).cuda()].cpu().numpy(), want["out"])
    assert rel_o <= 2e-3 and mx_o <= 2.0 ** -6, (rel_o, mx_o)


def test_peer_overflow_is_reported_by_every_rank_and_next_step_works():
    cfg = synth.MoeConfig("ep_over", H=256, I=128, E=8, k=2, fmt=0, T=64, seed=3, zipf_s=1.4)
    world, T_local = 2, 32
    x = synth.gen_inputs(cfg, 64).cuda()
    _, aux = reference(cfg, x)
    per_rank = torch.bincount((aux["ids"].reshape(-1) // 4).long(), minlength=2)
    cap = int(per_rank.max().item()) - 1      # one row short on the busier rank
    ranks = Ranks(cfg, world, T_local, cap=cap)
    try:
        xs = [x[:32].contiguous(), x[32:].contiguous()]
        outs, errs = ranks.step(xs, check=False)
        assert len(errs) >= 2 and all("inconsistent group table" in e for e in errs), errs
        # a step that fits goes through on the same state afterwards
        small = [x[:8].contiguous(), x[32:40].contiguous()]
        outs, _ = ranks.step(small)
        ref, _ = reference(cfg, torch.cat(small, 0))
        got = torch.cat([outs[0], outs[1]], 0)
        assert ((got - ref).norm() / ref.norm()).item() <= 2e-3
    finally:
        ranks.close()


def test_peer_wait_runs_out_when_a_rank_never_joins():
    """Rank 1 never steps: rank 0's waits give up after wait_ms, the status says so, and the
    context keeps working (a later single-GPU call on it succeeds)."""
    cfg = synth.MoeConfig("ep_wait", H=256, I=128, E=8, k=2, fmt=0, T=16, seed=4)
    ranks = Ranks(cfg, 2, 8, cap=32, wait_ms=50, active=[0])
    try:
        x = synth.gen_inputs(cfg, 16).cuda()
        outs, errs = ranks.step([x[:8].contiguous(), None], check=False)
        assert errs and all("bounded wait timed out" in e for e in errs), errs
        ids, w = ranks.layers[0].route(x[:8].contiguous())
        ranks.ctxs[0].synchronize()
        assert ids.shape == (8, 2)
    finally:
        ranks.close()
