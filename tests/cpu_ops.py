"""CPU stand-in for strata_b200.api.MoeLayer built on the oracle: lets the expert-parallel
exchange logic run under gloo without a GPU.  Test infrastructure only."""
import ctypes as C

import numpy as np
import torch

from oracle import oracle as O
from strata_b200 import synth
from tests import helpers as Hh


class OracleOps:
    def __init__(self, cfg, expert_begin, expert_count):
        self.cfg, self.ebeg, self.n = cfg, expert_begin, expert_count
        self.router_w, self.bias = synth.gen_router(cfg)
        self.spec = O.router_spec(cfg.E, cfg.k, cfg.score_kind, cfg.normalize, cfg.norm_init, cfg.weight_scale)
        self.experts, self._keep = Hh.oracle_experts(cfg, range(expert_begin, expert_begin + expert_count))
        self.shared, self._keep2 = Hh.oracle_shared(cfg)

    def route(self, x):
        logits = O.router_logits(Hh.np_u16(x), Hh.np_u16(self.router_w))
        rc, ids, w = O.route(self.spec, logits, self.bias.numpy() if self.bias is not None else None)
        assert rc == 0
        return torch.from_numpy(ids.astype(np.int32)), torch.from_numpy(w)

    def group(self, ids, expert_begin=0, n_experts=None, want_inv=False):
        n_experts = self.cfg.E if n_experts is None else n_experts
        flat = ids.reshape(-1).numpy().astype(np.int64) - expert_begin
        ok = (flat >= 0) & (flat < n_experts)
        idx = np.nonzero(ok)[0]
        order = idx[np.argsort(flat[idx], kind="stable")]
        counts = np.bincount(flat[idx], minlength=n_experts).astype(np.int32)
        offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        perm = np.zeros(flat.size, np.int32)
        perm[:order.size] = order
        inv = np.full(flat.size, -1, np.int32)
        inv[order] = np.arange(order.size, dtype=np.int32)
        out = (torch.from_numpy(counts), torch.from_numpy(offsets), torch.from_numpy(perm))
        return out + (torch.from_numpy(inv),) if want_inv else out

    def gather_rows(self, src, index, index_div=1, n=None):
        n = index.numel() if n is None else n
        return src[(index[:n].long() // index_div)].contiguous()

    def experts_grouped(self, rows, offsets):
        cfg = self.cfg
        xf = rows.float().numpy()
        y = np.zeros((rows.shape[0], cfg.H), np.float32)
        a = np.empty(cfg.I, np.float32)
        u = np.empty(cfg.I, np.float32)
        off = offsets.numpy()
        for le in range(self.n):
            for pos in range(off[le], off[le + 1]):
                rc = O.port().orc_expert_ffn(C.byref(self.experts[self.ebeg + le]),
                                             xf[pos].ctypes.data_as(O.f32p), 1.0, 0, 0,
                                             a.ctypes.data_as(O.f32p), u.ctypes.data_as(O.f32p),
                                             y[pos].ctypes.data_as(O.f32p))
                assert rc == 0
        return torch.from_numpy(y)

    def combine(self, y, inv, weights, x_shared=None, out=None):
        cfg = self.cfg
        T = weights.shape[0]
        yv, iv, wv = y.numpy(), inv.numpy().reshape(T, cfg.k), weights.numpy()
        o = np.zeros((T, cfg.H), np.float32)
        for t in range(T):
            for r in range(cfg.k):
                if iv[t, r] >= 0:
                    o[t] = o[t] + yv[iv[t, r]] * wv[t, r]
            if cfg.output_scale != 1.0:
                o[t] = o[t] * np.float32(cfg.output_scale)
            if x_shared is not None and self.shared is not None:
                xf = x_shared[t].float().numpy()
                a = np.empty(cfg.I_shared, np.float32)
                u = np.empty(cfg.I_shared, np.float32)
                ys = np.empty(cfg.H, np.float32)
                rc = O.port().orc_expert_ffn(C.byref(self.shared), xf.ctypes.data_as(O.f32p), 1.0, 0, 0,
                                             a.ctypes.data_as(O.f32p), u.ctypes.data_as(O.f32p),
                                             ys.ctypes.data_as(O.f32p))
                assert rc == 0
                o[t] = o[t] + ys
        return torch.from_numpy(o)
