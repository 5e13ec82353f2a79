"""The oracle's view of a synthetic layer (checker glue: TEST INFRASTRUCTURE ONLY, like the rest of oracle/)."""
import numpy as np
import torch

from oracle import oracle as O
from strata_b200 import synth


def np_u16(t):
    """bf16 torch tensor -> uint16 numpy (bit pattern)."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def oracle_experts(cfg, needed):
    """ctypes Expert array of length E with host weights for the experts in `needed`."""
    arr = (O.Expert * cfg.E)()
    keep = []
    for e in sorted(set(int(v) for v in needed)):
        mats = []
        for role in synth.ROLES:
            rows, cols = cfg.role_shape(role)
            p, s = synth.gen_expert_range(cfg, role, e, e + 1, "cpu")
            p = np.ascontiguousarray(p[0].numpy())
            s = np.ascontiguousarray(s[0].numpy())
            keep += [p, s]
            g = synth.NVFP4_GLOBAL[role] if cfg.fmt == synth.FMT_NVFP4 else 1.0
            mats.append(O.make_matrix(cfg.fmt, rows, cols, p, s, g))
        arr[e].gate, arr[e].up, arr[e].down = mats
        arr[e].activation, arr[e].gate_beta, arr[e].linear_beta = cfg.activation, cfg.gate_beta, cfg.linear_beta
    return arr, keep


def oracle_shared(cfg):
    sh = synth.gen_shared(cfg)
    if not sh:
        return None, []
    ex = O.Expert()
    keep = []
    mats = []
    for role in synth.ROLES:
        w = np.ascontiguousarray(np_u16(sh[role]))
        keep.append(w)
        mats.append(O.make_matrix(O.FMT_BF16, w.shape[0], w.shape[1], w))
    ex.gate, ex.up, ex.down = mats
    ex.activation, ex.gate_beta, ex.linear_beta = cfg.activation, cfg.gate_beta, cfg.linear_beta
    return ex, keep


def oracle_desc(cfg, T, accumulate_double=False, combine_order=O.COMBINE_RANK_ORDER):
    d = O.LayerDesc()
    d.T, d.H, d.I, d.E, d.k = T, cfg.H, cfg.I, cfg.E, cfg.k
    d.router = O.router_spec(cfg.E, cfg.k, cfg.score_kind, cfg.normalize, cfg.norm_init, cfg.weight_scale)
    d.output_scale = cfg.output_scale
    d.combine_order = combine_order
    d.coef_before_down = 0
    d.accumulate_double = int(accumulate_double)
    d.I_shared = cfg.I_shared
    return d


def run_oracle(cfg, x_bf16, token_subset=None, accumulate_double=False):
    """Routing for all tokens, expert outputs for the subset.  x_bf16: torch bf16 [T,H] (CPU)."""
    T = x_bf16.shape[0]
    w, b = synth.gen_router(cfg)
    desc = oracle_desc(cfg, T, accumulate_double)
    # routing first (cheap) to learn which experts the subset needs
    logits = O.router_logits(np_u16(x_bf16), np_u16(w))
    rc, ids, wts = O.route(desc.router, logits, b.numpy() if b is not None else None)
    assert rc == 0
    sub = np.arange(T, dtype=np.uint32) if token_subset is None else np.asarray(token_subset, np.uint32)
    experts, keep = oracle_experts(cfg, ids[sub].reshape(-1))
    shared, keep2 = oracle_shared(cfg)
    res = O.moe_layer(desc, np_u16(x_bf16), np_u16(w), b.numpy() if b is not None else None, experts,
                      shared, sub)
    assert res["rc"] == 0
    res["subset"] = sub
    return res


def run_oracle_latent(cfg, x_bf16, token_subset=None):
    """LatentMoE (cfg.H_model > 0): routing for all tokens, outputs [len(subset), H_model] for the subset."""
    import ctypes as C
    T = x_bf16.shape[0]
    w, b = synth.gen_router(cfg)
    lat = synth.gen_latent(cfg)
    desc = oracle_desc(cfg, T)
    xs, ws = np_u16(x_bf16), np_u16(w)
    ids = np.empty((T, cfg.k), np.uint32)
    wts = np.empty((T, cfg.k), np.float32)
    bias = np.ascontiguousarray(b.numpy()) if b is not None else None
    down, up = np_u16(lat["down"]), np_u16(lat["up"])
    norm = np.ascontiguousarray(lat["norm"].numpy())
    lib = O.port()
    def call(experts, shared, sub, out):
        return lib.orc_latent_moe_layer(
            C.byref(desc), cfg.H_model, float(cfg.rms_epsilon), xs.ctypes.data_as(O.u16p), ws.ctypes.data_as(O.u16p),
            bias.ctypes.data_as(O.f32p) if bias is not None else None, down.ctypes.data_as(O.u16p),
            up.ctypes.data_as(O.u16p), norm.ctypes.data_as(O.f32p), experts, C.byref(shared) if shared is not None else None,
            sub.ctypes.data_as(O.u32p) if sub is not None else None, 0 if sub is None else len(sub),
            ids.ctypes.data_as(O.u32p), wts.ctypes.data_as(O.f32p), out.ctypes.data_as(O.f32p) if out is not None else None)
    assert call(None, None, None, None) == 0            # routing only: which experts does the subset need
    sub = np.arange(T, dtype=np.uint32) if token_subset is None else np.asarray(token_subset, np.uint32)
    experts, keep = oracle_experts(cfg, ids[sub].reshape(-1))
    shared, keep2 = oracle_shared(cfg)
    out = np.empty((len(sub), cfg.H_model), np.float32)
    assert call(experts, shared, sub, out) == 0
    return dict(ids=ids, weights=wts, out=out, subset=sub)


def error_metrics(got, want):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    rel_l2 = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
    rms = np.sqrt(np.mean(want ** 2))
    max_abs_over_rms = np.abs(got - want).max() / max(rms, 1e-30)
    return rel_l2, max_abs_over_rms
