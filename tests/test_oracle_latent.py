"""The plain-C LatentMoE restatement (oracle/moe_oracle.c: orc_latent_moe_layer) against the reference's own
kimi_latent_moe_layer compiled unmodified (oracle/_ref), at the shape its contract fixes: hidden 7168, latent 3584,
896 MXFP4 experts of width 3072, top-16, two BF16 shared experts, SiTU-GLU.  The reference's BF16 projections and
MXFP4 matvecs use AVX2 summation orders, so outputs are compared within FP32 reassociation, expert ids exactly."""
import ctypes as C

import numpy as np

from oracle import layer_check as Hh
from oracle import oracle as O
from strata_b200 import synth


def test_latent_moe_matches_compiled_reference(ref):
    cfg = synth.CONFIGS["kimi"]
    T = 2
    x = synth.gen_inputs(cfg, T)
    mine = Hh.run_oracle_latent(cfg, x)
    # the same tensors for the reference call
    w, b = synth.gen_router(cfg)
    lat = synth.gen_latent(cfg)
    sh = synth.gen_shared(cfg)
    bias = np.zeros(cfg.E, np.float32) if b is None else np.ascontiguousarray(b.numpy())
    keep, ptrs = [], (C.c_void_p * (cfg.E * 6))()
    for e in sorted(set(int(v) for v in mine["ids"].reshape(-1))):
        for r, role in enumerate(synth.ROLES):
            p, s = synth.gen_expert_range(cfg, role, e, e + 1, "cpu")
            p, s = np.ascontiguousarray(p[0].numpy()), np.ascontiguousarray(s[0].numpy())
            keep += [p, s]
            ptrs[e * 6 + 2 * r] = p.ctypes.data
            ptrs[e * 6 + 2 * r + 1] = s.ctypes.data
    xf = np.ascontiguousarray(x.float().numpy())
    out = np.empty((T, cfg.H_model), np.float32)
    ids = np.empty((T, cfg.k), np.uint32)
    wts = np.empty((T, cfg.k), np.float32)
    u16 = lambda t: Hh.np_u16(t).ctypes.data_as(O.u16p)
    keep += [Hh.np_u16(t) for t in (w, lat["down"], lat["up"], sh["gate"], sh["up"], sh["down"])]
    norm = np.ascontiguousarray(lat["norm"].numpy())
    rc = ref.ref_kimi_latent_moe(out.ctypes.data_as(O.f32p), xf.ctypes.data_as(O.f32p), T, keep[-6].ctypes.data_as(O.u16p),
                                 bias.ctypes.data_as(O.f32p), keep[-5].ctypes.data_as(O.u16p),
                                 keep[-4].ctypes.data_as(O.u16p), norm.ctypes.data_as(O.f32p),
                                 keep[-3].ctypes.data_as(O.u16p), keep[-2].ctypes.data_as(O.u16p),
                                 keep[-1].ctypes.data_as(O.u16p), ptrs, ids.ctypes.data_as(O.u32p),
                                 wts.ctypes.data_as(O.f32p))
    assert rc == 0
    assert np.array_equal(ids, mine["ids"])                     # same selection, same rank order
    assert np.allclose(wts, mine["weights"], rtol=2e-6, atol=0)  # logits differ in the last bits between the two orders
    rel, mx = Hh.error_metrics(mine["out"], out)
    assert rel <= 2e-5 and mx <= 2e-4, (rel, mx)
