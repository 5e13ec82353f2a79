"""Every benchmark configuration at its REAL shape against the CPU oracle, through the C ABI.

Routing (logits, expert ids, routing weights) and grouping (counts, offsets, permutation) are
compared bit for bit over ALL tokens; the layer output is compared on a handful of tokens (the
oracle regenerates only the experts those tokens route to), within the bars of the task: relative
L2 <= 1e-2 and max-abs <= 2^-6 x RMS of the oracle's FP32-accumulate result.  The shapes follow
the reference's own full-shape command test (tests/test_cuda_backend.cpp:1509-1574: the GLM INT4
command at hidden 6144 / intermediate 2048).

  c1 / c1_sigmoid at 64 and 256 tokens   hybrid route: weight-streaming gate/up + tensor-core down
  c2 at 4096 tokens                      INT4-g128 on the tcgen05 path, 128 rows per expert, 128-token tiles
  c3 at 16384 tokens                     MXFP4 on the tcgen05 path, 512 rows per expert, 192-token tiles
  c3, one rank's share of an 8-GPU run   32 resident experts, the rows they receive (grouped stage call)
  c4 at 256 tokens                       896 experts, top-16, Zipf-biased router, mixed dispatch
"""
import gc

import numpy as np
import pytest
import torch

from oracle import oracle as O
from strata_b200 import MoeContext, MoeLayer, synth
from tests import helpers as Hh

pytestmark = pytest.mark.gpu

REL_L2, MAX_ABS = 1e-2, 2.0 ** -6
TENSOR_TIGHT = 2e-3      # tensor-core path: the SwiGLU output is one f16 (11-bit significand)


@pytest.fixture(scope="module")
def ctx():
    return MoeContext(0)


def release(*objs):
    for o in objs:
        if hasattr(o, "close"):
            o.close()
    gc.collect()
    torch.cuda.empty_cache()


def check_routing(aux, ref, weights_exact=True):
    assert np.array_equal(aux["logits"].cpu().numpy().view(np.uint32), ref["logits"].view(np.uint32))
    assert np.array_equal(aux["ids"].cpu().numpy().astype(np.uint32), ref["ids"])
    if weights_exact:
        assert np.array_equal(aux["weights"].cpu().numpy().view(np.uint32), ref["weights"].view(np.uint32))
    assert np.array_equal(aux["counts"].cpu().numpy().astype(np.uint32), ref["counts"])
    assert np.array_equal(aux["offsets"].cpu().numpy().astype(np.uint32), ref["offsets"])
    assert np.array_equal(aux["perm"].cpu().numpy().astype(np.uint32), ref["perm"])


def full_layer(ctx, cfg, T, sub, tight):
    layer = synth.build_layer(cfg, "cuda", T=T)
    ml = MoeLayer(ctx, cfg, max_tokens=T)
    ml.load_synth(layer)
    out, aux = ml.forward(layer.x, want_aux=True)
    ctx.synchronize()
    out2 = ml.forward(layer.x)
    ctx.synchronize()
    assert torch.equal(out, out2)                      # bit-reproducible run to run
    sub = np.asarray(sub)
    ref = Hh.run_oracle(cfg, layer.x.cpu(), token_subset=sub)
    check_routing(aux, ref)
    if T >= 512 and cfg.score_kind != synth.SCORE_SOFTMAX:
        # without the logits in the aux outputs a batch this large takes the fast router (tensor-core projection,
        # exact recheck): ids, rank order, counts and permutation must be bit-identical all the same
        before = ctx.stats()
        out3, aux3 = ml.forward(layer.x, want_aux=True, aux_logits=False)
        ctx.synchronize()
        after = ctx.stats()
        assert after.router_fast_tokens - before.router_fast_tokens == T
        assert after.router_rechecked_tokens - before.router_rechecked_tokens <= T // 100
        assert np.array_equal(aux3["ids"].cpu().numpy().astype(np.uint32), ref["ids"])
        assert np.array_equal(aux3["weights"].cpu().numpy().view(np.uint32), ref["weights"].view(np.uint32))
        assert after.router_worst_error <= 0.25, after.router_worst_error
        assert np.array_equal(aux3["counts"].cpu().numpy().astype(np.uint32), ref["counts"])
        assert np.array_equal(aux3["perm"].cpu().numpy().astype(np.uint32), ref["perm"])
        assert torch.equal(out3, out)
        del out3, aux3
    rel, mx = Hh.error_metrics(out[torch.from_numpy(sub).cuda()].cpu().numpy(), ref["out"])
    counts = aux["counts"].cpu().numpy()
    release(ml)
    del layer, out, out2, aux
    release()
    assert rel <= REL_L2 and mx <= MAX_ABS, (rel, mx)
    assert rel <= tight, rel
    return counts


@pytest.mark.parametrize("name,T", [("c1", 256), ("c1_sigmoid", 256), ("c1", 64), ("c1_sigmoid", 64)])
def test_c1_batch_sizes_of_the_sweep(ctx, name, T):
    # 10 (T=256) and 2.5 (T=64) rows per expert: the routes the benchmark's sweep takes
    full_layer(ctx, synth.CONFIGS[name], T, [0, 1, T // 2, T - 1], TENSOR_TIGHT)


def test_c2_int4_prefill_full_shape(ctx):
    counts = full_layer(ctx, synth.CONFIGS["c2"], 4096, [0, 1, 1777, 2048, 4095], TENSOR_TIGHT)
    assert counts.sum() == 4096 * 8 and counts.min() > 64       # every expert is on the tensor-core path


def test_c3_mxfp4_prefill_full_shape(ctx):
    counts = full_layer(ctx, synth.CONFIGS["c3"], 16384, [0, 8191, 12345, 16383], TENSOR_TIGHT)
    assert counts.sum() == 16384 * 8 and counts.min() > 192     # several 192-token tiles per expert


def test_c4_896_experts_zipf_full_shape(ctx):
    counts = full_layer(ctx, synth.CONFIGS["c4"], 256, [0, 100, 255], TENSOR_TIGHT)
    # the Zipf bias makes a few experts hot (tensor-core path inside the step) and leaves many idle
    assert counts.max() >= 24 and (counts == 0).any(), (counts.max(), (counts == 0).sum())


def test_c3_one_rank_share(ctx):
    """What rank 3 of an 8-GPU run computes: its 32 resident experts over the rows every rank sends
    them, through the grouped stage call, against the oracle's per-expert result."""
    cfg = synth.CONFIGS["c3"]
    T, world, rank = 16384, 8, 3
    B = cfg.E // world
    layer = synth.build_layer(cfg, "cuda", expert_begin=rank * B, expert_end=(rank + 1) * B, T=T)
    router = MoeLayer(ctx, cfg, max_tokens=T, expert_begin=rank * B, expert_count=B, max_pairs=T * cfg.k // 4)
    router.load_synth(layer)
    ids, w = router.route(layer.x)
    counts, offsets, perm = router.group(ids, rank * B, B)
    ctx.synchronize()
    ids_h = ids.cpu().numpy().astype(np.uint32)
    rcounts, roffsets, rperm = O.group(ids_h, cfg.E)
    lo, hi = int(roffsets[rank * B]), int(roffsets[(rank + 1) * B])
    n = hi - lo
    assert np.array_equal(counts.cpu().numpy().astype(np.uint32), rcounts[rank * B:(rank + 1) * B])
    assert np.array_equal(perm.cpu().numpy().astype(np.uint32)[:n], rperm[lo:hi])
    rows = router.gather_rows(layer.x, perm, cfg.k, n=n)
    y = router.experts_grouped(rows, offsets)
    ctx.synchronize()
    # oracle: a few rows of a few local experts
    x_h = layer.x.cpu()
    yh = y.cpu().numpy()
    off = offsets.cpu().numpy().astype(np.int64)
    picks = [(0, 0), (7, 100), (31, int(counts[31].item()) - 1)]
    experts, keep = Hh.oracle_experts(cfg, [rank * B + le for le, _ in picks])
    got, want = [], []
    import ctypes as C
    for le, r in picks:
        pos = int(off[le]) + r
        tok = int(rperm[lo + pos]) // cfg.k
        xf = np.ascontiguousarray(x_h[tok].float().numpy())
        a = np.empty(cfg.I, np.float32)
        u = np.empty(cfg.I, np.float32)
        out = np.empty(cfg.H, np.float32)
        f32p = C.POINTER(C.c_float)
        rc = O.port().orc_expert_ffn(C.byref(experts[rank * B + le]), xf.ctypes.data_as(f32p), C.c_float(1.0), 0, 0,
                                     a.ctypes.data_as(f32p), u.ctypes.data_as(f32p), out.ctypes.data_as(f32p))
        assert rc == 0
        got.append(yh[pos])
        want.append(out)
    rel, mx = Hh.error_metrics(np.stack(got), np.stack(want))
    release(router)
    assert rel <= TENSOR_TIGHT and mx <= MAX_ABS, (rel, mx)
