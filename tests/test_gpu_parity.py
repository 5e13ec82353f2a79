"""CUDA path against the CPU oracle through the C ABI (needs a B200).

Bars (from the task's north star): expert ids, permutation, counts and offsets bit-exact;
dequantised weights bit-exact; layer output within relative L2 1e-2 and max-abs 2^-6 x RMS of
the oracle's FP32-accumulate result.  The kernels accumulate in FP32 as well, so a much tighter
bound is asserted alongside to catch layout or indexing mistakes early.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from strata_b200 import MoeContext, MoeLayer, synth
from tests import helpers as Hh

pytestmark = pytest.mark.gpu

REL_L2, MAX_ABS = 1e-2, 2.0 ** -6
TIGHT_REL_L2 = 2e-4          # weight-streaming kernels: activations carried as an f16 hi/lo pair
TENSOR_REL_L2 = 1e-3         # tensor-core kernels: one f16 per activation element


def tight_bound(cfg, T):
    """From 8 rows per expert on, the down projection (from 12 on, both GEMMs) runs on the tensor-core path."""
    if cfg.I_shared and T >= 24:
        return 2e-3          # shared expert on the tensor-core path: BF16 activation between its GEMMs
    if cfg.fmt != synth.FMT_BF16 and T * cfg.k >= 8 * cfg.E:
        return TENSOR_REL_L2
    return TIGHT_REL_L2


@pytest.fixture(scope="module")
def ctx():
    return MoeContext(0)


def small(fmt, **kw):
    base = dict(name=f"small{fmt}", H=512, I=256, E=16, k=4, fmt=fmt, T=8, seed=3)
    base.update(kw)
    return synth.MoeConfig(**base)


SMALL_CASES = [
    small(synth.FMT_MXFP4),
    small(synth.FMT_NVFP4, I_shared=128),
    small(synth.FMT_INT4, norm_init=1e-20, weight_scale=2.5),
    small(synth.FMT_MXFP4, T=1, name="one_token"),
    small(synth.FMT_MXFP4, T=37, E=8, k=3, H=384, I=128, name="ragged"),
    small(synth.FMT_NVFP4, T=19, score_kind=synth.SCORE_SOFTMAX, name="softmax"),
    small(synth.FMT_INT4, T=5, score_kind=synth.SCORE_SIGMOID_PLAIN, E=32, k=16, name="kimi_like"),
    small(synth.FMT_NVFP4, T=9, output_scale=2.5, I_shared=256, name="laguna_like"),
    small(synth.FMT_MXFP4, T=8, zipf_s=1.1, E=64, k=8, name="zipf_bias"),
    small(synth.FMT_BF16, T=6, name="plain_bf16"),
    small(synth.FMT_MXFP4, T=7, activation=1, gate_beta=2.5, linear_beta=4.0, name="situ_stream"),
    small(synth.FMT_NVFP4, T=80, E=8, k=2, activation=1, gate_beta=1.5, linear_beta=2.0, I_shared=128, name="situ_tensor"),
    small(synth.FMT_INT4, T=5, activation=1, gate_beta=3.0, linear_beta=3.0, name="situ_int4"),
    small(synth.FMT_BF16, T=40, E=8, k=2, name="plain_bf16_rows"),
    small(synth.FMT_MXFP4, T=33, E=32, k=6, score_kind=synth.SCORE_SQRTSOFTPLUS, weight_scale=1.5, name="dsv4_router"),
    # shapes the bulk-copy ring kernels accept (MXFP4 needs K % 512 == 0 on both GEMMs, NVFP4 K % 256 == 0)
    small(synth.FMT_MXFP4, I=512, name="ring_mx"),
    small(synth.FMT_MXFP4, I=512, T=13, name="ring_mx_two_token_tiles"),
    small(synth.FMT_MXFP4, H=1024, I=512, T=23, E=4, k=2, name="ring_mx_passes"),
    small(synth.FMT_NVFP4, H=768, I=256, T=11, E=8, k=2, name="ring_nv_short_last_stage"),
    small(synth.FMT_MXFP4, H=1536, I=1024, T=5, E=8, k=3, name="ring_mx_three_stages"),
]


def run_layer(ctx, cfg, T=None):
    layer = synth.build_layer(cfg, "cuda", T=T)
    ml = MoeLayer(ctx, cfg, max_tokens=layer.x.shape[0])
    ml.load_synth(layer)
    out, aux = ml.forward(layer.x, want_aux=True)
    ctx.synchronize()
    return layer, ml, out, aux


@pytest.mark.parametrize("cfg", SMALL_CASES, ids=lambda c: c.name)
def test_small_layer_matches_oracle(ctx, cfg):
    layer, ml, out, aux = run_layer(ctx, cfg)
    ref = Hh.run_oracle(cfg, layer.x.cpu())
    assert np.array_equal(aux["logits"].cpu().numpy().view(np.uint32), ref["logits"].view(np.uint32))
    assert np.array_equal(aux["ids"].cpu().numpy().astype(np.uint32), ref["ids"])
    assert np.array_equal(aux["weights"].cpu().numpy().view(np.uint32), ref["weights"].view(np.uint32))
    assert np.array_equal(aux["counts"].cpu().numpy().astype(np.uint32), ref["counts"])
    assert np.array_equal(aux["offsets"].cpu().numpy().astype(np.uint32), ref["offsets"])
    assert np.array_equal(aux["perm"].cpu().numpy().astype(np.uint32), ref["perm"])
    rel, mx = Hh.error_metrics(out.cpu().numpy(), ref["out"])
    assert rel <= REL_L2 and mx <= MAX_ABS
    assert rel <= tight_bound(cfg, layer.x.shape[0]), rel


@pytest.mark.parametrize("fmt,wide", [(synth.FMT_MXFP4, True), (synth.FMT_MXFP4, False),
                                      (synth.FMT_NVFP4, True), (synth.FMT_INT4, False), (synth.FMT_BF16, False)])
def test_dequantised_weights_bit_exact(ctx, fmt, wide):
    # wide MXFP4 scales force the general BF16 decoders; narrow ones take the f16 path
    cfg = small(fmt, H=256, I=128, E=4, k=2, name=f"deq{fmt}")
    layer = synth.build_layer(cfg, "cuda")
    if fmt == synth.FMT_MXFP4 and not wide:
        for role in synth.ROLES:
            s = layer.scales[role]
            layer.scales[role] = (torch.arange(s.numel(), device="cuda") % 27 + 100).to(torch.uint8).view_as(s)
    if fmt == synth.FMT_MXFP4 and wide:
        # widen the scale spread over every legal E8M0 byte, including block scales >= 4
        for role in synth.ROLES:
            s = layer.scales[role]
            layer.scales[role] = (torch.arange(s.numel(), device="cuda") % 254 + 1).to(torch.uint8).view_as(s)
    if fmt == synth.FMT_NVFP4:
        # every finite E4M3 byte, including subnormal and negative block scales
        for role in synth.ROLES:
            s = layer.scales[role]
            v = (torch.arange(s.numel(), device="cuda") % 256)
            v = torch.where((v & 0x7F) == 0x7F, torch.zeros_like(v), v)
            layer.scales[role] = v.to(torch.uint8).view_as(s)
    ml = MoeLayer(ctx, cfg)
    ml.set_router(layer.router_w, layer.bias)
    for r, role in enumerate(synth.ROLES):
        for e in range(cfg.E):
            ml.set_expert(e, r, layer.packed[role][e], layer.scales[role][e], 1.0)
    for r, role in enumerate(synth.ROLES):
        rows, cols = cfg.role_shape(role)
        for e in (0, cfg.E - 1):
            got = ml.dequant_export(e, r).numpy()
            p = layer.packed[role][e].cpu().numpy()
            s = layer.scales[role][e].cpu().numpy()
            want = O.dequant(O.make_matrix(fmt, rows, cols, p, s, 1.0), device_zero=True)
            # zero sign is canonicalised: the CPU tables and the device decode of the reference
            # disagree on nibble 0x8 themselves
            got = got + 0.0
            want = want + 0.0
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (role, e)


def test_nvfp4_global_scale_within_one_ulp(ctx):
    cfg = small(synth.FMT_NVFP4, H=256, I=128, E=2, k=1, name="deq_global")
    layer = synth.build_layer(cfg, "cuda")
    ml = MoeLayer(ctx, cfg)
    ml.load_synth(layer)
    got = ml.dequant_export(1, 0).numpy()
    p, s = layer.packed["gate"][1].cpu().numpy(), layer.scales["gate"][1].cpu().numpy()
    want = O.dequant(O.make_matrix(O.FMT_NVFP4, cfg.I, cfg.H, p, s, synth.NVFP4_GLOBAL["gate"]))
    assert np.all(np.abs(got - want) <= np.spacing(np.abs(want).astype(np.float32)))


@pytest.mark.parametrize("name,T,n_check", [("c0", 8, 8), ("c1", 16, 6), ("c1_sigmoid", 4, 4)])
def test_full_size_decode_configs(ctx, name, T, n_check):
    cfg = synth.CONFIGS[name]
    layer, ml, out, aux = run_layer(ctx, cfg, T=T)
    sub = np.arange(T)[:n_check]
    ref = Hh.run_oracle(cfg, layer.x.cpu(), token_subset=sub)
    assert np.array_equal(aux["logits"].cpu().numpy().view(np.uint32), ref["logits"].view(np.uint32))
    assert np.array_equal(aux["ids"].cpu().numpy().astype(np.uint32), ref["ids"])
    assert np.array_equal(aux["counts"].cpu().numpy().astype(np.uint32), ref["counts"])
    assert np.array_equal(aux["perm"].cpu().numpy().astype(np.uint32), ref["perm"])
    rel, mx = Hh.error_metrics(out.cpu().numpy()[sub], ref["out"])
    assert rel <= REL_L2 and mx <= MAX_ABS
    assert rel <= TIGHT_REL_L2, rel


def test_forward_host_round_trip_and_determinism(ctx):
    cfg = small(synth.FMT_MXFP4, T=8, name="host")
    layer, ml, out, aux = run_layer(ctx, cfg)
    xh = layer.x.cpu().pin_memory()
    oh = torch.empty(cfg.T, cfg.H, dtype=torch.float32).pin_memory()
    ml.forward_host(xh, oh)
    assert torch.equal(oh, out.cpu())
    out2 = ml.forward(layer.x)
    ctx.synchronize()
    assert torch.equal(out2, out)      # bit-reproducible run to run


@pytest.mark.parametrize("chunks", [0, 3])
def test_forward_host_in_chunks_is_bit_identical(ctx, chunks, monkeypatch):
    """A large host-buffer call runs in token chunks with the copies overlapped (two by default when every expert still
    gets a full tile per chunk, any count on request): the result equals the device-resident one-piece call bit for bit
    -- tokens are independent."""
    if chunks:
        monkeypatch.setenv("STRATA_MOE_HOST_CHUNKS", str(chunks))
    cfg = small(synth.FMT_MXFP4, T=4100, E=8, k=2, H=512, I=256, name=f"host_chunks{chunks}")
    layer, ml, out, aux = run_layer(ctx, cfg)
    xh = layer.x.cpu().pin_memory()
    oh = torch.empty(cfg.T, cfg.H, dtype=torch.float32).pin_memory()
    ml.forward_host(xh, oh)
    assert torch.equal(oh, out.cpu())
    ml.forward_host(xh, oh)                 # and again: the staging halves are reused
    assert torch.equal(oh, out.cpu())


def test_empty_page_is_a_no_op(ctx):
    cfg = small(synth.FMT_MXFP4, name="empty")
    layer = synth.build_layer(cfg, "cuda")
    ml = MoeLayer(ctx, cfg)
    ml.load_synth(layer)
    out = ml.forward(layer.x[:0])
    ctx.synchronize()
    assert out.shape[0] == 0


def test_large_group_path_matches_small_path(ctx):
    # > 4096 pairs exercises the segmented histogram/scan/scatter kernels
    cfg = small(synth.FMT_MXFP4, T=1500, E=64, k=6, H=256, I=128, name="grp")
    layer = synth.build_layer(cfg, "cuda")
    ml = MoeLayer(ctx, cfg)
    ml.load_synth(layer)
    ids, w = ml.route(layer.x)
    counts, offsets, perm = ml.group(ids)
    ctx.synchronize()
    rc, rcounts, roffsets, rperm = 0, *O.group(ids.cpu().numpy().astype(np.uint32), cfg.E)
    assert np.array_equal(counts.cpu().numpy().astype(np.uint32), rcounts)
    assert np.array_equal(offsets.cpu().numpy().astype(np.uint32), roffsets)
    assert np.array_equal(perm.cpu().numpy().astype(np.uint32), rperm)
    # expert-parallel slice: only experts [16, 48)
    c2, o2, p2 = ml.group(ids, 16, 32)
    ctx.synchronize()
    n = int(roffsets[48] - roffsets[16])
    assert np.array_equal(c2.cpu().numpy().astype(np.uint32), rcounts[16:48])
    assert np.array_equal(p2.cpu().numpy().astype(np.uint32)[:n], rperm[roffsets[16]:roffsets[48]])


@pytest.mark.parametrize("fmt", [synth.FMT_MXFP4, synth.FMT_NVFP4])
def test_general_bf16_decoder_path(ctx, fmt, monkeypatch):
    # the FP4 formats normally take the f16 weight-streaming kernels; an expert whose MXFP4
    # scales span more than 26 octaves falls back to the general BF16 decoders, forced here
    monkeypatch.setenv("STRATA_MOE_NO_F16_PATH", "1")
    cfg = small(fmt, T=11, name=f"general{fmt}")
    layer, ml, out, aux = run_layer(ctx, cfg)
    ref = Hh.run_oracle(cfg, layer.x.cpu())
    assert np.array_equal(aux["ids"].cpu().numpy().astype(np.uint32), ref["ids"])
    rel, mx = Hh.error_metrics(out.cpu().numpy(), ref["out"])
    assert rel <= TIGHT_REL_L2 and mx <= MAX_ABS


PREFILL_TIGHT = 2e-3   # the tensor-core path keeps the SwiGLU output in f16 (11-bit significand)


@pytest.mark.parametrize("fmt", [synth.FMT_MXFP4, synth.FMT_NVFP4, synth.FMT_INT4])
def test_prefill_path_matches_oracle(ctx, fmt):
    # 600 tokens x top-2 over 8 experts: ~150 rows per expert -> tcgen05 grouped GEMM path,
    # ragged groups (row counts that are not multiples of 16 or 128)
    cfg = small(fmt, T=600, E=8, k=2, H=512, I=256, name=f"prefill{fmt}",
                I_shared=0, norm_init=1e-20 if fmt == synth.FMT_INT4 else 0.0)
    layer, ml, out, aux = run_layer(ctx, cfg)
    ref = Hh.run_oracle(cfg, layer.x.cpu())
    assert np.array_equal(aux["ids"].cpu().numpy().astype(np.uint32), ref["ids"])
    assert np.array_equal(aux["perm"].cpu().numpy().astype(np.uint32), ref["perm"])
    rel, mx = Hh.error_metrics(out.cpu().numpy(), ref["out"])
    assert rel <= REL_L2 and mx <= MAX_ABS
    assert rel <= PREFILL_TIGHT, rel


def test_prefill_path_tiny_and_empty_groups(ctx, monkeypatch):
    # force the tensor-core path on a page where most experts get 0-3 rows
    monkeypatch.setenv("STRATA_MOE_PREFILL_MIN_ROWS", "0")
    cfg = small(synth.FMT_NVFP4, T=5, E=16, k=2, H=256, I=128, name="prefill_tiny")
    layer, ml, out, aux = run_layer(ctx, cfg)
    ref = Hh.run_oracle(cfg, layer.x.cpu())
    rel, mx = Hh.error_metrics(out.cpu().numpy(), ref["out"])
    assert rel <= PREFILL_TIGHT and mx <= MAX_ABS


def test_prefill_and_streaming_paths_agree(ctx, monkeypatch):
    cfg = small(synth.FMT_MXFP4, T=300, E=8, k=2, H=512, I=256, name="paths")
    layer, ml, out_tc, _ = run_layer(ctx, cfg)
    monkeypatch.setenv("STRATA_MOE_NO_PREFILL_PATH", "1")   # switches are read when a layer is created
    ml2 = MoeLayer(ctx, cfg, max_tokens=layer.x.shape[0])
    ml2.load_synth(layer)
    out_stream = ml2.forward(layer.x)
    ctx.synchronize()
    rel, mx = Hh.error_metrics(out_tc.cpu().numpy(), out_stream.cpu().numpy())
    assert rel <= PREFILL_TIGHT


@pytest.mark.parametrize("fmt", [synth.FMT_MXFP4, synth.FMT_NVFP4])
def test_ring_and_register_streaming_kernels_agree(ctx, fmt, monkeypatch):
    # the same small batch through the bulk-copy ring kernels and through the register-streaming ones
    cfg = small(fmt, H=1024, I=512, T=9, E=8, k=3, name=f"ring_vs_reg{fmt}")
    layer, ml, out_ring, _ = run_layer(ctx, cfg)
    monkeypatch.setenv("STRATA_MOE_NO_STREAM_RING", "1")   # switches are read when a layer is created
    ml2 = MoeLayer(ctx, cfg, max_tokens=layer.x.shape[0])
    ml2.load_synth(layer)
    out_reg = ml2.forward(layer.x)
    ctx.synchronize()
    rel, mx = Hh.error_metrics(out_ring.cpu().numpy(), out_reg.cpu().numpy())
    assert rel <= 1e-5, rel        # same products, different FP32 summation order


@pytest.mark.parametrize("T,E,k,kind", [(1, 128, 4, synth.SCORE_SIGMOID), (8, 256, 6, synth.SCORE_SQRTSOFTPLUS),
                                        (16, 64, 8, synth.SCORE_SIGMOID), (13, 896, 16, synth.SCORE_SIGMOID_PLAIN)])
def test_decode_front_end_matches_separate_kernels(ctx, T, E, k, kind, monkeypatch):
    """At most 16 tokens: the whole-row logits kernel and the fused route + group + convert kernel against the staged
    logits kernel and the separate route / group / convert kernels: every routing and grouping output and the layer
    output bit for bit (the arithmetic is the same, only the launches differ)."""
    cfg = small(synth.FMT_MXFP4, T=T, E=E, k=k, H=512, I=512, score_kind=kind, zipf_s=0.7, name=f"front{T}_{E}_{k}")
    layer, ml, out, aux = run_layer(ctx, cfg)
    monkeypatch.setenv("STRATA_MOE_NO_SMALL_FRONT", "1")
    ml2 = MoeLayer(ctx, cfg, max_tokens=T)
    ml2.load_synth(layer)
    out2, aux2 = ml2.forward(layer.x, want_aux=True)
    ctx.synchronize()
    for key in ("logits", "ids", "weights", "counts", "offsets", "perm"):
        a, b = aux[key].cpu().numpy(), aux2[key].cpu().numpy()
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), key
    assert torch.equal(out, out2)
    ref = Hh.run_oracle(cfg, layer.x.cpu())
    assert np.array_equal(aux["logits"].cpu().numpy().view(np.uint32), ref["logits"].view(np.uint32))
    assert np.array_equal(aux["perm"].cpu().numpy().astype(np.uint32), ref["perm"])


def test_ring_kernels_with_sixteen_row_token_tiles(ctx, monkeypatch):
    # by default the ring kernels only take batches whose groups fit an 8-row tile; their 16-row variant on request
    monkeypatch.setenv("STRATA_MOE_STREAM_RING_MAX_ROWS", "16")
    cfg = small(synth.FMT_MXFP4, H=1024, I=512, T=23, E=4, k=2, name="ring_mx_sixteen")
    layer, ml, out, aux = run_layer(ctx, cfg)
    ref = Hh.run_oracle(cfg, layer.x.cpu())
    rel, mx = Hh.error_metrics(out.cpu().numpy(), ref["out"])
    assert rel <= REL_L2 and mx <= MAX_ABS, (rel, mx)


def test_shared_expert_on_tensor_core_path(ctx):
    # 200 tokens: the BF16 shared expert runs as a one-group grouped GEMM, the routed NVFP4
    # experts (50 rows each on average) take the tensor-core path as well
    cfg = small(synth.FMT_NVFP4, T=200, I_shared=256, output_scale=2.5, name="shared_tc")
    layer, ml, out, aux = run_layer(ctx, cfg)
    ref = Hh.run_oracle(cfg, layer.x.cpu())
    assert np.array_equal(aux["ids"].cpu().numpy().astype(np.uint32), ref["ids"])
    rel, mx = Hh.error_metrics(out.cpu().numpy(), ref["out"])
    assert rel <= PREFILL_TIGHT and mx <= MAX_ABS, (rel, mx)


def test_prefill_path_odd_hidden_size(ctx):
    # H = 384: not a multiple of 256, so the down projection takes the single-tile mode and the
    # last packed staging block of every row is half filled
    cfg = small(synth.FMT_MXFP4, T=400, E=8, k=2, H=384, I=128, name="prefill_odd")
    layer, ml, out, aux = run_layer(ctx, cfg)
    ref = Hh.run_oracle(cfg, layer.x.cpu())
    rel, mx = Hh.error_metrics(out.cpu().numpy(), ref["out"])
    assert rel <= PREFILL_TIGHT and mx <= MAX_ABS, (rel, mx)


def test_mixed_dispatch_under_a_skewed_router(ctx, monkeypatch):
    """A Zipf-biased router gives a few experts many rows and most experts few: inside one step the
    hot experts run on the tensor-core path and the rest on the weight-streaming kernels."""
    monkeypatch.setenv("STRATA_MOE_MIXED_MIN_TOKENS", "1")   # the default only switches it on from 128 tokens
    cfg = small(synth.FMT_MXFP4, T=64, E=64, k=6, zipf_s=1.3, name="skewed")
    layer, ml, out, aux = run_layer(ctx, cfg)
    counts = aux["counts"].cpu().numpy()
    assert counts.max() >= 24 and ((counts > 0) & (counts < 24)).any(), counts
    assert counts.sum() * 1.0 / cfg.E < 8           # the step as a whole is in the streaming regime
    ref = Hh.run_oracle(cfg, layer.x.cpu())
    assert np.array_equal(aux["ids"].cpu().numpy().astype(np.uint32), ref["ids"])
    rel, mx = Hh.error_metrics(out.cpu().numpy(), ref["out"])
    assert rel <= TENSOR_REL_L2 and mx <= MAX_ABS, (rel, mx)


@pytest.mark.parametrize("kind,zipf,dup", [(synth.SCORE_SIGMOID, 0.0, False), (synth.SCORE_SIGMOID_PLAIN, 1.1, False),
                                           (synth.SCORE_SQRTSOFTPLUS, 0.0, False), (synth.SCORE_SIGMOID, 0.0, True)])
def test_fast_router_is_bit_exact(ctx, kind, zipf, dup, monkeypatch):
    """Tensor-core projection + exact recheck against the canonical router: expert ids in rank order and routing
    weights bit for bit (the selected logits are recomputed in the canonical summation order).
    `dup` makes two experts identical, so that every token has an exact tie."""
    monkeypatch.setenv("STRATA_MOE_FAST_ROUTER_MIN_TOKENS", "1")
    cfg = small(synth.FMT_MXFP4, T=700, E=128, k=8, H=512, I=256, score_kind=kind, zipf_s=zipf,
                weight_scale=1.5, name=f"fast_router{kind}{int(dup)}")
    layer = synth.build_layer(cfg, "cuda")
    if dup:
        layer.router_w[77] = layer.router_w[3]
    ml = MoeLayer(ctx, cfg, max_tokens=cfg.T)
    ml.load_synth(layer)
    ids_x, w_x, _ = ml.route(layer.x, want_logits=True)      # canonical projection
    before = ctx.stats()
    ids_f, w_f = ml.route(layer.x)                            # fast path
    ctx.synchronize()
    after = ctx.stats()
    assert after.router_fast_tokens - before.router_fast_tokens == cfg.T
    rechecked = after.router_rechecked_tokens - before.router_rechecked_tokens
    assert torch.equal(ids_f, ids_x)
    assert torch.equal(w_f.view(torch.int32), w_x.view(torch.int32))
    assert 0.0 < after.router_worst_error <= 0.5      # the bound the selection assumes, with room to spare
    if dup:
        # tokens whose selection holds a twin have an exact tie; the canonical rule (lower index first) decides it on the
        # recomputed logits, inside the fast path
        touched = int(((ids_x == 3) | (ids_x == 77)).any(dim=1).sum().item())
        assert touched > 0
    assert rechecked <= cfg.T // 50


def test_workspace_guard_zones_stay_intact():
    """Ragged shapes through every expert path on a fresh context (small workspaces, so an overrun lands in a guard
    zone and not in slack): the canary bytes around all workspaces are intact afterwards."""
    c = MoeContext(0)
    for cfg in (small(synth.FMT_MXFP4, T=13, E=8, k=3, H=1024, I=512, name="guard_ring"),
                small(synth.FMT_NVFP4, T=37, E=8, k=2, H=768, I=256, name="guard_stream"),
                small(synth.FMT_INT4, T=333, E=8, k=2, H=512, I=256, norm_init=1e-20, name="guard_prefill"),
                small(synth.FMT_MXFP4, T=64, E=64, k=6, zipf_s=1.3, name="guard_mixed"),
                small(synth.FMT_NVFP4, T=200, I_shared=256, name="guard_shared")):
        layer = synth.build_layer(cfg, "cuda")
        ml = MoeLayer(c, cfg, max_tokens=layer.x.shape[0])
        ml.load_synth(layer)
        ml.forward(layer.x)
        c.synchronize()
        c.check_canaries()
        ml.close()


def test_state_hash_of_the_output(ctx):
    """strata_moe_stable_bf16_hash of a layer's output equals the oracle's hash of the same values (the reference's
    "[state]" diagnostic), and two runs of the layer hash alike."""
    cfg = small(synth.FMT_MXFP4, T=9, name="hash")
    layer, ml, out, aux = run_layer(ctx, cfg)
    h = ctx.stable_bf16_hash(out)
    assert h == O.stable_bf16_hash(out.cpu().numpy())
    assert ctx.stable_bf16_hash(ml.forward(layer.x)) == h


@pytest.mark.parametrize("T,E,S,k", [(5, 256, 2, 6), (300, 128, 1, 8), (33, 64, 0, 4)])
def test_inkling_sink_router(ctx, T, E, S, k):
    """Gate projection over routed + sink rows and the sink router against the oracle (which is pinned bit for bit to
    the compiled inkling_route_sigmoid_sink): logits, ids and every weight bit-exact; one forced exact tie."""
    H = 512
    g = torch.Generator().manual_seed(T * 1000 + E)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w = (torch.randn(E + S, H, generator=g) * 0.08).to(torch.bfloat16)
    w[11] = w[2]                                            # twins: identical logits for every token
    bias = (torch.randn(E, generator=g) * 0.05).float()
    bias[11] = bias[2]
    scale = float(np.float32(2.5) * np.float32(0.75))
    logits = ctx.project_rows(x.cuda(), w.cuda())
    ids, wr, ws = ctx.route_sink(logits, bias.cuda(), E, S, k, scale)
    ctx.synchronize()
    ref_logits = O.router_logits(Hh.np_u16(x), Hh.np_u16(w))
    assert np.array_equal(logits.cpu().numpy().view(np.uint32), ref_logits.view(np.uint32))
    rc, rids, rw = O.route_sigmoid_sink(ref_logits, bias.numpy(), E, S, k, np.float32(scale))
    assert rc == 0
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), rids[:, :k])
    assert np.array_equal(wr.cpu().numpy().view(np.uint32), rw[:, :k].view(np.uint32))
    if S:
        assert np.array_equal(ws.cpu().numpy().view(np.uint32), np.ascontiguousarray(rw[:, k:]).view(np.uint32))
    assert ((rids[:, :k] == 2).any(axis=1) >= (rids[:, :k] == 11).any(axis=1)).all()   # the lower twin goes first


@pytest.mark.parametrize("kind", [synth.SCORE_SIGMOID, synth.SCORE_SQRTSOFTPLUS])
def test_hash_routing_weights(ctx, kind):
    """Experts given per token (hash routing): ids are passed through, weights equal the oracle's bit for bit
    (the sqrt-softplus rule included: expf and log1pf follow the host libm's algorithms step by step)."""
    import ctypes as C
    cfg = small(synth.FMT_MXFP4, T=9, E=32, k=4, score_kind=kind, weight_scale=1.5, name=f"hash{kind}")
    layer = synth.build_layer(cfg, "cuda")
    ml = MoeLayer(ctx, cfg, max_tokens=cfg.T)
    ml.load_synth(layer)
    rng = np.random.default_rng(8)
    table = np.stack([rng.choice(cfg.E, size=cfg.k, replace=False) for _ in range(cfg.T)]).astype(np.int32)
    ids, w = ml.route_hash(layer.x, torch.from_numpy(table).cuda())
    _, _, logits = ml.route(layer.x, want_logits=True)
    ctx.synchronize()
    assert np.array_equal(ids.cpu().numpy(), table)
    spec = O.router_spec(cfg.E, cfg.k, kind, normalize=True, weight_scale=1.5)
    lg = logits.cpu().numpy()
    f32p, u32p = C.POINTER(C.c_float), C.POINTER(C.c_uint32)
    want = np.empty((cfg.T, cfg.k), np.float32)
    tmp = np.empty(cfg.k, np.uint32)
    for t in range(cfg.T):
        row = np.ascontiguousarray(table[t].astype(np.uint32))
        assert O.port().orc_route_given_row(C.byref(spec), np.ascontiguousarray(lg[t]).ctypes.data_as(f32p),
                                            row.ctypes.data_as(u32p), tmp.ctypes.data_as(u32p),
                                            want[t].ctypes.data_as(f32p)) == 0
    got = w.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
