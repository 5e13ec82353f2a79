"""ctypes bindings to the CPU checkers.  TEST INFRASTRUCTURE ONLY.

`port`  = oracle/libmoe_oracle.so  (plain-C restatement, oracle/moe_oracle.c)
`ref`   = oracle/_ref/libstrata_ref.so (the reference's own CPU code behind oracle/ref_shim.cpp)

Only tests/, __graft_entry__.smoke() and bench.py's CPU legs import this module.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

FMT_MXFP4, FMT_NVFP4, FMT_INT4, FMT_BF16 = 0, 1, 2, 3
SCORE_SIGMOID, SCORE_SIGMOID_PLAIN, SCORE_SOFTMAX, SCORE_SQRTSOFTPLUS = 0, 1, 2, 3
COMBINE_RANK_ORDER, COMBINE_JOB_ORDER = 0, 1

u8p = C.POINTER(C.c_uint8)
u16p = C.POINTER(C.c_uint16)
u32p = C.POINTER(C.c_uint32)
f32p = C.POINTER(C.c_float)


class Matrix(C.Structure):
    _fields_ = [("fmt", C.c_int32), ("rows", C.c_uint32), ("cols", C.c_uint32),
                ("packed", C.c_void_p), ("scales", C.c_void_p), ("global_scale", C.c_float)]


class Expert(C.Structure):
    _fields_ = [("gate", Matrix), ("up", Matrix), ("down", Matrix), ("activation", C.c_int32),
                ("gate_beta", C.c_float), ("linear_beta", C.c_float)]


class RouterSpec(C.Structure):
    _fields_ = [("experts", C.c_uint32), ("top_k", C.c_uint32), ("score_kind", C.c_int32),
                ("normalize", C.c_int32), ("norm_init", C.c_float), ("weight_scale", C.c_float),
                ("softcap", C.c_float)]


class LayerDesc(C.Structure):
    _fields_ = [("T", C.c_uint32), ("H", C.c_uint32), ("I", C.c_uint32), ("E", C.c_uint32),
                ("k", C.c_uint32), ("router", RouterSpec), ("output_scale", C.c_float),
                ("combine_order", C.c_int32), ("coef_before_down", C.c_int32),
                ("accumulate_double", C.c_int32), ("I_shared", C.c_uint32)]


class RefExpertPtrs(C.Structure):
    _fields_ = [("gate_packed", C.c_void_p), ("gate_scales", C.c_void_p),
                ("up_packed", C.c_void_p), ("up_scales", C.c_void_p),
                ("down_packed", C.c_void_p), ("down_scales", C.c_void_p),
                ("gate_global", C.c_float), ("up_global", C.c_float), ("down_global", C.c_float)]


_port = None
_ref = None


def port():
    global _port
    if _port is None:
        path = os.path.join(HERE, "libmoe_oracle.so")
        if not os.path.exists(path):
            from . import build
            build.build_port()
        lib = C.CDLL(path)
        lib.orc_bf16_to_f32.restype = C.c_float
        lib.orc_bf16_to_f32.argtypes = [C.c_uint16]
        lib.orc_f32_to_bf16.restype = C.c_uint16
        lib.orc_f32_to_bf16.argtypes = [C.c_float]
        lib.orc_e2m1.restype = C.c_float
        lib.orc_e2m1.argtypes = [C.c_uint32, C.c_int]
        lib.orc_e8m0.restype = C.c_float
        lib.orc_e8m0.argtypes = [C.c_uint32, C.c_int]
        lib.orc_e4m3.restype = C.c_float
        lib.orc_e4m3.argtypes = [C.c_uint32]
        lib.orc_sigmoid.restype = C.c_float
        lib.orc_sigmoid.argtypes = [C.c_float]
        lib.orc_silu.restype = C.c_float
        lib.orc_silu.argtypes = [C.c_float]
        lib.orc_expf_replica.restype = C.c_float
        lib.orc_expf_replica.argtypes = [C.c_float, C.c_int]
        lib.orc_log1pf_replica.restype = C.c_float
        lib.orc_log1pf_replica.argtypes = [C.c_float]
        lib.orc_dequant_row.argtypes = [C.POINTER(Matrix), C.c_uint32, C.c_int, f32p]
        lib.orc_matvec.argtypes = [C.POINTER(Matrix), f32p, f32p, C.c_uint32, C.c_uint32, C.c_int]
        lib.orc_router_logits.restype = None
        lib.orc_router_logits.argtypes = [u16p, u16p, C.c_uint32, C.c_uint32, C.c_uint32, f32p]
        lib.orc_route.argtypes = [C.POINTER(RouterSpec), f32p, f32p, C.c_uint32, u32p, f32p]
        lib.orc_group.restype = None
        lib.orc_group.argtypes = [u32p, C.c_uint32, C.c_uint32, C.c_uint32, u32p, u32p, u32p]
        lib.orc_moe_layer.argtypes = [C.POINTER(LayerDesc), u16p, u16p, f32p, C.POINTER(Expert),
                                      C.POINTER(Expert), u32p, C.c_uint32, f32p, u32p, f32p, u32p,
                                      u32p, u32p, f32p]
        lib.orc_expert_ffn.argtypes = [C.POINTER(Expert), f32p, C.c_float, C.c_int, C.c_int, f32p, f32p, f32p]
        lib.orc_route_given_row.argtypes = [C.POINTER(RouterSpec), f32p, u32p, u32p, f32p]
        lib.orc_situ_glu.argtypes = [C.c_float] * 4
        lib.orc_situ_glu.restype = C.c_float
        lib.orc_bf16_round.argtypes = [C.c_float]
        lib.orc_bf16_round.restype = C.c_float
        lib.orc_quantize_e4m3_value.argtypes = [C.c_float]
        lib.orc_quantize_e4m3_value.restype = C.c_float
        lib.orc_quantize_activation_e4m3.argtypes = [f32p, C.c_uint64]
        lib.orc_quantize_activation_e4m3.restype = None
        lib.orc_dsv4_expert.argtypes = [f32p, f32p, u8p, u8p, u8p, u8p, u8p, u8p, C.c_uint32, C.c_uint32,
                                        C.c_float, C.c_float, f32p]
        lib.orc_dsv4_fp8_shared.argtypes = [f32p, f32p, u8p, u8p, u8p, u8p, u8p, u8p, C.c_uint32, C.c_uint32,
                                            C.c_float, f32p]
        lib.orc_latent_moe_layer.argtypes = [C.POINTER(LayerDesc), C.c_uint32, C.c_float, u16p, u16p, f32p, u16p, u16p, f32p,
                                             C.POINTER(Expert), C.POINTER(Expert), u32p, C.c_uint32, u32p, f32p, f32p]
        lib.orc_experts_all.argtypes = [C.POINTER(LayerDesc), u16p, C.POINTER(Expert), u32p, f32p,
                                        u32p, u32p, f32p]
        _port = lib
    return _port


def ref():
    """The compiled reference, or None when it was never built on this machine."""
    global _ref
    if _ref is None:
        path = os.path.join(HERE, "_ref", "libstrata_ref.so")
        if not os.path.exists(path):
            from . import build
            if build.build_reference() is None:
                return None
        lib = C.CDLL(path)
        for name in ("ref_fp4_e2m1", "ref_fp8_e4m3", "ref_mxfp4_scale", "ref_dsv4_e8m0"):
            getattr(lib, name).restype = C.c_float
            getattr(lib, name).argtypes = [C.c_uint8]
        for name in ("ref_sigmoid", "ref_silu"):
            getattr(lib, name).restype = C.c_float
            getattr(lib, name).argtypes = [C.c_float]
        for name in ("ref_glm_route", "ref_kimi_route", "ref_dsv4_route"):
            getattr(lib, name).argtypes = [f32p, f32p, C.c_uint32, C.c_uint32, C.c_float, u32p, f32p]
        lib.ref_laguna_route.argtypes = [f32p, f32p, C.c_uint32, C.c_uint32, C.c_int, C.c_float,
                                         u32p, f32p]
        lib.ref_inkling_route_sink.argtypes = [f32p, f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_float,
                                               u32p, f32p]
        lib.ref_kimi_mxfp4_matvec.argtypes = [f32p, f32p, u8p, u8p, C.c_uint32, C.c_uint32]
        lib.ref_dsv4_fp4_matvec.argtypes = [f32p, f32p, u8p, u8p, C.c_uint32, C.c_uint32]
        lib.ref_laguna_nvfp4_matvec.argtypes = [f32p, f32p, u8p, u8p, C.c_float, C.c_uint32,
                                                C.c_uint32, C.c_uint32, C.c_uint32]
        lib.ref_inkling_nvfp4_matvec.argtypes = [f32p, f32p, u8p, u8p, C.c_float, C.c_uint32, C.c_uint32]
        lib.ref_glm_int4_matvec_scalar.argtypes = [f32p, f32p, u8p, u8p, C.c_uint32, C.c_uint32]
        lib.ref_glm_int4_matvec_rows.argtypes = [f32p, f32p, u8p, u8p, C.c_uint32, C.c_uint32,
                                                 C.c_uint32, C.c_uint32]
        lib.ref_dsv4_host_expert.argtypes = [f32p, f32p, u8p, u8p, u8p, u8p, u8p, u8p, C.c_uint32,
                                             C.c_uint32, C.c_float, C.c_float, C.c_int]
        lib.ref_cpu_experts.restype = C.c_int64
        lib.ref_dsv4_route_hash.argtypes = [f32p, u32p, C.c_uint32, C.c_uint32, C.c_float, u32p, f32p]
        lib.ref_dsv4_quantize.argtypes = [f32p, C.c_uint32]
        lib.ref_kimi_situ_glu.argtypes = [f32p, f32p, f32p, C.c_uint32, C.c_float, C.c_float]
        lib.ref_dsv4_tile_shard.restype = C.c_uint64
        lib.ref_dsv4_tile_shard.argtypes = [u8p, u8p, u8p, u8p, u8p, u8p, u8p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64]
        lib.ref_parse_route_trace.restype = C.c_int64
        lib.ref_parse_route_trace.argtypes = [C.c_char_p, C.POINTER(C.c_uint64), u32p, f32p, C.c_uint64, C.c_uint64]
        lib.ref_kimi_latent_moe.argtypes = [f32p, f32p, C.c_uint32, u16p, f32p, u16p, u16p, f32p, u16p, u16p, u16p,
                                            C.POINTER(C.c_void_p), u32p, f32p]
        lib.ref_cpu_experts.argtypes = [C.c_int, C.c_uint32, C.c_uint32, C.c_uint32,
                                        C.POINTER(RefExpertPtrs), f32p, u32p, u32p, f32p, C.c_uint32]
        _ref = lib
    return _ref


# ----------------------------------------------------------------- numpy helpers
def _p(a, t):
    return a.ctypes.data_as(t)


def _vp(a):
    return C.c_void_p(a.ctypes.data) if a is not None else C.c_void_p(0)


def make_matrix(fmt, rows, cols, packed, scales=None, global_scale=1.0):
    """packed / scales are C-contiguous numpy arrays kept alive by the caller."""
    m = Matrix()
    m.fmt, m.rows, m.cols = fmt, rows, cols
    m.packed = packed.ctypes.data if packed is not None else None
    m.scales = scales.ctypes.data if scales is not None else None
    m.global_scale = float(global_scale)
    return m


def dequant(m, device_zero=False):
    out = np.empty((m.rows, m.cols), np.float32)
    lib = port()
    for r in range(m.rows):
        rc = lib.orc_dequant_row(C.byref(m), r, int(device_zero), _p(out[r], f32p))
        assert rc == 0
    return out


def matvec(m, x, double=False):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(m.rows, np.float32)
    rc = port().orc_matvec(C.byref(m), _p(x, f32p), _p(y, f32p), 0, m.rows, int(double))
    assert rc == 0
    return y


def router_logits(x_bf16, wg_bf16):
    """x_bf16 [T,H] uint16, wg_bf16 [E,H] uint16 -> fp32 [T,E] in the reference's GPU order."""
    x_bf16 = np.ascontiguousarray(x_bf16, np.uint16)
    wg_bf16 = np.ascontiguousarray(wg_bf16, np.uint16)
    T, H = x_bf16.shape
    E = wg_bf16.shape[0]
    out = np.empty((T, E), np.float32)
    port().orc_router_logits(_p(x_bf16, u16p), _p(wg_bf16, u16p), T, H, E, _p(out, f32p))
    return out


def router_spec(experts, top_k, score_kind=SCORE_SIGMOID, normalize=True, norm_init=0.0,
                weight_scale=1.0, softcap=0.0):
    s = RouterSpec()
    s.experts, s.top_k, s.score_kind = experts, top_k, score_kind
    s.normalize, s.norm_init, s.weight_scale, s.softcap = int(normalize), norm_init, weight_scale, softcap
    return s


def route(spec, logits, bias=None):
    logits = np.ascontiguousarray(logits, np.float32)
    T = logits.shape[0]
    ids = np.empty((T, spec.top_k), np.uint32)
    w = np.empty((T, spec.top_k), np.float32)
    b = np.ascontiguousarray(bias, np.float32) if bias is not None else None
    rc = port().orc_route(C.byref(spec), _p(logits, f32p), _p(b, f32p) if b is not None else None,
                          T, _p(ids, u32p), _p(w, f32p))
    return rc, ids, w


def stable_bf16_hash(values):
    values = np.ascontiguousarray(values, np.float32)
    lib = port()
    lib.orc_stable_bf16_hash.restype = C.c_uint64
    lib.orc_stable_bf16_hash.argtypes = [f32p, C.c_size_t]
    return int(lib.orc_stable_bf16_hash(_p(values, f32p), values.size))


def route_sigmoid_sink(logits, bias, experts, sinks, top_k, scale):
    """Inkling's sink router over logits [T, experts + sinks]: ids / weights [T, top_k + sinks]."""
    logits = np.ascontiguousarray(logits, np.float32)
    bias = np.ascontiguousarray(bias, np.float32)
    T = logits.shape[0]
    ids = np.empty((T, top_k + sinks), np.uint32)
    w = np.empty((T, top_k + sinks), np.float32)
    scratch = np.empty(experts, np.float32)
    lib = port()
    lib.orc_route_sigmoid_sink.argtypes = [f32p, f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, f32p, u32p, f32p]
    for t in range(T):
        rc = lib.orc_route_sigmoid_sink(_p(logits[t], f32p), _p(bias, f32p), experts, sinks, top_k, scale,
                                        _p(scratch, f32p), _p(ids[t], u32p), _p(w[t], f32p))
        if rc:
            return rc, ids, w
    return 0, ids, w


def group(ids, experts):
    ids = np.ascontiguousarray(ids, np.uint32)
    T, k = ids.shape
    counts = np.empty(experts, np.uint32)
    offsets = np.empty(experts + 1, np.uint32)
    perm = np.empty(T * k, np.uint32)
    port().orc_group(_p(ids, u32p), T, k, experts, _p(counts, u32p), _p(offsets, u32p),
                     _p(perm, u32p))
    return counts, offsets, perm


def moe_layer(desc, x_bf16, router_w, bias, experts, shared=None, token_subset=None,
              want_output=True):
    """experts: ctypes array of Expert (length E).  Returns dict of numpy results."""
    x_bf16 = np.ascontiguousarray(x_bf16, np.uint16)
    router_w = np.ascontiguousarray(router_w, np.uint16)
    T, E, k, H = desc.T, desc.E, desc.k, desc.H
    logits = np.empty((T, E), np.float32)
    ids = np.empty((T, k), np.uint32)
    w = np.empty((T, k), np.float32)
    counts = np.empty(E, np.uint32)
    offsets = np.empty(E + 1, np.uint32)
    perm = np.empty(T * k, np.uint32)
    sub = None
    n = T
    if token_subset is not None:
        sub = np.ascontiguousarray(token_subset, np.uint32)
        n = len(sub)
    out = np.empty((n, H), np.float32) if want_output else None
    b = np.ascontiguousarray(bias, np.float32) if bias is not None else None
    rc = port().orc_moe_layer(
        C.byref(desc), _p(x_bf16, u16p), _p(router_w, u16p), _p(b, f32p) if b is not None else None,
        experts, C.byref(shared) if shared is not None else None,
        _p(sub, u32p) if sub is not None else None, n, _p(logits, f32p), _p(ids, u32p), _p(w, f32p),
        _p(counts, u32p), _p(offsets, u32p), _p(perm, u32p),
        _p(out, f32p) if out is not None else None)
    return dict(rc=rc, logits=logits, ids=ids, weights=w, counts=counts, offsets=offsets, perm=perm,
                out=out)
