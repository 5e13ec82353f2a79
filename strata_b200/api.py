"""ctypes binding of include/strata_moe.h.  torch is used only for device memory and streams."""
import ctypes as C
import os
import weakref

import torch

from . import synth

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

EXPORTS = [
    "strata_moe_create", "strata_moe_destroy", "strata_moe_last_error", "strata_moe_synchronize",
    "strata_moe_get_stats", "strata_moe_set_timing", "strata_moe_get_phase_ms", "strata_moe_layer_create",
    "strata_moe_layer_destroy", "strata_moe_set_router", "strata_moe_set_expert",
    "strata_moe_set_shared", "strata_moe_forward", "strata_moe_forward_host", "strata_moe_route",
    "strata_moe_group", "strata_moe_gather_rows", "strata_moe_combine", "strata_moe_experts_grouped", "strata_moe_dequant_export",
    "strata_moe_enqueue_dense", "strata_moe_collect_dense", "strata_moe_group_static",
    "strata_moe_ep_window_bytes", "strata_moe_ep_window_alloc", "strata_moe_ep_window_open",
    "strata_moe_ep_window_close", "strata_moe_ep_window_free", "strata_moe_ep_create", "strata_moe_ep_destroy",
    "strata_moe_ep_begin", "strata_moe_ep_dispatch", "strata_moe_ep_experts", "strata_moe_ep_finish",
    "strata_moe_ep_forward", "strata_moe_ep_abandon", "strata_moe_ep_last_counts",
    "strata_moe_experts_grouped_dsv4", "strata_moe_quantize_e4m3", "strata_moe_combine_dsv4",
    "strata_moe_route_hash", "strata_moe_project_rows", "strata_moe_route_sink", "strata_moe_stable_bf16_hash", "strata_moe_check_canaries",
    "strata_moe_forward_routed", "strata_moe_latent_create", "strata_moe_latent_destroy", "strata_moe_latent_experts",
    "strata_moe_latent_set_router", "strata_moe_latent_set_projections", "strata_moe_latent_set_shared",
    "strata_moe_latent_forward",
    "strata_moe_device_count", "strata_moe_weight_upload", "strata_moe_weight_release", "strata_moe_command_enqueue",
    "strata_moe_command_collect", "strata_moe_command_enqueue_rows_dsv4", "strata_moe_command_collect_rows_dsv4",
]

SRC_HOST, SRC_DEVICE_COPY, SRC_DEVICE_BORROW = 0, 1, 2


class StrataMoeError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"strata_moe error {code}: {message}")
        self.code = code


class LayerDesc(C.Structure):
    _fields_ = [("hidden", C.c_uint32), ("intermediate", C.c_uint32), ("experts", C.c_uint32),
                ("top_k", C.c_uint32), ("format", C.c_int32), ("score_kind", C.c_int32),
                ("normalize", C.c_int32), ("norm_init", C.c_float), ("weight_scale", C.c_float),
                ("output_scale", C.c_float), ("softcap", C.c_float),
                ("shared_intermediate", C.c_uint32), ("expert_begin", C.c_uint32),
                ("expert_count", C.c_uint32), ("max_tokens", C.c_uint32), ("max_pairs", C.c_uint32),
                ("activation", C.c_int32), ("gate_beta", C.c_float), ("linear_beta", C.c_float)]


class Aux(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("ids", C.c_void_p), ("weights", C.c_void_p),
                ("counts", C.c_void_p), ("offsets", C.c_void_p), ("perm", C.c_void_p)]


class Stats(C.Structure):
    _fields_ = [("forward_calls", C.c_uint64), ("kernel_launches", C.c_uint64),
                ("h2d_bytes", C.c_uint64), ("d2h_bytes", C.c_uint64), ("weight_bytes", C.c_uint64),
                ("last_forward_ms", C.c_float), ("router_fast_tokens", C.c_uint64),
                ("router_rechecked_tokens", C.c_uint64), ("command_calls", C.c_uint64),
                ("workspace_allocations", C.c_uint64), ("router_worst_error", C.c_float)]


def library_path():
    return os.path.join(HERE, "libstrata_moe.so")


def load_library():
    """Loads the CUDA library; raises when it has not been built (there is no fallback)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        raise StrataMoeError(-5, f"{path} is missing: run `python -m strata_b200.build` (needs nvcc)")
    lib = C.CDLL(path)
    vp, u32, i32, f32 = C.c_void_p, C.c_uint32, C.c_int, C.c_float
    lib.strata_moe_create.argtypes = [i32, vp, C.POINTER(vp)]
    lib.strata_moe_destroy.argtypes = [vp]
    lib.strata_moe_destroy.restype = None
    lib.strata_moe_last_error.argtypes = [vp]
    lib.strata_moe_last_error.restype = C.c_char_p
    lib.strata_moe_synchronize.argtypes = [vp]
    lib.strata_moe_get_stats.argtypes = [vp, C.POINTER(Stats)]
    lib.strata_moe_set_timing.argtypes = [vp, i32]
    lib.strata_moe_set_timing.restype = None
    lib.strata_moe_get_phase_ms.argtypes = [vp, C.POINTER(C.c_float)]
    lib.strata_moe_layer_create.argtypes = [vp, C.POINTER(LayerDesc), C.POINTER(vp)]
    lib.strata_moe_layer_destroy.argtypes = [vp]
    lib.strata_moe_layer_destroy.restype = None
    lib.strata_moe_set_router.argtypes = [vp, vp, vp, i32]
    lib.strata_moe_set_expert.argtypes = [vp, u32, i32, vp, vp, f32, i32]
    lib.strata_moe_set_shared.argtypes = [vp, i32, vp, i32]
    lib.strata_moe_forward.argtypes = [vp, vp, u32, vp, C.POINTER(Aux)]
    lib.strata_moe_forward_host.argtypes = [vp, vp, u32, vp]
    lib.strata_moe_route.argtypes = [vp, vp, u32, vp, vp, vp]
    lib.strata_moe_route_hash.argtypes = [vp, vp, u32, vp, vp, vp, vp]
    lib.strata_moe_project_rows.argtypes = [vp, vp, u32, u32, vp, u32, vp]
    lib.strata_moe_stable_bf16_hash.argtypes = [vp, vp, C.c_size_t, C.POINTER(C.c_uint64)]
    lib.strata_moe_route_sink.argtypes = [vp, vp, vp, u32, u32, u32, u32, C.c_float, vp, vp, vp]
    lib.strata_moe_group.argtypes = [vp, vp, u32, u32, u32, vp, vp, vp, vp]
    lib.strata_moe_gather_rows.argtypes = [vp, vp, u32, vp, u32, u32, vp]
    lib.strata_moe_combine.argtypes = [vp, vp, vp, vp, vp, u32, vp]
    lib.strata_moe_experts_grouped.argtypes = [vp, vp, u32, vp, vp]
    lib.strata_moe_dequant_export.argtypes = [vp, u32, i32, vp]
    lib.strata_moe_enqueue_dense.argtypes = [vp, vp, u32, vp, vp, u32, i32]
    lib.strata_moe_collect_dense.argtypes = [vp, vp, vp]
    lib.strata_moe_group_static.argtypes = [vp, vp, u32, u32, u32, vp, vp, vp, vp, C.c_char_p, C.c_size_t]
    lib.strata_moe_ep_window_bytes.argtypes = [C.POINTER(LayerDesc), u32, u32]
    lib.strata_moe_ep_window_bytes.restype = C.c_size_t
    lib.strata_moe_ep_window_alloc.argtypes = [vp, C.c_size_t, C.POINTER(vp), vp]
    lib.strata_moe_ep_window_open.argtypes = [vp, vp, C.POINTER(vp)]
    lib.strata_moe_ep_window_close.argtypes = [vp, vp]
    lib.strata_moe_ep_window_free.argtypes = [vp, vp]
    lib.strata_moe_ep_create.argtypes = [vp, u32, u32, u32, C.POINTER(vp), u32, C.POINTER(vp)]
    lib.strata_moe_ep_destroy.argtypes = [vp]
    lib.strata_moe_ep_destroy.restype = None
    lib.strata_moe_ep_begin.argtypes = [vp, vp, u32]
    lib.strata_moe_ep_dispatch.argtypes = [vp]
    lib.strata_moe_ep_experts.argtypes = [vp, u32]
    lib.strata_moe_ep_finish.argtypes = [vp, vp]
    lib.strata_moe_ep_forward.argtypes = [vp, vp, u32, vp, u32]
    lib.strata_moe_ep_abandon.argtypes = [vp]
    lib.strata_moe_ep_last_counts.argtypes = [vp, C.POINTER(u32), C.POINTER(u32), C.POINTER(u32)]
    lib.strata_moe_experts_grouped_dsv4.argtypes = [vp, vp, u32, vp, vp, f32, vp]
    lib.strata_moe_quantize_e4m3.argtypes = [vp, vp, u32, u32]
    lib.strata_moe_combine_dsv4.argtypes = [vp, vp, vp, vp, u32, vp]
    lib.strata_moe_forward_routed.argtypes = [vp, vp, u32, vp, vp, vp]
    lib.strata_moe_latent_create.argtypes = [vp, C.POINTER(LayerDesc), u32, f32, C.POINTER(vp)]
    lib.strata_moe_latent_destroy.argtypes = [vp]
    lib.strata_moe_latent_destroy.restype = None
    lib.strata_moe_latent_experts.argtypes = [vp]
    lib.strata_moe_latent_experts.restype = C.c_void_p
    lib.strata_moe_latent_set_router.argtypes = [vp, vp, vp, i32]
    lib.strata_moe_latent_set_projections.argtypes = [vp, vp, vp, vp, i32]
    lib.strata_moe_latent_set_shared.argtypes = [vp, i32, vp, i32]
    lib.strata_moe_latent_forward.argtypes = [vp, vp, u32, vp, vp, vp]
    _LIB = lib
    return lib


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def group_static(ids, expert_begin, n_experts, stream=None, want_inv=True):
    """strata_moe_group_static on torch tensors: the grouping call that allocates nothing inside the
    library (the output tensors here are the caller's).  Raises StrataMoeError with the library's text."""
    lib = load_library()
    flat = ids.reshape(-1)
    dev = ids.device
    counts = torch.empty(n_experts, dtype=torch.int32, device=dev)
    offsets = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    perm = torch.empty(flat.numel(), dtype=torch.int32, device=dev)
    inv = torch.empty(flat.numel(), dtype=torch.int32, device=dev) if want_inv else None
    stream = torch.cuda.current_stream(dev) if stream is None else stream
    err = C.create_string_buffer(256)
    rc = lib.strata_moe_group_static(C.c_void_p(stream.cuda_stream), _ptr(flat), flat.numel(), expert_begin,
                                     n_experts, _ptr(counts), _ptr(offsets), _ptr(perm), _ptr(inv), err, 256)
    if rc != 0:
        raise StrataMoeError(rc, err.value.decode())
    return counts, offsets, perm, inv


class MoeContext:
    """One per process and device (strata_moe_ctx)."""

    def __init__(self, device=0, stream=None):
        self.lib = load_library()
        if not torch.cuda.is_available():
            raise StrataMoeError(-5, "no CUDA device: this library has no CPU path")
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        # the library runs on this torch stream; callers on another stream are ordered against it
        # by MoeLayer (wait_stream on both sides of every call)
        self.stream = stream if stream is not None else torch.cuda.Stream(self.device)
        h = C.c_void_p()
        rc = self.lib.strata_moe_create(device, C.c_void_p(self.stream.cuda_stream), C.byref(h))
        if rc != 0:
            raise StrataMoeError(rc, "strata_moe_create failed (needs an sm_100 device)")
        self.h = h
        # objects that hold pointers into this context; closed before it, whatever order the
        # garbage collector picks
        self._children = weakref.WeakSet()

    def enter(self):
        """Orders the library's stream after the caller's current stream."""
        cur = torch.cuda.current_stream(self.device)
        if cur.cuda_stream != self.stream.cuda_stream:
            self.stream.wait_stream(cur)

    def leave(self):
        """Orders the caller's current stream after the library's stream."""
        cur = torch.cuda.current_stream(self.device)
        if cur.cuda_stream != self.stream.cuda_stream:
            cur.wait_stream(self.stream)

    def check(self, rc):
        if rc != 0:
            raise StrataMoeError(rc, self.lib.strata_moe_last_error(self.h).decode())

    def synchronize(self):
        self.check(self.lib.strata_moe_synchronize(self.h))

    def stats(self):
        s = Stats()
        self.check(self.lib.strata_moe_get_stats(self.h, C.byref(s)))
        return s

    def check_canaries(self):
        """Raises when a kernel wrote outside one of the context's workspaces."""
        self.check(self.lib.strata_moe_check_canaries(self.h))

    def stable_bf16_hash(self, values):
        """The reference's per-layer state hash of an fp32 device tensor (FNV-1a over its BF16 rounding)."""
        h = C.c_uint64()
        self.enter()
        self.check(self.lib.strata_moe_stable_bf16_hash(self.h, _ptr(values), values.numel(), C.byref(h)))
        self.leave()
        return int(h.value)

    def project_rows(self, x, w):
        """logits [T, rows] of BF16 x [T, H] against BF16 w [rows, H] in the router's canonical summation order."""
        T, H = x.shape
        out = torch.empty(T, w.shape[0], dtype=torch.float32, device=x.device)
        self.enter()
        self.check(self.lib.strata_moe_project_rows(self.h, _ptr(x), T, H, _ptr(w), w.shape[0], _ptr(out)))
        self.leave()
        return out

    def route_sink(self, logits, bias, routed_experts, sinks, top_k, scale):
        """Inkling's sink router: (ids [T, k], weights [T, k], sink weights [T, sinks])."""
        T, dev = logits.shape[0], logits.device
        ids = torch.empty(T, top_k, dtype=torch.int32, device=dev)
        w = torch.empty(T, top_k, dtype=torch.float32, device=dev)
        ws = torch.empty(T, max(sinks, 1), dtype=torch.float32, device=dev)
        self.enter()
        self.check(self.lib.strata_moe_route_sink(self.h, _ptr(logits), _ptr(bias), T, routed_experts, sinks, top_k,
                                                  scale, _ptr(ids), _ptr(w), _ptr(ws)))
        self.leave()
        return ids, w, ws[:, :sinks]

    def quantize_e4m3(self, values):
        """In-place E4M3 activation quantisation of fp32 [rows, cols] (one power-of-two scale per 128 columns)."""
        self.enter()
        self.check(self.lib.strata_moe_quantize_e4m3(self.h, _ptr(values), values.shape[0], values.shape[1]))
        self.leave()
        return values

    def set_timing(self, on):
        self.lib.strata_moe_set_timing(self.h, int(on))

    PHASES = ("router_logits", "route", "group", "gather", "gate_up", "down", "shared", "combine")

    def phase_ms(self):
        out = (C.c_float * 8)()
        self.check(self.lib.strata_moe_get_phase_ms(self.h, out))
        return dict(zip(self.PHASES, [float(v) for v in out]))

    def close(self):
        if self.h:
            for order in (2, 1, 0):          # ep states, then windows, then layers
                for child in list(self._children):
                    if getattr(child, "_close_order", 0) == order:
                        child.close()
            self.lib.strata_moe_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MoeLayer:
    """One MoE layer (strata_moe_layer): resident weights + workspaces."""

    def __init__(self, ctx, cfg, max_tokens=None, expert_begin=0, expert_count=None, max_pairs=0):
        self.ctx, self.cfg, self.lib = ctx, cfg, ctx.lib
        d = LayerDesc()
        d.hidden, d.intermediate, d.experts, d.top_k = cfg.H, cfg.I, cfg.E, cfg.k
        d.format, d.score_kind, d.normalize = cfg.fmt, cfg.score_kind, int(cfg.normalize)
        d.norm_init, d.weight_scale, d.output_scale, d.softcap = cfg.norm_init, cfg.weight_scale, cfg.output_scale, 0.0
        d.shared_intermediate = cfg.I_shared
        d.expert_begin = expert_begin
        d.expert_count = cfg.E - expert_begin if expert_count is None else expert_count
        d.max_tokens = cfg.T if max_tokens is None else max_tokens
        d.max_pairs = max_pairs
        d.activation = getattr(cfg, "activation", 0)
        d.gate_beta, d.linear_beta = getattr(cfg, "gate_beta", 1.0), getattr(cfg, "linear_beta", 1.0)
        self.desc = d
        h = C.c_void_p()
        ctx.check(self.lib.strata_moe_layer_create(ctx.h, C.byref(d), C.byref(h)))
        self.h = h
        self._keep = []
        ctx._children.add(self)

    # ---- weights -------------------------------------------------------------------
    def set_router(self, gate_bf16, bias=None):
        src = SRC_DEVICE_BORROW if gate_bf16.is_cuda else SRC_HOST
        self._keep += [gate_bf16, bias]
        self.ctx.check(self.lib.strata_moe_set_router(self.h, _ptr(gate_bf16), _ptr(bias), src))

    def set_expert(self, expert, role, packed, scales, global_scale=1.0):
        src = SRC_DEVICE_BORROW if packed.is_cuda else SRC_HOST
        self._keep += [packed, scales]
        self.ctx.check(self.lib.strata_moe_set_expert(self.h, expert, role, _ptr(packed), _ptr(scales),
                                                      float(global_scale), src))

    def set_shared(self, role, w):
        src = SRC_DEVICE_BORROW if w.is_cuda else SRC_HOST
        self._keep.append(w)
        self.ctx.check(self.lib.strata_moe_set_shared(self.h, role, _ptr(w), src))

    def load_synth(self, layer):
        """Registers every tensor of a synth.SynthLayer (borrowed in place when on the GPU)."""
        self.ctx.enter()
        self.set_router(layer.router_w, layer.bias)
        for r, role in enumerate(synth.ROLES):
            p, s = layer.packed[role], layer.scales[role]
            for le in range(layer.expert_end - layer.expert_begin):
                self.set_expert(layer.expert_begin + le, r, p[le], s[le], layer.global_scale(role))
            if layer.shared:
                self.set_shared(r, layer.shared[role])

    # ---- compute -------------------------------------------------------------------
    def forward(self, x, out=None, want_aux=False, aux_logits=True):
        """aux_logits=False leaves the logits out of the aux outputs: asking for them makes the library
        compute every logit in the canonical order, which large batches otherwise avoid."""
        T = x.shape[0]
        dev = x.device
        if out is None:
            out = torch.empty(T, self.cfg.H, dtype=torch.float32, device=dev)
        if T == 0:
            return (out, None) if want_aux else out
        aux_t = None
        aux = None
        if want_aux:
            E, k = self.cfg.E, self.cfg.k
            aux_t = dict(logits=torch.empty(T, E, dtype=torch.float32, device=dev),
                         ids=torch.empty(T, k, dtype=torch.int32, device=dev),
                         weights=torch.empty(T, k, dtype=torch.float32, device=dev),
                         counts=torch.empty(E, dtype=torch.int32, device=dev),
                         offsets=torch.empty(E + 1, dtype=torch.int32, device=dev),
                         perm=torch.empty(T * k, dtype=torch.int32, device=dev))
            if not aux_logits:
                aux_t["logits"] = None
            aux = Aux(*[(v.data_ptr() if v is not None else None) for v in aux_t.values()])
        self.ctx.enter()
        self.ctx.check(self.lib.strata_moe_forward(self.h, _ptr(x), T, _ptr(out),
                                                   C.byref(aux) if aux is not None else None))
        self.ctx.leave()
        return (out, aux_t) if want_aux else out

    def forward_host(self, x_host, out_host):
        self.ctx.check(self.lib.strata_moe_forward_host(self.h, _ptr(x_host), x_host.shape[0], _ptr(out_host)))
        return out_host

    def route(self, x, want_logits=False):
        T, dev = x.shape[0], x.device
        ids = torch.empty(T, self.cfg.k, dtype=torch.int32, device=dev)
        w = torch.empty(T, self.cfg.k, dtype=torch.float32, device=dev)
        logits = torch.empty(T, self.cfg.E, dtype=torch.float32, device=dev) if want_logits else None
        self.ctx.enter()
        self.ctx.check(self.lib.strata_moe_route(self.h, _ptr(x), T, _ptr(logits), _ptr(ids), _ptr(w)))
        self.ctx.leave()
        return (ids, w, logits) if want_logits else (ids, w)

    def route_hash(self, x, token_experts):
        """Weights for given experts per token (hash routing); returns (ids, weights)."""
        T, dev = x.shape[0], x.device
        ids = torch.empty(T, self.cfg.k, dtype=torch.int32, device=dev)
        w = torch.empty(T, self.cfg.k, dtype=torch.float32, device=dev)
        self.ctx.enter()
        self.ctx.check(self.lib.strata_moe_route_hash(self.h, _ptr(x), T, _ptr(token_experts), None, _ptr(ids), _ptr(w)))
        self.ctx.leave()
        return ids, w

    def group(self, ids, expert_begin=0, n_experts=None, want_inv=False):
        n_experts = self.cfg.E if n_experts is None else n_experts
        flat = ids.reshape(-1)
        dev = ids.device
        counts = torch.empty(n_experts, dtype=torch.int32, device=dev)
        offsets = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
        perm = torch.empty(flat.numel(), dtype=torch.int32, device=dev)
        inv = torch.empty(flat.numel(), dtype=torch.int32, device=dev) if want_inv else None
        self.ctx.enter()
        self.ctx.check(self.lib.strata_moe_group(self.h, _ptr(flat), flat.numel(), expert_begin, n_experts,
                                                 _ptr(counts), _ptr(offsets), _ptr(perm), _ptr(inv)))
        self.ctx.leave()
        return (counts, offsets, perm, inv) if want_inv else (counts, offsets, perm)

    def gather_rows(self, src, index, index_div=1, n=None):
        """dst[i] = src[index[i] // index_div] for i < n (rows of any dtype, 16-byte multiples)."""
        n = index.numel() if n is None else n
        dst = torch.empty((n,) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
        if n:
            row_bytes = src[0].numel() * src.element_size()
            self.ctx.enter()
            self.ctx.check(self.lib.strata_moe_gather_rows(self.h, _ptr(src), row_bytes, _ptr(index), index_div,
                                                           n, _ptr(dst)))
            self.ctx.leave()
        return dst

    def combine(self, y, inv, weights, x_shared=None, out=None):
        T = weights.shape[0]
        if out is None:
            out = torch.empty(T, self.cfg.H, dtype=torch.float32, device=weights.device)
        if T:
            self.ctx.enter()
            self.ctx.check(self.lib.strata_moe_combine(self.h, _ptr(y), _ptr(inv), _ptr(weights), _ptr(x_shared),
                                                       T, _ptr(out)))
            self.ctx.leave()
        return out

    def experts_grouped(self, rows, offsets, y=None):
        if y is None:
            y = torch.empty(rows.shape[0], self.cfg.H, dtype=torch.float32, device=rows.device)
        self.ctx.enter()
        self.ctx.check(self.lib.strata_moe_experts_grouped(self.h, _ptr(rows), rows.shape[0], _ptr(offsets), _ptr(y)))
        self.ctx.leave()
        return y

    def experts_grouped_dsv4(self, rows_f32, offsets, coefficients=None, swiglu_limit=10.0, y=None):
        """Bit-exact DeepSeek-V4 expert arithmetic on fp32 rows in group order (MXFP4-format weights)."""
        if y is None:
            y = torch.empty(rows_f32.shape[0], self.cfg.H, dtype=torch.float32, device=rows_f32.device)
        self.ctx.enter()
        self.ctx.check(self.lib.strata_moe_experts_grouped_dsv4(self.h, _ptr(rows_f32), rows_f32.shape[0],
                                                                _ptr(offsets), _ptr(coefficients),
                                                                float(swiglu_limit), _ptr(y)))
        self.ctx.leave()
        return y

    def combine_dsv4(self, y, inv, tokens, shared_rows=None, out=None):
        if out is None:
            out = torch.empty(tokens, self.cfg.H, dtype=torch.float32, device=y.device)
        self.ctx.enter()
        self.ctx.check(self.lib.strata_moe_combine_dsv4(self.h, _ptr(y), _ptr(inv), _ptr(shared_rows), tokens, _ptr(out)))
        self.ctx.leave()
        return out

    def dequant_export(self, expert, role):
        rows, cols = self.cfg.role_shape(synth.ROLES[role])
        out = torch.empty(rows, cols, dtype=torch.float32)
        self.ctx.check(self.lib.strata_moe_dequant_export(self.h, expert, role, _ptr(out)))
        return out

    def enqueue_dense(self, hidden_f32_host, experts, coefs, with_shared=False):
        ex = torch.tensor(list(experts), dtype=torch.int32)
        cf = torch.tensor(list(coefs), dtype=torch.float32)
        self._dense_keep = (hidden_f32_host, ex, cf)
        self.ctx.check(self.lib.strata_moe_enqueue_dense(self.h, _ptr(hidden_f32_host), hidden_f32_host.shape[0],
                                                         _ptr(ex), _ptr(cf), len(ex), int(with_shared)))

    def collect_dense(self, n_experts, rows, with_shared=False):
        routed = torch.empty(n_experts, rows, self.cfg.H, dtype=torch.float32)
        shared = torch.empty(rows, self.cfg.H, dtype=torch.float32) if with_shared else None
        self.ctx.check(self.lib.strata_moe_collect_dense(self.h, _ptr(routed), _ptr(shared)))
        return routed, shared

    def close(self):
        if self.h:
            if self.ctx.h:               # a closed context has already closed this layer
                self.lib.strata_moe_layer_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class LatentMoe:
    """strata_moe_latent: the LatentMoE wrapper (router and shared experts on cfg.H_model wide rows, routed experts
    on the cfg.H wide latent)."""

    _close_order = 0

    def __init__(self, ctx, cfg, max_tokens=None):
        assert cfg.H_model, "configuration has no latent"
        self.ctx, self.cfg, self.lib = ctx, cfg, ctx.lib
        d = LayerDesc()
        d.hidden, d.intermediate, d.experts, d.top_k = cfg.H, cfg.I, cfg.E, cfg.k
        d.format, d.score_kind, d.normalize = cfg.fmt, cfg.score_kind, int(cfg.normalize)
        d.norm_init, d.weight_scale, d.output_scale, d.softcap = cfg.norm_init, cfg.weight_scale, cfg.output_scale, 0.0
        d.shared_intermediate = cfg.I_shared
        d.expert_begin, d.expert_count = 0, cfg.E
        d.max_tokens = cfg.T if max_tokens is None else max_tokens
        d.max_pairs = 0
        d.activation, d.gate_beta, d.linear_beta = cfg.activation, cfg.gate_beta, cfg.linear_beta
        h = C.c_void_p()
        ctx.check(self.lib.strata_moe_latent_create(ctx.h, C.byref(d), cfg.H_model, float(cfg.rms_epsilon), C.byref(h)))
        self.h = h
        self._keep = []
        ctx._children.add(self)

    def load_synth(self, layer):
        self.ctx.enter()
        src = lambda t: SRC_DEVICE_BORROW if t.is_cuda else SRC_HOST
        self._keep += [layer.router_w, layer.bias, layer.latent, layer.shared, layer.packed, layer.scales]
        self.ctx.check(self.lib.strata_moe_latent_set_router(self.h, _ptr(layer.router_w), _ptr(layer.bias), src(layer.router_w)))
        lt = layer.latent
        self.ctx.check(self.lib.strata_moe_latent_set_projections(self.h, _ptr(lt["down"]), _ptr(lt["up"]), _ptr(lt["norm"]),
                                                                  src(lt["down"])))
        experts = C.c_void_p(self.lib.strata_moe_latent_experts(self.h))
        for r, role in enumerate(synth.ROLES):
            p, s = layer.packed[role], layer.scales[role]
            for e in range(self.cfg.E):
                self.ctx.check(self.lib.strata_moe_set_expert(experts, e, r, _ptr(p[e]), _ptr(s[e]),
                                                              float(layer.global_scale(role)), src(p)))
            if layer.shared:
                self.ctx.check(self.lib.strata_moe_latent_set_shared(self.h, r, _ptr(layer.shared[role]), src(layer.shared[role])))

    def forward(self, x, want_routing=False):
        T, dev = x.shape[0], x.device
        out = torch.empty(T, self.cfg.H_model, dtype=torch.float32, device=dev)
        ids = torch.empty(T, self.cfg.k, dtype=torch.int32, device=dev)
        w = torch.empty(T, self.cfg.k, dtype=torch.float32, device=dev)
        self.ctx.enter()
        self.ctx.check(self.lib.strata_moe_latent_forward(self.h, _ptr(x), T, _ptr(out), _ptr(ids), _ptr(w)))
        self.ctx.leave()
        return (out, ids, w) if want_routing else out

    def close(self):
        if self.h:
            if self.ctx.h:
                self.lib.strata_moe_latent_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class EpWindow:
    """A rank's exchange window (device memory that peers map).  `handle` is the 64-byte token a
    peer process passes to EpWindow.open."""

    _close_order = 1

    def __init__(self, ctx, ptr, handle=None, owned=True):
        self.ctx, self.ptr, self.handle, self.owned = ctx, ptr, handle, owned
        ctx._children.add(self)

    @staticmethod
    def bytes_needed(layer, world, row_capacity):
        n = load_library().strata_moe_ep_window_bytes(C.byref(layer.desc), world, row_capacity)
        if n == 0:
            raise StrataMoeError(-1, "bad window geometry")
        return n

    @classmethod
    def alloc(cls, ctx, nbytes):
        p = C.c_void_p()
        h = C.create_string_buffer(64)
        ctx.check(ctx.lib.strata_moe_ep_window_alloc(ctx.h, nbytes, C.byref(p), h))
        return cls(ctx, p.value, h.raw, True)

    @classmethod
    def open(cls, ctx, handle):
        p = C.c_void_p()
        ctx.check(ctx.lib.strata_moe_ep_window_open(ctx.h, C.create_string_buffer(handle, 64), C.byref(p)))
        return cls(ctx, p.value, handle, False)

    def close(self):
        if self.ptr and self.ctx.h:
            fn = self.ctx.lib.strata_moe_ep_window_free if self.owned else self.ctx.lib.strata_moe_ep_window_close
            self.ctx.check(fn(self.ctx.h, C.c_void_p(self.ptr)))
        self.ptr = None


class EpState:
    """strata_moe_ep: one rank of an expert-parallel layer over peer-mapped windows."""

    _close_order = 2

    def __init__(self, layer, rank, world, row_capacity, window_ptrs, wait_ms=0):
        self.layer, self.ctx, self.lib = layer, layer.ctx, layer.lib
        self.h = None
        self.world = world
        self.ctx._children.add(self)
        arr = (C.c_void_p * world)(*[C.c_void_p(p) for p in window_ptrs])
        h = C.c_void_p()
        self.ctx.check(self.lib.strata_moe_ep_create(layer.h, rank, world, row_capacity, arr, wait_ms, C.byref(h)))
        self.h = h

    def begin(self, x):
        self._x = x
        self.ctx.enter()
        self.ctx.check(self.lib.strata_moe_ep_begin(self.h, _ptr(x), x.shape[0]))

    def dispatch(self):
        self.ctx.check(self.lib.strata_moe_ep_dispatch(self.h))

    def experts(self, expected_rows=0):
        self.ctx.check(self.lib.strata_moe_ep_experts(self.h, expected_rows))

    def finish(self, out=None):
        x = self._x
        if out is None:
            out = torch.empty(x.shape[0], self.layer.cfg.H, dtype=torch.float32, device=x.device)
        self.ctx.check(self.lib.strata_moe_ep_finish(self.h, _ptr(out)))
        self.ctx.leave()
        return out

    def forward(self, x, out=None, expected_rows=0, join=True):
        """join=False leaves the caller's stream un-ordered against this step (the caller joins later with
        ctx.leave()): several steps on different contexts can then be in flight together."""
        if out is None:
            out = torch.empty(x.shape[0], self.layer.cfg.H, dtype=torch.float32, device=x.device)
        self.ctx.enter()
        self.ctx.check(self.lib.strata_moe_ep_forward(self.h, _ptr(x), x.shape[0], _ptr(out), expected_rows))
        if join:
            self.ctx.leave()
        return out

    def abandon(self):
        self.ctx.check(self.lib.strata_moe_ep_abandon(self.h))

    def last_counts(self):
        """(token rows sent to each owner, token rows received, (token, expert) rows computed) of the last step."""
        sent = (C.c_uint32 * self.world)()
        recv, pairs = C.c_uint32(0), C.c_uint32(0)
        self.ctx.check(self.lib.strata_moe_ep_last_counts(self.h, sent, C.byref(recv), C.byref(pairs)))
        return list(sent), recv.value, pairs.value

    def close(self):
        if self.h:
            if self.ctx.h and self.layer.h:
                self.lib.strata_moe_ep_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
