"""Seeded synthetic MoE layers with the shapes and value distributions of the five
benchmark configurations.

Real checkpoints are not available offline, so every tensor is generated from a
counter-based hash (splitmix64 over the element index) that gives bit-identical bytes on
CPU and on CUDA and lets any single expert be generated on its own.  That is what allows
a full-size layer to live only on the GPU while the CPU checker regenerates just the
experts a sampled token routes to.

Layouts are the checkpoint-native ones the reference consumes:
  MXFP4  packed u8 [rows, cols/2] (low nibble = even column) + E8M0 u8 [rows, cols/32]
  NVFP4  packed u8 [rows, cols/2] + E4M3 u8 [rows, cols/16] + one fp32 global scale,
         w = e2m1 * (e4m3 / global)
  INT4   u32 words [rows, cols/8], nibble j of a word = column 8w+j, value raw-8,
         BF16 scale [rows, cols/128]
gate/up are [I, H], down is [H, I]; all row-major (K contiguous).
"""
from dataclasses import dataclass, field, replace

import numpy as np
import torch

FMT_MXFP4, FMT_NVFP4, FMT_INT4, FMT_BF16 = 0, 1, 2, 3
SCORE_SIGMOID, SCORE_SIGMOID_PLAIN, SCORE_SOFTMAX, SCORE_SQRTSOFTPLUS = 0, 1, 2, 3
ROLES = ("gate", "up", "down")


@dataclass(frozen=True)
class MoeConfig:
    name: str
    H: int
    I: int
    E: int
    k: int
    fmt: int
    T: int
    score_kind: int = SCORE_SIGMOID
    normalize: bool = True
    norm_init: float = 0.0
    weight_scale: float = 1.0     # multiplied into each routing weight
    output_scale: float = 1.0     # multiplied into the summed routed output
    I_shared: int = 0             # BF16 shared expert width, 0 = none
    seed: int = 0
    zipf_s: float = 0.0           # > 0: Zipf(s) router bias over a seeded rank permutation
    activation: int = 0           # 0 = SwiGLU, 1 = SiTU-GLU (Kimi-K3), routed and shared experts alike
    gate_beta: float = 1.0
    linear_beta: float = 1.0
    H_model: int = 0              # > 0: LatentMoE (Kimi-K3): router and shared experts on H_model, experts on H
    rms_epsilon: float = 1e-5
    description: str = ""

    @property
    def Hx(self):
        """Width of the layer's input rows (the router's and the shared experts' K)."""
        return self.H_model or self.H

    def with_(self, **kw):
        return replace(self, **kw)

    def role_shape(self, role):
        return (self.I, self.H) if role in ("gate", "up") else (self.H, self.I)


CONFIGS = {
    # DeepSeek-V4-Flash-style decode: 256 experts, top-6 sigmoid, renormalised, MXFP4.
    "c0": MoeConfig("c0", H=4096, I=2048, E=256, k=6, fmt=FMT_MXFP4, T=8, seed=0,
                    description="DSV4-Flash-style MXFP4 decode, 8 tokens"),
    # Laguna-style NVFP4 + always-on BF16 shared expert, top-10.  BASELINE names softmax
    # scoring; the reference's own Laguna rule is sigmoid + renormalise + 2.5 output scale.
    "c1": MoeConfig("c1", H=3072, I=1024, E=256, k=10, fmt=FMT_NVFP4, T=256,
                    score_kind=SCORE_SOFTMAX, normalize=True, I_shared=1024, seed=0,
                    description="Laguna-style NVFP4 + shared expert, softmax top-10"),
    "c1_sigmoid": MoeConfig("c1_sigmoid", H=3072, I=1024, E=256, k=10, fmt=FMT_NVFP4, T=256,
                            score_kind=SCORE_SIGMOID, normalize=True, output_scale=2.5,
                            I_shared=1024, seed=0,
                            description="Laguna rule as the reference implements it"),
    # GLM-style INT4 W4A16 prefill: top-8 sigmoid, normaliser starts at 1e-20, scale 2.5.
    "c2": MoeConfig("c2", H=6144, I=2048, E=256, k=8, fmt=FMT_INT4, T=4096, norm_init=1e-20,
                    weight_scale=2.5, seed=0, description="GLM-style INT4-g128 prefill, 4096 tokens"),
    # Expert-parallel MXFP4 prefill.
    "c3": MoeConfig("c3", H=7168, I=2048, E=256, k=8, fmt=FMT_MXFP4, T=16384, seed=0,
                    description="EP MXFP4 prefill, 16384 tokens"),
    # Kimi-K3-style 896-expert decode with a Zipf-skewed selection bias.
    "c4": MoeConfig("c4", H=7168, I=1024, E=896, k=16, fmt=FMT_MXFP4, T=256,
                    score_kind=SCORE_SIGMOID_PLAIN, seed=1, zipf_s=1.1,
                    description="Kimi-K3-style 896-expert MXFP4 decode, Zipf(1.1) bias"),
    # Kimi-K3 LatentMoE at its real shape: route on 7168, 896 MXFP4 experts (top-16) on a 3584-wide latent,
    # two BF16 shared experts (6144 wide together), SiTU-GLU.
    "kimi": MoeConfig("kimi", H=3584, I=3072, E=896, k=16, fmt=FMT_MXFP4, T=4, score_kind=SCORE_SIGMOID_PLAIN,
                      I_shared=6144, seed=2, activation=1, gate_beta=4.0, linear_beta=25.0, H_model=7168,
                      description="Kimi-K3 LatentMoE, 896 experts on a 3584-wide latent"),
}


# --------------------------------------------------------------------------- hashing
def _s64(v):
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


_GOLDEN = _s64(0x9E3779B97F4A7C15)
_M1 = _s64(0xBF58476D1CE4E5B9)
_M2 = _s64(0x94D049BB133111EB)


def _lshr(z, n):
    return (z >> n) & ((1 << (64 - n)) - 1)


def hash64(start, count, seed, device):
    """splitmix64 of (index, seed) for index in [start, start+count) as int64."""
    idx = torch.arange(start, start + count, dtype=torch.int64, device=device)
    z = idx * _GOLDEN + _s64(seed * 0xD1B54A32D192ED03 + 0x632BE59BD9B4E019)
    z = (z ^ _lshr(z, 30)) * _M1
    z = (z ^ _lshr(z, 27)) * _M2
    return z ^ _lshr(z, 31)


def hash_bytes(start, count, seed, device, chunk=1 << 25):
    """count uniform bytes: byte j is byte (j % 8) of hash64(j // 8).  start, count % 8 == 0."""
    assert start % 8 == 0 and count % 8 == 0
    out = torch.empty(count, dtype=torch.uint8, device=device)
    words = count // 8
    for w0 in range(0, words, chunk):
        w1 = min(words, w0 + chunk)
        out[w0 * 8:w1 * 8] = hash64(start // 8 + w0, w1 - w0, seed, device).view(torch.uint8)
    return out


def _tensor_seed(cfg, name):
    h = 1469598103934665603
    for ch in f"{cfg.name}/{cfg.seed}/{name}".encode():
        h = ((h ^ ch) * 1099511628211) & ((1 << 64) - 1)
    return h >> 1


def e4m3_encode_table():
    """256 E4M3 bytes whose values are 2^u, u evenly spaced over [-4, 2], rounded to E4M3."""
    vals = []
    for j in range(256):
        v = 2.0 ** (-4.0 + 6.0 * (j + 0.5) / 256.0)
        e = int(np.floor(np.log2(v)))
        m = int(np.rint((v / 2.0 ** e - 1.0) * 8.0))
        if m == 8:
            e, m = e + 1, 0
        vals.append(((e + 7) << 3) | m)
    return np.array(vals, np.uint8)


NVFP4_GLOBAL = {"gate": 203.0, "up": 199.0, "down": 207.0}
MXFP4_SCALE_BYTE = 0x78


# ----------------------------------------------------------------- per-expert tensors
def expert_bytes(cfg, role):
    rows, cols = cfg.role_shape(role)
    packed = rows * cols // 2
    if cfg.fmt == FMT_MXFP4:
        return packed, rows * cols // 32
    if cfg.fmt == FMT_NVFP4:
        return packed, rows * cols // 16
    if cfg.fmt == FMT_INT4:
        return packed, rows * cols // 128 * 2
    if cfg.fmt == FMT_BF16:
        return rows * cols * 2, 0
    raise ValueError(cfg.fmt)


def gen_expert_range(cfg, role, e0, e1, device):
    """(packed u8 [e1-e0, packed_bytes], scales u8 [e1-e0, scale_bytes]) for experts e0..e1."""
    pb, sb = expert_bytes(cfg, role)
    n = e1 - e0
    packed = hash_bytes(e0 * pb, n * pb, _tensor_seed(cfg, role + ".packed"), device).view(n, pb)
    if cfg.fmt == FMT_BF16:
        # plain BF16 weights, uniform with std 0.02, built from byte pairs
        u = packed.view(torch.int16).to(torch.int32) & 0xFFFF
        val = (u.to(torch.float32) / 65536.0 - 0.5) * (0.02 * 12.0 ** 0.5)
        return val.to(torch.bfloat16).view(torch.uint8).view(n, pb), torch.zeros(n, 0, dtype=torch.uint8, device=device)
    raw = hash_bytes(e0 * sb, n * sb, _tensor_seed(cfg, role + ".scales"), device)
    if cfg.fmt == FMT_MXFP4:
        # constant 2^-7 with a -1/0/+1 octave jitter: dequantised std ~ 0.02; never 0x00/0xFF
        scales = (MXFP4_SCALE_BYTE - 1 + (raw % 3)).to(torch.uint8)
    elif cfg.fmt == FMT_NVFP4:
        table = torch.from_numpy(e4m3_encode_table()).to(device)
        scales = table[raw.long()]
    else:
        # BF16 of 0.02/4.61*(1+0.1*U): built from byte pairs (u16 -> U in [0,1))
        u = raw.view(torch.int16).to(torch.int32) & 0xFFFF
        val = (0.02 / 4.61) * (1.0 + 0.1 * (u.to(torch.float32) / 65536.0))
        scales = val.to(torch.bfloat16).view(torch.uint8)
    return packed, scales.view(n, sb)


@dataclass
class SynthLayer:
    cfg: MoeConfig
    device: torch.device
    x: torch.Tensor = None              # [T, H] bf16
    router_w: torch.Tensor = None       # [E, H] bf16
    bias: torch.Tensor = None           # [E] fp32 or None
    packed: dict = field(default_factory=dict)   # role -> u8 [E_local, bytes]
    scales: dict = field(default_factory=dict)
    shared: dict = field(default_factory=dict)   # role -> bf16 [rows, cols]
    latent: dict = field(default_factory=dict)   # LatentMoE: down / up (bf16), norm (fp32)
    expert_begin: int = 0
    expert_end: int = 0

    def global_scale(self, role):
        return NVFP4_GLOBAL[role] if self.cfg.fmt == FMT_NVFP4 else 1.0


def gen_inputs(cfg, T=None, seed=None):
    """Activations BF16 N(0,1) [T,H] (CPU tensor)."""
    T = cfg.T if T is None else T
    g = torch.Generator().manual_seed(1000 + (cfg.seed if seed is None else seed))
    return torch.randn(T, cfg.Hx, generator=g, dtype=torch.float32).to(torch.bfloat16)


def gen_router(cfg):
    """Router gate BF16 N(0, 0.02^2) [E,H] and selection bias (None or fp32 [E])."""
    g = torch.Generator().manual_seed(2000 + cfg.seed)
    w = (torch.randn(cfg.E, cfg.Hx, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    bias = None
    if cfg.zipf_s > 0:
        # selection probability ~ rank^-s over a seeded permutation of expert ranks; the bias
        # steers selection only (weights come from the unbiased scores).
        rank = torch.randperm(cfg.E, generator=g).to(torch.float32) + 1.0
        bias = (-cfg.zipf_s * 0.25 * torch.log(rank)).to(torch.float32)
    return w, bias


def gen_shared(cfg):
    """BF16 N(0, 0.02^2) shared expert (gate/up [Is,H], down [H,Is])."""
    if not cfg.I_shared:
        return {}
    g = torch.Generator().manual_seed(3000 + cfg.seed)
    out = {}
    for role in ROLES:
        rows, cols = (cfg.I_shared, cfg.Hx) if role != "down" else (cfg.Hx, cfg.I_shared)
        out[role] = (torch.randn(rows, cols, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    return out


def gen_latent(cfg):
    """LatentMoE projections: down BF16 [H, H_model] (latent ~ N(0, 1)), up BF16 [H_model, H], norm fp32 [H]."""
    if not cfg.H_model:
        return {}
    g = torch.Generator().manual_seed(4000 + cfg.seed)
    down = (torch.randn(cfg.H, cfg.H_model, generator=g, dtype=torch.float32) * cfg.H_model ** -0.5).to(torch.bfloat16)
    up = (torch.randn(cfg.H_model, cfg.H, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    norm = (1.0 + 0.1 * (torch.rand(cfg.H, generator=g, dtype=torch.float32) - 0.5)).contiguous()
    return {"down": down, "up": up, "norm": norm}


def build_layer(cfg, device, expert_begin=0, expert_end=None, T=None, with_weights=True):
    """Generate a layer (optionally only experts [expert_begin, expert_end)) on `device`."""
    device = torch.device(device)
    expert_end = cfg.E if expert_end is None else expert_end
    layer = SynthLayer(cfg, device, expert_begin=expert_begin, expert_end=expert_end)
    layer.x = gen_inputs(cfg, T).to(device)
    w, b = gen_router(cfg)
    layer.router_w = w.to(device)
    layer.bias = b.to(device) if b is not None else None
    layer.shared = {r: t.to(device) for r, t in gen_shared(cfg).items()}
    layer.latent = {r: t.to(device) for r, t in gen_latent(cfg).items()}
    if with_weights:
        for role in ROLES:
            p, s = gen_expert_range(cfg, role, expert_begin, expert_end, device)
            layer.packed[role], layer.scales[role] = p, s
    return layer
