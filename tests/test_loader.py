"""include/strata_moe_loader.hpp: safetensors parsing and the per-family tensor names, the DeepSeek-V4 tiled host
layout against the reference's own transform (compiled, oracle/_ref), strata.route_trace v2 against the reference's
own parser, and (on a GPU) a layer loaded from a checkpoint file against the same layer registered directly."""
import ctypes as C
import json
import os
import struct
import subprocess

import numpy as np
import pytest
import torch

from oracle import oracle as O
from strata_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def exe(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("loader") / "loader_test")
    lib_dir = os.path.join(ROOT, "strata_b200")
    r = subprocess.run(["g++", "-std=c++20", "-O1", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
                        os.path.join(ROOT, "tests", "cpp", "loader_test.cpp"), "-o", out, "-L", lib_dir,
                        "-lstrata_moe", f"-Wl,-rpath,{lib_dir}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    return out


@pytest.fixture(scope="module")
def exe_sanitized(tmp_path_factory):
    """The same program under AddressSanitizer and UndefinedBehaviorSanitizer (the reference builds its host layer
    that way in its sanitizer configuration, CMakeLists.txt:17, 194-200): the header-only loader parses untrusted
    file contents, which is where such a build earns its keep.  Only the CPU sub-commands run under it."""
    out = str(tmp_path_factory.mktemp("loader_san") / "loader_test_san")
    lib_dir = os.path.join(ROOT, "strata_b200")
    r = subprocess.run(["g++", "-std=c++20", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=all",
                        "-fno-omit-frame-pointer", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
                        os.path.join(ROOT, "tests", "cpp", "loader_test.cpp"), "-o", out, "-L", lib_dir,
                        "-lstrata_moe", f"-Wl,-rpath,{lib_dir}"], capture_output=True, text=True)
    if r.returncode != 0 and "sanitize" in r.stderr and ("cannot find" in r.stderr or "unrecognized" in r.stderr):
        pytest.skip("this toolchain has no sanitizer runtime")
    assert r.returncode == 0, r.stderr[-3000:]
    return out


@pytest.fixture(params=["plain", "sanitized"])
def cpu_exe(request):
    return request.getfixturevalue("exe" if request.param == "plain" else "exe_sanitized")


def fnv1a64(b):
    h = 1469598103934665603
    for v in b:
        h = ((h ^ v) * 1099511628211) & ((1 << 64) - 1)
    return h


def write_safetensors(path, tensors):
    """tensors: name -> (dtype string, shape, bytes)."""
    header, blob, at = {"__metadata__": {"format": "pt", "note": "a {nested} value, with [brackets]"}}, b"", 0
    for name, (dtype, shape, data) in tensors.items():
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [at, at + len(data)]}
        blob += data
        at += len(data)
    text = json.dumps(header).encode()
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + blob)


def laguna_checkpoint(cfg, layer_index):
    """A synthetic layer under the names the Laguna checkpoint uses."""
    layer = synth.build_layer(cfg, "cpu")
    p = f"model.layers.{layer_index}.mlp."
    t = {p + "gate.weight": ("BF16", (cfg.E, cfg.H), layer.router_w.view(torch.uint8).numpy().tobytes())}
    stems = {"gate": "gate_proj", "up": "up_proj", "down": "down_proj"}
    for role in synth.ROLES:
        rows, cols = cfg.role_shape(role)
        for e in range(cfg.E):
            base = f"{p}experts.{e}.{stems[role]}"
            t[base + ".weight_packed"] = ("U8", (rows, cols // 2), layer.packed[role][e].numpy().tobytes())
            t[base + ".weight_scale"] = ("F8_E4M3", (rows, cols // 16), layer.scales[role][e].numpy().tobytes())
            t[base + ".weight_global_scale"] = ("F32", (1,), struct.pack("<f", synth.NVFP4_GLOBAL[role]))
        t[f"{p}shared_expert.{stems[role]}.weight"] = ("BF16", tuple(layer.shared[role].shape),
                                                       layer.shared[role].view(torch.uint8).numpy().tobytes())
    return layer, t


def test_safetensors_index(cpu_exe, tmp_path):
    cfg = synth.MoeConfig("ckpt", H=256, I=128, E=4, k=2, fmt=synth.FMT_NVFP4, T=6, seed=11, I_shared=128)
    _, tensors = laguna_checkpoint(cfg, 7)
    path = str(tmp_path / "model-00001.safetensors")
    write_safetensors(path, tensors)
    r = subprocess.run([cpu_exe, "list", path], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    seen = {}
    for line in r.stdout.splitlines():
        name, dtype, shape, nbytes, h = line.split()
        seen[name] = (dtype, tuple(int(v) for v in shape.split("x")), int(nbytes), int(h, 16))
    assert set(seen) == set(tensors)
    for name, (dtype, shape, data) in tensors.items():
        assert seen[name] == (dtype, tuple(shape), len(data), fnv1a64(data)), name


def test_damaged_safetensors_files_are_rejected_cleanly(exe_sanitized, tmp_path):
    """Checkpoint files are untrusted input.  A valid file is damaged in seeded ways (bytes of the JSON header
    overwritten, the header length changed, the file cut short, offsets moved past the end) and read by the sanitizer
    build: every case must end with a parsed listing or a reported error, never with a sanitizer finding or a crash."""
    cfg = synth.MoeConfig("ckpt_fuzz", H=256, I=128, E=2, k=1, fmt=synth.FMT_NVFP4, T=2, seed=5, I_shared=128)
    _, tensors = laguna_checkpoint(cfg, 0)
    good = str(tmp_path / "good.safetensors")
    write_safetensors(good, tensors)
    blob = bytearray(open(good, "rb").read())
    hlen = struct.unpack("<Q", bytes(blob[:8]))[0]
    rng = np.random.default_rng(2024)
    cases = []
    for _ in range(60):                                   # header bytes overwritten
        b = bytearray(blob)
        for _ in range(int(rng.integers(1, 6))):
            b[8 + int(rng.integers(0, hlen))] = int(rng.integers(0, 256))
        cases.append(bytes(b))
    for v in (0, 1, 7, hlen - 1, hlen + 1, len(blob), len(blob) * 4, 2 ** 40, 2 ** 63, 2 ** 64 - 1):   # header length
        cases.append(struct.pack("<Q", v) + bytes(blob[8:]))
    for cut in (0, 4, 8, 9, 8 + hlen // 2, 8 + hlen, 8 + hlen + 1, len(blob) - 1):                        # truncation
        cases.append(bytes(blob[:cut]))
    text = bytes(blob[8:8 + hlen]).decode()
    for old, new in (('"data_offsets": [0,', '"data_offsets": [18446744073709551615,'), ('"shape": [', '"shape": [-1, '),
                     ('"dtype": "U8"', '"dtype": 7'), ('{', '[', ), ('"data_offsets"', '"data_offset"')):
        t = text.replace(old, new, 1).encode()
        t += b" " * ((8 - len(t) % 8) % 8)
        cases.append(struct.pack("<Q", len(t)) + t + bytes(blob[8 + hlen:]))
    verdicts = {0: 0, 1: 0}
    for i, data in enumerate(cases):
        path = str(tmp_path / f"case{i}.safetensors")
        with open(path, "wb") as f:
            f.write(data)
        r = subprocess.run([exe_sanitized, "list", path], capture_output=True, timeout=60)
        err = r.stderr.decode(errors="replace")     # a damaged tensor name need not be UTF-8 any more
        assert r.returncode in (0, 1), (i, r.returncode, err[-1500:])
        assert "Sanitizer" not in err and "runtime error" not in err, (i, err[-1500:])
        verdicts[r.returncode] += 1
    assert verdicts[1] >= 20, verdicts      # most damage must be noticed, not silently accepted


def test_tiled32_layout_round_trip_against_reference_transform(cpu_exe, ref, tmp_path):
    H, I, shards = 256, 128, 2
    rng = np.random.default_rng(3)
    t = {k: rng.integers(0, 256, n, dtype=np.uint8) for k, n in
         dict(w1=I * H // 2, s1=I * H // 32, w3=I * H // 2, s3=I * H // 32, w2=H * I // 2, s2=H * I // 32).items()}
    p = lambda a: a.ctypes.data_as(O.u8p)
    size = ref.ref_dsv4_tile_shard(None, p(t["w1"]), p(t["s1"]), p(t["w3"]), p(t["s3"]), p(t["w2"]), p(t["s2"]), H, I, 0, shards)
    assert size > 0
    files = []
    for s in range(shards):
        buf = np.zeros(size, np.uint8)
        assert ref.ref_dsv4_tile_shard(p(buf), p(t["w1"]), p(t["s1"]), p(t["w3"]), p(t["s3"]), p(t["w2"]), p(t["s2"]),
                                       H, I, s, shards) == size
        files.append(str(tmp_path / f"shard{s}.bin"))
        buf.tofile(files[-1])
    out = str(tmp_path / "canon")
    r = subprocess.run([cpu_exe, "untile", str(H), str(I), out] + files, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    for k, want in t.items():
        assert np.array_equal(np.fromfile(f"{out}.{k}", np.uint8), want), k


def test_damaged_tiled_shards_are_rejected_cleanly(exe_sanitized, ref, tmp_path):
    """The 32-row tiled host layout read with wrong sizes: truncated, empty, over-long shards and shapes that do not
    match the files must give a reported error under the sanitizer build, not a finding."""
    H, I, shards = 256, 128, 2
    rng = np.random.default_rng(9)
    t = {k: rng.integers(0, 256, n, dtype=np.uint8) for k, n in
         dict(w1=I * H // 2, s1=I * H // 32, w3=I * H // 2, s3=I * H // 32, w2=H * I // 2, s2=H * I // 32).items()}
    p = lambda a: a.ctypes.data_as(O.u8p)
    size = ref.ref_dsv4_tile_shard(None, p(t["w1"]), p(t["s1"]), p(t["w3"]), p(t["s3"]), p(t["w2"]), p(t["s2"]), H, I, 0, shards)
    good = []
    for sidx in range(shards):
        buf = np.zeros(size, np.uint8)
        ref.ref_dsv4_tile_shard(p(buf), p(t["w1"]), p(t["s1"]), p(t["w3"]), p(t["s3"]), p(t["w2"]), p(t["s2"]), H, I, sidx, shards)
        good.append(buf)

    def run(files, h=H, i=I):
        paths = []
        for n, data in enumerate(files):
            paths.append(str(tmp_path / f"d{len(os.listdir(tmp_path))}_{n}.bin"))
            np.asarray(data, np.uint8).tofile(paths[-1])
        r = subprocess.run([exe_sanitized, "untile", str(h), str(i), str(tmp_path / "out")] + paths, capture_output=True)
        err = r.stderr.decode(errors="replace")
        assert "Sanitizer" not in err and "runtime error" not in err, err[-1500:]
        return r.returncode

    assert run(good) == 0
    assert run([good[0][:-1], good[1]]) == 1                   # one byte short
    assert run([good[0], good[1][:size // 2]]) == 1            # half a shard
    assert run([good[0], np.zeros(0, np.uint8)]) == 1          # empty shard
    assert run([good[0], np.concatenate([good[1], good[1][:64]])]) == 1   # over-long
    assert run([good[0]]) in (0, 1)                            # a lone shard is a different, smaller split: either way no finding
    assert run(good, h=H * 2) == 1 and run(good, i=I * 2) == 1  # shapes that the files do not hold
    assert run(good, h=0) == 1 and run(good, i=0) == 1
    assert run(good, h=100) == 1                               # not a multiple of the tile


def test_route_trace_is_read_by_the_reference_parser(cpu_exe, ref, tmp_path):
    path = str(tmp_path / "routes.jsonl")
    assert subprocess.run([cpu_exe, "trace", path]).returncode == 0
    head = (C.c_uint64 * 50)()
    experts = np.zeros(64, np.uint32)
    coefs = np.zeros(64, np.float32)
    n = ref.ref_parse_route_trace(path.encode(), head, experts.ctypes.data_as(O.u32p), coefs.ctypes.data_as(O.f32p), 10, 64)
    assert n == 3
    rows = [tuple(head[i * 5 + j] for j in range(5)) for i in range(3)]
    assert rows[0][:4] == (42, 10, 3, 1) and rows[1][:4] == (42, 11, 3, 1) and rows[2][:4] == (43, 99, 7, 2)
    assert [r[4] & 0xFFFFFFFF for r in rows] == [3, 3, 1]
    assert list(experts[:7]) == [5, 1, 7, 2, 0, 3, 11]
    # the reference's parser skips the coefficients (its simulator only needs the experts); they are written
    # with max_digits10 so that any JSON reader recovers the float32 values exactly
    lines = [json.loads(l) for l in open(path)]
    assert lines[0] == {"schema": "strata.route_trace", "version": 2, "position_base": 0, "layer_base": 0,
                        "coefficient_encoding": "float32-roundtrip-decimal"}
    got = np.array(lines[1]["coefficients"] + lines[2]["coefficients"], np.float32)
    want = np.array([0.5, 0.25, 0.125, 0.3333333, 1.0e-7, 0.6666666], np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert lines[3]["coefficients"] == [] and lines[3]["phase"] == "decode"


@pytest.mark.gpu
def test_layer_loaded_from_a_checkpoint_equals_direct_registration(exe, tmp_path):
    from strata_b200 import MoeContext, MoeLayer
    cfg = synth.MoeConfig("ckpt", H=256, I=128, E=4, k=2, fmt=synth.FMT_NVFP4, T=6, seed=11, I_shared=128)
    layer, tensors = laguna_checkpoint(cfg, 7)
    path = str(tmp_path / "model-00001.safetensors")
    write_safetensors(path, tensors)
    xfile, ofile = str(tmp_path / "x.bin"), str(tmp_path / "out.bin")
    layer.x.view(torch.uint8).numpy().tofile(xfile)
    r = subprocess.run([exe, "forward", path, "laguna", "7", str(cfg.fmt), str(cfg.H), str(cfg.I), str(cfg.E), str(cfg.k),
                        str(cfg.I_shared), str(cfg.score_kind), xfile, str(cfg.T), ofile], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    got = np.fromfile(ofile, np.float32).reshape(cfg.T, cfg.H)
    ctx = MoeContext(0)
    dev = synth.build_layer(cfg, "cuda")
    ml = MoeLayer(ctx, cfg)
    ml.load_synth(dev)
    want = ml.forward(dev.x)
    ctx.synchronize()
    assert np.array_equal(got.view(np.uint32), want.cpu().numpy().view(np.uint32))
