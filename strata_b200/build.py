"""Compiles the CUDA kernels and the C ABI into strata_b200/libstrata_moe.so (sm_100a only)."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libstrata_moe.so")
SOURCES = ["api.cu", "router.cu", "group.cu", "decode.cu", "decode_fp4.cu", "decode_stream.cu", "combine.cu", "prefill.cu", "ep.cu", "dsv4_exact.cu", "latent.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=default"]


def _deps():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [
        os.path.join(HERE, "..", "include", "strata_moe.h"), os.path.abspath(__file__)]


def build(force=False, verbose=False):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    if not force and os.path.exists(LIB):
        t = os.path.getmtime(LIB)
        if all(os.path.getmtime(d) <= t for d in _deps()):
            return LIB
    flags = list(NVCC_FLAGS)
    if verbose:
        flags += ["-Xptxas", "-v"]
    objs, jobs = [], []
    for src in SOURCES:
        obj = os.path.join(CSRC, src[:-3] + ".o")
        objs.append(obj)
        jobs.append((src, subprocess.Popen([nvcc] + flags + ["-c", os.path.join(CSRC, src), "-o", obj],
                                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    ok = True
    for src, j in jobs:
        out, _ = j.communicate()
        if j.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src}\n{out}\n")
        ok &= j.returncode == 0
    if not ok:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([nvcc, "-shared", "-o", LIB] + objs + ["-lcudart_static", "-lpthread", "-ldl", "-lrt"])
    for o in objs:
        os.remove(o)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
