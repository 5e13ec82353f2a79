"""Builds the two CPU checkers.  TEST INFRASTRUCTURE ONLY.

  oracle/libmoe_oracle.so      the plain-C restatement (oracle/moe_oracle.c)
  oracle/_ref/libstrata_ref.so the reference's own CPU sources, compiled unmodified from
                               where they lie in the reference checkout, behind the
                               extern "C" doorway in oracle/ref_shim.cpp

The second one is only (re)built when a reference checkout is given (argument or the
STRATA_REFERENCE environment variable; failing both, a directory named `reference` beside the
repository is tried); a machine without the checkout uses the library built earlier.  The reference's CMake build is not used: it
requires libnuma, which is absent, so the listed files are compiled directly.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def default_reference():
    return os.environ.get("STRATA_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")

REF_SOURCES = [
    "kernels/cpu/dsv4_fp4_expert.cpp",
    "kernels/cpu/glm_int4.cpp",
    "src/platform/numerics.cpp",
    "src/platform/diagnostics.cpp",
    "src/platform/compressed_tensors.cpp",
    "src/platform/worker_pool.cpp",
    "src/platform/numa_topology.cpp",
    "src/platform/safetensors.cpp",
    "src/platform/json_cursor.cpp",
    "src/platform/trace.cpp",
    "src/models/dsv4/deepseek_ops.cpp",
    "src/models/glm52/glm_ops.cpp",
    "src/models/laguna/laguna_ops.cpp",
    "src/models/inkling/inkling_ops.cpp",
    "src/models/kimi_k3/kimi_k3_ops.cpp",
    "src/models/kimi_k3/kimi_k3_layer.cpp",
    "src/models/kimi_k3/kimi_k3_kv_cache.cpp",
    "src/models/common/model.cpp",
]


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_port(force=False):
    src = os.path.join(HERE, "moe_oracle.c")
    out = os.path.join(HERE, "libmoe_oracle.so")
    if force or _newer(out, [src]):
        subprocess.check_call(
            ["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-mfma", "-mavx2", "-shared", "-fPIC",
             "-fvisibility=hidden", "-o", out, src, "-lm"])
    return out


def build_reference(reference=None, force=False):
    reference = reference or default_reference()
    outdir = os.path.join(HERE, "_ref")
    out = os.path.join(outdir, "libstrata_ref.so")
    if not os.path.isdir(os.path.join(reference, "kernels", "cpu")):
        return out if os.path.exists(out) else None
    shim = os.path.join(HERE, "ref_shim.cpp")
    sources = [os.path.join(reference, s) for s in REF_SOURCES]
    if not (force or _newer(out, [shim] + sources)):
        return out
    os.makedirs(outdir, exist_ok=True)
    objs = []
    jobs = []
    for src in sources + [shim]:
        obj = os.path.join(outdir, os.path.basename(src) + ".o")
        objs.append(obj)
        jobs.append(subprocess.Popen(
            ["g++", "-std=c++20", "-O2", "-fPIC", "-w", "-I", os.path.join(reference, "include"),
             "-include", "algorithm", "-c", src, "-o", obj]))
    for j in jobs:
        if j.wait() != 0:
            raise RuntimeError("reference compile failed")
    subprocess.check_call(["g++", "-shared", "-o", out] + objs + ["-Wl,--no-undefined", "-lpthread"])
    for obj in objs:
        os.remove(obj)
    return out


# The reference's own CUDA backend (kernels/cuda/backend.cu, 17k lines, no build system needed: nvcc on the one file plus
# three host sources it calls into).  Second checker and "kernel to beat" on the GPU box: the reference's command tests,
# as ported in tests/cpp/backend_shim_test.cpp, are compiled HERE against the reference's own headers and this library
# (the GPU box has no reference checkout) into oracle/_ref/backend_shim_test_ref.
REF_CUDA_HOST_SOURCES = ["src/platform/attention.cpp", "src/platform/numerics.cpp", "src/platform/safetensors.cpp",
                         "src/platform/json_cursor.cpp"]


def build_reference_cuda(reference=None, force=False):
    reference = reference or default_reference()
    outdir = os.path.join(HERE, "_ref")
    lib = os.path.join(outdir, "libstrata_ref_cuda.so")
    exe = os.path.join(outdir, "backend_shim_test_ref")
    backend = os.path.join(reference, "kernels", "cuda", "backend.cu")
    if not os.path.exists(backend):
        return (lib, exe) if os.path.exists(lib) and os.path.exists(exe) else None
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    inc = os.path.join(reference, "include")
    os.makedirs(outdir, exist_ok=True)
    hosts = [os.path.join(reference, s) for s in REF_CUDA_HOST_SOURCES]
    if force or _newer(lib, [backend] + hosts):
        objs = [os.path.join(outdir, "backend.cu.o")]
        jobs = [subprocess.Popen([nvcc, "-std=c++20", "-gencode", "arch=compute_100a,code=sm_100a", "-w",
                                  "--expt-relaxed-constexpr", "--extended-lambda", "-O2", "-Xcompiler", "-fPIC",
                                  "-I", inc, "-c", backend, "-o", objs[0]])]
        for src in hosts:
            obj = os.path.join(outdir, os.path.basename(src) + ".o")
            objs.append(obj)
            jobs.append(subprocess.Popen(["g++", "-std=c++20", "-O2", "-fPIC", "-w", "-I", inc, "-include", "algorithm",
                                          "-c", src, "-o", obj]))
        for j in jobs:
            if j.wait() != 0:
                raise RuntimeError("reference CUDA backend compile failed")
        subprocess.check_call([nvcc, "-shared", "-o", lib] + objs +
                              ["-lcublas", "-lcudart_static", "-lpthread", "-ldl", "-lrt", "-Xlinker", "--no-undefined",
                               "-Xlinker", "-rpath=/usr/local/cuda/lib64"])
        for obj in objs:
            os.remove(obj)
    test_src = os.path.join(HERE, "..", "tests", "cpp", "backend_shim_test.cpp")
    port = build_port()
    if force or _newer(exe, [lib, test_src, port]):
        subprocess.check_call(["g++", "-std=c++20", "-O1", "-w", "-DSTRATA_TEST_REFERENCE_BACKEND", "-I", inc, test_src, "-o", exe,
                               "-L", outdir, "-lstrata_ref_cuda", "-L", HERE, "-lmoe_oracle",
                               "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,$ORIGIN/..", "-Wl,-rpath,/usr/local/cuda/lib64"])
    return lib, exe


if __name__ == "__main__":
    print(build_port(force="--force" in sys.argv))
    print(build_reference(force="--force" in sys.argv))
    print(build_reference_cuda(force="--force" in sys.argv))
