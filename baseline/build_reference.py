#!/usr/bin/env python3
"""Builds the reference's engine, unmodified, into ``baseline/_ref/ref_bench``.

The reference is a CMake project that fetches mdspan, CUTLASS, nlohmann_json and googletest over the
network (cmake/Deps.cmake) and links gRPC for its server.  Its engine, scheduler, model and kernels
need none of gRPC, and this image carries the other headers: CUTLASS (under flashinfer's data
folder), nlohmann/json.hpp (under cudnn_frontend's third-party folder) and the CUDA toolkit's
mdspan.  So the sources are compiled directly, with the reference's own options (C++20 for CUDA,
C++23 for the host, ``--use_fast_math``; cmake/CUDAConf.cmake, cmake/CXXConf.cmake), two stand-in
headers under ``baseline/shim`` (``mdspan/mdspan.hpp``, ``print``) and ``ref_driver.cc`` in place of
``src/server.cu`` and ``src/grpc_adapter.cc``.

    python baseline/build_reference.py [/path/to/firefly]
"""
import glob
import json
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

HOST = ["src/tensor.cc", "src/engine.cc", "src/scheduler.cc", "src/radix_tree.cc", "src/model_registry.cc",
        "src/allocator_cpu.cc", "src/tokenizer.cc"]
DEVICE = ["src/allocator_cuda.cu", "src/model/qwen_model.cu"] + \
         [f"src/kernels/{k}.cu" for k in ("activation", "add", "attention", "embedding", "linear", "norm", "rope", "sampling")]


def find_include(*parts):
    for base in {sysconfig.get_paths()["purelib"], *sys.path}:
        cand = os.path.join(base, *parts)
        if os.path.exists(cand):
            return cand
    raise SystemExit(f"header tree not found: {os.path.join(*parts)}")


def build(reference: str) -> str:
    os.makedirs(OUT, exist_ok=True)
    cutlass = find_include("flashinfer", "data", "cutlass", "include")
    json_dir = find_include("include", "cudnn_frontend", "thirdparty")
    inc = ["-I", os.path.join(reference, "include"), "-I", os.path.join(HERE, "shim"), "-I", cutlass, "-I", json_dir,
           "-I", "/usr/local/cuda/include"]
    objs = []
    for src in HOST:
        obj = os.path.join(OUT, os.path.basename(src) + ".o")
        subprocess.run(["g++", "-std=c++23", "-O2", "-fPIC", *inc, "-c", os.path.join(reference, src), "-o", obj], check=True)
        objs.append(obj)
    nv = ["nvcc", "-std=c++20", "--use_fast_math", "--expt-relaxed-constexpr", "-O2", "-gencode",
          "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
    for src in DEVICE:
        obj = os.path.join(OUT, os.path.basename(src) + ".o")
        subprocess.run([*nv, *inc, "-c", os.path.join(reference, src), "-o", obj], check=True)
        objs.append(obj)
    drv = os.path.join(OUT, "ref_driver.o")
    subprocess.run(["g++", "-std=c++23", "-O2", "-fPIC", *inc, "-c", os.path.join(HERE, "ref_driver.cc"), "-o", drv], check=True)
    exe = os.path.join(OUT, "ref_bench")
    subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", drv, *objs, "-o", exe, "-lcudart", "-lpthread"],
                   check=True)
    for o in glob.glob(os.path.join(OUT, "*.o")):
        os.unlink(o)
    return exe


if __name__ == "__main__":
    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FIREFLY_REFERENCE", "")
    if not where:
        try:
            with open(os.path.join(HERE, "..", "BASELINE.json")) as fh:
                where = json.load(fh).get("reference_path", "")
        except (OSError, ValueError):
            where = ""
    if not where:
        sys.exit("usage: python baseline/build_reference.py REFERENCE_SOURCES (or $FIREFLY_REFERENCE)")
    print(build(where))
