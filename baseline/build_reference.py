"""Builds the reference arm of bench.py: ember.cpp's interpreter with its CUDA half, unmodified,
straight from its source tree with nvcc, and the small timing driver beside this file.

    python baseline/build_reference.py [--reference /path/to/ember.cpp] [--out baseline/_ref]

ember.cpp is a scikit-build/CMake project whose configure step downloads nlohmann_json and
cpp-httplib, so `pip install` of it fails without a network.  Its interpreter needs neither the
download nor Boost: the sources below compile by hand (the same set its CPU tools are built from,
plus graph_ir_cuda.cu, cuda_kernels.cu and kv_quant.cu with -DHAS_CUDA, the definition its own
CMakeLists.txt gives its core library), against the nlohmann/json.hpp that this image carries in a
Python package.  Nothing of the reference is changed or copied into this repository: the objects
and the binary go to baseline/_ref (git-ignored), which travels to the GPU box with the snapshot.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import site
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["graph_ir.cpp", "graph_ir_ops.cpp", "graph_ir_expr.cpp", "graph_ir_mamba.cpp", "graph_ir_recurrence.cpp",
           "graph_ir_validate.cpp", "ir_digest.cpp", "cpu_attention.cpp", "utils.cpp", "logger.cpp", "quantization.cpp",
           "gguf_parser.cpp", "parallel_for.cpp", "model_config.cpp", "weight_management.cpp",
           "graph_ir_cuda.cu", "cuda_kernels.cu", "kv_quant.cu"]
# code for the B200 (sm_100) and PTX of the same version; -ffp-contract=off as ember.cpp's own build has it
FLAGS = ["-std=c++17", "-O3", "-DHAS_CUDA", "-gencode", "arch=compute_100,code=[sm_100,compute_100]",
         "-Xcompiler", "-fopenmp", "-Xcompiler", "-ffp-contract=off", "-w"]


def find_json_include() -> str | None:
    for base in site.getsitepackages():
        cand = os.path.join(base, "include", "cudnn_frontend", "thirdparty")
        if os.path.isfile(os.path.join(cand, "nlohmann", "json.hpp")):
            return cand
    return None


def binary(out: str | None = None) -> str:
    return os.path.join(out or os.path.join(HERE, "_ref"), "ref_bench")


def build(reference: str, out: str | None = None) -> str:
    out = out or os.path.join(HERE, "_ref")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    inc = find_json_include()
    if not os.path.isfile(os.path.join(reference, "graph_ir.cpp")):
        raise RuntimeError(f"{reference} does not hold ember.cpp's sources (graph_ir.cpp)")
    if inc is None:
        raise RuntimeError("nlohmann/json.hpp was not found in this image's Python packages")
    os.makedirs(out, exist_ok=True)

    def compile_one(src: str) -> str:
        path = src if os.path.isabs(src) else os.path.join(reference, src)
        obj = os.path.join(out, os.path.basename(src).rsplit(".", 1)[0] + ".o")
        r = subprocess.run([nvcc, *FLAGS, f"-I{reference}", f"-I{inc}", "-c", path, "-o", obj], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stderr[-3000:]}")
        print(f"  compiled {os.path.basename(src)}", flush=True)
        return obj

    print(f"building ember.cpp's interpreter from {reference} into {out} (a few minutes) ...", flush=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, SOURCES + [os.path.join(HERE, "ref_bench.cpp")]))
    exe = binary(out)
    r = subprocess.run([nvcc, "-gencode", "arch=compute_100,code=[sm_100,compute_100]", "-Xcompiler", "-fopenmp", *objs,
                        "-lcublas", "-Xlinker", "-rpath=/usr/local/cuda/lib64", "-o", exe], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"linking ref_bench failed:\n{r.stderr[-3000:]}")
    for obj in objs:
        os.remove(obj)
    print("built", exe)
    return exe


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--reference", default=os.environ.get("EMBER_REFERENCE", "/root/reference"))
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    try:
        build(args.reference, args.out)
    except RuntimeError as e:
        print(f"error: {e}", file=sys.stderr)
        sys.exit(1)
