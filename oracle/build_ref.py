#!/usr/bin/env python
"""Builds the reference's own CUDA operators as a comparison oracle for the GPU box: ``oracle/_ref/fastgl_ref.so``.

Test infrastructure, not product code: nothing under ``fastgl-ae_b200/`` loads the result.  Only
``tests/golden/make_ref_golden.py`` does, to write the fixtures that pin the CPU oracle and the CUDA kernels of this
repository to outputs of the reference itself.

The reference's extension (cuda_operators/setup.py) targets PyTorch 1.10 and sm_80.  Its sources are compiled from
where they lie, through a scratch copy that receives three mechanical edits and is deleted afterwards -- no reference
source is kept in this repository:

* ``AT_DISPATCH_*(x.type(), ...)`` -> ``x.scalar_type()`` (the overload taking ``.type()`` no longer exists);
* ``CHECK_GT(scale, 0)`` -> ``TORCH_CHECK(scale > 0)`` (cuda_hashtable.cuh:159, a glog macro that was never defined);
* the architecture flag (setup.py:18 builds sm_80 machine code only) -> ``compute_100a / sm_100a``.

The module is named ``fastgl_ref`` so that it cannot shadow this repository's ``fastgl``.  Compiling needs no GPU.

    python oracle/build_ref.py <dir holding cuda_operators/> [--force]
"""
from __future__ import annotations

import argparse
import os
import re
import shutil
import subprocess
import sys
import sysconfig
import tempfile
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "fastgl_ref.so")
SOURCES = ["aggregate_acc.cpp", "aggregate_acc_kernel.cu", "id_map.cu", "sample.cu", "utilis.cu"]
HEADERS = ["cuda_hashtable.cuh"]


def patched(text: str) -> str:
    text = re.sub(r"(AT_DISPATCH_[A-Z_]+\(\s*[A-Za-z_0-9]+)\.type\(\)", r"\1.scalar_type()", text)
    text = text.replace("CHECK_GT(scale, 0);", "TORCH_CHECK(scale > 0);")
    return text


def build(reference_dir: str, force: bool = False) -> str | None:
    src_dir = os.path.join(reference_dir, "cuda_operators")
    if not all(os.path.exists(os.path.join(src_dir, f)) for f in SOURCES + HEADERS):
        return None
    newest = max(os.path.getmtime(os.path.join(src_dir, f)) for f in SOURCES + HEADERS)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= max(newest, os.path.getmtime(__file__)):
        return OUT
    import torch
    from torch.utils import cpp_extension

    os.makedirs(OUT_DIR, exist_ok=True)
    tmp = tempfile.mkdtemp(prefix="fgl_ref_build_")
    try:
        for f in SOURCES + HEADERS:
            with open(os.path.join(src_dir, f)) as fin, open(os.path.join(tmp, f), "w") as fout:
                fout.write(patched(fin.read()))
        inc = [f"-I{p}" for p in cpp_extension.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
        defs = ["-DTORCH_EXTENSION_NAME=fastgl_ref", "-DTORCH_API_INCLUDE_EXTENSION_H",
                f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
        nvcc = os.path.join(cpp_extension.CUDA_HOME or "/usr/local/cuda", "bin", "nvcc")

        def compile_one(f: str) -> str:
            obj = os.path.join(tmp, f + ".o")
            if f.endswith(".cu"):
                cmd = [nvcc, "-c", f, "-o", obj, "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
                       "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-w"] + defs + inc
            else:
                cmd = ["g++", "-c", f, "-o", obj, "-O2", "-std=c++17", "-fPIC", "-w"] + defs + inc
            subprocess.run(cmd, cwd=tmp, check=True)
            return obj

        with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
            objs = list(pool.map(compile_one, SOURCES))
        lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
        cuda_lib = os.path.join(cpp_extension.CUDA_HOME or "/usr/local/cuda", "lib64")
        subprocess.run(["g++", "-shared", "-o", OUT] + objs +
                       [f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
                        "-ltorch_python", f"-L{cuda_lib}", "-lcudart"], check=True)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    return OUT


def load():
    """Import ``oracle/_ref/fastgl_ref.so`` (needs torch; importing needs no GPU).  None when it was not built."""
    if not os.path.exists(OUT):
        return None
    import importlib.util

    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location("fastgl_ref", OUT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("reference_dir")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    out = build(a.reference_dir, a.force)
    print(out if out else "reference sources not found: nothing built")
    sys.exit(0)
