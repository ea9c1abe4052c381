#!/usr/bin/env python3
"""Builds the REFERENCE engine (KleinSteven/pulse_infer, unmodified sources) for sm_100 with its CUDA path on,
plus ``ref_bench_driver.cu``, into ``baseline/_ref/ref_bench`` - the program ``bench.py --impl reference`` runs.

The reference is a C++/CMake project (no setup.py / pyproject.toml, so pip cannot install it) whose configure
step fetches spdlog, nlohmann-json and googletest from the network.  This script does by hand what its
``src/CMakeLists.txt`` does: every ``.cpp`` of core, layer, ops, model and runtime and every ``.cu`` of
``src/ops/kernels/cuda`` with ``PULSE_USE_CUDA`` defined and the reference's own nvcc flags
(``--expt-relaxed-constexpr --extended-lambda -use_fast_math``, CMakeLists.txt:108-110), linked with cudart and
cuBLAS; spdlog and nlohmann-json headers come from copies vendored inside installed Python packages.  The only
departure from the reference's build is the architecture list (``75;80;86`` there, sm_100 here).  The tokenizer and
the text-level batching engine are left out (they need tokenizer files; the driver feeds token ids to the model).

    python baseline/build_reference.py [--reference /path/to/pulse_infer]
"""
from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("PULSE_REFERENCE", "/root/reference"))
    ap.add_argument("--jobs", type=int, default=min(16, os.cpu_count() or 4))
    args = ap.parse_args()
    ref = os.path.abspath(args.reference)
    if not os.path.isdir(os.path.join(ref, "src", "ops", "kernels", "cuda")):
        print(f"no reference checkout at {ref}", file=sys.stderr)
        return 1
    site = sysconfig.get_paths()["purelib"]
    spdlog = os.path.join(site, "flashinfer", "data", "spdlog", "include")
    json_inc = os.path.join(site, "include", "cudnn_frontend", "thirdparty")
    for need in (spdlog, json_inc):
        if not os.path.isdir(need):
            print(f"vendored headers not found: {need}", file=sys.stderr)
            return 1
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    obj_dir = os.path.join(OUT, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    common = ["-std=c++20", "-O3", "-w", "-DPULSE_USE_CUDA", "-DSPDLOG_USE_STD_FORMAT=1", f"-I{ref}/include",
              f"-I{spdlog}", f"-I{json_inc}", f"-I{cuda_home}/include"]
    nvcc = ["nvcc", "-gencode", "arch=compute_100,code=sm_100", "--expt-relaxed-constexpr", "--extended-lambda",
            "-use_fast_math", *common]
    jobs = []
    cpps = []
    for pattern in ("src/core/*.cpp", "src/layer/*.cpp", "src/ops/*.cpp", "src/model/qwen3/model.cpp",
                    "src/model/qwen3/config.cpp", "src/runtime/*.cpp"):
        cpps += sorted(glob.glob(os.path.join(ref, pattern)))
    for src in cpps:
        obj = os.path.join(obj_dir, os.path.relpath(src, ref).replace(os.sep, "_") + ".o")
        jobs.append((["g++", *common, "-c", src, "-o", obj], obj))
    for src in sorted(glob.glob(os.path.join(ref, "src/ops/kernels/cuda/*.cu"))):
        obj = os.path.join(obj_dir, os.path.relpath(src, ref).replace(os.sep, "_") + ".o")
        jobs.append(([*nvcc, "-c", src, "-o", obj], obj))
    driver_obj = os.path.join(obj_dir, "ref_bench_driver.o")
    jobs.append(([*nvcc, "-c", os.path.join(HERE, "ref_bench_driver.cu"), "-o", driver_obj], driver_obj))

    def run(job):
        cmd, obj = job
        proc = subprocess.run(cmd, capture_output=True, text=True)
        print(("ok   " if proc.returncode == 0 else "FAIL ") + os.path.basename(obj), flush=True)
        return proc.returncode, proc.stderr[-3000:]

    print(f"compiling {len(jobs)} files of the reference for sm_100 (a minute or two) ...", flush=True)
    with ThreadPoolExecutor(args.jobs) as pool:
        results = list(pool.map(run, jobs))
    bad = [err for rc, err in results if rc != 0]
    if bad:
        print(bad[0], file=sys.stderr)
        return 1
    exe = os.path.join(OUT, "ref_bench")
    link = ["nvcc", "-gencode", "arch=compute_100,code=sm_100", *[obj for _, obj in jobs], "-o", exe, "-lcublas", "-lcudart"]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        print(proc.stderr[-3000:], file=sys.stderr)
        return 1
    with open(os.path.join(OUT, "BUILD_INFO.txt"), "w") as fh:
        fh.write(f"reference: {ref}\nflags: {' '.join(nvcc)}\n")
    print(f"built {exe}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
