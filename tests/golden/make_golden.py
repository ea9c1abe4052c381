"""Makes the golden outputs under tests/golden/: logits of the REFERENCE project's own CPU model code on
two tiny random models.

It compiles the reference's sources (core, layer, ops, model, runtime; no CUDA) together with
``ref_cpu_driver.cpp`` using vendored spdlog and nlohmann-json headers found in site-packages, writes
the tiny models A and B with this framework's seeded random-weights mode (stored as float32, values
rounded to bfloat16 first so that both precisions of the engine load the same numbers), runs the driver
on fixed prompts and stores tokens and logits in ``tiny_<name>.npz``.

Run from the repository root:  python tests/golden/make_golden.py --reference /path/to/pulse_infer
The reference requires ``lm_head.weight`` even for a tied model (src/model/qwen3/model.cpp:1009-1021), so
the copy of the folder that the driver reads gets one equal to the embedding.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import subprocess
import sys
import sysconfig
import tempfile

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from pulse_infer_b200.weights import SafetensorsFile, write_random_model, write_safetensors  # noqa: E402
from tiny_configs import CONFIGS, SEEDS  # noqa: E402

PROMPTS = {
    "A": [[3, 17, 200, 45, 9], list(np.random.RandomState(5).randint(0, 256, size=17))],
    "B": [[7], list(np.random.RandomState(6).randint(0, 515, size=23)), list(np.random.RandomState(7).randint(0, 515, size=40))],
}


def build_driver(reference: str, workdir: str) -> str:
    site = sysconfig.get_paths()["purelib"]
    spdlog = os.path.join(site, "flashinfer", "data", "spdlog", "include")
    json_inc = os.path.join(site, "include", "cudnn_frontend", "thirdparty")
    for need in (spdlog, json_inc):
        if not os.path.isdir(need):
            raise SystemExit(f"vendored headers not found: {need}")
    sources = []
    for pattern in ("src/core/allocastor.cpp", "src/core/logging.cpp", "src/core/safetensor.cpp", "src/core/tensor.cpp",
                    "src/core/var.cpp", "src/layer/*.cpp", "src/ops/*.cpp", "src/model/qwen3/model.cpp",
                    "src/model/qwen3/config.cpp", "src/runtime/*.cpp"):
        sources += sorted(glob.glob(os.path.join(reference, pattern)))
    exe = os.path.join(workdir, "ref_cpu_driver")
    cmd = ["g++", "-std=c++20", "-O1", "-w", "-DSPDLOG_USE_STD_FORMAT=1", f"-I{reference}/include", f"-I{spdlog}",
           f"-I{json_inc}", os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_cpu_driver.cpp"),
           *sources, "-o", exe]
    print("compiling the reference CPU model (about a minute) ...", flush=True)
    subprocess.run(cmd, check=True)
    return exe


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    out_dir = os.path.dirname(os.path.abspath(__file__))
    with tempfile.TemporaryDirectory() as work:
        exe = build_driver(args.reference, work)
        for name in ("A", "B"):
            cfg = CONFIGS[name]
            folder = os.path.join(work, f"tiny_{name}")
            write_random_model(cfg, SEEDS[name], folder, dtype="bfloat16")
            # the reference's Float32 model wants F32 tensors: same values, widened
            src = SafetensorsFile(os.path.join(folder, "model.safetensors"))
            tensors = {n: src.tensor(n).to(torch.float32) for n in src.names()}
            if "lm_head.weight" not in tensors:
                tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
            ref_folder = os.path.join(work, f"ref_{name}")
            os.makedirs(ref_folder)
            write_safetensors(os.path.join(ref_folder, "model.safetensors"), tensors)
            obj = cfg.to_json_dict()
            obj["torch_dtype"] = "float32"
            with open(os.path.join(ref_folder, "config.json"), "w") as fh:
                json.dump(obj, fh)
            arrays = {}
            for i, prompt in enumerate(PROMPTS[name]):
                raw = os.path.join(work, f"{name}_{i}.f32")
                subprocess.run([exe, ref_folder, raw, *[str(int(t)) for t in prompt]], check=True)
                logits = np.fromfile(raw, dtype="<f4").reshape(len(prompt), cfg.vocab_size)
                arrays[f"tokens_{i}"] = np.asarray(prompt, dtype=np.int32)
                arrays[f"logits_{i}"] = logits
            # a fingerprint of the weights, so that a change of the random generator is noticed
            arrays["weight_checksum"] = np.asarray(
                [float(sum(t.double().abs().sum() for t in tensors.values() if True))], dtype=np.float64)
            np.savez_compressed(os.path.join(out_dir, f"tiny_{name}.npz"), **arrays)
            print(f"wrote tiny_{name}.npz: {[a.shape for k, a in arrays.items() if k.startswith('logits')]}")


if __name__ == "__main__":
    main()
