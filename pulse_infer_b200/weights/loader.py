"""Loading a model's tensors from the safetensors files of its folder, by name.

The model says which tensors it wants (name, shape); the files say which they hold.  Every mismatch -
missing names, names nobody asked for, wrong shapes - is collected and reported in ONE error.

dtype policy: a tensor stored in bfloat16 stays bfloat16 in 'bfloat16' mode; a tensor stored in
32-bit stays 32-bit (products with such a matrix then run in 32-bit); in 'float32' mode everything
is converted to float32.  Float16 is converted to the mode's dtype.  Integer tensors become int32.

Reference parity: ``src/core/var.cpp:109-116,197-207`` (every file of the folder, duplicate names are
an error), ``var.cpp:61-75,161-164`` (shape / missing errors, reported one at a time there),
``src/model/qwen3/model.cpp:159-323,975-1021`` (the names).  The reference refuses a dtype other
than the model's; conversion here lets the float32 path load bfloat16 files.
"""
from __future__ import annotations

import os

import torch

from .safetensors_io import SafetensorsFile, list_weight_files


class WeightError(ValueError):
    """The files do not match the model; the message lists every problem."""

    def __init__(self, missing, unexpected, wrong_shape, duplicates=(), where=""):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.duplicates = sorted(duplicates)
        lines = [f"weights in '{where}' do not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " +
                         "; ".join(f"{n}: expected {list(e)}, got {list(g)}" for n, e, g in self.wrong_shape))
        if self.duplicates:
            lines.append(f"  tensors that appear in two files ({len(self.duplicates)}): " + ", ".join(self.duplicates))
        super().__init__("\n".join(lines))


def convert_for_mode(t: torch.Tensor, mode: str, device) -> torch.Tensor:
    """Move a file tensor to the device in the dtype the policy above gives it."""
    if t.dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool):
        return t.to(device=device, dtype=torch.int32)
    t = t.to(device)
    if mode == "float32":
        return t.to(torch.float32)
    if t.dtype == torch.bfloat16 or t.dtype == torch.float32:
        return t
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    return t.to(torch.bfloat16)   # float16


def index_folder(model_dir: str):
    files = list_weight_files(model_dir)
    if not files:
        raise FileNotFoundError(f"no .safetensors file in '{model_dir}'")
    opened, where, duplicates = [], {}, []
    for path in files:
        f = SafetensorsFile(path)
        opened.append(f)
        for name in f.names():
            if name in where:
                duplicates.append(name)    # var.cpp:197-203 "already exists"
            else:
                where[name] = f
    return opened, where, duplicates


def load_weights(model, model_dir: str, runtime) -> None:
    """Fill every part of ``model`` from the folder; raises WeightError listing all mismatches."""
    opened, where, duplicates = index_folder(model_dir)
    expected = model.expected_tensors()
    missing = [n for n, (_, _, spec) in expected.items() if n not in where and not spec.optional]
    unexpected = [n for n in where if n not in expected]
    wrong = []
    for name, (_, _, spec) in expected.items():
        if name in where:
            got = where[name].entries[name].shape
            if tuple(got) != tuple(spec.shape):
                wrong.append((name, tuple(spec.shape), tuple(got)))
    if missing or unexpected or wrong or duplicates:
        raise WeightError(missing, unexpected, wrong, duplicates, where=model_dir)

    by_part: dict[int, tuple] = {}
    for name, (part, rel, _) in expected.items():
        if name in where:
            by_part.setdefault(id(part), (part, {}))[1][rel] = name
    for _, part in model.named_parts():
        _, names = by_part.get(id(part), (part, {}))
        tensors = {rel: convert_for_mode(where[full].tensor(full), runtime.mode, runtime.device)
                   for rel, full in names.items()}
        part.load(tensors, runtime)
    model.finish_loading()
    for f in opened:
        f.close()
