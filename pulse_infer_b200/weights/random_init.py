"""Seeded random weights: either into a model folder (config.json + model.safetensors) or straight
into a model on the device.

Matrices and the embedding are N(0, 0.02); norm weights are 1 + N(0, 0.02).  Values come from a
counter-based generator (a 64-bit mix of seed, tensor number and element index; a normal deviate is
the centred sum of twelve 16-bit uniforms), written with integer tensor operations only, so the same
(seed, tensor order) gives the same bits on the CPU and on the GPU and no tensor depends on how many
were drawn before it.  The reference has no random-weights mode (its tests fill tensors by hand,
``tests/core/test_var_builder.cpp:16-24``).
"""
from __future__ import annotations

import json
import os

import torch

from ..config.registry import get_architecture
from .safetensors_io import write_safetensors

_STD = 0.02
_GOLDEN = -7046029254386353131          # 0x9E3779B97F4A7C15 as a signed 64-bit integer
_MIX1 = -4658895280553007687            # 0xBF58476D1CE4E5B9
_MIX2 = -7723592293110705685            # 0x94D049BB133111EB
_CHUNK = 1 << 24


def _lsr(x: torch.Tensor, n: int) -> torch.Tensor:
    """Logical shift right on int64 (torch's >> is arithmetic)."""
    return x if n == 0 else (x >> n) & ((1 << (64 - n)) - 1)


def _mix(z: torch.Tensor) -> torch.Tensor:
    z = (z ^ _lsr(z, 30)) * _MIX1
    z = (z ^ _lsr(z, 27)) * _MIX2
    return z ^ _lsr(z, 31)


def _wrap(v: int) -> int:
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


def normal_tensor(shape, seed: int, tensor_id: int, mean: float, std: float, dtype: torch.dtype, device) -> torch.Tensor:
    """A tensor of N(mean, std) deviates that depends on (seed, tensor_id, element index) only."""
    numel = 1
    for s in shape:
        numel *= s
    out = torch.empty(numel, dtype=dtype, device=device)
    key = _wrap((seed * 0x9E3779B97F4A7C15 + tensor_id * 0xD1342543DE82EF95 + 0x2545F4914F6CDD1D))
    for a in range(0, numel, _CHUNK):
        b = min(numel, a + _CHUNK)
        idx = torch.arange(a, b, dtype=torch.int64, device=device)
        base = _mix(idx * _GOLDEN + key)
        total = torch.zeros(b - a, dtype=torch.int64, device=device)
        for word in range(3):
            w = _mix(base + _wrap((word + 1) * _MIX1))
            for field in range(4):
                total += _lsr(w, 16 * field) & 0xFFFF
        # twelve uniforms on [0, 65535]: mean 6 * 65535, variance 12 * (65536^2 - 1) / 12
        z = (total - 6 * 65535).to(torch.float32) * (1.0 / 65536.0)
        out[a:b] = (z * std + mean).to(dtype)
    return out.reshape(tuple(shape))


def _storage_dtype(dtype: str) -> torch.dtype:
    if dtype in ("bfloat16", "bf16"):
        return torch.bfloat16
    if dtype in ("float32", "fp32", "f32"):
        return torch.float32
    raise ValueError(f"weights are written as 'bfloat16' or 'float32', not '{dtype}'")


def random_tensors(model, seed: int, dtype: torch.dtype, device, skip_optional: bool = True):
    """Yield (full name, part, relative name, tensor) for every tensor the model wants, in name order."""
    expected = model.expected_tensors()
    for tensor_id, name in enumerate(sorted(expected)):
        part, rel, spec = expected[name]
        if spec.optional and skip_optional:
            continue
        mean = 1.0 if spec.init == "ones_normal" else 0.0
        yield name, part, rel, normal_tensor(spec.shape, seed, tensor_id, mean, _STD, dtype, device)


def _spec_only_model(config):
    from ..parts.model import DecoderModel, Runtime
    arch = get_architecture(config.architecture)
    return DecoderModel(arch.build_spec(config), Runtime(torch.device("cpu"), "float32"))


def write_random_model(config, seed: int, out_dir: str, dtype: str | None = None) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with seeded random weights."""
    store = _storage_dtype(dtype or config.torch_dtype)
    os.makedirs(out_dir, exist_ok=True)
    model = _spec_only_model(config)
    tensors = {name: t for name, _, _, t in random_tensors(model, seed, store, torch.device("cpu"))}
    obj = config.to_json_dict()
    obj["torch_dtype"] = "bfloat16" if store == torch.bfloat16 else "float32"
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(obj, fh, indent=2)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors, metadata={"format": "pt", "seed": seed})
    return out_dir


def init_random_weights(model, seed: int, runtime, dtype: str = "bfloat16") -> None:
    """Fill a model on its device without going through files (large benchmark shapes)."""
    from .loader import convert_for_mode
    store = _storage_dtype(dtype)
    per_part: dict[int, tuple] = {}
    for _, part, rel, t in random_tensors(model, seed, store, runtime.device):
        per_part.setdefault(id(part), (part, {}))[1][rel] = convert_for_mode(t, runtime.mode, runtime.device)
    for _, part in model.named_parts():
        part.load(per_part.get(id(part), (part, {}))[1], runtime)
    model.finish_loading()
