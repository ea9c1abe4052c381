"""Putting an engine together: configuration -> model -> weights -> cache -> step function."""
from __future__ import annotations

import os

import torch

from .. import ops
from ..cache import CacheManager
from ..config.registry import get_architecture, load_config
from ..parts.model import DecoderModel, Runtime
from ..weights import init_random_weights, load_weights
from .step import ModelRunner


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("pulse_infer_b200 runs on a CUDA device (sm_100a) only; there is no CPU path. "
                           f"Asked for '{device}', torch.cuda.is_available() = {torch.cuda.is_available()}")
    return device


def build_model(config, runtime: Runtime, **spec_options) -> DecoderModel:
    arch = get_architecture(config.architecture)
    return DecoderModel(arch.build_spec(config, **spec_options), runtime)


def head_dims_of(model: DecoderModel) -> list:
    dims = set()
    for cs in model.cache_specs():
        if cs is not None and cs.head_dim % 16 == 0 and cs.head_dim <= 256:
            dims.add(cs.head_dim)
    return sorted(dims)


def page_bytes(model: DecoderModel, page_size: int, dtype: torch.dtype) -> int:
    """Bytes that one page id costs: keys and values of ``page_size`` tokens in every cache of the model."""
    item = torch.empty((), dtype=dtype).element_size()
    return sum(2 * cs.num_kv_heads * cs.head_dim * page_size * item for cs in model.cache_specs() if cs is not None)


def build_runner(model_dir: str | None = None, *, config=None, seed: int | None = None, dtype: str = "bfloat16",
                 device="cuda:0", page_size: int = 16, num_pages: int | None = None, max_tokens: int | None = None,
                 max_requests: int = 64, max_tokens_per_request: int | None = None,
                 max_tokens_per_step: int | None = None, attention_impl: str = "auto",
                 use_cuda_graphs: bool = False, kv_bytes: int | None = None, **spec_options) -> ModelRunner:
    """From a model folder (``model_dir``) or from a configuration plus a seed (random weights on the
    device) to a ready step function.  The page pool holds ``num_pages`` pages per layer group, or
    as many as fit in ``kv_bytes`` bytes, or enough for ``max_tokens`` tokens (none given: ``max_requests`` requests of the model's longest context,
    at most 2^20 tokens)."""
    device = require_cuda(device)
    runtime = Runtime(device, dtype, attention_impl)
    if model_dir is not None:
        config = load_config(model_dir)
    elif config is None:
        raise ValueError("give a model folder or a configuration")
    model = build_model(config, runtime, **spec_options)
    fast = runtime.mode == "bfloat16" and attention_impl != "simple"
    dims = head_dims_of(model)
    specs = [cs for cs in model.cache_specs() if cs is not None]
    needs_simple = not fast or any(cs.head_dim not in dims for cs in specs)
    ops.preload(dims if fast else (), simple_attention=needs_simple and bool(specs),
                float32_products=runtime.mode == "float32")
    with torch.cuda.device(device):
        if model_dir is not None:
            load_weights(model, model_dir, runtime)
        else:
            init_random_weights(model, 0 if seed is None else seed, runtime,
                                "bfloat16" if runtime.mode == "bfloat16" else "float32")
        if num_pages is None and kv_bytes is not None:
            num_pages = int(kv_bytes) // page_bytes(model, page_size, runtime.act_dtype)
            if num_pages <= 0:
                raise ValueError(f"{kv_bytes} bytes hold no page of {page_size} tokens of this model")
        if num_pages is None:
            if max_tokens is None:
                # every request slot at the model's longest context, capped at a million tokens
                max_tokens = min(max_requests * model.spec.max_position, 1 << 20)
            num_pages = (max_tokens + page_size - 1) // page_size
        per_request = max_tokens_per_request or min(model.spec.max_position, num_pages * page_size)
        cache = CacheManager(model.cache_specs(), model.state_specs(), page_size, num_pages, max_requests,
                             per_request, dtype=runtime.act_dtype, device=device)
    runner = ModelRunner(model, cache, runtime, max_tokens_per_step, use_cuda_graphs)
    runner.config = config
    return runner
