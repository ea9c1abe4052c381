"""Qwen3 dense as a ``ModelSpec``: pre-norm decoder blocks of grouped-query attention (per-head RMSNorm
of queries and keys, rotary positions) and a SwiGLU feed-forward, RMSNorm everywhere, optionally tied
output head.  Every number comes from the configuration.

Reference parity: ``src/model/qwen3/model.cpp:159-323`` (per-layer tensor names and shapes),
``model.cpp:975-1021`` (embedding, final norm, lm_head), ``model.cpp:152-157`` (q width = heads * head
size, one eps for all norms), ``model.cpp:824,838`` (rotary width = head size).  The reference rotates
adjacent pairs (``src/ops/kernels/cuda/rope_kernel.cu:102-123``); ``rope_pairing='half'`` selects the
split-halves convention instead.
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..config.registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def build_qwen3_spec(config: Qwen3Config, rope_pairing: str = "adjacent") -> ModelSpec:
    pairing = config.extra.get("rope_pairing", rope_pairing) if isinstance(config.extra, dict) else rope_pairing
    norm = lambda size, prefix: PartSpec("rmsnorm", dict(size=size, eps=config.rms_norm_eps), prefix)  # noqa: E731
    layers = []
    for i in range(config.num_hidden_layers):
        base = f"model.layers.{i}."
        layers.append(LayerSpec(
            arrangement="pre_norm",
            mixer=PartSpec("attention", dict(
                hidden_size=config.hidden_size, num_heads=config.num_attention_heads,
                num_kv_heads=config.num_key_value_heads, head_dim=config.head_dim, qk_norm=True,
                norm_eps=config.rms_norm_eps, position="rotary", window=config.layer_window(i)),
                base + "self_attn."),
            feed_forward=PartSpec("swiglu", dict(hidden_size=config.hidden_size,
                                                intermediate_size=config.intermediate_size), base + "mlp."),
            mixer_norm=norm(config.hidden_size, base + "input_layernorm."),
            feed_forward_norm=norm(config.hidden_size, base + "post_attention_layernorm."),
        ))
    return ModelSpec(
        embedding=PartSpec("token_embedding", dict(vocab_size=config.vocab_size, hidden_size=config.hidden_size),
                           "model.embed_tokens."),
        layers=tuple(layers),
        order=tuple(ScheduleEntry(layer=i, cache=i) for i in range(config.num_hidden_layers)),
        final_norm=norm(config.hidden_size, "model.norm."),
        lm_head=PartSpec("lm_head", dict(vocab_size=config.vocab_size, hidden_size=config.hidden_size,
                                         tied=config.tie_word_embeddings), "lm_head."),
        positions={"rotary": PartSpec("rotary", dict(theta=config.rope_theta, rotary_dim=config.head_dim,
                                                     pairing=pairing))},
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        max_position=config.max_position_embeddings,
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_qwen3_spec, model_type="qwen3")
