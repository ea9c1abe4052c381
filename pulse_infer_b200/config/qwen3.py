"""Qwen3 dense configuration, read from the architecture's own config.json keys.

Reference parity: ``include/pulse/model/qwen3/config.hpp:12-36`` (fields) and
``src/model/qwen3/config.cpp:231-380`` (loading, generation_config.json override of EOS and the
sampling defaults), validation ``config.cpp:209-227`` (all sizes positive, heads divisible by groups).

Beyond the reference, which reads none of them, the window keys of the same config.json are honoured:
``use_sliding_window``, ``sliding_window``, ``max_window_layers`` and ``layer_types`` decide, layer by
layer, whether a layer attends to all keys or to the last ``sliding_window`` of them.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

from .base import ConfigError, KeyReader, ModelConfig, read_json_file, resolve_model_dir

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    vocab_size: int = 0
    max_position_embeddings: int = 0
    rms_norm_eps: float = 0.0
    rope_theta: float = 0.0
    tie_word_embeddings: bool = False
    torch_dtype: str = "bfloat16"
    eos_token_ids: tuple = ()
    # per-layer attention kind, already resolved from the window keys; () means every layer is full
    layer_types: tuple = ()
    sliding_window: int | None = None
    # sampling defaults from generation_config.json (config.hpp:27-29); 0 means "not given"
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 0.0
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    # ---- derived sizes -------------------------------------------------------------------------
    @property
    def q_size(self) -> int:
        """Width of the query projection; it may differ from hidden_size (model.cpp:152)."""
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim  # config.hpp:33-35

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def layer_window(self, layer: int) -> int | None:
        """Number of keys layer ``layer`` sees, or None for all of them."""
        if self.layer_types and self.layer_types[layer] == SLIDING_ATTENTION:
            return self.sliding_window
        return None

    # ---- validation ------------------------------------------------------------------------------
    def validate(self) -> "Qwen3Config":
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config value '{name}' must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim ({self.head_dim}) must be even: rotation works on pairs")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        if self.layer_types:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError(
                    f"layer_types has {len(self.layer_types)} entries for {self.num_hidden_layers} layers")
            for kind in self.layer_types:
                if kind not in (FULL_ATTENTION, SLIDING_ATTENTION):
                    raise ConfigError(f"unknown layer type '{kind}' in layer_types")
            if SLIDING_ATTENTION in self.layer_types and not (self.sliding_window and self.sliding_window > 0):
                raise ConfigError("a sliding_attention layer needs a positive sliding_window")
        return self

    # ---- JSON ------------------------------------------------------------------------------------
    @classmethod
    def from_json_dict(cls, obj: dict, source: str = "<dict>", generation: dict | None = None,
                       generation_source: str = "<dict>") -> "Qwen3Config":
        r = KeyReader(obj, source)
        archs = r.str_list("architectures")
        architecture = archs[0] if archs else "Qwen3ForCausalLM"

        num_heads = r.int("num_attention_heads")
        hidden = r.int("hidden_size")
        # the reference insists on head_dim (config.cpp:262); a file without it means hidden/heads
        head_dim = r.int("head_dim", None)
        if head_dim is None:
            if num_heads <= 0 or hidden % num_heads != 0:
                raise ConfigError(f"Missing or invalid integer key 'head_dim' in '{source}'")
            head_dim = hidden // num_heads

        if r.has("rope_theta"):
            rope_theta = r.float("rope_theta")
        elif isinstance(obj.get("rope_parameters"), dict) and "rope_theta" in obj["rope_parameters"]:
            rope_theta = KeyReader(obj["rope_parameters"], source).float("rope_theta")
        else:
            raise ConfigError(f"Missing or invalid float key 'rope_theta' in '{source}'")
        for key in ("rope_scaling", "rope_parameters"):
            scaling = obj.get(key)
            if isinstance(scaling, dict):
                kind = scaling.get("rope_type", scaling.get("type", "default"))
                if kind not in (None, "default"):
                    raise ConfigError(f"'{key}' of type '{kind}' in '{source}' is not supported")

        # What the architecture's config.json can ask for and the parts here cannot do is refused, not ignored.  (The
        # reference never reads these keys and always computes without biases and with SiLU, model.cpp:208,225,242;
        # silu_kernel.cu:78-104.)
        for key in ("attention_bias", "mlp_bias"):
            if r.bool(key, False):
                raise ConfigError(f"'{key}': true in '{source}' is not supported: the projections here have no bias")
        act = r.str("hidden_act", "silu")
        if act not in ("silu", "swish"):
            raise ConfigError(f"'hidden_act': '{act}' in '{source}' is not supported: the feed-forward here is SiLU-gated")
        dropout = r.float("attention_dropout", 0.0)
        if dropout != 0.0:
            raise ConfigError(f"'attention_dropout': {dropout} in '{source}' is not supported (inference only)")

        layers = r.int("num_hidden_layers")
        window = r.int("sliding_window", None)
        layer_types = r.str_list("layer_types")
        use_window = r.bool("use_sliding_window", False)
        if layer_types is None:
            if use_window and window is not None:
                first = r.int("max_window_layers", layers)
                layer_types = tuple(SLIDING_ATTENTION if i >= first else FULL_ATTENTION for i in range(layers))
            else:
                layer_types = ()
        if SLIDING_ATTENTION not in layer_types:
            layer_types, window = (), None

        eos = r.int_list("eos_token_id")
        temperature, top_k, top_p = 0.0, 0, 0.0
        if generation is not None:
            g = KeyReader(generation, generation_source)
            g_eos = g.int_list("eos_token_id")
            if g_eos:
                eos = g_eos  # generation_config.json wins (config.cpp:339-346)
            temperature = g.float("temperature", 0.0)
            top_k = g.int("top_k", 0)
            top_p = g.float("top_p", 0.0)

        known = {"architectures", "num_attention_heads", "hidden_size", "head_dim", "rope_theta", "num_hidden_layers",
                 "sliding_window", "layer_types", "use_sliding_window", "max_window_layers", "eos_token_id",
                 "intermediate_size", "num_key_value_heads", "vocab_size", "max_position_embeddings",
                 "rms_norm_eps", "tie_word_embeddings", "torch_dtype", "dtype", "attention_bias", "mlp_bias", "hidden_act",
                 "attention_dropout"}
        cfg = cls(
            architecture=architecture,
            hidden_size=hidden,
            intermediate_size=r.int("intermediate_size"),
            num_hidden_layers=layers,
            num_attention_heads=num_heads,
            num_key_value_heads=r.int("num_key_value_heads", num_heads),
            head_dim=head_dim,
            vocab_size=r.int("vocab_size"),
            max_position_embeddings=r.int("max_position_embeddings"),
            rms_norm_eps=r.float("rms_norm_eps"),
            rope_theta=rope_theta,
            tie_word_embeddings=r.bool("tie_word_embeddings", False),
            torch_dtype=r.str("torch_dtype", None) or r.str("dtype", "bfloat16"),
            eos_token_ids=tuple(eos),
            layer_types=tuple(layer_types),
            sliding_window=window,
            temperature=temperature, top_k=top_k, top_p=top_p,
            extra={k: v for k, v in obj.items() if k not in known},
        )
        return cfg.validate()

    @classmethod
    def load(cls, path: str) -> "Qwen3Config":
        model_dir = resolve_model_dir(path)
        config_path = os.path.join(model_dir, "config.json")
        obj = read_json_file(config_path)
        gen_path = os.path.join(model_dir, "generation_config.json")
        generation = read_json_file(gen_path) if os.path.isfile(gen_path) else None
        return cls.from_json_dict(obj, config_path, generation, gen_path)

    def to_json_dict(self) -> dict:
        obj = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": self.torch_dtype,
            "hidden_act": "silu",
        }
        if self.eos_token_ids:
            obj["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.layer_types:
            obj["use_sliding_window"] = True
            obj["sliding_window"] = self.sliding_window
            obj["layer_types"] = list(self.layer_types)
        return obj
