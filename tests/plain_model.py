"""A plain, slow implementation of the Qwen3 dense decoder, written from the reference engine's formulas.

Whole sequences, no cache, no batching, one function per part, numpy only.  It shares no code with
``pulse_infer_b200`` (it reads safetensors through the framework's file reader only in the tests'
helper, never in these functions).  Precision is a parameter: float64 gives the value the engine is
measured against; float32 shows what plain 32-bit arithmetic gives.

Where it comes from (paths inside the reference project):
* ``embedding``        include/pulse/ops/kernels/embedding_kernel.hpp:10-26
* ``rms_norm``         include/pulse/ops/kernels/rmsnorm_kernel.hpp:11-35
* ``linear``           include/pulse/ops/kernels/matmul_kernel.hpp:10-38 with src/layer/linear.cpp:213
* ``rope``             include/pulse/ops/kernels/rope_kernel.hpp:11-49
* ``attention``        include/pulse/ops/kernels/mha_kernel.hpp:47-87 (softmax 12-29)
* ``swiglu``           src/model/qwen3/model.cpp:416-440 with include/pulse/ops/kernels/silu_kernel.hpp:10-15
* ``decoder_layer``    src/model/qwen3/model.cpp:325-464
* ``forward``          src/model/qwen3/model.cpp:1093-1177
* samplers             src/scheduler/continuous_batch_engine.cpp:20-62, demo/qwen3_infer.cpp:229-423

It was compared once with the reference's own model code, compiled for the CPU, on tiny random
models; the outputs and the script that made them are under ``tests/golden/``.

Extensions that the reference does not have and that therefore rest on the formulas stated here:
the window (a query at position p sees keys p - window + 1 .. p), the 'half' rotary pairing, and a
layer order given as a list.
"""
from __future__ import annotations

import math

import numpy as np


# ---------------------------------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------------------------------
def embedding(table: np.ndarray, tokens) -> np.ndarray:
    """Row gather; an id outside the table leaves a row of zeros (embedding_kernel.hpp:18-20)."""
    out = np.zeros((len(tokens), table.shape[1]), dtype=table.dtype)
    for i, t in enumerate(tokens):
        if 0 <= t < table.shape[0]:
            out[i] = table[t]
    return out


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """x * (1 / sqrt(mean(x^2) + eps)) * w over the last axis (rmsnorm_kernel.hpp:20-33)."""
    mean_sq = np.mean(x * x, axis=-1, keepdims=True)
    inv = 1.0 / np.sqrt(mean_sq + x.dtype.type(eps))
    return x * inv * weight


def linear(x: np.ndarray, weight: np.ndarray) -> np.ndarray:
    """y = x W^T with W [out, in], no bias (linear.cpp:213, matmul_kernel.hpp:23-35)."""
    return x @ weight.T


def rope(x: np.ndarray, positions, theta: float, rotary_dim: int, pairing: str = "adjacent") -> np.ndarray:
    """x [T, heads, d].  angle = pos / theta^(2i / rot) for pair i (rope_kernel.hpp:28-41).
    'adjacent': pair i is elements (2i, 2i+1), as the reference rotates; 'half': (i, i + rot/2)."""
    out = x.copy()
    pairs = rotary_dim // 2
    i = np.arange(pairs, dtype=np.float64)
    div = np.power(np.float64(theta), 2.0 * i / rotary_dim)
    ang = np.asarray(positions, dtype=np.float64)[:, None] / div[None, :]       # [T, pairs]
    cos = np.cos(ang).astype(x.dtype)[:, None, :]
    sin = np.sin(ang).astype(x.dtype)[:, None, :]
    if pairing == "adjacent":
        a, b = x[..., 0:rotary_dim:2], x[..., 1:rotary_dim:2]
        out[..., 0:rotary_dim:2] = a * cos - b * sin
        out[..., 1:rotary_dim:2] = a * sin + b * cos
    elif pairing == "half":
        a, b = x[..., :pairs], x[..., pairs:rotary_dim]
        out[..., :pairs] = a * cos - b * sin
        out[..., pairs:rotary_dim] = a * sin + b * cos
    else:
        raise ValueError(pairing)
    return out


def softmax(s: np.ndarray) -> np.ndarray:
    """exp(s - max) / sum (mha_kernel.hpp:12-29)."""
    e = np.exp(s - np.max(s))
    return e / np.sum(e)


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, window: int | None = None,
              scale: float | None = None) -> np.ndarray:
    """q [T, nq, d], k and v [T, nkv, d], all positions of one sequence.  Query t sees keys 0..t
    (mha_kernel.hpp:66-72), or t - window + 1 .. t with a window.  kv head = head / (nq / nkv)
    (mha_kernel.hpp:63); score = q.k / sqrt(d) (mha_kernel.hpp:58,70); output = sum_j p_j v_j."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    scale = q.dtype.type(1.0 / math.sqrt(d)) if scale is None else q.dtype.type(scale)
    out = np.zeros_like(q)
    for h in range(nq):
        kvh = h // group
        for t in range(T):
            lo = 0 if window is None else max(0, t - window + 1)
            s = (k[lo:t + 1, kvh, :] @ q[t, h, :]) * scale
            p = softmax(s)
            out[t, h, :] = p @ v[lo:t + 1, kvh, :]
    return out


def silu(x: np.ndarray) -> np.ndarray:
    return x / (1.0 + np.exp(-x))       # silu_kernel.hpp:12-14


def swiglu(x: np.ndarray, w_gate, w_up, w_down) -> np.ndarray:
    """down(silu(gate(x)) * up(x)) (model.cpp:416-440)."""
    return linear(silu(linear(x, w_gate)) * linear(x, w_up), w_down)


# ---------------------------------------------------------------------------------------------------
# a layer and the whole model
# ---------------------------------------------------------------------------------------------------
def layer_keys_values(x_normed, w, prefix, cfg, positions, pairing):
    """Projected, normalised and rotated keys, and raw values, of one layer (model.cpp:343-404)."""
    nkv, d = cfg["num_key_value_heads"], cfg["head_dim"]
    T = x_normed.shape[0]
    k = linear(x_normed, w[prefix + "self_attn.k_proj.weight"]).reshape(T, nkv, d)
    v = linear(x_normed, w[prefix + "self_attn.v_proj.weight"]).reshape(T, nkv, d)
    k = rms_norm(k, w[prefix + "self_attn.k_norm.weight"], cfg["rms_norm_eps"])
    k = rope(k, positions, cfg["rope_theta"], d, pairing)
    return k, v


def decoder_layer(h, w, prefix, cfg, positions, window=None, pairing="adjacent", shared_kv=None):
    """One pre-norm block (model.cpp:325-464).  Returns the new hidden state and this layer's (k, v).
    ``shared_kv``: use these keys and values instead of projecting own ones."""
    nq, d, eps = cfg["num_attention_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    T = h.shape[0]
    x = rms_norm(h, w[prefix + "input_layernorm.weight"], eps)                       # model.cpp:335
    q = linear(x, w[prefix + "self_attn.q_proj.weight"]).reshape(T, nq, d)           # model.cpp:340
    q = rms_norm(q, w[prefix + "self_attn.q_norm.weight"], eps)                      # model.cpp:359
    q = rope(q, positions, cfg["rope_theta"], d, pairing)                            # model.cpp:363-367
    k, v = shared_kv if shared_kv is not None else layer_keys_values(x, w, prefix, cfg, positions, pairing)
    a = attention(q, k, v, window).reshape(T, nq * d)                                # model.cpp:406-413
    h = h + linear(a, w[prefix + "self_attn.o_proj.weight"])                         # model.cpp:419-427
    x = rms_norm(h, w[prefix + "post_attention_layernorm.weight"], eps)              # model.cpp:429
    h = h + swiglu(x, w[prefix + "mlp.gate_proj.weight"], w[prefix + "mlp.up_proj.weight"],
                   w[prefix + "mlp.down_proj.weight"])                               # model.cpp:434-461
    return h, (k, v)


def layer_windows(cfg) -> list:
    """Per layer: the window, or None.  From config.json: ``layer_types`` if present, else layers with
    index >= max_window_layers when use_sliding_window is true."""
    L = cfg["num_hidden_layers"]
    window = cfg.get("sliding_window")
    types = cfg.get("layer_types")
    if types is None and cfg.get("use_sliding_window") and window:
        first = cfg.get("max_window_layers", L)
        types = ["sliding_attention" if i >= first else "full_attention" for i in range(L)]
    if not types:
        return [None] * L
    return [window if t == "sliding_attention" else None for t in types]


def forward(cfg: dict, w: dict, tokens, dtype=np.float64, pairing: str = "adjacent", order=None) -> np.ndarray:
    """Logits [T, vocab] at every position of one sequence (model.cpp:1093-1177, applied to each token
    with all earlier ones as context).  ``cfg`` holds config.json's keys; ``w`` the tensors by name.
    ``order``: list of (layer, cache) pairs; a layer whose cache was filled by an earlier entry and that
    has no key projection of its own reads that entry's keys and values."""
    w = {k: np.asarray(v, dtype=dtype) for k, v in w.items()}
    T = len(tokens)
    positions = np.arange(T)
    windows = layer_windows(cfg)
    h = embedding(w["model.embed_tokens.weight"], tokens)                             # model.cpp:1108
    if order is None:
        order = [(i, i) for i in range(cfg["num_hidden_layers"])]
    caches = {}
    for layer, cache in order:
        prefix = f"model.layers.{layer}."
        reads_only = (prefix + "self_attn.k_proj.weight") not in w
        shared = caches[cache] if reads_only else None
        h, kv = decoder_layer(h, w, prefix, cfg, positions, windows[layer], pairing, shared)
        if not reads_only:
            caches[cache] = kv
    x = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])                      # model.cpp:1124
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]   # model.cpp:1129,1152
    return linear(x, head)


# ---------------------------------------------------------------------------------------------------
# samplers
# ---------------------------------------------------------------------------------------------------
def greedy(logits: np.ndarray) -> int:
    """First maximum wins (continuous_batch_engine.cpp:28-36: strict '>')."""
    best = 0
    for i in range(1, len(logits)):
        if logits[i] > logits[best]:
            best = i
    return best


def kept_set(logits: np.ndarray, temperature: float, top_k: int, top_p: float):
    """Indices that temperature / top-k / top-p sampling may return, with their weights
    (demo/qwen3_infer.cpp:336-409): the k largest logits (earlier index stays on equal logits), weights
    exp((logit - max) / temperature), then the shortest prefix in descending order whose cumulative
    share reaches top_p.  Logits equal to the last kept one are kept as well."""
    n = len(logits)
    order = sorted(range(n), key=lambda i: (-logits[i], i))
    if 0 < top_k < n:
        order = order[:top_k]
    mx = logits[order[0]]
    weights = np.array([math.exp((logits[i] - mx) / temperature) for i in order])
    if 0.0 < top_p < 1.0:
        total = weights.sum()
        cum, keep = 0.0, 0
        for j, wgt in enumerate(weights):
            cum += wgt / total
            keep = j + 1
            if cum >= top_p:
                break
        last = logits[order[keep - 1]]
        while keep < len(order) and logits[order[keep]] == last:
            keep += 1
        order, weights = order[:keep], weights[:keep]
    return order, weights


def splitmix64(z: int) -> int:
    mask = (1 << 64) - 1
    z = (z + 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    return z ^ (z >> 31)


def uniform_from(seed: int, counter: int) -> float:
    """The engine's counter-based draw in [0, 1): 24 bits of a 64-bit mix of (seed, counter)."""
    mask = (1 << 64) - 1
    r = splitmix64(splitmix64(seed & mask) ^ ((counter * 0xD1342543DE82EF95) & mask))
    return (r >> 40) / 16777216.0


def sample(logits: np.ndarray, temperature: float, top_k: int, top_p: float, seed: int, counter: int) -> int:
    """Inverse-CDF draw over the kept set, walked in index order, with u = uniform_from(seed, counter)."""
    if temperature <= 0.0:
        return greedy(logits)
    order, weights = kept_set(logits, temperature, top_k, top_p)
    pairs = sorted(zip(order, weights))
    target = uniform_from(seed, counter) * sum(wgt for _, wgt in pairs)
    cum = 0.0
    for idx, wgt in pairs:
        cum += wgt
        if cum >= target:
            return idx
    return pairs[-1][0]
