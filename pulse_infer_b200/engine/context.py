"""What one step is made of: the batch as segments, and the device-side metadata the kernels read.

A step is a list of segments.  A segment is the next tokens of one request: a portion of its prompt of
any length, or one decoded token.  The tokens of all segments are laid end to end (T tokens in all);
per token the kernels get its absolute position and its request's slot, per segment the offset of its
first token, its slot, its start position and its length.  All of this travels in ONE int32 buffer
(one host-to-device copy per step).

Reference parity: ``src/scheduler/continuous_batch_engine.cpp:151-164`` flattens chunks the same way
into tokens / positions / seq ids; the reference then uploads a block table with one row per *token*
(``src/model/qwen3/model.cpp:1273-1281``), whereas here tokens point at their request's row.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

import numpy as np
import torch

from .. import ops


@dataclass
class Segment:
    """Next tokens of one request.  ``want``: indices into ``tokens`` whose logits are asked for."""
    request_id: object
    tokens: list
    want: list = field(default_factory=list)
    # filled in by the step function from the cache manager
    slot: int = -1
    start: int = -1
    offset: int = -1      # row of the segment's first token in the step's flat token list


@dataclass
class CacheView:
    """What a mixer sees of the cache for one execution of its layer."""
    keys: torch.Tensor | None          # [pages, nkv, page_size, d]
    values: torch.Tensor | None
    block_table: torch.Tensor | None   # int32 [slots, max_pages]
    page_size: int
    state: torch.Tensor | None = None  # [slots, *shape] fixed-size state of this layer, if it asked for one


@dataclass
class AttentionScratch:
    max_splits: int
    acc: torch.Tensor | None
    ml: torch.Tensor | None
    split_keys: int = ops.SPLIT_KEYS
    # key splitting of the prompt kernel (short portions behind long contexts): shares per query block and their scratch
    prompt_splits: int = 1
    prompt_acc: torch.Tensor | None = None
    prompt_ml: torch.Tensor | None = None
    # single tokens on the tcgen05 decode kernel: its workspace (the key ranges above are then not used)
    decode_ws: "ops.DecodeWorkspace | None" = None


class StepContext:
    """Device metadata of one step.  Built by ``StepContext.build``; a captured decode step keeps one
    context alive and refills its buffer in place (``refill``)."""

    FIELDS = ("tokens", "positions", "token_slot", "token_seg", "seg_off", "seg_slot", "seg_start", "seg_len",
              "want_rows")

    def __init__(self, runtime, cache_manager):
        self.runtime = runtime
        self.cache_manager = cache_manager
        self.act_dtype = runtime.act_dtype
        self.device = runtime.device
        self.position_data: dict = {}
        self.segments: list = []
        self._scratch: dict = {}
        self.splits_bound: int | None = None     # fixed number of key ranges (captured steps)
        # fixed keys per range (captured steps): {(kv heads, head size): keys}; else chosen per step
        self.split_keys: dict | None = None
        self.error_count: torch.Tensor | None = None
        self.upcoming_weights = None
        self.prefetch_hints = os.environ.get("PULSE_PREFETCH", "1") != "0"
        self.prefetch_bytes = int(float(os.environ.get("PULSE_PREFETCH_MB", "4")) * (1 << 20))
        self.num_tokens = 0

    # ---- layout of the metadata buffer -------------------------------------------------------------
    @staticmethod
    def layout(num_tokens: int, num_segments: int, num_wanted: int) -> dict:
        sizes = {"tokens": num_tokens, "positions": num_tokens, "token_slot": num_tokens, "token_seg": num_tokens,
                 "seg_off": num_segments, "seg_slot": num_segments, "seg_start": num_segments,
                 "seg_len": num_segments, "want_rows": num_wanted}
        offsets, at = {}, 0
        for name in StepContext.FIELDS:
            offsets[name] = (at, sizes[name])
            at += (sizes[name] + 3) // 4 * 4          # keep every field 16-byte aligned
        offsets["_total"] = (0, max(at, 4))
        return offsets

    @staticmethod
    def pack(segments: list) -> tuple:
        """Host side: the metadata buffer of a batch, as a numpy array, plus its shape facts."""
        T = sum(len(s.tokens) for s in segments)
        R = len(segments)
        W = sum(len(s.want) for s in segments)
        lay = StepContext.layout(T, R, W)
        buf = np.zeros(lay["_total"][1], dtype=np.int32)

        def view(name):
            a, n = lay[name]
            return buf[a:a + n]
        tok, pos, tslot, tseg = view("tokens"), view("positions"), view("token_slot"), view("token_seg")
        soff, sslot, sstart, slen, want = (view("seg_off"), view("seg_slot"), view("seg_start"), view("seg_len"),
                                           view("want_rows"))
        at, w = 0, 0
        for i, s in enumerate(segments):
            n = len(s.tokens)
            s.offset = at
            tok[at:at + n] = s.tokens
            pos[at:at + n] = np.arange(s.start, s.start + n, dtype=np.int32)
            tslot[at:at + n] = s.slot
            tseg[at:at + n] = i
            soff[i], sslot[i], sstart[i], slen[i] = at, s.slot, s.start, n
            for j in s.want:
                if not (0 <= j < n):
                    raise ValueError(f"request '{s.request_id}': wanted place {j} is outside its {n} tokens")
                want[w] = at + j
                w += 1
            at += n
        return buf, lay, (T, R, W)

    @classmethod
    def build(cls, segments: list, runtime, cache_manager) -> "StepContext":
        ctx = cls(runtime, cache_manager)
        buf, lay, (T, R, W) = cls.pack(segments)
        host = torch.from_numpy(buf)
        if ctx.device.type == "cuda":
            host = host.pin_memory()
        ctx.buffer = host.to(ctx.device, non_blocking=True)
        ctx._bind(segments, lay, T, R, W)
        ctx.error_count = torch.zeros(1, dtype=torch.int32, device=ctx.device)
        return ctx

    def _bind(self, segments, lay, T, R, W) -> None:
        self.segments = segments
        self.num_tokens, self.num_segments, self.num_wanted = T, R, W
        for name in self.FIELDS:
            a, n = lay[name]
            setattr(self, name, self.buffer[a:a + n])
        lens = [len(s.tokens) for s in segments]
        self.max_seg_len = max(lens) if lens else 0
        self.has_prompt = any(n > 1 for n in lens)
        self.has_decode = any(n == 1 for n in lens)
        self.decode_starts = [s.start for s in segments if len(s.tokens) == 1]
        self.decode_pos_max = max(self.decode_starts, default=0)
        self._scratch = {}

    # ---- prefetch hints --------------------------------------------------------------------------------
    PREFETCH_MAX_TOKENS = 16      # only steps this small stream their weights once (decode); others reuse them

    def prefetch(self, weights):
        """The tensor to hand to a small kernel as "the next product's weights", or None when a hint would
        not help (large steps, float32 path, hints switched off)."""
        if weights is None or not self.prefetch_hints or self.num_tokens > self.PREFETCH_MAX_TOKENS:
            return None
        if weights.dtype != torch.bfloat16 or not weights.is_cuda:
            return None
        limit = self.prefetch_bytes // weights.element_size()
        return weights if weights.numel() <= limit else weights.reshape(-1)[:limit]

    # ---- what parts ask for --------------------------------------------------------------------------
    def cache_view(self, cache_index, layer_index) -> CacheView:
        cm = self.cache_manager
        state = cm.state.get(layer_index)
        if cache_index is None:
            return CacheView(None, None, None, cm.page_size, state)
        group = cm.group_for_cache(cache_index)
        keys, values = group.kv(cache_index)
        return CacheView(keys, values, group.device_table, cm.page_size, state)

    def _decode_workspace(self, head_dim: int):
        """One workspace per head size for all layers and steps of a runtime: they run one after the other on one stream."""
        held = getattr(self.runtime, "decode_workspaces", None)
        if held is None:
            held = {}
            try:
                self.runtime.decode_workspaces = held
            except AttributeError:
                pass
        ws = held.get(head_dim)
        if ws is None:
            ws = held[head_dim] = ops.attention_decode_workspace(head_dim, self.device)
        return ws

    def attention_scratch(self, num_heads: int, head_dim: int, window, num_kv_heads: int = 1) -> AttentionScratch:
        """Scratch of the decode attention: the workspace of the tcgen05 kernel, or for the mma.sync kernel partial
        outputs and (max, sum) pairs per key range; and the shares of the prompt kernel."""
        key = (num_heads, head_dim, window)
        sc = self._scratch.get(key)
        if sc is None:
            if not self.has_decode:
                sc = AttentionScratch(1, None, None)
            elif ops.decode_on_tcgen05(head_dim, self.cache_manager.page_size, num_heads // max(num_kv_heads, 1), self.act_dtype,
                                       self.num_segments):
                sc = AttentionScratch(1, None, None, decode_ws=self._decode_workspace(head_dim))
            else:
                split_keys = (self.split_keys or {}).get((num_kv_heads, head_dim)) or ops.choose_split_keys(
                    len(self.decode_starts), num_kv_heads, self.decode_pos_max, head_dim)
                # the widest request decides: with a window that is not always the one at the highest position
                splits = self.splits_bound or ops.attention_splits_bound(self.decode_starts, window, split_keys)
                if splits > 1:
                    rows = self.num_tokens * num_heads
                    acc = torch.empty((rows, splits, head_dim), dtype=torch.float32, device=self.device)
                    ml = torch.empty((rows, splits, 2), dtype=torch.float32, device=self.device)
                    sc = AttentionScratch(splits, acc, ml, split_keys)
                else:
                    sc = AttentionScratch(1, None, None, split_keys)
            if self.has_prompt and ops.attention_tcgen05_usable(head_dim, self.cache_manager.page_size) \
                    and self.act_dtype == torch.bfloat16:
                portions = [(s.start, len(s.tokens)) for s in self.segments if len(s.tokens) > 1]
                shares = ops.choose_prompt_splits(portions, num_heads // max(num_kv_heads, 1), num_kv_heads, window)
                if shares > 1:
                    rows = self.num_tokens * num_heads
                    sc.prompt_splits = shares
                    sc.prompt_acc = torch.empty((rows, shares, head_dim), dtype=torch.float32, device=self.device)
                    sc.prompt_ml = torch.empty((rows, shares, 2), dtype=torch.float32, device=self.device)
            self._scratch[key] = sc
        return sc
