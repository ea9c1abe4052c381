"""Python side of the hand-written sm_100a kernels: loads the libraries built from ``csrc/`` and
wraps each entry point in a function that checks its tensors and launches on torch's current stream.

There is no fallback: if a library cannot be built or loaded, or the tensors are not on a CUDA
device, the call raises.  Matrix products in bfloat16 go to cuBLAS through ``torch.mm`` (the
reference engine uses cuBLAS for every product, src/ops/kernels/cuda/matmul_kernel.cu:132-154);
the float32 path uses the repository's own fp32-FMA kernel so that no reduced-precision mode can
take part.
"""
from __future__ import annotations

import ctypes
import math
import os
from ctypes import c_float, c_int, c_void_p

import torch

from ..csrc import build

F32, BF16 = 0, 1
SPLIT_KEYS = 256          # keys per range of the split decode attention (a multiple of the 64-key tile)
_LIBS: dict = {}
LAUNCHES = 0              # kernels of this repository launched through these wrappers (graph replays add theirs)


def count_launches(n: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n


class KernelError(RuntimeError):
    pass


def _lib(name: str, head_dim: int | None = None) -> ctypes.CDLL:
    key = (name, head_dim)
    lib = _LIBS.get(key)
    if lib is None:
        path = build.library_path(name, head_dim)
        try:
            lib = ctypes.CDLL(path)
        except OSError as exc:
            raise KernelError(f"cannot load kernel library {path}: {exc}") from exc
        lib.pi_last_error.restype = ctypes.c_char_p
        _LIBS[key] = lib
    return lib


def _check(lib, rc: int, what: str, launches: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += launches
    if rc != 0:
        raise KernelError(f"{what} failed (code {rc}): {lib.pi_last_error().decode(errors='replace')}")


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}")


def _p(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _prefetch_args(t: torch.Tensor | None):
    """(pointer, bytes) of weights that small kernels may ask the L2 to fetch ahead of the next product."""
    if t is None:
        return c_void_p(0), ctypes.c_ulonglong(0)
    return c_void_p(t.data_ptr()), ctypes.c_ulonglong(t.numel() * t.element_size())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on a CUDA device only; got a tensor on " + str(t.device))


def _need_contig(**tensors) -> None:
    for name, t in tensors.items():
        if t is not None and not t.is_contiguous():
            raise KernelError(f"tensor '{name}' must be contiguous")


def preload(head_dims=(), simple_attention: bool = False, float32_products: bool = False) -> None:
    """Build and load what a model needs, so that the first step does not pay for it.  Everything else
    (sampling, for instance) is built when it is first called."""
    _lib("elementwise")
    if float32_products:
        _lib("gemm_f32")
    else:
        _lib("gemm_small_m")
        _lib("gemm_tcgen05")
    if simple_attention:
        _lib("attention_simple")
    for d in head_dims:
        _lib("attention_mma", d)
        if not float32_products and d in (64, 128) and os.environ.get("PULSE_TCGEN05_ATTENTION", "1") != "0":
            _lib("attention_tcgen05", d)


# ---- embedding --------------------------------------------------------------------------------------
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """tokens int32 [T], table [V, H] (bf16 or fp32) -> fp32 residual [T, H]."""
    _need_cuda(tokens, table)
    _need_contig(tokens=tokens, table=table)
    if tokens.dtype != torch.int32:
        raise KernelError("token ids must be int32")
    T, (V, H) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    lib = _lib("elementwise")
    _check(lib, lib.pi_embed(_p(tokens), _p(table), c_int(_code(table.dtype)), _p(out), c_int(T), c_int(H), c_int(V),
                             _stream()), "embedding")
    return out


# ---- fused residual add + RMSNorm ---------------------------------------------------------------------
def add_rmsnorm(hidden: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: torch.Tensor | None = None, out: torch.Tensor | None = None,
                prefetch: torch.Tensor | None = None) -> torch.Tensor:
    """hidden fp32 [T, H].  Without ``rows``: hidden += delta in place and the norm of every row is
    returned.  With ``rows`` (int32 [n]): the norm of hidden[rows] + delta[rows]; hidden is not changed."""
    _need_cuda(hidden, delta, weight, rows)
    _need_contig(hidden=hidden, delta=delta, weight=weight, rows=rows)
    if hidden.dtype != torch.float32:
        raise KernelError("the residual stream must be float32")
    T, H = hidden.shape
    if delta is not None and (delta.shape != hidden.shape or delta.dtype != out_dtype):
        raise KernelError(f"delta must be {tuple(hidden.shape)} of {out_dtype}, got {tuple(delta.shape)} of {delta.dtype}")
    if weight.shape != (H,):
        raise KernelError(f"norm weight must have shape ({H},), got {tuple(weight.shape)}")
    n = T if rows is None else rows.numel()
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("rows must be int32")
    if out is None:
        out = torch.empty((n, H), dtype=out_dtype, device=hidden.device)
    lib = _lib("elementwise")
    _check(lib, lib.pi_add_rmsnorm(_p(hidden), _p(delta), _p(weight), c_int(_code(weight.dtype)), _p(out),
                                   c_int(_code(out_dtype)), _p(rows), c_int(n), c_int(H), c_float(eps),
                                   *_prefetch_args(prefetch), _stream()), "add_rmsnorm")
    return out


# ---- SiLU(gate) * up ------------------------------------------------------------------------------------
def silu_mul(gate_up: torch.Tensor, out: torch.Tensor | None = None, prefetch: torch.Tensor | None = None,
             blocked: bool = False) -> torch.Tensor:
    """gate_up [T, 2*I] -> [T, I].  Columns are [all gate | all up], or with ``blocked`` blocks of 16:
    8 gate features followed by their 8 up features."""
    _need_cuda(gate_up)
    _need_contig(gate_up=gate_up)
    T, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("gate_up must have an even number of columns")
    inter = two_i // 2
    if out is None:
        out = torch.empty((T, inter), dtype=gate_up.dtype, device=gate_up.device)
    lib = _lib("elementwise")
    _check(lib, lib.pi_silu_mul(_p(gate_up), _p(out), c_int(_code(gate_up.dtype)), c_int(T), c_int(inter),
                                c_int(1 if blocked else 0), *_prefetch_args(prefetch), _stream()), "silu_mul")
    return out


# ---- rotation tables --------------------------------------------------------------------------------------
def rope_table(positions: torch.Tensor, divisors: torch.Tensor):
    """positions int32 [T], divisors float64 [pairs] (theta^(2i/rot)) -> cos, sin fp32 [T, pairs]."""
    _need_cuda(positions, divisors)
    _need_contig(positions=positions, divisors=divisors)
    if positions.dtype != torch.int32 or divisors.dtype != torch.float64:
        raise KernelError("positions must be int32 and divisors float64")
    T, pairs = positions.numel(), divisors.numel()
    cos = torch.empty((T, pairs), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    lib = _lib("elementwise")
    _check(lib, lib.pi_rope_table(_p(positions), _p(divisors), _p(cos), _p(sin), c_int(T), c_int(pairs), _stream()),
           "rope_table")
    return cos, sin


# ---- fused per-head norm + rotation + paged key/value write ---------------------------------------------
def qk_norm_rope_write(qkv: torch.Tensor, q_weight, k_weight, eps: float, cos, sin, adjacent_pairs: bool,
                       kcache, vcache, block_table, token_slot: torch.Tensor, positions: torch.Tensor,
                       page_size: int, nq: int, nkv: int, head_dim: int, error_count: torch.Tensor,
                       prefetch: torch.Tensor | None = None) -> None:
    """qkv [T, (nq + 2*nkv) * d]: query heads are normalised and rotated in place; key heads are
    normalised, rotated and written to ``kcache``; value heads are copied to ``vcache`` (both
    [pages, nkv, page_size, d]).  ``q_weight``/``k_weight`` None: no per-head norm.  ``cos``/``sin``
    None: no rotation.  ``nkv`` = 0 for a layer that only reads another layer's cache."""
    _need_cuda(qkv, q_weight, k_weight, cos, sin, kcache, vcache, block_table, token_slot, positions, error_count)
    _need_contig(qkv=qkv, kcache=kcache, vcache=vcache, block_table=block_table, cos=cos, sin=sin)
    T, width = qkv.shape
    if width != (nq + 2 * nkv) * head_dim:
        raise KernelError(f"qkv has {width} columns, expected (nq + 2 nkv) * d = {(nq + 2 * nkv) * head_dim}")
    has_norm = q_weight is not None
    if has_norm and (q_weight.shape != (head_dim,) or (nkv and k_weight.shape != (head_dim,))):
        raise KernelError("per-head norm weights must have shape (head_dim,)")
    rot_pairs = 0 if cos is None else cos.shape[1]
    if cos is not None and (cos.shape != (T, rot_pairs) or sin.shape != cos.shape or cos.dtype != torch.float32):
        raise KernelError("rotation tables must be float32 [T, pairs]")
    if nkv:
        if kcache.dtype != qkv.dtype or vcache.dtype != qkv.dtype or kcache.shape != vcache.shape:
            raise KernelError("key and value pages must match the activation dtype and each other")
        if kcache.shape[1:] != (nkv, page_size, head_dim):
            raise KernelError(f"pages must be [n, {nkv}, {page_size}, {head_dim}], got {tuple(kcache.shape)}")
    wdtype = q_weight.dtype if has_norm else torch.float32
    lib = _lib("elementwise")
    _check(lib, lib.pi_qk_norm_rope_write(
        _p(qkv), c_int(width), c_int(_code(qkv.dtype)), _p(q_weight), _p(k_weight if nkv else q_weight),
        c_int(_code(wdtype)), c_float(eps), c_int(1 if has_norm else 0), _p(cos), _p(sin), c_int(rot_pairs),
        c_int(1 if adjacent_pairs else 0), _p(kcache), _p(vcache), _p(block_table),
        c_int(block_table.shape[1] if block_table is not None else 0), _p(token_slot), _p(positions),
        c_int(page_size), c_int(nq), c_int(nkv), c_int(head_dim), c_int(T), _p(error_count),
        *_prefetch_args(prefetch), _stream()), "qk_norm_rope_write")


# ---- attention ------------------------------------------------------------------------------------------------
def attention_simple(q: torch.Tensor, q_stride: int, kcache, vcache, block_table, token_slot, positions,
                     num_tokens: int, nq: int, nkv: int, head_dim: int, page_size: int, window: int | None,
                     scale: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """Plain paged attention (float32 or bfloat16).  ``q`` holds the query heads of token t at
    element offset t * q_stride.  Returns [T, nq * d]."""
    _need_cuda(q, kcache, vcache, block_table, token_slot, positions)
    _need_contig(kcache=kcache, vcache=vcache, block_table=block_table)
    if out is None:
        out = torch.empty((num_tokens, nq * head_dim), dtype=q.dtype, device=q.device)
    lib = _lib("attention_simple")
    _check(lib, lib.pi_attention_simple(
        _p(q), c_int(q_stride), _p(kcache), _p(vcache), c_int(_code(q.dtype)), _p(block_table),
        c_int(block_table.shape[1]), _p(token_slot), _p(positions), _p(out), c_int(num_tokens), c_int(nq), c_int(nkv),
        c_int(head_dim), c_int(page_size), c_int(window or 0), c_float(scale), _stream()), "attention_simple")
    return out


_SM_COUNT: int | None = None


def sm_count() -> int:
    """Streaming multiprocessors of the current CUDA device (148 on a B200); launch shapes are sized from it."""
    global _SM_COUNT
    if _SM_COUNT is None:
        _SM_COUNT = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count \
            if torch.cuda.is_available() else 148
    return _SM_COUNT


def choose_split_keys(num_decode: int, num_kv_heads: int, max_pos: int, head_dim: int | None = None) -> int:
    """Keys per range of the split decode attention of the mma.sync kernel (from measurements on B200): it wants
    several CTAs per SM, so short ranges for a small batch and long ones (less start-up cost per byte) for a large one.
    (The tcgen05 decode kernel cuts the keys of a step into equal spans by itself.)"""
    forced = os.environ.get("PULSE_SPLIT_KEYS")
    if forced:
        return int(forced)
    tiles = (max_pos + 256) // 256
    ctas = num_decode * max(num_kv_heads, 1) * tiles
    sms = sm_count()
    if ctas > 48 * sms:
        return 2048
    if ctas > 16 * sms:
        return 1024
    if ctas > 6 * sms:
        return 512
    return SPLIT_KEYS


def attention_num_splits(pos: int, window: int | None, split_keys: int = SPLIT_KEYS) -> int:
    """Key ranges a decoding request whose newest token sits at ``pos`` is cut into (depends on its own
    length and the window only, never on the batch)."""
    w = window or 0
    lo = max(0, pos - w + 1) if w > 0 else 0
    lo_al = (lo // 64) * 64
    return (pos + 1 - lo_al + split_keys - 1) // split_keys


def attention_splits_bound(positions, window: int | None, split_keys: int = SPLIT_KEYS) -> int:
    """The width the scratch of the split decode attention needs for requests whose newest tokens sit at
    ``positions``: the largest count among them.  Without a window that is the count at the highest position; with
    one it is not (the window's first key is rounded down to a multiple of 64, so the count swings by one with
    pos % 64) - every position is looked at."""
    if not positions:
        return 1
    if not window:
        return attention_num_splits(max(positions), None, split_keys)
    return max(attention_num_splits(p, window, split_keys) for p in set(positions))


TCGEN05_ATTENTION = os.environ.get("PULSE_TCGEN05_ATTENTION", "1") != "0"


TCGEN05_DECODE = os.environ.get("PULSE_TCGEN05_DECODE", "1") != "0"     # single tokens on the persistent tcgen05 kernel


def attention_decode_tcgen05_usable(head_dim: int, page_size: int, group: int) -> bool:
    return TCGEN05_ATTENTION and head_dim in (64, 128) and page_size in (8, 16, 32, 64) and 1 <= group <= 16


DECODE_SPAN_MIN = int(os.environ.get("PULSE_DECODE_SPAN_MIN", "2"))     # shortest span of a CTA of the decode kernel, in units (key tiles + costs)
DECODE_PAIR_COST = int(os.environ.get("PULSE_DECODE_PAIR_COST", "2"))    # units a (request, kv head) pair counts for beside its key tiles


class DecodeWorkspace:
    """What the tcgen05 decode attention kernel keeps between its CTAs: the partial results of (request, kv head) pairs
    whose keys were cut between CTAs, two slots of 16 heads per CTA, and a counter per CTA that says how many pieces of
    the pair that begins there have been delivered.  Its size does not depend on the batch or on the context.  The
    counters are zero between launches; launches that share a workspace must not overlap (one stream)."""

    def __init__(self, head_dim: int, device):
        self.ctas = sm_count()
        self.head_dim = head_dim
        self.acc = torch.empty(self.ctas * 2 * 16 * head_dim, dtype=torch.float32, device=device)
        self.ml = torch.empty(self.ctas * 2 * 16 * 2, dtype=torch.float32, device=device)
        self.count = torch.zeros(self.ctas, dtype=torch.int32, device=device)


def attention_decode_workspace(head_dim: int, device) -> DecodeWorkspace:
    return DecodeWorkspace(head_dim, device)


def attention_tcgen05_usable(head_dim: int, page_size: int) -> bool:
    return TCGEN05_ATTENTION and head_dim in (64, 128) and page_size in (8, 16, 32, 64, 128)


def choose_prompt_splits(portions, group: int, num_kv_heads: int, window: int | None) -> int:
    """How many CTAs share the key tiles of a query block in the prompt attention kernel.  ``portions``: (start, length)
    of the step's segments of more than one token.  A query block is 256 rows (tokens x heads of a group); a step with
    few of them behind a long context - a short portion of a long prompt - would leave most SMs idle while a few walk
    thousands of keys, so their keys are cut into shares.  1 when the blocks fill the GPU or the contexts are short."""
    forced = os.environ.get("PULSE_PROMPT_SPLITS")
    if forced:
        return max(1, int(forced))
    if not portions:
        return 1
    ctas = sum((n * group + 255) // 256 for _, n in portions) * max(num_kv_heads, 1)
    keys = max((min(start + n, (window or (start + n)) + n)) for start, n in portions)
    tiles = (keys + 127) // 128
    sms = sm_count()
    if ctas * 2 > sms or tiles < 8:
        return 1
    return max(1, min(sms // ctas, tiles // 4, 16))


def attention_tcgen05(q: torch.Tensor, q_stride: int, kcache, vcache, block_table, seg_off, seg_slot, seg_start, seg_len,
                      num_tokens: int, num_segments: int, max_seg_len: int, nq: int, nkv: int, head_dim: int,
                      page_size: int, window: int | None, scale: float, out: torch.Tensor, splits: int = 1,
                      part_acc: torch.Tensor | None = None, part_ml: torch.Tensor | None = None,
                      token_seg: torch.Tensor | None = None) -> torch.Tensor:
    """Prompt portions (segments of more than one token) on tcgen05 tensor cores; rows of single-token
    segments in ``out`` are left untouched (see csrc/attention_tcgen05.cu).  ``splits`` > 1: that many CTAs share the
    key tiles of every query block and a second kernel combines their shares; needs float32 scratch ``part_acc``
    [tokens * nq * splits * head_dim], ``part_ml`` [tokens * nq * splits * 2] and ``token_seg`` (int32 [tokens])."""
    _need_cuda(q, kcache, vcache, block_table, seg_off, seg_slot, seg_start, seg_len, out, part_acc, part_ml, token_seg)
    _need_contig(kcache=kcache, vcache=vcache, block_table=block_table)
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16:
        raise KernelError("the tcgen05 attention kernel takes bfloat16 only")
    if splits > 1:
        need = num_tokens * nq * splits
        if (part_acc is None or part_ml is None or token_seg is None or part_acc.numel() < need * head_dim
                or part_ml.numel() < need * 2 or part_acc.dtype != torch.float32 or part_ml.dtype != torch.float32):
            raise KernelError("scratch for the split prompt attention is missing or too small")
    lib = _lib("attention_tcgen05", head_dim)
    _check(lib, lib.pi_attention_tcgen05(
        _p(q), c_int(q_stride), _p(kcache), _p(vcache), ctypes.c_longlong(kcache.shape[0]), _p(block_table),
        c_int(block_table.shape[1]), _p(seg_off), _p(seg_slot), _p(seg_start), _p(seg_len), _p(out), c_int(num_segments),
        c_int(max_seg_len), c_int(nq), c_int(nkv), c_int(page_size), c_int(window or 0), c_float(scale), c_int(splits),
        _p(part_acc), _p(part_ml), _p(token_seg), c_int(num_tokens), _stream()),
        "attention_tcgen05", launches=2 if splits > 1 else 1)
    return out


def attention_tcgen05_loaded_status() -> int:
    """The first non-zero status among the tcgen05 attention libraries that this process has loaded."""
    for (name, head_dim) in list(_LIBS):
        if name == "attention_tcgen05":
            status = attention_tcgen05_status(head_dim)
            if status:
                return status
    return 0


def attention_tcgen05_status(head_dim: int) -> int:
    lib = _lib("attention_tcgen05", head_dim)
    status = ctypes.c_uint(0)
    _check(lib, lib.pi_attention_tcgen05_status(ctypes.byref(status)), "attention_tcgen05_status", launches=0)
    return int(status.value)


def attention_mma(q: torch.Tensor, q_stride: int, kcache, vcache, block_table, seg_off, seg_slot, seg_start, seg_len,
                  token_seg, num_tokens: int, num_segments: int, max_seg_len: int, has_prompt: bool, has_decode: bool,
                  max_splits: int, part_acc, part_ml, nq: int, nkv: int, head_dim: int, page_size: int,
                  window: int | None, scale: float, out: torch.Tensor | None = None,
                  split_keys: int = SPLIT_KEYS, prefetch: torch.Tensor | None = None,
                  prompt_on_tcgen05: bool = True, decode_on_tcgen05: bool | None = None, prompt_splits: int = 1,
                  prompt_acc: torch.Tensor | None = None, prompt_ml: torch.Tensor | None = None,
                  decode_ws: DecodeWorkspace | None = None) -> torch.Tensor:
    """Tensor-core paged attention for bfloat16 over request segments.  Prompt portions (segments of several tokens)
    and single tokens are separate kernels: for head sizes 64 / 128 the tcgen05 kernels of csrc/attention_tcgen05.cu
    (``prompt_on_tcgen05`` / ``decode_on_tcgen05``; the decode kernel cuts the keys of the step into equal spans by
    itself and wants ``decode_ws``, made here when missing), otherwise - and for sizes those do not take - the
    mma.sync kernels of csrc/attention_mma.cu with key ranges of ``split_keys`` keys, ``max_splits`` of them at most,
    in ``part_acc`` / ``part_ml``.  ``prompt_splits`` / ``prompt_acc`` / ``prompt_ml``: key splitting of the tcgen05
    prompt kernel (see ``attention_tcgen05``)."""
    _need_cuda(q, kcache, vcache, block_table, seg_off, seg_slot, seg_start, seg_len, token_seg, part_acc, part_ml)
    _need_contig(kcache=kcache, vcache=vcache, block_table=block_table)
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16:
        raise KernelError("the tensor-core attention kernel takes bfloat16 only")
    if out is None:
        out = torch.empty((num_tokens, nq * head_dim), dtype=q.dtype, device=q.device)
    if decode_on_tcgen05 is None:
        decode_on_tcgen05 = TCGEN05_DECODE
    if has_prompt and prompt_on_tcgen05 and attention_tcgen05_usable(head_dim, page_size):
        # prompt portions on the tcgen05 kernel, single tokens (if any) on the decode kernel below
        attention_tcgen05(q, q_stride, kcache, vcache, block_table, seg_off, seg_slot, seg_start, seg_len, num_tokens,
                          num_segments, max_seg_len, nq, nkv, head_dim, page_size, window, scale, out,
                          splits=prompt_splits, part_acc=prompt_acc, part_ml=prompt_ml, token_seg=token_seg)
        if not has_decode:
            return out
        has_prompt = False
    decode_mode = 1 if has_decode else 0
    if has_decode and decode_on_tcgen05 and attention_decode_tcgen05_usable(head_dim, page_size, nq // nkv):
        # single tokens on the persistent tcgen05 kernel, which also adds up the pieces of requests it has cut
        ws = _decode_workspace(decode_ws, head_dim, q.device)
        tlib = _lib("attention_tcgen05", head_dim)
        _check(tlib, tlib.pi_attention_decode_tcgen05(
            _p(q), c_int(q_stride), _p(kcache), _p(vcache), ctypes.c_longlong(kcache.shape[0]), _p(block_table),
            c_int(block_table.shape[1]), _p(seg_off), _p(seg_slot), _p(seg_start), _p(seg_len), _p(out), _p(ws.acc),
            _p(ws.ml), _p(ws.count), c_int(ws.ctas), c_int(DECODE_SPAN_MIN), c_int(DECODE_PAIR_COST), c_int(num_segments), c_int(nq), c_int(nkv),
            c_int(page_size), c_int(window or 0), c_float(scale), _stream()), "attention_decode_tcgen05")
        if not has_prompt:
            return out
        decode_mode = 0
    if decode_mode and max_splits > 1:
        need = num_tokens * nq * max_splits
        if part_acc is None or part_acc.numel() < need * head_dim or part_ml.numel() < need * 2:
            raise KernelError("scratch for the split decode attention is missing or too small")
    lib = _lib("attention_mma", head_dim)
    _check(lib, lib.pi_attention_mma_prefetch(
        _p(q), c_int(q_stride), _p(kcache), _p(vcache), _p(block_table), c_int(block_table.shape[1]), _p(seg_off),
        _p(seg_slot), _p(seg_start), _p(seg_len), _p(token_seg), _p(out), _p(part_acc), _p(part_ml), c_int(max_splits),
        c_int(split_keys), c_int(num_tokens), c_int(num_segments), c_int(max_seg_len), c_int(1 if has_prompt else 0),
        c_int(decode_mode), c_int(nq), c_int(nkv), c_int(page_size), c_int(window or 0), c_float(scale),
        *_prefetch_args(prefetch), _stream()), "attention_mma",
        launches=int(has_prompt) + int(decode_mode == 1) + int(decode_mode > 0 and max_splits > 1))
    return out


FUSE_ROPE = os.environ.get("PULSE_FUSE_ROPE", "1") != "0"     # steps of single tokens: norm, rotation and page write inside the attention kernel


def _decode_workspace(ws: DecodeWorkspace | None, head_dim: int, device) -> DecodeWorkspace:
    if ws is None:
        return DecodeWorkspace(head_dim, device)
    if ws.head_dim < head_dim or ws.acc.device != device:
        raise KernelError(f"the decode workspace was made for head size {ws.head_dim} on {ws.acc.device}")
    return ws


DECODE_MAX_SEGMENTS = 1024      # requests per step that the tcgen05 decode kernel takes (FD_MAX_SEGS in csrc/attention_tcgen05.cu)


def decode_on_tcgen05(head_dim: int, page_size: int, group: int, act_dtype: torch.dtype, num_segments: int = 0) -> bool:
    """Whether single tokens of such a layer go to the tcgen05 decode kernel (which cuts the keys by itself) rather
    than to the mma.sync kernel with its key ranges; a step of more than DECODE_MAX_SEGMENTS segments does not."""
    return (TCGEN05_DECODE and act_dtype == torch.bfloat16 and num_segments <= DECODE_MAX_SEGMENTS
            and attention_decode_tcgen05_usable(head_dim, page_size, group))


def attention_decode_fused_usable(head_dim: int, page_size: int, group: int, adjacent_pairs: bool,
                                  act_dtype: torch.dtype) -> bool:
    """Whether a step that holds single tokens only can leave per-head norm, rotation and the page write of the new
    keys and values to the tcgen05 decode attention kernel (``attention_decode_fused``)."""
    return FUSE_ROPE and adjacent_pairs and decode_on_tcgen05(head_dim, page_size, group, act_dtype)


def attention_decode_fused(qkv: torch.Tensor, kcache, vcache, block_table, seg_off, seg_slot, seg_start, seg_len,
                           num_segments: int, nq: int, nkv: int, head_dim: int, page_size: int, window: int | None,
                           scale: float, q_weight, k_weight, eps: float, cos, sin, error_count: torch.Tensor,
                           workspace: DecodeWorkspace | None = None, out: torch.Tensor | None = None,
                           span_min: int | None = None, pair_cost: int | None = None) -> torch.Tensor:
    """A step of single tokens, straight from the q/k/v product: ``qkv`` [T, (nq + 2 nkv) d] raw.  The tcgen05 decode
    kernel normalises and rotates the queries as it loads them, writes each token's (normalised, rotated) key and its
    value into their page before it reads that page, and adds up the pieces of the requests whose keys it has cut
    between CTAs (``workspace``; made here when missing).  ``q_weight``/``k_weight`` None: no per-head norm;
    ``cos``/``sin`` None: no rotation (pairs are adjacent elements).  Returns [T, nq * d]."""
    _need_cuda(qkv, kcache, vcache, block_table, seg_off, seg_slot, seg_start, seg_len, q_weight, k_weight, cos, sin,
               error_count)
    _need_contig(qkv=qkv, kcache=kcache, vcache=vcache, block_table=block_table, cos=cos, sin=sin)
    T, width = qkv.shape
    if qkv.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or vcache.dtype != torch.bfloat16:
        raise KernelError("the fused decode attention takes bfloat16 only")
    if width != (nq + 2 * nkv) * head_dim or T != num_segments:
        raise KernelError("the fused decode attention takes one row of (nq + 2 nkv) * d raw projections per single-token segment")
    if kcache.shape[1:] != (nkv, page_size, head_dim) or vcache.shape != kcache.shape:
        raise KernelError(f"pages must be [n, {nkv}, {page_size}, {head_dim}], got {tuple(kcache.shape)}")
    has_norm = q_weight is not None
    if has_norm and (k_weight is None or q_weight.shape != (head_dim,) or k_weight.shape != (head_dim,)
                     or q_weight.dtype != k_weight.dtype):
        raise KernelError("per-head norm weights must both have shape (head_dim,) and one dtype")
    rot_pairs = 0 if cos is None else cos.shape[1]
    if cos is not None and (cos.shape != (T, rot_pairs) or sin.shape != cos.shape or cos.dtype != torch.float32):
        raise KernelError("rotation tables must be float32 [T, pairs]")
    ws = _decode_workspace(workspace, head_dim, qkv.device)
    if out is None:
        out = torch.empty((T, nq * head_dim), dtype=qkv.dtype, device=qkv.device)
    tlib = _lib("attention_tcgen05", head_dim)
    _check(tlib, tlib.pi_attention_decode_tcgen05_fused(
        _p(qkv), c_int(width), _p(kcache), _p(vcache), ctypes.c_longlong(kcache.shape[0]), _p(block_table),
        c_int(block_table.shape[1]), _p(seg_off), _p(seg_slot), _p(seg_start), _p(seg_len), _p(out), _p(ws.acc), _p(ws.ml),
        _p(ws.count), c_int(ws.ctas), c_int(span_min or DECODE_SPAN_MIN), c_int(DECODE_PAIR_COST if pair_cost is None else pair_cost),
        c_int(num_segments), c_int(nq), c_int(nkv),
        c_int(page_size), c_int(window or 0), c_float(scale), _p(q_weight), _p(k_weight),
        c_int(_code(q_weight.dtype) if has_norm else BF16), c_float(eps), _p(cos), _p(sin), c_int(rot_pairs), _p(error_count),
        _stream()), "attention_decode_tcgen05_fused")
    return out


# ---- matrix products -----------------------------------------------------------------------------------------------
def gemm_f32(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """x fp32 [M, K], weight fp32 [N, K] -> fp32 [M, N] with fp32 FMA in a fixed k order."""
    _need_cuda(x, weight)
    if x.dtype != torch.float32 or weight.dtype != torch.float32:
        raise KernelError("gemm_f32 takes float32 operands")
    if x.stride(-1) != 1 or weight.stride(-1) != 1:
        raise KernelError("gemm_f32 needs unit stride along k")
    M, K = x.shape
    N, K2 = weight.shape
    if K != K2:
        raise KernelError(f"inner sizes differ: {K} vs {K2}")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    lib = _lib("gemm_f32")
    _check(lib, lib.pi_gemm_f32_nt(_p(x), c_int(x.stride(0)), _p(weight), c_int(weight.stride(0)), _p(out),
                                   c_int(out.stride(0)), c_int(M), c_int(N), c_int(K), _stream()), "gemm_f32")
    return out


FUSE_NORMS = os.environ.get("PULSE_FUSE_NORMS", "1") != "0"   # decoding: norms prepared / finished inside the products
SMALL_M_ROWS = 16         # up to this many rows the weight-streaming kernel is used instead of cuBLAS


class NormedRows:
    """The input of an RMSNorm over a few rows of the 32-bit residual, prepared by the product that last added to
    the residual (``linear(..., residual=h, next_norm=...)``): ``scaled`` = bf16(h * norm weight) and ``partials``
    [32, slots] = sums of h^2 per row and 16-feature tile.  The weight-streaming product takes both and scales
    its outputs by rsqrt(mean(h^2) + eps), so the norm needs no kernel of its own; ``materialize()`` runs the norm
    kernel for everyone else.  ``owner`` says whose norm this is (any object, compared by identity)."""

    def __init__(self, hidden: torch.Tensor, weight: torch.Tensor, eps: float, act_dtype: torch.dtype,
                 scaled: torch.Tensor, partials: torch.Tensor, owner=None):
        self.hidden, self.weight, self.eps, self.act_dtype = hidden, weight, float(eps), act_dtype
        self.scaled, self.partials, self.owner = scaled, partials, owner
        self.shape, self.dtype = hidden.shape, act_dtype
        self._value: torch.Tensor | None = None

    def materialize(self) -> torch.Tensor:
        if self._value is None:
            self._value = add_rmsnorm(self.hidden, None, self.weight, self.eps, self.act_dtype)
        return self._value


def gemm_small_m(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype, out: torch.Tensor | None = None,
                 gated: bool = False, residual: torch.Tensor | None = None, row_ssq: tuple | None = None,
                 emit_norm: torch.Tensor | None = None):
    """x bf16 [M <= 32, K], weight bf16 [N, K] -> [M, N] in bf16 or fp32: every weight read once.
    ``gated``: weight rows are gate/up features interleaved in blocks of 8 (see ``interleave_gate_up``) and the
    result is silu(gate) * up, [M, N / 2] bf16.
    ``residual`` (float32 [M, N]): the result is added to it in place and it is returned.  With ``emit_norm``
    (the weight [N] of the RMSNorm that follows) the kernel also writes bf16(residual * emit_norm) and the
    per-tile sums of residual^2, and (residual, scaled, partials) is returned.
    ``row_ssq`` = (partials, eps): x is such a ``scaled`` tensor; outputs are scaled by rsqrt(mean + eps) per row."""
    _need_cuda(x, weight)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise KernelError("gemm_small_m takes bfloat16 operands")
    if x.stride(-1) != 1 or weight.stride(-1) != 1:
        raise KernelError("gemm_small_m needs unit stride along k")
    M, K = x.shape
    N, K2 = weight.shape
    if K != K2:
        raise KernelError(f"inner sizes differ: {K} vs {K2}")
    lib = _lib("gemm_small_m")
    if emit_norm is not None and residual is None:
        raise KernelError("gemm_small_m: preparing the next norm goes with the residual epilogue")
    if not gated and residual is None and row_ssq is None:
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        _check(lib, lib.pi_gemm_small_m(_p(x), c_int(x.stride(0)), _p(weight), c_int(weight.stride(0)), _p(out),
                                        c_int(_code(out_dtype)), c_int(out.stride(0)), c_int(M), c_int(N), c_int(K),
                                        _stream()), "gemm_small_m")
        return out
    scaled = partials = None
    if residual is not None:
        if gated or residual.dtype != torch.float32 or tuple(residual.shape) != (M, N) or residual.stride(-1) != 1:
            raise KernelError("gemm_small_m: the residual is float32 [M, N] and goes with a plain product")
        _need_cuda(residual)
        out, epilogue = residual, 2
        if emit_norm is not None:
            _need_cuda(emit_norm)
            if emit_norm.numel() != N or not emit_norm.is_contiguous():
                raise KernelError("gemm_small_m: the next norm's weight must hold N contiguous values")
            scaled = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
            partials = torch.empty((32, lib.pi_gemm_small_m_tiles(c_int(N))), dtype=torch.float32, device=x.device)
    else:
        if emit_norm is not None:
            raise KernelError("gemm_small_m: preparing the next norm goes with the residual epilogue")
        epilogue = 1 if gated else 0
        if gated:
            out_dtype = torch.bfloat16
        if out is None:
            out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
    ssq, eps = row_ssq if row_ssq is not None else (None, 0.0)
    if ssq is not None:
        _need_cuda(ssq)
        if ssq.dtype != torch.float32 or ssq.dim() != 2 or ssq.shape[0] != 32 or not ssq.is_contiguous():
            raise KernelError("gemm_small_m: the partial sums are float32 [32, slots]")
    _check(lib, lib.pi_gemm_small_m_fused(
        _p(x), c_int(x.stride(0)), _p(weight), c_int(weight.stride(0)), _p(out), c_int(_code(out.dtype)),
        c_int(out.stride(0)), c_int(M), c_int(N), c_int(K), c_int(epilogue), _p(ssq),
        c_int(ssq.shape[1] if ssq is not None else 0), c_float(eps), _p(emit_norm),
        c_int(_code(emit_norm.dtype) if emit_norm is not None else BF16), _p(scaled),
        c_int(scaled.stride(0) if scaled is not None else 0), _p(partials), _stream()), "gemm_small_m_fused")
    if scaled is not None:
        return out, scaled, partials
    return out


def gemm_tcgen05(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, gated: bool = False,
                 out: torch.Tensor | None = None, max_ctas: int = 0, mode: int = 0) -> torch.Tensor:
    """x bf16 [M, K], weight bf16 [N, K] -> [M, N] on tcgen05 tensor cores (TMEM accumulators, TMA loads).
    ``gated``: weight rows are gate/up features interleaved in blocks of 8 (see ``interleave_gate_up``) and the
    result is silu(gate) * up, [M, N / 2] bf16.  ``mode``: 0 chosen from M, 1 single CTAs, 2 CTA pairs."""
    _need_cuda(x, weight)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise KernelError("gemm_tcgen05 takes bfloat16 operands")
    if x.stride(-1) != 1 or weight.stride(-1) != 1:
        raise KernelError("gemm_tcgen05 needs unit stride along k")
    M, K = x.shape
    N, K2 = weight.shape
    if K != K2:
        raise KernelError(f"inner sizes differ: {K} vs {K2}")
    if out is None:
        out = torch.empty((M, N // 2 if gated else N), dtype=out_dtype, device=x.device)
    lib = _lib("gemm_tcgen05")
    _check(lib, lib.pi_gemm_tcgen05(_p(x), c_int(x.stride(0)), _p(weight), c_int(weight.stride(0)), _p(out),
                                    c_int(_code(out.dtype)), c_int(out.stride(0)), c_int(M), c_int(N), c_int(K),
                                    c_int(1 if gated else 0), c_int(max_ctas), c_int(mode), _stream()), "gemm_tcgen05")
    return out


def gemm_tcgen05_status() -> int:
    """0 if every bounded wait of the tcgen05 kernels launched so far was met (synchronises the device)."""
    lib = _lib("gemm_tcgen05")
    status = ctypes.c_uint(0)
    _check(lib, lib.pi_gemm_tcgen05_status(ctypes.byref(status)), "gemm_tcgen05_status", launches=0)
    return int(status.value)


GATE_BLOCK = 8    # gate / up features per block of the interleaved layout


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, K] gate and up weights -> [2I, K] with rows in blocks of 16: 8 gate rows, then their 8 up rows.
    A 16-row tile of the small-M product and every 32-column chunk of the tcgen05 product's epilogue then
    hold gate and up of the same features."""
    I, K = gate.shape
    B = GATE_BLOCK
    if I % B:
        raise KernelError(f"the interleaved layout needs an intermediate size that is a multiple of {B}")
    return torch.stack([gate.view(I // B, B, K), up.view(I // B, B, K)], dim=1).reshape(2 * I, K).contiguous()


def small_m_usable(rows: int, K: int, weight: torch.Tensor) -> bool:
    """Whether ``linear`` would put a product of this many rows with this weight on the weight-streaming kernel."""
    return (rows <= SMALL_M_ROWS and weight.dtype == torch.bfloat16 and K % 8 == 0 and weight.stride(-1) == 1
            and weight.stride(0) % 8 == 0 and weight.data_ptr() % 16 == 0)


def linear(x, weight: torch.Tensor, out_dtype: torch.dtype | None = None, residual: torch.Tensor | None = None,
           next_norm: tuple | None = None, out: torch.Tensor | None = None):
    """y = x W^T with W [out, in] (src/layer/linear.cpp:213).  A bfloat16 weight runs on tensor cores with
    32-bit accumulation: up to SMALL_M_ROWS rows on the weight-streaming kernel, more on cuBLAS.  A float32
    weight runs on the fp32-FMA kernel, whatever the activation dtype.
    ``x`` may be ``NormedRows``: the weight-streaming kernel finishes the norm itself, otherwise it is computed
    first.  ``residual`` (float32 [rows, out]): where the weight-streaming kernel runs, y is added to it in
    place and None is returned - or, with ``next_norm`` = (weight, eps, owner) of the RMSNorm that follows, the
    ``NormedRows`` that its consumer takes; otherwise y is returned and the caller adds it.
    ``out`` ([rows, out] of ``out_dtype``, contiguous; plain bfloat16-weight products only): where y is written."""
    if out is not None and (residual is not None or tuple(out.shape) != (x.shape[0], weight.shape[0])
                            or not out.is_contiguous() or weight.dtype != torch.bfloat16
                            or out.dtype != (out_dtype or torch.bfloat16)):
        raise KernelError("linear: `out` goes with a plain bfloat16-weight product and must be [rows, out] of the output dtype")
    if isinstance(x, NormedRows):
        sc = x.scaled
        if (x._value is None and small_m_usable(sc.shape[0], sc.shape[1], weight) and residual is None
                and (out_dtype or torch.bfloat16) in (torch.bfloat16, torch.float32)):
            return gemm_small_m(sc, weight, out_dtype or torch.bfloat16, out=out, row_ssq=(x.partials, x.eps))
        x = x.materialize()
    _need_cuda(x, weight)
    out_dtype = out_dtype or x.dtype
    if weight.dtype == torch.float32:
        y = gemm_f32(x if x.dtype == torch.float32 else x.float(), weight)
        return y if out_dtype == torch.float32 else y.to(out_dtype)
    if weight.dtype != torch.bfloat16:
        raise KernelError(f"weights must be bfloat16 or float32, not {weight.dtype}")
    xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    if (small_m_usable(xb.shape[0], xb.shape[1], weight) and xb.stride(-1) == 1 and xb.stride(0) % 8 == 0
            and xb.data_ptr() % 16 == 0 and out_dtype in (torch.bfloat16, torch.float32)):
        if residual is not None:
            if next_norm is not None and out_dtype == torch.bfloat16 and FUSE_NORMS:
                nw, eps, owner = next_norm
                _, scaled, partials = gemm_small_m(xb, weight, torch.float32, residual=residual, emit_norm=nw)
                return NormedRows(residual, nw, eps, out_dtype, scaled, partials, owner)
            gemm_small_m(xb, weight, torch.float32, residual=residual)
            return None
        return gemm_small_m(xb, weight, out_dtype, out=out)
    if out_dtype == torch.bfloat16:
        return torch.mm(xb, weight.t(), out=out) if out is not None else torch.mm(xb, weight.t())
    if out is not None:
        return torch.mm(xb, weight.t(), out_dtype=torch.float32, out=out)
    return torch.mm(xb, weight.t(), out_dtype=torch.float32)


# ---- sampling ---------------------------------------------------------------------------------------------------------
def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """logits fp32 [n, V] -> int32 [n]; the lowest index wins ties."""
    _need_cuda(logits)
    if logits.dtype != torch.float32 or logits.stride(-1) != 1:
        raise KernelError("logits must be float32 with unit stride")
    n, V = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    lib = _lib("sampling")
    words = lib.pi_argmax_scratch_floats(c_int(n), c_int(V))
    scratch = torch.empty((words,), dtype=torch.float32, device=logits.device) if words else None
    _check(lib, lib.pi_argmax(_p(logits), c_int(logits.stride(0)), c_int(n), c_int(V), _p(out), _p(scratch), _stream()),
           "argmax", launches=2 if words else 1)
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           seeds: torch.Tensor, counters: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Per-row temperature / top-k / top-p sampling; temperature <= 0 means greedy for that row.
    seeds and counters are int64 (read as unsigned); the uniform draw depends on them only."""
    _need_cuda(logits, temperature, top_k, top_p, seeds, counters)
    n, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(-1) != 1:
        raise KernelError("logits must be float32 with unit stride")
    if (temperature.dtype != torch.float32 or top_p.dtype != torch.float32 or top_k.dtype != torch.int32
            or seeds.dtype != torch.int64 or counters.dtype != torch.int64):
        raise KernelError("sampling parameters: temperature/top_p float32, top_k int32, seeds/counters int64")
    for name, t in (("temperature", temperature), ("top_k", top_k), ("top_p", top_p), ("seeds", seeds), ("counters", counters)):
        if t.numel() != n or not t.is_contiguous():
            raise KernelError(f"sampling parameter '{name}' must hold one contiguous value per row")
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    lib = _lib("sampling")
    _check(lib, lib.pi_sample(_p(logits), c_int(logits.stride(0)), c_int(n), c_int(V), _p(temperature), _p(top_k),
                              _p(top_p), _p(seeds), _p(counters), _p(out), _stream()), "sample")
    return out


def sample_entries(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                   seeds: torch.Tensor, row_entry: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """As ``sample``, with the options in tables that outlive the step: ``row_entry`` int64 [n, 2] gives, per row, the
    table entry it uses and its draw counter."""
    _need_cuda(logits, temperature, top_k, top_p, seeds, row_entry)
    n, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(-1) != 1:
        raise KernelError("logits must be float32 with unit stride")
    if (temperature.dtype != torch.float32 or top_p.dtype != torch.float32 or top_k.dtype != torch.int32
            or seeds.dtype != torch.int64 or row_entry.dtype != torch.int64):
        raise KernelError("sampling tables: temperature/top_p float32, top_k int32, seeds int64; row_entry int64")
    entries = temperature.numel()
    for name, t in (("top_k", top_k), ("top_p", top_p), ("seeds", seeds)):
        if t.numel() != entries or not t.is_contiguous():
            raise KernelError(f"sampling table '{name}' must hold {entries} contiguous values")
    if tuple(row_entry.shape) != (n, 2) or not row_entry.is_contiguous():
        raise KernelError("row_entry must be contiguous int64 [rows, 2]")
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    lib = _lib("sampling")
    _check(lib, lib.pi_sample_entries(_p(logits), c_int(logits.stride(0)), c_int(n), c_int(V), _p(temperature), _p(top_k),
                                      _p(top_p), _p(seeds), _p(row_entry), _p(out), _stream()), "sample_entries")
    return out


def logit_edit(logits: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor, values: torch.Tensor, set_value: bool) -> None:
    """logits[rows[i], tokens[i]] += values[i] (or = values[i]); pairs must be distinct."""
    _need_cuda(logits, rows, tokens, values)
    n = rows.numel()
    lib = _lib("sampling")
    _check(lib, lib.pi_logit_edit(_p(logits), c_int(logits.stride(0)), c_int(logits.shape[1]), _p(rows), _p(tokens),
                                  _p(values), c_int(n), c_int(1 if set_value else 0), _stream()), "logit_edit")
