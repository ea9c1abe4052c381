"""Kernel entry points.  ``from pulse_infer_b200 import ops`` then ``ops.embed(...)`` and so on."""
from . import kernels
from .kernels import (BF16, F32, SPLIT_KEYS, DECODE_MAX_SEGMENTS, KernelError, NormedRows, add_rmsnorm, argmax, attention_mma, attention_num_splits, attention_splits_bound, choose_prompt_splits, choose_split_keys,
                      attention_simple, attention_decode_fused, attention_decode_fused_usable, attention_decode_workspace, decode_on_tcgen05, DecodeWorkspace, attention_tcgen05, attention_tcgen05_status, attention_tcgen05_loaded_status, attention_tcgen05_usable, attention_decode_tcgen05_usable, embed, gemm_f32, gemm_small_m, gemm_tcgen05, gemm_tcgen05_status, interleave_gate_up, linear, logit_edit, preload, qk_norm_rope_write, rope_table,
                      sample, sample_entries, silu_mul, small_m_usable)

__all__ = ["DECODE_MAX_SEGMENTS", "BF16", "F32", "SPLIT_KEYS", "KernelError", "NormedRows", "add_rmsnorm", "argmax", "attention_mma",
           "attention_num_splits", "attention_splits_bound", "choose_prompt_splits", "choose_split_keys", "attention_simple", "attention_decode_fused", "attention_decode_fused_usable", "attention_decode_workspace", "decode_on_tcgen05", "DecodeWorkspace", "attention_tcgen05", "attention_tcgen05_status", "attention_tcgen05_loaded_status", "attention_tcgen05_usable", "attention_decode_tcgen05_usable", "embed", "gemm_f32", "gemm_small_m", "gemm_tcgen05", "gemm_tcgen05_status", "interleave_gate_up", "linear", "logit_edit", "preload",
           "qk_norm_rope_write", "rope_table", "sample", "sample_entries", "silu_mul", "small_m_usable"]
