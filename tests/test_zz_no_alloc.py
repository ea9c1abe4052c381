"""The allocation-free attention entry point, called through its exported C symbol.

Some hosts of the kernel library cannot allocate device memory around a launch (they run inside
another framework's memory plan, or all device memory was handed out at start-up), so they cannot
provide the scratch that the split decode attention needs.  ``pi_attention_mma_noalloc`` keeps that
scratch in a fixed array inside the library instead.  This test calls it with ctypes, the way such a
host would, twice in a row on different inputs (the array keeps the first call's contents), and wants
the same output as the regular entry point that is given scratch of its own.

It is collected last on purpose: a run that stops at the first failure has then run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

from gpu_util import PagedKV, need_gpu, segments_to_device

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, q, kv, meta, segs, out, max_splits, nq, nkv, d, page, window, scale, has_decode=None):
    p = lambda t: c_void_p(t.data_ptr())  # noqa: E731
    lens = [n for _, _, n in segs]
    if has_decode is None:
        has_decode = int(any(n == 1 for n in lens))
    return lib.pi_attention_mma_noalloc(
        p(q), c_int(nq * d), p(kv.kcache), p(kv.vcache), p(kv.table_dev), c_int(kv.table_dev.shape[1]),
        p(meta["seg_off"]), p(meta["seg_slot"]), p(meta["seg_start"]), p(meta["seg_len"]), p(meta["token_seg"]), p(out),
        c_int(max_splits), c_int(256), c_int(meta["T"]), c_int(len(segs)), c_int(max(lens)),
        c_int(int(any(n > 1 for n in lens))), c_int(has_decode), c_int(nq), c_int(nkv), c_int(page),
        c_int(window or 0), c_float(scale), c_void_p(torch.cuda.current_stream().cuda_stream))


def test_noalloc_entry_matches_regular_entry_twice():
    dev = need_gpu()
    from pulse_infer_b200 import ops
    from pulse_infer_b200.csrc import build
    nq, nkv, d, page = 8, 2, 64, 16
    lib = ctypes.CDLL(build.library_path("attention_mma", d))
    lib.pi_last_error.restype = ctypes.c_char_p
    assert lib.pi_attention_noalloc_scratch_bytes() == 8 * 1024 * 1024
    scale = 1.0 / math.sqrt(d)
    cases = [  # (sequence lengths, segments (slot, start, n), window): decodes long enough to be split ...
        ([1000, 700, 90], [(0, 999, 1), (1, 699, 1), (2, 60, 30)], None),
        ([1300, 300], [(1, 299, 1), (0, 1299, 1)], 600),
        ([200, 90], [(0, 199, 1), (1, 89, 1)], None),        # ... and short ones: a single range, no scratch used
    ]
    for call, (lengths, segs, window) in enumerate(cases):
        kv = PagedKV(lengths, nkv, d, page, torch.bfloat16, dev, seed=call)
        meta = segments_to_device(segs, dev)
        T = meta["T"]
        q = torch.randn(T, nq * d, generator=torch.Generator().manual_seed(call)).to(torch.bfloat16).to(dev)
        lens = [n for _, _, n in segs]
        splits = max(ops.attention_num_splits(st, window) for _, st, n in segs if n == 1)
        assert (splits > 1) == (call < 2)
        acc = torch.empty(T * nq * splits * d, dtype=torch.float32, device=dev)
        ml = torch.empty(T * nq * splits * 2, dtype=torch.float32, device=dev)
        want = ops.attention_mma(q, nq * d, kv.kcache, kv.vcache, kv.table_dev, meta["seg_off"], meta["seg_slot"],
                                 meta["seg_start"], meta["seg_len"], meta["token_seg"], T, len(segs), max(lens),
                                 any(n > 1 for n in lens), any(n == 1 for n in lens), splits, acc, ml, nq, nkv, d, page,
                                 window, scale, prompt_on_tcgen05=False, decode_on_tcgen05=False)      # the same library as the entry under test
        got = torch.full_like(want, float("nan"))
        before = torch.cuda.memory_allocated()
        rc = _call_noalloc(lib, q, kv, meta, segs, got, splits, nq, nkv, d, page, window, scale)
        assert rc == 0, lib.pi_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        # same kernels, same arithmetic: the tolerance of the attention tests (0.03) is far from needed
        assert torch.isfinite(got.float()).all()
        assert float((got.float() - want.float()).abs().max()) <= 0.03
        assert torch.equal(got, want)


def test_noalloc_entry_refuses_sizes_beyond_its_array():
    dev = need_gpu()
    from pulse_infer_b200.csrc import build
    nq, nkv, d, page = 32, 8, 128, 16
    lib = ctypes.CDLL(build.library_path("attention_mma", d))
    lib.pi_last_error.restype = ctypes.c_char_p
    segs = [(i, 4095, 1) for i in range(64)]
    meta = segments_to_device(segs, dev)
    dummy = torch.zeros(64 * nq * d, dtype=torch.bfloat16, device=dev)
    table = torch.zeros(64, 256, dtype=torch.int32, device=dev)

    class KV:
        kcache = vcache = dummy
        table_dev = table
    # 64 tokens x 32 heads x 16 ranges x 130 floats = 17 MB > 8 MiB: refused before anything is launched
    rc = _call_noalloc(lib, dummy, KV, meta, segs, dummy, 16, nq, nkv, d, page, None, 0.1)
    assert rc == -1
    text = lib.pi_last_error().decode()
    assert "bytes of scratch" in text and "8388608" in text
    # "only merge what is already in the scratch" makes no sense for an array nobody else can write: refused
    rc = _call_noalloc(lib, dummy, KV, meta, segs, dummy, 2, nq, nkv, d, page, None, 0.1, has_decode=2)
    assert rc == -1 and "has_decode" in lib.pi_last_error().decode()
    torch.cuda.synchronize()


def test_noalloc_entry_at_the_edge_of_its_array():
    """The largest scratch that fits is taken (and gives the regular entry's output), the next size up is refused.
    A call needs rows * ranges * (head size + 2) * 4 bytes; with head size 64 that is 264 bytes per (row, range):
    31,775 of them are 8,388,600 bytes (8 bytes below the 8 MiB array), 31,776 are 256 bytes over."""
    dev = need_gpu()
    from pulse_infer_b200 import ops
    from pulse_infer_b200.csrc import build
    d, page = 64, 16
    lib = ctypes.CDLL(build.library_path("attention_mma", d))
    lib.pi_last_error.restype = ctypes.c_char_p
    limit = lib.pi_attention_noalloc_scratch_bytes()
    scale = 1.0 / math.sqrt(d)
    # 31 tokens x 25 heads x 41 ranges = 31,775 entries; the requests themselves use two or three of the 41 ranges
    nq, nkv, splits = 25, 5, 41
    lengths = [300 + 17 * i for i in range(31)]
    segs = [(i, n - 1, 1) for i, n in enumerate(lengths)]
    assert len(segs) * nq * splits * (d + 2) * 4 == limit - 8
    kv = PagedKV(lengths, nkv, d, page, torch.bfloat16, dev, seed=5)
    meta = segments_to_device(segs, dev)
    T = meta["T"]
    q = torch.randn(T, nq * d, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(dev)
    acc = torch.empty(T * nq * splits * d, dtype=torch.float32, device=dev)
    ml = torch.empty(T * nq * splits * 2, dtype=torch.float32, device=dev)
    want = ops.attention_mma(q, nq * d, kv.kcache, kv.vcache, kv.table_dev, meta["seg_off"], meta["seg_slot"],
                             meta["seg_start"], meta["seg_len"], meta["token_seg"], T, len(segs), 1, False, True, splits,
                             acc, ml, nq, nkv, d, page, None, scale, prompt_on_tcgen05=False, decode_on_tcgen05=False)
    got = torch.full_like(want, float("nan"))
    rc = _call_noalloc(lib, q, kv, meta, segs, got, splits, nq, nkv, d, page, None, scale)
    assert rc == 0, lib.pi_last_error().decode()
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # 32 tokens x 3 heads x 331 ranges = 31,776 entries: 256 bytes more than the array holds
    segs = [(0, 10, 1)] * 32
    meta = segments_to_device(segs, dev)
    assert 32 * 3 * 331 * (d + 2) * 4 == limit + 256
    rc = _call_noalloc(lib, q, kv, meta, segs, got, 331, 3, 3, d, page, None, scale)
    assert rc == -1 and "bytes of scratch" in lib.pi_last_error().decode()
    torch.cuda.synchronize()
