"""Host-side facts of a step that need no GPU: the metadata buffer and the width of the split-attention scratch."""
import numpy as np
import torch

from pulse_infer_b200 import ops
from pulse_infer_b200.cache import CacheManager
from pulse_infer_b200.engine.context import Segment, StepContext
from pulse_infer_b200.parts.base import CacheSpec
from pulse_infer_b200.parts.model import Runtime


def test_key_range_count_is_not_monotone_under_a_window():
    """The window's first key is rounded down to a multiple of 64, so a request at a lower position can need more
    key ranges than one at a higher position."""
    assert ops.attention_num_splits(511, 256, 256) == 1
    assert ops.attention_num_splits(300, 256, 256) == 2
    assert ops.attention_splits_bound([511, 300], 256, 256) == 2
    assert ops.attention_splits_bound([511], 256, 256) == 1
    assert ops.attention_splits_bound([], 256, 256) == 1


def test_bound_covers_every_position():
    rng = np.random.RandomState(0)
    for window in (None, 24, 150, 256, 300, 1000, 4096):
        for split_keys in (128, 256, 512, 2048):
            positions = [int(p) for p in rng.randint(0, 9000, size=40)] + [0, 63, 64, 255, 256, 4095, 4096, 4159]
            bound = ops.attention_splits_bound(positions, window, split_keys)
            counts = [ops.attention_num_splits(p, window, split_keys) for p in positions]
            assert bound == max(counts)
            if window:
                # a window of w keys never needs more than ceil((w + 63) / split_keys) ranges
                assert bound <= (window + 63 + split_keys - 1) // split_keys
            else:
                assert bound == ops.attention_num_splits(max(positions), None, split_keys)


def test_step_context_sizes_the_scratch_for_the_widest_request():
    runtime = Runtime(torch.device("cpu"), "bfloat16")
    cache = CacheManager([CacheSpec(1, 32, 256)], [None], 16, 64, 4, 1024, allocate_pools=False)
    segs = [Segment("a", [1], [0]), Segment("b", [2], [0]), Segment("c", [3, 4, 5], [2])]
    for s, (slot, start) in zip(segs, ((0, 511), (1, 300), (2, 0))):
        s.slot, s.start = slot, start
    ctx = StepContext.build(segs, runtime, cache)
    assert ctx.has_decode and ctx.has_prompt and ctx.decode_starts == [511, 300] and ctx.decode_pos_max == 511
    ctx.split_keys = {(1, 32): 256}
    sc = ctx.attention_scratch(num_heads=2, head_dim=32, window=256, num_kv_heads=1)
    assert sc.max_splits == 2 and sc.split_keys == 256
    assert sc.acc.shape == (ctx.num_tokens * 2, 2, 32) and sc.ml.shape == (ctx.num_tokens * 2, 2, 2)
    # without a window the highest position decides
    sc = ctx.attention_scratch(num_heads=2, head_dim=32, window=None, num_kv_heads=1)
    assert sc.max_splits == 2        # 512 keys in ranges of 256


def test_step_context_gives_the_tcgen05_decode_kernel_its_workspace_up_to_1024_requests():
    """Head size 128 in bfloat16: single tokens go to the tcgen05 decode kernel, which needs one workspace per runtime
    (kept across steps) and no key ranges; a step of more requests than that kernel takes falls back to key ranges."""
    runtime = Runtime(torch.device("cpu"), "bfloat16")
    for count, spans in ((3, True), (ops.DECODE_MAX_SEGMENTS, True), (ops.DECODE_MAX_SEGMENTS + 1, False)):
        cache = CacheManager([CacheSpec(2, 128, None)], [None], 16, 64, count, 4096, allocate_pools=False)
        segs = [Segment(i, [1], [0]) for i in range(count)]
        for i, s in enumerate(segs):
            s.slot, s.start = i, 3000 + (i % 7)
        ctx = StepContext.build(segs, runtime, cache)
        sc = ctx.attention_scratch(num_heads=8, head_dim=128, window=None, num_kv_heads=2)
        assert (sc.decode_ws is not None) == spans
        if spans:
            assert sc.max_splits == 1 and sc.acc is None
            assert sc.decode_ws is runtime.decode_workspaces[128]
            assert int(sc.decode_ws.count.abs().sum()) == 0 and sc.decode_ws.acc.numel() == sc.decode_ws.ctas * 2 * 16 * 128
            again = StepContext.build(segs, runtime, cache).attention_scratch(8, 128, None, 2)
            assert again.decode_ws is sc.decode_ws
        else:
            assert sc.max_splits == ops.attention_splits_bound([s.start for s in segs], None, sc.split_keys) and sc.acc is not None
