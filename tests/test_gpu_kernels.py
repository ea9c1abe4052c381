"""Each kernel alone against a plain reference, at sizes other than the engine tests use."""
import math

import numpy as np
import pytest
import torch

import plain_model
from gpu_util import PagedKV, dense_attention, need_gpu, segments_to_device

pytestmark = pytest.mark.gpu


def _ops():
    from pulse_infer_b200 import ops
    return ops


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding(dtype):
    dev, ops = need_gpu(), _ops()
    table = torch.randn(1000, 202).to(dtype)
    tokens = torch.tensor([0, 999, 5, 5, 123, 1000, -1], dtype=torch.int32)
    out = ops.embed(tokens.to(dev), table.to(dev)).cpu()
    want = torch.from_numpy(plain_model.embedding(table.float().numpy(), tokens.tolist()))
    assert out.dtype == torch.float32 and torch.equal(out, want)


@pytest.mark.parametrize("hidden", [4096, 202, 77, 1536, 5120, 8192, 9000])
@pytest.mark.parametrize("act,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32)])
def test_add_rmsnorm(hidden, act, wdt):
    dev, ops = need_gpu(), _ops()
    g = torch.Generator().manual_seed(hidden)
    h = torch.randn(9, hidden, generator=g) * 3
    delta = torch.randn(9, hidden, generator=g).to(act)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(wdt)
    eps = 1e-5
    hd = h.clone().to(dev)
    x = ops.add_rmsnorm(hd, delta.to(dev), w.to(dev), eps, act).cpu()
    s = h.double() + delta.double()
    want = plain_model.rms_norm(s.numpy(), w.double().numpy(), eps)
    assert torch.allclose(hd.cpu().double(), s, atol=1e-6, rtol=1e-6)          # the residual is 32-bit
    tol = 1e-5 if act == torch.float32 else 2 ** -8
    assert np.abs(x.double().numpy() - want).max() <= tol * np.abs(want).max()
    # without a delta, and gathered rows that leave the residual untouched
    x0 = ops.add_rmsnorm(h.clone().to(dev), None, w.to(dev), eps, act).cpu()
    assert np.abs(x0.double().numpy() - plain_model.rms_norm(h.double().numpy(), w.double().numpy(), eps)).max() <= tol * 4
    rows = torch.tensor([7, 0, 7, 3], dtype=torch.int32)
    hd2 = h.clone().to(dev)
    xr = ops.add_rmsnorm(hd2, delta.to(dev), w.to(dev), eps, act, rows=rows.to(dev)).cpu()
    assert torch.equal(hd2.cpu(), h)
    assert np.abs(xr.double().numpy() - want[rows.long().numpy()]).max() <= tol * np.abs(want).max()


@pytest.mark.parametrize("inter", [12288, 222, 7, 224])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(inter, dtype):
    dev, ops = need_gpu(), _ops()
    gu = (torch.randn(5, 2 * inter, generator=torch.Generator().manual_seed(1)) * 4).to(dtype)
    out = ops.silu_mul(gu.to(dev)).cpu().double().numpy()
    g, u = gu[:, :inter].double().numpy(), gu[:, inter:].double().numpy()
    want = plain_model.silu(g) * u
    tol = 1e-6 if dtype == torch.float32 else 2 ** -8
    assert np.abs(out - want).max() <= tol * max(1.0, np.abs(want).max())
    if inter % 8 == 0:       # the same values with gate and up columns interleaved in blocks of 8
        blocked = torch.stack([gu[:, :inter].view(5, inter // 8, 8), gu[:, inter:].view(5, inter // 8, 8)], dim=2)
        out_b = ops.silu_mul(blocked.reshape(5, 2 * inter).contiguous().to(dev), blocked=True).cpu().double().numpy()
        assert np.array_equal(out_b, out)


def test_rope_table_large_positions():
    dev, ops = need_gpu(), _ops()
    pos = torch.tensor([0, 1, 17, 4095, 131071], dtype=torch.int32)
    rot, theta = 96, 1e6
    div = torch.tensor([theta ** (2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64)
    cos, sin = ops.rope_table(pos.to(dev), div.to(dev))
    ang = pos.double()[:, None] / div[None, :]
    assert (cos.cpu().double() - torch.cos(ang)).abs().max() < 1e-7
    assert (sin.cpu().double() - torch.sin(ang)).abs().max() < 1e-7


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,rot,adjacent,page", [(6, 2, 48, 48, True, 8), (8, 1, 32, 16, False, 16),
                                                        (5, 5, 80, 80, False, 4), (4, 2, 256, 256, True, 16)])
def test_qk_norm_rope_write(dtype, nq, nkv, d, rot, adjacent, page):
    dev, ops = need_gpu(), _ops()
    g = torch.Generator().manual_seed(nq * d)
    segs = [(1, 13, 9), (0, 0, 5), (2, 40, 1)]            # (slot, start, length)
    meta = segments_to_device(segs, dev)
    T = meta["T"]
    qkv = torch.randn(T, (nq + 2 * nkv) * d, generator=g).to(dtype)
    qw = (1 + 0.2 * torch.randn(d, generator=g)).to(dtype)
    kw = (1 + 0.2 * torch.randn(d, generator=g)).to(dtype)
    eps, theta = 1e-5, 10000.0
    pages = 24
    table = torch.full((3, 16), -1, dtype=torch.int32)
    perm = torch.randperm(pages, generator=g).tolist()
    for slot, start, n in segs:
        for i in range((start + n + page - 1) // page):
            table[slot, i] = perm.pop()
    kc = torch.zeros(pages, nkv, page, d, dtype=dtype, device=dev)
    vc = torch.zeros_like(kc)
    div = torch.tensor([theta ** (2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64, device=dev)
    cos, sin = ops.rope_table(meta["positions"], div)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    dq = qkv.clone().to(dev)
    ops.qk_norm_rope_write(dq, qw.to(dev), kw.to(dev), eps, cos, sin, adjacent, kc, vc, table.to(dev),
                           meta["token_slot"], meta["positions"], page, nq, nkv, d, err)
    assert int(err.item()) == 0
    x = qkv.double().numpy().reshape(T, nq + 2 * nkv, d)
    positions = meta["positions"].cpu().numpy()
    pairing = "adjacent" if adjacent else "half"
    q_want = plain_model.rope(plain_model.rms_norm(x[:, :nq], qw.double().numpy(), eps), positions, theta, rot, pairing)
    k_want = plain_model.rope(plain_model.rms_norm(x[:, nq:nq + nkv], kw.double().numpy(), eps), positions, theta, rot, pairing)
    v_want = x[:, nq + nkv:]
    tol = 2e-6 if dtype == torch.float32 else 2 ** -7
    got = dq.cpu().double().numpy().reshape(T, nq + 2 * nkv, d)
    assert np.abs(got[:, :nq] - q_want).max() <= tol * np.abs(q_want).max()
    assert np.array_equal(got[:, nq:], x[:, nq:])                      # key/value columns are left alone
    kcc, vcc = kc.cpu().double().numpy(), vc.cpu().double().numpy()
    tslot = meta["token_slot"].cpu().numpy()
    for t in range(T):
        p = int(table[tslot[t], positions[t] // page]); s = positions[t] % page
        assert np.abs(kcc[p, :, s] - k_want[t]).max() <= tol * np.abs(k_want).max()
        assert np.array_equal(vcc[p, :, s], v_want[t])
    # nothing else was written
    written = np.zeros((pages, page), dtype=bool)
    for t in range(T):
        written[int(table[tslot[t], positions[t] // page]), positions[t] % page] = True
    assert not kcc.transpose(0, 2, 1, 3)[~written].any() and not vcc.transpose(0, 2, 1, 3)[~written].any()
    # a token whose page is missing is counted, not written
    bad = table.clone(); bad[2, 40 // page] = -1
    ops.qk_norm_rope_write(qkv.clone().to(dev), qw.to(dev), kw.to(dev), eps, cos, sin, adjacent, kc, vc, bad.to(dev),
                           meta["token_slot"], meta["positions"], page, nq, nkv, d, err)
    assert int(err.item()) == 2 * nkv


def _attention_case(ops, dev, dtype, impl, nq, nkv, d, page, window, segs, lengths, seed=0, spike=None, prompt_splits=1,
                    decode_ws=None):
    """segs: (slot, start, n) with start + n <= lengths[slot]; queries random; returns max error / scale."""
    kv = PagedKV(lengths, nkv, d, page, dtype, dev, seed=seed)
    meta = segments_to_device(segs, dev)
    T = meta["T"]
    g = torch.Generator().manual_seed(seed + 1)
    q = torch.randn(T, nq, d, generator=g).to(dtype)
    if spike is not None:
        slot, key_pos, head = spike
        kvh = head // (nq // nkv)
        # the spiked key is a large multiple of the LAST query of that slot's segment, head `head`
        t_last = [o + n - 1 for (s, st, n), o in zip(segs, meta["seg_off"].tolist()) if s == slot][0]
        big = (q[t_last, head].double() * 6.0).to(dtype)
        page_id = int(kv.table[slot, key_pos // page])
        kv.kcache[page_id, kvh, key_pos % page] = big.to(dev)
        kv.k_dense[slot][key_pos, kvh] = big.double()
    scale = 1.0 / math.sqrt(d)
    qflat = q.reshape(T, nq * d).contiguous().to(dev)
    if impl == "simple":
        out = ops.attention_simple(qflat, nq * d, kv.kcache, kv.vcache, kv.table_dev, meta["token_slot"],
                                   meta["positions"], T, nq, nkv, d, page, window, scale)
    else:
        lens = [n for _, _, n in segs]
        dec_pos = max([st for _, st, n in segs if n == 1], default=0)
        splits = ops.attention_num_splits(dec_pos, window) if any(n == 1 for n in lens) else 1
        acc = torch.empty(T * nq * splits * d, dtype=torch.float32, device=dev)
        ml = torch.empty(T * nq * splits * 2, dtype=torch.float32, device=dev)
        # scratch of the split prompt kernel starts as NaN: a share that is read without having been written shows
        pacc = torch.full((T * nq * prompt_splits * d,), float("nan"), dtype=torch.float32, device=dev) if prompt_splits > 1 else None
        pml = torch.full((T * nq * prompt_splits * 2,), float("nan"), dtype=torch.float32, device=dev) if prompt_splits > 1 else None
        out = ops.attention_mma(qflat, nq * d, kv.kcache, kv.vcache, kv.table_dev, meta["seg_off"], meta["seg_slot"],
                                meta["seg_start"], meta["seg_len"], meta["token_seg"], T, len(segs), max(lens),
                                any(n > 1 for n in lens), any(n == 1 for n in lens), splits, acc, ml, nq, nkv, d, page,
                                window, scale, prompt_on_tcgen05=(impl == "tcgen05"), decode_on_tcgen05=(impl == "tcgen05"),
                                prompt_splits=prompt_splits, prompt_acc=pacc, prompt_ml=pml, decode_ws=decode_ws)
        if impl == "tcgen05":
            if not ops.attention_tcgen05_usable(d, page):
                pytest.skip("the tcgen05 kernel takes head sizes 64 / 128 and page sizes 8..128")
            assert ops.attention_tcgen05_status(d) == 0
    out = out.cpu().double().reshape(T, nq, d)
    worst = 0.0
    for (slot, start, n), off in zip(segs, meta["seg_off"].tolist()):
        want = dense_attention(q[off:off + n].double(), kv.k_dense[slot], kv.v_dense[slot],
                               list(range(start, start + n)), window, scale)
        err = float((out[off:off + n] - want).abs().max())
        if not math.isfinite(err):
            return float("inf")               # max() would drop a NaN
        worst = max(worst, err)
    return worst


ATTN_SHAPES = [  # nq, nkv, d, page
    (8, 2, 128, 16), (6, 3, 64, 8), (4, 2, 16, 8), (8, 1, 32, 16), (6, 2, 48, 16), (3, 3, 64, 4), (32, 8, 128, 16), (5, 1, 80, 8), (2, 1, 256, 16),
    (40, 2, 64, 16), (12, 1, 64, 16), (16, 1, 32, 8), (7, 7, 96, 16)]


@pytest.mark.parametrize("nq,nkv,d,page", ATTN_SHAPES)
@pytest.mark.parametrize("window", [None, 37])
def test_attention_simple_float32(nq, nkv, d, page, window):
    dev, ops = need_gpu(), _ops()
    lengths = [150, 70, 301, 9]
    segs = [(0, 100, 50), (1, 69, 1), (2, 0, 301), (3, 7, 2)]
    err = _attention_case(ops, dev, torch.float32, "simple", nq, nkv, d, page, window, segs, lengths)
    assert err < 2e-5


@pytest.mark.parametrize("nq,nkv,d,page", [s for s in ATTN_SHAPES if s[2] % 16 == 0])
@pytest.mark.parametrize("window", [None, 37])
@pytest.mark.parametrize("impl", ["mma", "simple", "tcgen05"])
def test_attention_bfloat16_prompt_and_decode(nq, nkv, d, page, window, impl):
    dev, ops = need_gpu(), _ops()
    if impl == "tcgen05" and not ops.attention_tcgen05_usable(d, page):
        pytest.skip("the tcgen05 kernel takes head sizes 64 / 128 and page sizes 8..128")
    lengths = [150, 70, 301, 9, 1000]
    # portions at odd offsets, single tokens at page edges (63|64, 255|256), one long decode that is split
    segs = [(0, 100, 50), (1, 69, 1), (2, 0, 301), (3, 7, 2), (4, 999, 1)]
    err = _attention_case(ops, dev, torch.bfloat16, impl, nq, nkv, d, page, window, segs, lengths)
    assert err < 0.03      # bfloat16 probabilities and outputs: about 2^-7 of values of order one


@pytest.mark.parametrize("ctx", [1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 255, 256, 257, 511, 512, 513, 1300])
@pytest.mark.parametrize("impl", ["mma", "tcgen05"])
def test_attention_decode_every_edge(ctx, impl):
    dev, ops = need_gpu(), _ops()
    err = _attention_case(ops, dev, torch.bfloat16, impl, 8, 2, 64, 16, None, [(0, ctx - 1, 1)], [ctx], seed=ctx)
    assert err < 0.03


@pytest.mark.parametrize("nq,nkv,d,page", [(32, 8, 128, 16), (16, 1, 64, 8), (6, 3, 128, 64), (5, 5, 64, 32)])
@pytest.mark.parametrize("window", [None, 100, 700])
def test_attention_tcgen05_decode_many_requests(nq, nkv, d, page, window):
    """More items than SMs would take at once, requests of very different lengths (one to several key ranges, the
    last one partial), a prompt portion in the same step: the persistent decode kernel, its ring and the merge."""
    dev, ops = need_gpu(), _ops()
    lengths = [3000, 1, 257, 1025, 640, 129, 2049, 64, 513, 90, 1500, 31]
    segs = [(i, n - 1, 1) for i, n in enumerate(lengths)]
    segs[4] = (4, 500, 140)                                # a portion among the single tokens
    err = _attention_case(ops, dev, torch.bfloat16, "tcgen05", nq, nkv, d, page, window, segs, lengths, seed=nq + page)
    assert err < 0.03


@pytest.mark.parametrize("impl,dtype", [("mma", torch.bfloat16), ("tcgen05", torch.bfloat16), ("simple", torch.bfloat16),
                                        ("simple", torch.float32)])
@pytest.mark.parametrize("key_pos", [0, 15, 16, 300, 511, 512, 700])
def test_attention_finds_one_far_key(impl, dtype, key_pos):
    """One key among hundreds carries nearly all the weight: the output must be that key's value."""
    dev, ops = need_gpu(), _ops()
    nq, nkv, d, page = 8, 2, 64, 16
    lengths = [800]
    for segs in ([(0, 799, 1)], [(0, 760, 40)]):
        kv_err = _attention_case(ops, dev, dtype, impl, nq, nkv, d, page, None, segs, lengths, seed=3,
                                 spike=(0, key_pos, 5))
        assert kv_err < (0.03 if dtype == torch.bfloat16 else 1e-4)


def test_attention_window_edge_exact():
    """Keys just outside the window hold huge values; any leak shows."""
    dev, ops = need_gpu(), _ops()
    for impl, dtype in (("mma", torch.bfloat16), ("tcgen05", torch.bfloat16), ("simple", torch.float32)):
        for window in (1, 16, 17, 64, 65):
            err = _attention_case(ops, dev, dtype, impl, 4, 2, 64, 16, window, [(0, 190, 10), (1, 99, 1)], [200, 100])
            assert err < (0.03 if dtype == torch.bfloat16 else 2e-5)


@pytest.mark.parametrize("nq,nkv,d,page", [(8, 2, 128, 16), (6, 6, 64, 8), (10, 2, 128, 64), (4, 1, 64, 128), (3, 1, 128, 32)])
@pytest.mark.parametrize("window", [None, 1, 130, 300])
def test_attention_tcgen05_long_portions(nq, nkv, d, page, window):
    """Portions of several 128-row tiles over several 128-key tiles, starting inside a page and inside a tile;
    windows that end inside a tile and span more than one; a single token beside them goes to the decode kernel."""
    dev, ops = need_gpu(), _ops()
    lengths = [700, 131, 1029, 40]
    segs = [(0, 100, 600), (1, 0, 131), (2, 517, 512), (3, 39, 1)]
    err = _attention_case(ops, dev, torch.bfloat16, "tcgen05", nq, nkv, d, page, window, segs, lengths, seed=nq + page)
    assert err < 0.03


@pytest.mark.parametrize("nq,nkv,d,page", [(8, 2, 128, 16), (6, 6, 64, 8), (16, 1, 64, 64), (32, 8, 128, 16), (5, 5, 128, 32), (12, 2, 64, 16)])
@pytest.mark.parametrize("window", [None, 300])
@pytest.mark.parametrize("norm,rot,span_min,pair_cost", [(True, 1.0, 2, 0), (True, 0.5, 1, 1), (False, 1.0, 3, 2), (True, 0.0, 40, 5)])
def test_attention_decode_fused_matches_the_separate_kernels(nq, nkv, d, page, window, norm, rot, span_min, pair_cost):
    """A step of single tokens with per-head norm, rotation and the page write done inside the tcgen05 decode kernel,
    against the separate kernels (qk_norm_rope_write, then the mma.sync attention): the same keys and values in the
    pages (values bitwise, keys to one rounding), untouched pages untouched, the same attention output; requests of 1
    to 1,300 keys, so that the newest key sits in a first, a middle and a last tile, and spans of at least 1, 2, 3 and
    40 units with 0 to 5 units of cost per pair, so that requests are cut in different places or not at all.  Both
    calls share one workspace."""
    dev, ops = need_gpu(), _ops()
    lengths = [1, 17, 128, 129, 700, 1300, 513, 64]
    segs = [(i, n - 1, 1) for i, n in enumerate(lengths)]
    kv = PagedKV(lengths, nkv, d, page, torch.bfloat16, dev, seed=nq + d, fill_garbage=False)
    meta = segments_to_device(segs, dev)
    T = meta["T"]
    g = torch.Generator().manual_seed(d + page)
    qkv = torch.randn(T, (nq + 2 * nkv) * d, generator=g).to(torch.bfloat16).to(dev)
    qw = (1 + 0.3 * torch.randn(d, generator=g)).to(torch.bfloat16).to(dev) if norm else None
    kw = (1 + 0.3 * torch.randn(d, generator=g)).to(torch.bfloat16).to(dev) if norm else None
    pairs = int(d // 2 * rot)
    cos = sin = None
    if pairs:
        ang = torch.rand(T, pairs, generator=g) * 6.28
        cos, sin = torch.cos(ang).to(dev), torch.sin(ang).to(dev)
    eps, scale = 1e-5, 1.0 / math.sqrt(d)
    split_keys = 256
    splits = max(ops.attention_num_splits(st, window, split_keys) for _, st, _ in segs)
    err1 = torch.zeros(1, dtype=torch.int32, device=dev)
    err2 = torch.zeros(1, dtype=torch.int32, device=dev)

    def scratch():
        return (torch.empty(T * nq * splits * d, dtype=torch.float32, device=dev),
                torch.empty(T * nq * splits * 2, dtype=torch.float32, device=dev))
    # the separate kernels
    k1, v1, q1 = kv.kcache.clone(), kv.vcache.clone(), qkv.clone()
    ops.qk_norm_rope_write(q1, qw, kw, eps, cos, sin, True, k1, v1, kv.table_dev, meta["token_slot"], meta["positions"], page,
                           nq, nkv, d, err1)
    acc, ml = scratch()
    want = ops.attention_mma(q1, q1.shape[1], k1, v1, kv.table_dev, meta["seg_off"], meta["seg_slot"], meta["seg_start"],
                             meta["seg_len"], meta["token_seg"], T, T, 1, False, True, splits, acc, ml, nq, nkv, d, page, window,
                             scale, split_keys=split_keys, decode_on_tcgen05=False)
    # one kernel; its workspace starts as NaN: a piece that is read without having been written shows
    ws = ops.attention_decode_workspace(d, dev)
    ws.acc.fill_(float("nan")); ws.ml.fill_(float("nan"))
    k2, v2 = kv.kcache.clone(), kv.vcache.clone()
    got = ops.attention_decode_fused(qkv.clone(), k2, v2, kv.table_dev, meta["seg_off"], meta["seg_slot"], meta["seg_start"],
                                     meta["seg_len"], T, nq, nkv, d, page, window, scale, qw, kw, eps, cos, sin, err2,
                                     workspace=ws, span_min=span_min, pair_cost=pair_cost)
    assert ops.attention_tcgen05_status(d) == 0 and int(err1.item()) == 0 and int(err2.item()) == 0
    assert int(ws.count.abs().sum().item()) == 0                          # the counters are left ready for the next launch
    assert torch.isfinite(got.float()).all()
    assert torch.equal(v2, v1)                                           # values: a copy
    kd = (k2.float() - k1.float()).abs()
    assert float(kd.max()) <= 2 ** -7 * float(k1.float().abs().max())    # keys: the same arithmetic, at most a rounding apart
    changed = (k2 != kv.kcache).flatten(2).any(-1).sum().item()          # (page, head) rows that were written
    assert 0 < changed <= T * nkv
    diff = float((got.float() - want.float()).abs().max())
    assert diff <= 2e-2 * float(want.float().abs().max()) + 1e-3, diff
    # a missing page is counted, not written
    bad = kv.table_dev.clone()
    bad[5, (lengths[5] - 1) // page] = -1
    k3, v3 = kv.kcache.clone(), kv.vcache.clone()
    ops.attention_decode_fused(qkv.clone(), k3, v3, bad, meta["seg_off"], meta["seg_slot"], meta["seg_start"], meta["seg_len"],
                               T, nq, nkv, d, page, window, scale, qw, kw, eps, cos, sin, err2, workspace=ws, span_min=span_min, pair_cost=pair_cost)
    assert int(err2.item()) == nkv and ops.attention_tcgen05_status(d) == 0
    assert int(ws.count.abs().sum().item()) == 0


@pytest.mark.parametrize("nq,nkv,d,page", [(8, 2, 128, 16), (32, 8, 128, 16), (12, 3, 64, 8), (16, 1, 64, 64), (40, 8, 128, 32)])
@pytest.mark.parametrize("window", [None, 700])
@pytest.mark.parametrize("span_min,pair_cost", [(1, 0), (4, 2), (7, 1), (2, 9)])
def test_attention_decode_spans_of_unequal_requests(nq, nkv, d, page, window, span_min, pair_cost, monkeypatch):
    """The tcgen05 decode kernel gives every CTA an equal span of the step's key tiles: requests of 3 to 5,000 keys in
    one step (some inside one span, some cut two or twenty times), against the dense reference.  One key far back in
    the longest request is made to stand out, so a piece that is dropped or counted twice shows; a prompt portion in
    the same step is not touched by the decode kernel's spans; three launches share one workspace."""
    dev, ops = need_gpu(), _ops()
    monkeypatch.setattr(ops.kernels, "DECODE_SPAN_MIN", span_min)
    monkeypatch.setattr(ops.kernels, "DECODE_PAIR_COST", pair_cost)
    lengths = [5000, 3, 129, 1200, 77, 2047, 640, 128, 300, 1]
    ws = ops.attention_decode_workspace(d, dev)
    ws.acc.fill_(float("nan")); ws.ml.fill_(float("nan"))
    decodes = [(i, n - 1, 1) for i, n in enumerate(lengths)]
    others = [sg for sg in decodes if sg[0] != 8]
    steps = [decodes, [sg for sg in decodes if sg[0] in (0, 3, 4, 9)], others[:5] + [(8, 100, 200)] + others[5:]]
    for call, segs in enumerate(steps):
        spike = (0, 1234 if window is None else 4500, nq - 1)
        err = _attention_case(ops, dev, torch.bfloat16, "tcgen05", nq, nkv, d, page, window, segs, lengths, seed=call + nq,
                              spike=spike, decode_ws=ws)
        assert err < 0.03, (call, err)
        assert int(ws.count.abs().sum().item()) == 0


@pytest.mark.parametrize("nq,nkv,d,page", [(8, 2, 128, 16), (12, 3, 64, 8), (16, 1, 64, 64)])
@pytest.mark.parametrize("fused", [False, True])
def test_attention_decode_reads_no_shared_memory_it_has_not_written(nq, nkv, d, page, fused, monkeypatch):
    """The pages behind the end of a request's last key tile are never loaded into the decode kernel's ring, and what
    lies there in shared memory must not reach the output (a probability of exactly zero times a NaN is a NaN).  A test
    build of the library fills every SM's shared memory with NaN bit patterns right before the kernel runs; requests
    whose lengths end anywhere in a tile - one key, a page, a tile less one, several tiles and a bit - must still give
    the reference's output.  (Checked once that a kernel which neither clears its ring nor those rows fails here.)"""
    import ctypes
    dev, ops = need_gpu(), _ops()
    from pulse_infer_b200.csrc import build
    monkeypatch.setenv("PULSE_NVCC_FLAGS", "-DFD_POISON_TEST")
    test_lib = ctypes.CDLL(build.library_path("attention_tcgen05", d))
    monkeypatch.delenv("PULSE_NVCC_FLAGS")
    lengths = [1, page, page + 1, 127, 128, 129, 200, 383, 700, 1025]
    segs = [(i, n - 1, 1) for i, n in enumerate(lengths)]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for window in (None, 150):
        if fused:
            kv = PagedKV(lengths, nkv, d, page, torch.bfloat16, dev, seed=d + page, fill_garbage=False)
            meta = segments_to_device(segs, dev)
            T = meta["T"]
            g = torch.Generator().manual_seed(page)
            qkv = torch.randn(T, (nq + 2 * nkv) * d, generator=g).to(torch.bfloat16).to(dev)
            err = torch.zeros(1, dtype=torch.int32, device=dev)
            k1, v1, q1 = kv.kcache.clone(), kv.vcache.clone(), qkv.clone()
            ops.qk_norm_rope_write(q1, None, None, 1e-6, None, None, True, k1, v1, kv.table_dev, meta["token_slot"],
                                   meta["positions"], page, nq, nkv, d, err)
            splits = max(ops.attention_num_splits(st, window, 256) for _, st, _ in segs)
            acc = torch.empty(T * nq * splits * d, dtype=torch.float32, device=dev)
            ml = torch.empty(T * nq * splits * 2, dtype=torch.float32, device=dev)
            want = ops.attention_mma(q1, q1.shape[1], k1, v1, kv.table_dev, meta["seg_off"], meta["seg_slot"], meta["seg_start"],
                                     meta["seg_len"], meta["token_seg"], T, T, 1, False, True, splits, acc, ml, nq, nkv, d, page,
                                     window, 1.0 / math.sqrt(d), split_keys=256, decode_on_tcgen05=False)
            ws = ops.attention_decode_workspace(d, dev)
            assert test_lib.pi_attention_tcgen05_test_poison_shared(stream) == 0
            torch.cuda.synchronize()
            got = ops.attention_decode_fused(qkv.clone(), kv.kcache.clone(), kv.vcache.clone(), kv.table_dev, meta["seg_off"],
                                             meta["seg_slot"], meta["seg_start"], meta["seg_len"], T, nq, nkv, d, page, window,
                                             1.0 / math.sqrt(d), None, None, 1e-6, None, None, err, workspace=ws)
            assert torch.isfinite(got.float()).all()
            assert float((got.float() - want.float()).abs().max()) <= 2e-2 * float(want.float().abs().max()) + 1e-3
        else:
            orig = ops.kernels.attention_mma

            def poisoned(*a, **kw):
                orig(*a, **kw)                                     # libraries loaded, workspace kernels out of the way
                assert test_lib.pi_attention_tcgen05_test_poison_shared(stream) == 0
                torch.cuda.synchronize()
                return orig(*a, **kw)
            monkeypatch.setattr(ops, "attention_mma", poisoned)
            err = _attention_case(ops, dev, torch.bfloat16, "tcgen05", nq, nkv, d, page, window, segs, lengths, seed=3)
            monkeypatch.setattr(ops, "attention_mma", orig)
            assert err < 0.03, err                     # NaN compares false
    assert ops.attention_tcgen05_status(d) == 0


@pytest.mark.parametrize("seed", list(range(24)))
def test_attention_decode_spans_random_steps(seed, monkeypatch):
    """Random decode steps for the tcgen05 decode kernel: 1 to 24 requests of 1 to 3,000 keys (many short ones, a few
    long ones), 1 to 8 kv heads with groups of 1 to 16, both head sizes, every page size, with and without a window,
    random span and cost settings - against the dense reference, on one workspace per head size that every case of
    the run shares."""
    dev, ops = need_gpu(), _ops()
    rng = np.random.RandomState(1000 + seed)
    d = int(rng.choice([64, 128]))
    page = int(rng.choice([8, 16, 32, 64]))
    nkv = int(rng.choice([1, 2, 3, 8]))
    group = int(rng.choice([1, 2, 4, 5, 8, 16]))
    if nkv * group > 32:
        group = 4
    nq = nkv * group
    window = None if rng.rand() < 0.5 else int(rng.randint(100, 3000))
    count = int(rng.randint(1, 25))
    lengths = [int(rng.randint(1, 3001)) if rng.rand() < 0.3 else int(rng.randint(1, 200)) for _ in range(count)]
    monkeypatch.setattr(ops.kernels, "DECODE_SPAN_MIN", int(rng.choice([1, 2, 4])))
    monkeypatch.setattr(ops.kernels, "DECODE_PAIR_COST", int(rng.choice([0, 1, 2, 4])))
    ws = _SHARED_DECODE_WS.get(d)
    if ws is None:
        ws = _SHARED_DECODE_WS[d] = ops.attention_decode_workspace(d, dev)
        ws.acc.fill_(float("nan")); ws.ml.fill_(float("nan"))
    segs = [(i, n - 1, 1) for i, n in enumerate(lengths)]
    order = rng.permutation(count)
    segs = [segs[i] for i in order]                       # the step need not list its requests in slot order
    longest = int(np.argmax(lengths))
    spike = None
    if lengths[longest] > 300:
        lo = 0 if window is None else max(0, lengths[longest] - window)
        spike = (longest, int(rng.randint(lo, lengths[longest] - 1)), int(rng.randint(0, nq)))
    err = _attention_case(ops, dev, torch.bfloat16, "tcgen05", nq, nkv, d, page, window, segs, lengths, seed=seed, spike=spike,
                          decode_ws=ws)
    assert err < 0.03, (seed, nq, nkv, d, page, window, lengths, err)
    assert int(ws.count.abs().sum().item()) == 0


_SHARED_DECODE_WS: dict = {}


@pytest.mark.parametrize("nq,nkv,d,page", [(8, 2, 128, 16), (6, 6, 64, 8), (4, 1, 64, 128), (32, 8, 128, 16)])
@pytest.mark.parametrize("window", [None, 130, 900])
@pytest.mark.parametrize("shares", [2, 3, 7, 16])
def test_attention_tcgen05_portions_with_shared_keys(nq, nkv, d, page, window, shares):
    """Short portions behind long contexts with the key tiles of every query block cut into shares (2 to 16 CTAs a
    block; with 16 some shares of the short contexts are empty), combined by the merge kernel; a single token beside
    them is untouched by it.  One key far back is made to stand out, so a share that is dropped or counted twice shows."""
    dev, ops = need_gpu(), _ops()
    lengths = [2300, 131, 1500, 40]
    segs = [(0, 2200, 100), (1, 0, 131), (2, 1400, 40), (3, 39, 1)]
    err = _attention_case(ops, dev, torch.bfloat16, "tcgen05", nq, nkv, d, page, window, segs, lengths, seed=nq + shares,
                          spike=(0, 5, nq - 1) if window is None else (0, 2300 - window + 3, nq - 1), prompt_splits=shares)
    assert err < 0.03


def test_prompt_shares_are_chosen_from_the_step():
    """CPU arithmetic of ``choose_prompt_splits``: shares only when the query blocks leave SMs idle and contexts are long."""
    ops = _ops()
    sms = ops.kernels.sm_count()
    assert ops.choose_prompt_splits([], 4, 8, None) == 1
    assert ops.choose_prompt_splits([(0, 2048)], 4, 8, None) == 1                    # 256 blocks: the GPU is full
    assert ops.choose_prompt_splits([(100, 128)], 4, 8, None) == 1                   # two key tiles: nothing to share
    few = ops.choose_prompt_splits([(16384, 128)], 4, 8, None)                       # 16 CTAs walking 129 key tiles
    assert few == min(sms // 16, 16)
    assert ops.choose_prompt_splits([(16384, 128)], 4, 8, 1024) == min(sms // 16, (1152 + 127) // 128 // 4, 16)


@pytest.mark.parametrize("M,N,K", [(1, 515, 96), (33, 515, 100), (64, 64, 16), (130, 77, 1000), (7, 4096, 4096)])
def test_gemm_f32_true_32bit(M, N, K):
    dev, ops = need_gpu(), _ops()
    g = torch.Generator().manual_seed(M + N)
    x, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    out = ops.gemm_f32(x.to(dev), w.to(dev)).cpu()
    want = x.double() @ w.double().t()
    bound = 2e-7 * K * float((x.abs().double() @ w.abs().double().t()).max())     # k roundings of eps/2
    assert float((out.double() - want).abs().max()) <= bound
    # tf32 would be off by about 1e-3 relative; make sure we are nowhere near
    assert float((out.double() - want).abs().max()) <= 1e-5 * float(want.abs().max()) * math.sqrt(K)
    # a row's result does not depend on the rows around it
    one = ops.gemm_f32(x[M // 2:M // 2 + 1].contiguous().to(dev), w.to(dev)).cpu()
    assert torch.equal(one[0], out[M // 2])


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("N,K", [(515, 96), (4096, 4096), (64, 8), (1000, 12288), (50, 200)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_small_m(M, N, K, out_dtype):
    dev, ops = need_gpu(), _ops()
    g = torch.Generator().manual_seed(M * 1000 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    out = ops.gemm_small_m(x.to(dev), w.to(dev), out_dtype).cpu()
    want = x.double() @ w.double().t()
    err = float((out.double() - want).abs().max())
    scale = float(want.abs().max())
    assert err <= (2e-5 if out_dtype == torch.float32 else 2 ** -8) * scale + 1e-6
    # a row's result does not depend on the rows around it: bitwise while the launch shape is the same (up to 8
    # rows here), to rounding when more rows pick another split of K
    if M > 1:
        one = ops.gemm_small_m(x[M - 1:].contiguous().to(dev), w.to(dev), out_dtype).cpu()
        if M <= 8:
            assert torch.equal(one[0], out[M - 1])
        else:
            assert float((one[0].double() - out[M - 1].double()).abs().max()) <= 2 ** -7 * scale


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1, 256, 128), (300, 515, 200), (257, 1000, 4096), (2048, 1024, 1024)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05(M, N, K, out_dtype):
    """The tcgen05 / TMEM / TMA product against a float64 product; every bounded wait must have been met."""
    dev, ops = need_gpu(), _ops()
    g = torch.Generator().manual_seed(M + N + K)
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.5).to(torch.bfloat16)
    out = ops.gemm_tcgen05(x.to(dev), w.to(dev), out_dtype).cpu()
    assert ops.gemm_tcgen05_status() == 0
    want = x.double() @ w.double().t()
    scale = float(want.abs().max())
    assert float((out.double() - want).abs().max()) <= (1e-5 if out_dtype == torch.float32 else 2 ** -8) * scale + 1e-6
    # fewer CTAs than tiles: the persistent loop and both accumulator buffers are exercised
    again = ops.gemm_tcgen05(x.to(dev), w.to(dev), out_dtype, max_ctas=3).cpu()
    assert ops.gemm_tcgen05_status() == 0 and torch.equal(again, out)


def test_gemm_tcgen05_wait_that_runs_out_is_reported_and_the_next_launch_works(monkeypatch, model_folders):
    """The give-up path of the bounded waits, made to run: a test build of the product (a small poll limit, and a
    hook that makes the producer leave out the loads of one pipeline stage - a barrier that nothing completes) is
    put in place of the engine's library.  The launch returns, the status word names the wait of the MMA warp on that
    stage, the step function's error check raises, and the launch after that is right again with status 0.
    Nothing traps and nothing spins without a limit: every role falls through to the common exit, which frees the
    tensor memory; no copy and no MMA is in flight at that point (the only loads of the problem were left out)."""
    import ctypes
    dev, ops = need_gpu(), _ops()
    from pulse_infer_b200.csrc import build
    from pulse_infer_b200.engine import StepError
    from test_gpu_engine import _runner
    monkeypatch.setenv("PULSE_NVCC_FLAGS", "-DTC_TEST_HOOKS -DTC_SPIN_LIMIT=65536")
    test_lib = ctypes.CDLL(build.library_path("gemm_tcgen05"))
    monkeypatch.delenv("PULSE_NVCC_FLAGS")
    test_lib.pi_last_error.restype = ctypes.c_char_p
    test_lib.pi_gemm_tcgen05_spin_limit.restype = ctypes.c_uint
    assert test_lib.pi_gemm_tcgen05_spin_limit() == 65536
    regular = ops.kernels._lib("gemm_tcgen05")
    with pytest.raises(AttributeError):
        regular.pi_gemm_tcgen05_test_skip_load                                   # the engine's library has no such hook
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(128, 64, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    w = (torch.randn(256, 64, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    want = (x.double() @ w.double().t()).cpu()
    runner = _runner(model_folders["D"], "bfloat16")
    assert ops.gemm_tcgen05_status() == 0
    monkeypatch.setitem(ops.kernels._LIBS, ("gemm_tcgen05", None), test_lib)
    # a normal launch of the test build is right
    out = ops.gemm_tcgen05(x, w, torch.float32)
    assert ops.gemm_tcgen05_status() == 0
    assert float((out.cpu().double() - want).abs().max()) <= 1e-5 * float(want.abs().max()) + 1e-6
    # the next launch leaves out the loads of its only stage (one tile, one k step)
    test_lib.pi_gemm_tcgen05_test_skip_load(ctypes.c_int(0))
    ops.gemm_tcgen05(x, w, torch.float32, out=torch.zeros_like(out))
    torch.cuda.synchronize()                                                  # the kernel gave up and returned
    with pytest.raises(StepError, match="tcgen05 product"):
        runner.check_device_errors()                                          # reads (and clears) the status word
    # what the status word held: code 3 (MMA warp waiting for a loaded stage), iteration 0
    test_lib.pi_gemm_tcgen05_test_skip_load(ctypes.c_int(0))
    ops.gemm_tcgen05(x, w, torch.float32, out=torch.zeros_like(out))
    assert ops.gemm_tcgen05_status() == (3 << 24) | 0
    # and the launch after it works, status 0
    out = ops.gemm_tcgen05(x, w, torch.float32)
    assert ops.gemm_tcgen05_status() == 0
    assert float((out.cpu().double() - want).abs().max()) <= 1e-5 * float(want.abs().max()) + 1e-6
    runner.check_device_errors()


@pytest.mark.parametrize("M,I,K", [(1, 224, 192), (8, 12288, 256), (5, 8, 64), (16, 1000, 520), (32, 176, 4096)])
def test_gemm_small_m_gated_epilogue(M, I, K):
    """The weight-streaming product with SiLU(gate) * up as its epilogue, against float64."""
    dev, ops = need_gpu(), _ops()
    g = torch.Generator().manual_seed(M + I)
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    gate = (torch.randn(I, K, generator=g) * 0.3).to(torch.bfloat16)
    up = (torch.randn(I, K, generator=g) * 0.3).to(torch.bfloat16)
    w = ops.interleave_gate_up(gate.to(dev), up.to(dev))
    out = ops.gemm_small_m(x.to(dev), w, torch.bfloat16, gated=True).cpu()
    assert out.shape == (M, I) and out.dtype == torch.bfloat16
    want = plain_model.silu((x.double() @ gate.double().t()).numpy()) * (x.double() @ up.double().t()).numpy()
    assert np.abs(out.double().numpy() - want).max() <= 2 ** -8 * np.abs(want).max() + 1e-6
    # the unfused route gives the same values up to the extra rounding of the [M, 2I] intermediate
    two = ops.silu_mul(ops.gemm_small_m(x.to(dev), w, torch.bfloat16), blocked=True).cpu()
    assert np.abs(two.double().numpy() - want).max() <= 2 ** -6 * np.abs(want).max() + 1e-6


@pytest.mark.parametrize("M,H,N,K", [(1, 4096, 6144, 1024), (8, 200, 515, 96), (16, 1024, 4096, 520), (13, 48, 224, 4104), (5, 16, 16, 8)])
@pytest.mark.parametrize("wdt", [torch.bfloat16, torch.float32])
def test_gemm_small_m_prepares_and_finishes_a_norm(M, H, N, K, wdt):
    """h += a W1^T as the epilogue of a product that also prepares the RMSNorm of the new h; the next product
    finishes that norm: norm(h) W2^T, plain and with SiLU * up behind it.  Each against float64."""
    dev, ops = need_gpu(), _ops()
    g = torch.Generator().manual_seed(M * 7 + N)
    a = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    w1 = (torch.randn(H, K, generator=g) * 0.3).to(torch.bfloat16)
    h0 = torch.randn(M + 2, H + 8, generator=g) * 3
    h0[1] *= 40.0                                             # rows of very different size: the scale is per row
    nw = (1 + 0.2 * torch.randn(H, generator=g)).to(wdt)
    w2 = (torch.randn(N, H, generator=g) * 0.3).to(torch.bfloat16)
    eps = 1e-5
    # the residual epilogue alone: r += x W^T in 32-bit, nothing else touched
    hd = h0.clone().to(dev)
    assert ops.linear(a.to(dev), w1.to(dev), torch.bfloat16, residual=hd[1:M + 1, :H]) is None
    want_h = h0.double()
    want_h[1:M + 1, :H] += a.double() @ w1.double().t()
    bound = 4e-6 * float((a.abs().double() @ w1.abs().double().t()).max() + h0.abs().max()) + 1e-6
    assert float((hd.cpu().double() - want_h).abs().max()) <= bound
    assert torch.equal(hd.cpu()[0], h0[0]) and torch.equal(hd.cpu()[:, H:], h0[:, H:])
    # with the next norm prepared: the same residual, and a description that the next product finishes
    hd2 = h0[1:M + 1, :H].contiguous().to(dev)
    owner = object()
    rows = ops.linear(a.to(dev), w1.to(dev), torch.bfloat16, residual=hd2, next_norm=(nw.to(dev), eps, owner))
    assert isinstance(rows, ops.NormedRows) and rows.owner is owner and torch.equal(hd2.cpu(), hd.cpu()[1:M + 1, :H])
    normed = plain_model.rms_norm(want_h[1:M + 1, :H].numpy(), nw.double().numpy(), eps)
    want = normed @ w2.double().numpy().T
    out = ops.linear(rows, w2.to(dev), torch.bfloat16).cpu()
    assert out.dtype == torch.bfloat16 and np.abs(out.double().numpy() - want).max() <= 2 ** -7 * np.abs(want).max() + 1e-6
    # the unfused route (norm kernel, then the product) agrees to bf16 rounding, and materialize() is that norm
    x = rows.materialize()
    assert np.abs(x.cpu().double().numpy() - normed).max() <= 2 ** -8 * np.abs(normed).max()
    two = ops.gemm_small_m(x, w2.to(dev), torch.bfloat16).cpu()
    assert np.abs(two.double().numpy() - want).max() <= 2 ** -6 * np.abs(want).max() + 1e-6
    if N % 16 == 0:                                           # finishing the norm + gated epilogue
        I = N // 2
        want_g = plain_model.silu(normed @ w2[:I].double().numpy().T) * (normed @ w2[I:].double().numpy().T)
        wi = ops.interleave_gate_up(w2[:I].contiguous().to(dev), w2[I:].contiguous().to(dev))
        got = ops.gemm_small_m(rows.scaled, wi, torch.bfloat16, gated=True, row_ssq=(rows.partials, rows.eps)).cpu()
        # gate and up each carry the rounding of the bf16 inputs (2^-9 an element, not averaged out when H is 16),
        # their product carries both, and the result is rounded once more
        assert got.shape == (M, I) and np.abs(got.double().numpy() - want_g).max() <= 2 ** -6 * np.abs(want_g).max() + 1e-6


@pytest.mark.parametrize("M,I,K", [(200, 224, 192), (130, 200, 64)])
def test_gemm_tcgen05_gated_epilogue(M, I, K):
    dev, ops = need_gpu(), _ops()
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    gate = (torch.randn(I, K, generator=g) * 0.3).to(torch.bfloat16)
    up = (torch.randn(I, K, generator=g) * 0.3).to(torch.bfloat16)
    w = ops.interleave_gate_up(gate.to(dev), up.to(dev))
    out = ops.gemm_tcgen05(x.to(dev), w, torch.bfloat16, gated=True).cpu()
    assert ops.gemm_tcgen05_status() == 0 and out.shape == (M, I)
    want = plain_model.silu((x.double() @ gate.double().t()).numpy()) * (x.double() @ up.double().t()).numpy()
    assert np.abs(out.double().numpy() - want).max() <= 2 ** -7 * np.abs(want).max()


def test_linear_bfloat16_and_mixed():
    dev, ops = need_gpu(), _ops()
    g = torch.Generator().manual_seed(0)
    x = torch.randn(17, 200, generator=g).to(torch.bfloat16)
    w = torch.randn(515, 200, generator=g).to(torch.bfloat16)
    want = x.double() @ w.double().t()
    y32 = ops.linear(x.to(dev), w.to(dev), torch.float32).cpu()
    assert y32.dtype == torch.float32 and float((y32.double() - want).abs().max()) < 1e-3
    yb = ops.linear(x.to(dev), w.to(dev), torch.bfloat16).cpu()
    assert yb.dtype == torch.bfloat16 and float((yb.double() - want).abs().max()) < 0.02 * float(want.abs().max())
    yf = ops.linear(x.to(dev), w.float().to(dev), torch.bfloat16).cpu()      # a weight kept in 32-bit
    assert float((yf.double() - want).abs().max()) < 0.02 * float(want.abs().max())


def test_argmax_lowest_index_wins():
    dev, ops = need_gpu(), _ops()
    logits = torch.randn(6, 151936, generator=torch.Generator().manual_seed(0))
    logits[0, 777] = 50.0; logits[0, 90000] = 50.0
    logits[1, 151935] = 60.0
    logits[2, 0] = 60.0
    logits[3, 5] = float("nan"); logits[3, 6] = 70.0
    got = ops.argmax(logits.to(dev)).cpu().tolist()
    assert got[:4] == [777, 151935, 0, 6]
    assert got[4:] == [plain_model.greedy(logits[i].numpy()) for i in (4, 5)]
    small = torch.tensor([[1.0, 3.0, 3.0, 2.0, 3.0]] * 2)
    assert ops.argmax(small.to(dev)).cpu().tolist() == [1, 1]


def _sample(ops, dev, logits, temp, k, p, seed, counters):
    n = logits.shape[0]
    f = lambda v, dt: torch.full((n,), v, dtype=dt, device=dev)  # noqa: E731
    return ops.sample(logits.to(dev), f(temp, torch.float32), f(k, torch.int32), f(p, torch.float32),
                      f(seed, torch.int64), torch.tensor(counters, dtype=torch.int64, device=dev)).cpu().tolist()


@pytest.mark.parametrize("vocab", [515, 40000])
@pytest.mark.parametrize("temp,k,p", [(0.8, 0, 0.0), (1.3, 20, 0.0), (0.6, 20, 0.95), (1.0, 0, 0.5), (0.7, 1, 0.0)])
def test_sampling_matches_plain_sampler(vocab, temp, k, p):
    dev, ops = need_gpu(), _ops()
    base = torch.randn(vocab, generator=torch.Generator().manual_seed(vocab)) * 2.5
    base[3] = base[11] = base.max() + 0.5                      # a tie at the top
    n = 64
    logits = base.repeat(n, 1).contiguous()
    counters = list(range(n))
    got = _sample(ops, dev, logits, temp, k, p, 1234, counters)
    order, _ = plain_model.kept_set(base.double().numpy(), temp, k, p)
    assert set(got) <= set(order)
    # same uniform numbers, same walk: tokens agree except where rounding of the cumulative sums decides
    want = [plain_model.sample(base.double().numpy(), temp, k, p, 1234, c) for c in counters]
    agree = sum(int(a == b) for a, b in zip(got, want))
    assert agree >= n - 2
    assert _sample(ops, dev, logits[:4], 0.0, k, p, 1, [0, 1, 2, 3]) == [3, 3, 3, 3]   # temperature 0 is greedy


def test_sampling_distribution():
    dev, ops = need_gpu(), _ops()
    base = torch.tensor([2.0, 1.0, 0.0, -1.0, 1.5, -30.0])
    n = 4000
    got = _sample(ops, dev, base.repeat(n, 1).contiguous(), 1.0, 0, 0.0, 99, list(range(n)))
    freq = np.bincount(got, minlength=6) / n
    prob = torch.softmax(base.double(), 0).numpy()
    assert np.abs(freq - prob).max() < 0.03
    # the draw depends on (seed, counter) only, not on the row's place in the batch
    again = _sample(ops, dev, base.repeat(5, 1).contiguous(), 1.0, 0, 0.0, 99, [7, 7, 3, 7, 3])
    assert again[0] == again[1] == again[3] == got[7] and again[2] == again[4] == got[3]


def test_logit_edit():
    dev, ops = need_gpu(), _ops()
    logits = torch.zeros(3, 100, device=dev)
    mk = lambda v, dt: torch.tensor(v, dtype=dt, device=dev)  # noqa: E731
    ops.logit_edit(logits, mk([0, 2, 2], torch.int32), mk([5, 7, 99], torch.int32), mk([-1.5, -1.5, -1.5], torch.float32), False)
    ops.logit_edit(logits, mk([1], torch.int32), mk([0], torch.int32), mk([float("-inf")], torch.float32), True)
    out = logits.cpu()
    assert out[0, 5] == -1.5 and out[2, 7] == -1.5 and out[2, 99] == -1.5 and out[1, 0] == float("-inf")
    assert out.isfinite().sum() == 299 and (out == 0).sum() == 296


def test_kernels_refuse_what_they_do_not_take():
    """A size or layout a kernel does not take is refused with a message, never computed wrongly."""
    dev, ops = need_gpu(), _ops()
    KernelError = ops.KernelError
    bf = lambda *shape: torch.zeros(*shape, dtype=torch.bfloat16, device=dev)       # noqa: E731
    i32 = lambda *v: torch.tensor(v, dtype=torch.int32, device=dev)                 # noqa: E731
    # tcgen05 prompt attention: page sizes 8..128 only, head sizes 64 / 128 only, bfloat16 only
    kc, vc = bf(4, 2, 4, 64), bf(4, 2, 4, 64)
    args = (bf(8, 4 * 64), 4 * 64, kc, vc, i32(0, 1).view(1, 2), i32(0), i32(0), i32(0), i32(8), 8, 1, 8, 4, 2, 64)
    with pytest.raises(KernelError, match="page size"):
        ops.attention_tcgen05(*args, 4, None, 0.125, bf(8, 4 * 64))
    with pytest.raises(Exception, match="head size"):
        ops.attention_tcgen05(bf(8, 4 * 48), 4 * 48, bf(4, 2, 8, 48), bf(4, 2, 8, 48), i32(0, 1).view(1, 2), i32(0), i32(0),
                              i32(0), i32(8), 8, 1, 8, 4, 2, 48, 8, None, 0.125, bf(8, 4 * 48))
    with pytest.raises(KernelError, match="bfloat16"):
        ops.attention_tcgen05(args[0].float(), *args[1:], 8, None, 0.125, bf(8, 4 * 64))
    assert not ops.attention_tcgen05_usable(96, 16) and not ops.attention_decode_tcgen05_usable(128, 16, 20)
    assert not ops.attention_decode_tcgen05_usable(128, 128, 4)
    # weight-streaming product: at most 32 rows, k a multiple of 8, the fused forms only in their combinations
    w = bf(64, 64)
    with pytest.raises(KernelError, match="at most 32"):
        ops.gemm_small_m(bf(33, 64), w, torch.bfloat16)
    with pytest.raises(KernelError, match="multiples of 8"):
        ops.gemm_small_m(bf(4, 60), bf(64, 60), torch.bfloat16)
    with pytest.raises(KernelError, match="gated"):
        ops.gemm_small_m(bf(4, 64), bf(24, 64), torch.bfloat16, gated=True)          # 24 rows: not whole blocks of 16
    with pytest.raises(KernelError, match="residual"):
        ops.gemm_small_m(bf(4, 64), w, torch.float32, residual=torch.zeros(4, 32, device=dev))
    with pytest.raises(KernelError, match="residual"):
        ops.gemm_small_m(bf(4, 64), w, torch.bfloat16, emit_norm=bf(64))
    # tcgen05 product: bfloat16 operands, gated output needs whole blocks
    with pytest.raises(KernelError, match="bfloat16"):
        ops.gemm_tcgen05(torch.zeros(4, 64, device=dev), w)
    with pytest.raises(KernelError, match="gated"):
        ops.gemm_tcgen05(bf(4, 64), bf(24, 64), torch.bfloat16, gated=True)
    # nothing above left an error behind
    assert ops.gemm_tcgen05_status() == 0 and ops.attention_tcgen05_loaded_status() == 0
