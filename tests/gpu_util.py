"""Helpers of the GPU tests: a randomly paged key/value cache and dense references of the kernels."""
import math

import numpy as np
import torch


def need_gpu():
    import pytest
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


class PagedKV:
    """Keys and values of several sequences scattered over pages in a shuffled order."""

    def __init__(self, lengths, nkv, d, page_size, dtype, device, seed=0, extra_pages=3, fill_garbage=True):
        g = torch.Generator().manual_seed(seed)
        self.lengths, self.nkv, self.d, self.page_size = list(lengths), nkv, d, page_size
        pages_per = [(n + page_size - 1) // page_size for n in lengths]
        total = sum(pages_per) + extra_pages
        perm = torch.randperm(total, generator=g).tolist()
        max_pages = max(pages_per) + 2
        self.table = torch.full((len(lengths), max_pages), -1, dtype=torch.int32)
        self.k_dense = [torch.randn(n, nkv, d, generator=g) for n in lengths]
        self.v_dense = [torch.randn(n, nkv, d, generator=g) for n in lengths]
        # pages start out holding large garbage: a kernel that reads beyond a sequence's end shows up
        kc = torch.full((total, nkv, page_size, d), 1e4 if fill_garbage else 0.0)
        vc = torch.full((total, nkv, page_size, d), -1e4 if fill_garbage else 0.0)
        at = 0
        for s, n in enumerate(lengths):
            for i in range(pages_per[s]):
                page = perm[at]; at += 1
                self.table[s, i] = page
                lo, hi = i * page_size, min(n, (i + 1) * page_size)
                kc[page, :, :hi - lo] = self.k_dense[s][lo:hi].transpose(0, 1)
                vc[page, :, :hi - lo] = self.v_dense[s][lo:hi].transpose(0, 1)
        self.kcache = kc.to(dtype).to(device)
        self.vcache = vc.to(dtype).to(device)
        # what the kernels see after rounding to the storage dtype
        self.k_dense = [k.to(dtype).double() for k in self.k_dense]
        self.v_dense = [v.to(dtype).double() for v in self.v_dense]
        self.table_dev = self.table.to(device)


def dense_attention(q, k, v, q_positions, window, scale):
    """q [n, nq, d] (float64) at absolute positions q_positions over keys k, v [len, nkv, d]."""
    n, nq, d = q.shape
    nkv = k.shape[1]
    G = nq // nkv
    out = torch.zeros(n, nq, d, dtype=torch.float64)
    for i, pos in enumerate(q_positions):
        lo = max(0, pos - window + 1) if window else 0
        for h in range(nq):
            kk, vv = k[lo:pos + 1, h // G], v[lo:pos + 1, h // G]
            p = torch.softmax((kk @ q[i, h]) * scale, 0)
            out[i, h] = p @ vv
    return out


def segments_to_device(segs, device):
    """segs: list of (slot, start, length).  Returns the device arrays the kernels take."""
    T = sum(n for _, _, n in segs)
    tok_slot = torch.zeros(T, dtype=torch.int32); pos = torch.zeros(T, dtype=torch.int32)
    tok_seg = torch.zeros(T, dtype=torch.int32)
    off, at = [], 0
    for i, (slot, start, n) in enumerate(segs):
        off.append(at)
        tok_slot[at:at + n] = slot; pos[at:at + n] = torch.arange(start, start + n); tok_seg[at:at + n] = i
        at += n
    mk = lambda x: torch.tensor(x, dtype=torch.int32, device=device)  # noqa: E731
    return dict(T=T, token_slot=tok_slot.to(device), positions=pos.to(device), token_seg=tok_seg.to(device),
                seg_off=mk(off), seg_slot=mk([s for s, _, _ in segs]), seg_start=mk([s for _, s, _ in segs]),
                seg_len=mk([n for _, _, n in segs]))
