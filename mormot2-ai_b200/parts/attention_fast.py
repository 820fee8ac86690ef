"""The tensor-core attention kernels of the bfloat16 path (``csrc/attention_mma.cu``): which
kernel takes a call, and how a sequence's pages are shared out over CTAs."""
from __future__ import annotations

from typing import Tuple

import torch

from .. import kernels as K
from ..cache.pages import pages_for

FAST_HEAD_DIMS = (64, 128)


def decode_split(line, T: int, nh: int, nkv: int, sms: int, window: int) -> Tuple[int, int]:
    """(splits, pages per split) for a decode step of T tokens: enough CTAs to fill the GPU a
    few times over, sized by the most pages that a sequence can hold in this line (not by the
    lengths of the moment: a captured launch must stay valid as sequences grow)."""
    pages = line.max_pages
    if window > 0:
        pages = min(pages, pages_for(window) + 1)
    subs = (nh // nkv + 15) // 16
    groups = max(1, T * nkv * subs)
    # a CTA has four warps that take pages in turn: one page a warp (then 2, 4, ...) until the
    # grid is no more than eight CTAs for every SM
    per_warp = 1
    while groups * -(-pages // (4 * per_warp)) > 8 * sms and 4 * per_warp < pages:
        per_warp *= 2
    pages_per_split = min(pages, 4 * per_warp)
    return -(-pages // pages_per_split), pages_per_split


def run(rt, q, q_stride, out, step, line, nh, nkv, hd, window, scale) -> bool:
    """True if a fast kernel took the call; False: the caller uses the general kernel."""
    if hd not in FAST_HEAD_DIMS or q.dtype != torch.bfloat16 or q_stride % 8 or q.data_ptr() % 16:
        return False
    if step.decode:
        splits, pps = decode_split(line, step.T, nh, nkv, rt.sms, window)
        need = step.T * nh * splits * (hd + 2)
        if rt.workspace is None or rt.workspace.numel() < need:
            return False
        K.attention_decode(q, q_stride, out, step, line, nh, nkv, hd, window, scale, splits, pps,
                           rt.workspace)
        return True
    if out.stride(0) % 8 or out.data_ptr() % 16:
        return False
    K.attention_prefill(q, q_stride, out, step, line, nh, nkv, hd, window, scale)
    return True
