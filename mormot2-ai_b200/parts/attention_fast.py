"""The tensor-core attention kernels of the bfloat16 path (``csrc/attention_mma.cu``): which
kernel takes a call, and how a sequence's pages are shared out over CTAs."""
from __future__ import annotations


import torch

from .. import kernels as K
from ..cache.pages import pages_for

FAST_HEAD_DIMS = (64, 128)
MAX_DECODE_SPLITS = 8       # the splits of a sequence are one thread-block cluster


def decode_splits(line, T: int, nh: int, nkv: int, sms: int, window: int) -> int:
    """Over how many CTAs the pages of a sequence are dealt out in a decode step of T tokens.
    Every CTA pays a fixed price (index loads before its first key, the merge at its end), so
    few, long CTAs win: as many as give one round of two CTAs per SM, at most 8 (the splits of a
    sequence form a thread-block cluster that merges through shared memory, and beyond that the
    merge costs more than the shorter CTAs save: measured at batch 1),
    and no more than the most pages that a sequence can hold in this line (the lengths of the
    moment do not count: a captured launch must stay valid as sequences grow)."""
    pages = line.max_pages
    if window > 0:
        pages = min(pages, pages_for(window) + 1)
    subs = (nh // nkv + 15) // 16
    groups = max(1, T * nkv * subs)
    return max(1, min((2 * sms) // groups, pages, MAX_DECODE_SPLITS))


MANY_SPLITS_MOST = 32       # CTAs that share one long sequence through scratch memory, at most


def decode_many_splits(step, nh: int, nkv: int, sms: int) -> int:
    """A batch so small that even eight splits a sequence leave SMs idle (one or two sequences
    at eight KV heads) whose longest sequence is long (``step.long``): a cluster's eight CTAs at
    ≈ 50 GB/s each then stream it at less than half the memory's rate. Returns how many CTAs
    share a sequence's pages through scratch memory and a second kernel that adds them up
    (about one CTA per SM), or 0 where the cluster form serves. The engine captures passes
    with ``step.long`` as graphs of their own, so the choice may depend on it."""
    subs = (nh // nkv + 15) // 16
    groups = max(1, step.T * nkv * subs)
    if not step.long or groups * MAX_DECODE_SPLITS > sms:
        return 0
    return min(sms // groups, MANY_SPLITS_MOST)


def run(rt, q, q_stride, out, step, line, nh, nkv, hd, window, scale) -> bool:
    """True if a fast kernel took the call; False: the caller uses the general kernel."""
    if hd not in FAST_HEAD_DIMS or q.dtype != torch.bfloat16 or q_stride % 8 or q.data_ptr() % 16:
        return False
    if step.decode:
        many = decode_many_splits(step, nh, nkv, rt.sms) if window == 0 else 0
        if many > MAX_DECODE_SPLITS and step.T * nh * many * (hd + 2) <= rt.attention_scratch.numel():
            K.attention_decode(q, q_stride, out, step, line, nh, nkv, hd, window, scale, many,
                               rt.attention_scratch, rt.error_word)
            return True
        splits = decode_splits(line, step.T, nh, nkv, rt.sms, window)
        K.attention_decode_clusters(q, q_stride, out, step, line, nh, nkv, hd, window, scale,
                                    splits, rt.error_word)
        return True
    if out.stride(0) % 8 or out.data_ptr() % 16:
        return False
    if hd == 128 and q.stride(1) == 1:
        # S and O in tensor memory, tiles by TMA (csrc/attention_tc.cu)
        K.attention_prefill_tc(q, q_stride, out, step, line, nh, nkv, hd, window, scale,
                               rt.error_word)
        return True
    K.attention_prefill(q, q_stride, out, step, line, nh, nkv, hd, window, scale,
                        rt.error_word)
    return True
