"""The tensor-core attention kernels of the bfloat16 path (``csrc/attention_mma.cu``)."""
from __future__ import annotations


def run(rt, q, q_stride, out, step, line, nh, nkv, hd, window, scale) -> bool:
    """True if a fast kernel took the call; False: the caller uses the general kernel."""
    return False
