"""Helpers of the GPU tests: a step context and a cache line made by hand, so that a kernel or
a part can be run alone."""
import numpy as np
import torch

from mormot2_ai_b200.cache.pages import PAGE, pages_for
from mormot2_ai_b200.cache.storage import CacheLine
from mormot2_ai_b200.engine.batch import StepBuffers

DEV = "cuda:0"


def make_step(seqs, max_tokens=4096, max_seqs=64):
    """seqs = [(slot, past, tokens, want)] -> StepContext on the device."""
    return StepBuffers(max_tokens, max_seqs, torch.device(DEV)).fill(seqs)


def make_line(n_slots, max_len, kv_heads, head_dim, dtype, window=0, ring_pages=0, seed=0,
              scramble=True):
    """A cache line with every slot's pages mapped (scrambled over the pool, so that a kernel
    that ignores the page table is found out)."""
    per = ring_pages if ring_pages else pages_for(max_len)
    n_pages = n_slots * per + 3
    rng = np.random.default_rng(seed)
    ids = rng.permutation(n_pages)[:n_slots * per] if scramble else np.arange(n_slots * per)
    table = torch.tensor(ids.reshape(n_slots, per), dtype=torch.int32, device=DEV)
    k = torch.zeros((n_pages, kv_heads, PAGE, head_dim), dtype=dtype, device=DEV)
    v = torch.zeros_like(k)
    return CacheLine(k, v, table, per, ring_pages, window, kv_heads, head_dim)


def fill_line(line, slot, keys, values, first_pos=0):
    """Writes keys/values [n, kv_heads, head_dim] (CPU float tensors) at positions
    first_pos.. of the slot, through the page table, as the kernels address them."""
    n = keys.shape[0]
    table = line.page_table.cpu()
    for i in range(n):
        pos = first_pos + i
        lp = pos // PAGE
        if line.ring_pages:
            lp %= line.ring_pages
        page = int(table[slot, lp])
        line.k[page, :, pos % PAGE, :] = keys[i].to(line.k.dtype).to(DEV)
        line.v[page, :, pos % PAGE, :] = values[i].to(line.v.dtype).to(DEV)


def read_line(line, slot, pos):
    table = line.page_table.cpu()
    lp = pos // PAGE
    if line.ring_pages:
        lp %= line.ring_pages
    page = int(table[slot, lp])
    return line.k[page, :, pos % PAGE, :].float().cpu(), line.v[page, :, pos % PAGE, :].float().cpu()
