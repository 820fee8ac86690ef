"""The entry point that allocates nothing (csrc/no_alloc.h), called through its exported C
symbol as a host without an allocator would call it, against the existing entry point that
takes the caller's scratch and against a float64 restatement of attention: two calls in a row
with different inputs (the second must not see what the first left in the shared scratch),
and the refusal beyond its limit. This file is named to be collected last."""
import ctypes
import math

import numpy as np
import pytest
import torch

from mormot2_ai_b200 import kernels as K
from mormot2_ai_b200.csrc import build
from tests.gpu_helpers import DEV, fill_line, make_line, make_step

pytestmark = pytest.mark.gpu

_vp, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
ARGTYPES = [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _f, _i,
            _vp, _vp]
LIMIT = 4 * 1024 * 1024          # MB_ATTENTION_DECODE_STATIC_FLOATS


def static_entry():
    lib = build.load_library("attention_mma")
    fn = lib.mb_attention_decode_static          # the exported C symbol
    fn.argtypes, fn.restype = ARGTYPES, _i
    return lib, fn


def call_static(fn, q, out, step, line, nh, nkv, hd, window, scale, splits):
    return fn(q.data_ptr(), nh * hd, out.data_ptr(), out.stride(0), line.k.data_ptr(),
              line.v.data_ptr(), line.page_table.data_ptr(), line.max_pages, line.ring_pages,
              step.tok_slot.data_ptr(), step.tok_pos.data_ptr(),
              out.shape[0], nh, nkv, hd, window, scale, splits, None,
              torch.cuda.current_stream().cuda_stream)


def case(seed, lens, nh, nkv, hd, window):
    """A cache line, a decode step of one token per sequence, the queries, and what went into
    the cache (rounded to bfloat16 as the cache holds it)."""
    rng = np.random.default_rng(seed)
    line = make_line(len(lens), 640, nkv, hd, torch.bfloat16, window=window, seed=seed)
    kv = []
    for slot, n in enumerate(lens):
        k = torch.tensor(rng.standard_normal((n, nkv, hd)), dtype=torch.float32).bfloat16().float()
        v = torch.tensor(rng.standard_normal((n, nkv, hd)), dtype=torch.float32).bfloat16().float()
        fill_line(line, slot, k, v)
        kv.append((k.numpy(), v.numpy()))
    step = make_step([(slot, n - 1, [0], []) for slot, n in enumerate(lens)])
    q = torch.tensor(rng.standard_normal((len(lens), nh * hd)), dtype=torch.float32)
    return line, step, q.bfloat16().to(DEV), kv


def attention_in_float64(q, keys, values, nh, nkv, hd, pos, window, scale):
    """One query row at position pos over keys[0..pos], or the last `window` of them."""
    lo = max(0, pos + 1 - window) if window else 0
    out = np.zeros((nh, hd))
    for h in range(nh):
        g = h // (nh // nkv)
        s = keys[lo:pos + 1, g].astype(np.float64) @ q[h].astype(np.float64) * scale
        p = np.exp(s - s.max())
        out[h] = (p @ values[lo:pos + 1, g].astype(np.float64)) / p.sum()
    return out


def test_two_calls_in_a_row_equal_the_existing_entry_point():
    lib, fn = static_entry()
    nh, nkv, hd = 8, 2, 128
    scale = 1 / math.sqrt(hd)
    before = torch.cuda.memory_allocated()
    for seed, lens, window, splits in ((1, [600, 3, 129], 0, 4), (2, [64, 500], 90, 10)):
        line, step, q, kv = case(seed, lens, nh, nkv, hd, window)
        want = torch.empty(len(lens), nh * hd, dtype=torch.bfloat16, device=DEV)
        scratch = torch.empty(len(lens) * nh * splits * (hd + 2), device=DEV)
        K.attention_decode(q, nh * hd, want, step, line, nh, nkv, hd, window, scale, splits,
                           scratch)
        got = torch.full_like(want, 7.0)
        allocated = torch.cuda.memory_allocated()
        rc = call_static(fn, q, got, step, line, nh, nkv, hd, window, scale, splits)
        assert rc == 0, lib.mb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == allocated
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 1.2e-2 * max(1.0, want.float().abs().max().item()), err
        assert torch.equal(got, want)        # the same kernels on the same inputs
        # and both against attention restated in float64 on what the cache holds
        qf = q.float().cpu().numpy().reshape(len(lens), nh, hd)
        plain = np.stack([attention_in_float64(qf[b], kv[b][0], kv[b][1], nh, nkv, hd, n - 1,
                                               window, scale).reshape(-1)
                          for b, n in enumerate(lens)])
        err = np.abs(got.float().cpu().numpy() - plain).max()
        assert err <= 1.2e-2 * max(1.0, np.abs(plain).max()), err


def test_sizes_beyond_the_limit_are_refused():
    lib, fn = static_entry()
    nh, nkv, hd = 32, 8, 128
    line, step, q, _ = case(3, [10] * 64, nh, nkv, hd, 0)
    out = torch.full((64, nh * hd), 3.0, dtype=torch.bfloat16, device=DEV)
    assert 64 * nh * 16 * (hd + 2) > LIMIT
    rc = call_static(fn, q, out, step, line, nh, nkv, hd, 0, 0.1, 16)
    assert rc != 0
    message = lib.mb_last_error().decode()
    assert "scratch" in message and str(LIMIT) in message
    torch.cuda.synchronize()
    assert float(out.float().min()) == 3.0          # nothing was launched
    assert 64 * nh * 15 * (hd + 2) <= LIMIT         # the largest size still fits
    assert call_static(fn, q, out, step, line, nh, nkv, hd, 0, 0.1, 15) == 0
    torch.cuda.synchronize()
