"""The Python face of the native kernels: each function takes CUDA tensors, checks what the
kernel cannot check itself, and launches on the current stream. Nothing here computes in
PyTorch, and nothing falls back: without a GPU or the compiled libraries it raises
``KernelError``.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build
from .errors import KernelError

F32, BF16 = 0, 1
EPI_STORE, EPI_ADD, EPI_SWIGLU, EPI_SWIGLU_PAIRS = 0, 1, 2, 3
PAGE = 64  # positions per cache page (MB_PAGE in csrc/common.cuh)

_c = ctypes
_vp, _i, _f, _d, _ll = _c.c_void_p, _c.c_int, _c.c_float, _c.c_double, _c.c_longlong


def code_of(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"tensors of {dtype} are not supported by the kernels")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("a kernel was given a tensor that is not on the GPU")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream of the current device as the integer that the kernels take."""
    if _raw_stream is not None:                     # the short way (no Stream object)
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def require_gpu() -> None:
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this library computes on a B200 only (no CPU path)")
    major, minor = torch.cuda.get_device_capability()
    if major != 10:
        raise KernelError(f"the kernels are built for sm_100a; this device is sm_{major}{minor}")


class Launches:
    """How many kernels of this library were launched (a graph replay counts the kernels that
    were captured into it)."""
    count = 0


CLASS_OF = {"mb_gemm_tc": "products", "mb_gemm_simt": "products",
            "mb_attention_simt": "attention", "mb_attention_decode": "attention",
            "mb_attention_decode_clusters": "attention", "mb_attention_prefill": "attention",
            "mb_attention_prefill_tc": "attention", "mb_rmsnorm": "norms",
            "mb_qk_norm_rope_store": "rotary", "mb_embed": "embedding", "mb_swiglu": "activation",
            "mb_argmax": "sampling", "mb_sample": "sampling", "mb_sample_filtered": "sampling",
            "mb_advance_decode": "sampling"}


class Timing:
    """Times every kernel call by its class while it is open (CUDA events around each call,
    which also keeps a kernel from starting under the tail of the one before: a diagnosis, not
    the speed of the product path). The role of the reference's ``TTimedBackend``
    (``demos/infer/llm-bench.lpr:58-236``).

        with Timing() as t:
            engine.step(...)
        t.shares()   # {"products": ms, "attention": ms, ...}, after a synchronize

    The time between the end of one call and the start of the next (the host preparing the
    next launch, other work on the stream) is booked as ``between``, so that the classes add
    up to the time from the first call to the last.
    """
    current: Optional["Timing"] = None

    def __init__(self):
        self.events = []

    def __enter__(self):
        Timing.current = self
        return self

    def __exit__(self, *exc):
        Timing.current = None

    def shares(self, start=None, end=None) -> dict:
        """``start``, ``end``: events recorded before the first and after the last call, whose
        distance to them is booked as ``between`` too."""
        torch.cuda.synchronize()
        out: dict = {}
        last = start
        for name, e0, e1 in self.events:
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
            if last is not None:
                out["between"] = out.get("between", 0.0) + last.elapsed_time(e0)
            last = e1
        if end is not None and last is not None:
            out["between"] = out.get("between", 0.0) + last.elapsed_time(end)
        return out


def read_trace() -> list:
    """The kernels' own timeline, from a build with ``MORMOT_B200_NVCC_FLAGS=-DMB_TRACE``: every
    CTA of the decode kernels (matrix products, RMSNorm, q/k norm + rotary, decode attention)
    leaves its start and end on the GPU's nanosecond timer. Returns ``[(start_ns, end_ns,
    kind)]`` of all CTAs since the last call, sorted by start (``kind``: "product", "norm",
    "rotary", "attention"); empty in an ordinary build. Unlike ``Timing`` this does not change
    the schedule: it shows a step as it runs inside a CUDA graph, kernels overlapping where
    programmatic dependent launch lets them."""
    names = {1: "product", 2: "norm", 3: "rotary", 4: "attention"}
    rows = []
    cap = 1 << 17
    buf = (_c.c_ulonglong * (2 * cap))()
    for lib in ("gemm_tc", "elementwise", "rope", "attention_mma"):
        handle = build.load_library(lib)
        if not hasattr(handle, "mb_trace_read"):
            continue
        n = handle.mb_trace_read(buf, cap)
        mask = (1 << 56) - 1
        rows += [(buf[2 * i] & mask, buf[2 * i + 1] & mask, names.get(buf[2 * i] >> 56, "?"))
                 for i in range(n)]
    rows.sort()
    return rows


def _call(libname: str, fn: str, argtypes, *args, launches: int = 1) -> None:
    lib = build.load_library(libname)
    f = getattr(lib, fn)
    if f.argtypes is None:
        f.argtypes = argtypes
        f.restype = _i
    timing = Timing.current
    if timing is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    rc = f(*args)
    if rc != 0:
        raise KernelError(lib.mb_last_error().decode(errors="replace"))
    if timing is not None:
        e1.record()
        timing.events.append((CLASS_OF.get(fn, "other"), e0, e1))
    Launches.count += launches


def _contig(t: torch.Tensor, what: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{what} is not contiguous")


# ------------------------------------------------------------------------------ elementwise
def embed(table: torch.Tensor, ids: torch.Tensor, x: torch.Tensor) -> None:
    """x[t, :] = table[ids[t], :] as float32."""
    T, H = x.shape
    _contig(table, "the embedding"), _contig(x, "x")
    assert ids.dtype == torch.int32 and x.dtype == torch.float32 and table.shape[1] == H
    _call("elementwise", "mb_embed", [_vp, _i, _vp, _vp, _i, _i, _i, _vp],
          _ptr(table), code_of(table.dtype), _ptr(ids), _ptr(x), T, H, table.shape[0], _stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: Optional[torch.Tensor],
            rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
            partial: Optional[torch.Tensor] = None) -> None:
    """out[r] = w * x[rows[r] or r] / rms(x). ``partial`` [parts, T, H] float32 is first added
    into x (the split results of the matrix product before)."""
    H = x.shape[-1]
    R = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
    assert x.dtype == torch.float32 and w.numel() == H
    _contig(x, "x")
    parts, stride = 0, 0
    if partial is not None:
        assert partial.dtype == torch.float32 and partial.is_contiguous()
        parts, stride = partial.shape[0], partial.stride(0)
    _call("elementwise", "mb_rmsnorm",
          [_vp, _vp, _i, _ll, _vp, _i, _f, _vp, _i, _vp, _i, _i, _vp],
          _ptr(x), _ptr(partial), parts, stride, _ptr(w), code_of(w.dtype), float(eps),
          _ptr(out), code_of(out.dtype) if out is not None else F32, _ptr(rows), R, H, _stream())


def add_partials(x: torch.Tensor, partial: torch.Tensor) -> None:
    """x += partial[0] + partial[1] + ... (float32 [parts, T, H]), in that order."""
    assert x.dtype == torch.float32 and partial.dtype == torch.float32 and partial.is_contiguous()
    _contig(x, "x")
    T, H = x.shape
    _call("elementwise", "mb_rmsnorm",
          [_vp, _vp, _i, _ll, _vp, _i, _f, _vp, _i, _vp, _i, _i, _vp],
          _ptr(x), _ptr(partial), partial.shape[0], partial.stride(0), None, F32, 0.0, None, F32,
          None, T, H, _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[T, I] = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.dtype == out.dtype
    _contig(gate_up, "gate_up"), _contig(out, "out")
    _call("elementwise", "mb_swiglu", [_vp, _vp, _i, _i, _i, _vp],
          _ptr(gate_up), _ptr(out), code_of(out.dtype), T, I, _stream())


def qk_norm_rope_store(qkv, q_norm, k_norm, eps, inv_freq, rot_dim, step, line, nh, nkv, hd,
                       write_kv: bool, partial: Optional[torch.Tensor] = None,
                       q_out: Optional[torch.Tensor] = None) -> None:
    """Per-head norm of q and k, rotary positions, q in place (or into ``q_out``), k and v into
    the cache line. ``partial`` [parts, T, width] float32: the split sums of the q/k/v product,
    which stand for ``qkv`` (then None) and are added up here."""
    if partial is not None:
        assert partial.dtype == torch.float32 and partial.is_contiguous() and q_out is not None
        T, width = partial.shape[1], partial.shape[2]
        dtype_code = code_of(q_out.dtype)
    else:
        T, width = qkv.shape
        _contig(qkv, "qkv")
        dtype_code = code_of(qkv.dtype)
    assert width == (nh + 2 * nkv) * hd
    if rot_dim > 0 and inv_freq is None:
        raise KernelError("a rotary encoding without its frequencies (is the position "
                          "encoding bound?)")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() < rot_dim // 2):
        raise KernelError(f"{inv_freq.numel()} frequencies for {rot_dim} rotating values")
    if (q_norm is None) != (k_norm is None):
        raise KernelError("q_norm and k_norm come together")
    wd = code_of(q_norm.dtype) if q_norm is not None else F32
    _call("rope", "mb_qk_norm_rope_store",
          [_vp, _vp, _i, _ll, _vp, _i, _vp, _vp, _i, _f, _vp, _i, _vp, _vp, _vp, _i, _i,
           _vp, _vp, _i, _i, _i, _i, _i, _vp],
          _ptr(qkv), _ptr(partial), partial.shape[0] if partial is not None else 0,
          partial.stride(0) if partial is not None else 0, _ptr(q_out), dtype_code,
          _ptr(q_norm), _ptr(k_norm), wd, float(eps),
          _ptr(inv_freq), rot_dim, _ptr(step.tok_slot), _ptr(step.tok_pos),
          _ptr(line.page_table), line.max_pages, line.ring_pages, _ptr(line.k), _ptr(line.v),
          T, nh, nkv, hd, 1 if write_kv else 0, _stream())


# ------------------------------------------------------------------------------ products
def gemm_simt(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPI_STORE) -> None:
    """c = a · wᵀ (store), c += a · wᵀ (add, float32 c), or SwiGLU over w = [gate; up]
    (EPI_SWIGLU) or over a w whose rows alternate gate, up (EPI_SWIGLU_PAIRS)."""
    M, K = a.shape
    N = c.shape[1]
    assert w.shape[1] == K
    assert w.shape[0] == (2 * N if epilogue in (EPI_SWIGLU, EPI_SWIGLU_PAIRS) else N)
    assert c.shape[0] == M and a.stride(1) == 1 and c.stride(1) == 1
    _contig(w, "the weight")
    _call("gemm_simt", "mb_gemm_simt",
          [_vp, _i, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp],
          _ptr(a), code_of(a.dtype), a.stride(0), _ptr(w), code_of(w.dtype), _ptr(c),
          code_of(c.dtype), c.stride(0), M, N, K, epilogue, _stream())


# ------------------------------------------------------------------------------ attention
def attention_simt(q: torch.Tensor, q_stride: int, out: torch.Tensor, step, line, nh, nkv, hd,
                   window: int, scale: float) -> None:
    T = out.shape[0]
    _contig(out, "out")
    _call("attention_simt", "mb_attention_simt",
          [_vp, _i, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f,
           _vp],
          _ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(line.k), _ptr(line.v),
          code_of(out.dtype), _ptr(line.page_table), line.max_pages, line.ring_pages,
          _ptr(step.tok_seq), _ptr(step.tok_pos), _ptr(step.seq_slot), T, nh, nkv, hd,
          window, float(scale), _stream())


# ------------------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: torch.Tensor,
           scratch: Optional[torch.Tensor] = None) -> None:
    """out[r] = arg-max of row r; with ``scratch`` (8 bytes per row and 2048 values) wide rows
    are read by many CTAs."""
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    nbytes = scratch.numel() * scratch.element_size() if scratch is not None else 0
    _call("sampling", "mb_argmax", [_vp, _ll, _i, _i, _vp, _vp, _ll, _vp],
          _ptr(logits), logits.stride(0), rows, V, _ptr(out), _ptr(scratch), nbytes, _stream(),
          launches=2 if scratch is not None and V > 4 * 2048 else 1)


def sample(logits: torch.Tensor, temperature: float, state_index: torch.Tensor,
           states: torch.Tensor, out: torch.Tensor) -> None:
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert states.dtype == torch.int64 and state_index.dtype == torch.int32
    _call("sampling", "mb_sample", [_vp, _ll, _i, _i, _d, _vp, _vp, _vp, _vp],
          _ptr(logits), logits.stride(0), rows, V, float(temperature), _ptr(state_index),
          _ptr(states), _ptr(out), _stream())


# ------------------------------------------------------------------------------ tensor cores
def gemm_tc_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    lib = build.load_library("gemm_tc")
    f = lib.mb_gemm_tc_supported
    if f.argtypes is None:
        f.argtypes = [_vp, _i, _vp, _i, _i, _i]
        f.restype = _i
    return bool(f(_ptr(a), a.stride(0), _ptr(w), a.shape[0], w.shape[0], w.shape[1]))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, add: bool,
            workspace: Optional[torch.Tensor], error: torch.Tensor, sms: int,
            swiglu: bool = False, defer: bool = False) -> int:
    """c = a · wᵀ (or c += for a float32 c) with bfloat16 a [M, K] and w [N, K] on the tensor
    cores; ``swiglu``: w's rows alternate gate and up and c [M, N / 2] = silu(gate) · up.
    ``workspace``: float32 scratch for split sums; ``error``: int32 device word. ``defer``:
    when K was split (the return value, the number of splits, is above 1) the partial sums stay
    in the workspace as [splits, M, N] and c is not touched."""
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert a.stride(1) == 1 and c.stride(1) == 1 and c.shape == (M, N // 2 if swiglu else N)
    _contig(w, "the weight")
    _call("gemm_tc", "mb_gemm_tc",
          [_vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _ll, _i, _vp, _i, _vp],
          _ptr(a), a.stride(0), _ptr(w), _ptr(c), code_of(c.dtype), c.stride(0), M, N, K,
          3 if swiglu else (1 if add else 0), _ptr(workspace),
          workspace.numel() if workspace is not None else 0, 1 if defer else 0,
          _ptr(error), sms, _stream())
    # the split of K adds one kernel that sums the partial products
    lib = build.load_library("gemm_tc")
    Launches.count += lib.mb_gemm_tc_last_launches() - 1
    return lib.mb_gemm_tc_last_splits()


def wait_selftest(error: torch.Tensor, code: int, tries: int = 2048) -> bool:
    """Runs one bounded wait that nothing ends (a barrier without anyone to arrive at it),
    with a limit of ``tries`` polls. True if the wait gave up, as it must; ``error`` (int32
    device word) then holds ``code``. The kernel returns by itself either way."""
    gave_up = torch.zeros(1, dtype=torch.int32, device=error.device)
    _call("gemm_tc", "mb_wait_selftest", [_vp, _i, _c.c_uint, _vp, _vp],
          _ptr(error), code, tries, _ptr(gave_up), _stream())
    return bool(gave_up.item())


def advance_decode(tok_ids: torch.Tensor, tok_pos: torch.Tensor, chosen: torch.Tensor,
                   history: Optional[torch.Tensor]) -> None:
    """The chosen tokens become the next step's ids, every position moves on by one."""
    B = tok_ids.numel()
    assert chosen.dtype == torch.int32 and chosen.numel() == B
    _call("elementwise", "mb_advance_decode", [_vp, _vp, _vp, _vp, _i, _vp],
          _ptr(tok_ids), _ptr(tok_pos), _ptr(chosen), _ptr(history), B, _stream())


def sample_filtered(logits: torch.Tensor, sampling, state_index: torch.Tensor,
                    states: torch.Tensor, scratch: torch.Tensor, out: torch.Tensor) -> None:
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert scratch.dtype == torch.int64 and scratch.is_contiguous() and scratch.shape[0] >= rows
    _call("sampling", "mb_sample_filtered",
          [_vp, _ll, _i, _i, _d, _i, _d, _d, _vp, _vp, _vp, _ll, _vp, _vp],
          _ptr(logits), logits.stride(0), rows, V, float(sampling.temperature),
          int(sampling.top_k), float(sampling.top_p), float(sampling.min_p), _ptr(state_index),
          _ptr(states), _ptr(scratch), scratch.shape[1], _ptr(out), _stream())


def attention_decode(q: torch.Tensor, q_stride: int, out: torch.Tensor, step, line, nh, nkv, hd,
                     window: int, scale: float, splits: int, scratch: torch.Tensor,
                     error: Optional[torch.Tensor] = None) -> None:
    """Attention of single tokens (a decode step) over the paged cache on the tensor cores; the
    pages of a sequence are dealt out over ``splits`` CTAs."""
    T = out.shape[0]
    _contig(out, "out")
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert scratch.dtype == torch.float32 and scratch.is_contiguous()
    _call("attention_mma", "mb_attention_decode",
          [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _f, _i,
           _vp, _ll, _vp, _vp],
          _ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(line.k), _ptr(line.v),
          _ptr(line.page_table), line.max_pages, line.ring_pages, _ptr(step.tok_slot),
          _ptr(step.tok_pos), T, nh, nkv, hd, window, float(scale),
          splits, _ptr(scratch), scratch.numel(), _ptr(error), _stream(), launches=2)


def attention_decode_clusters(q: torch.Tensor, q_stride: int, out: torch.Tensor, step, line, nh,
                              nkv, hd, window: int, scale: float, splits: int,
                              error: Optional[torch.Tensor] = None) -> None:
    """``attention_decode`` with the splits of a (token, group of heads) as one thread-block
    cluster that merges through its shared memory: no scratch, one kernel; at most 8 splits."""
    T = out.shape[0]
    _contig(out, "out")
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    _call("attention_mma", "mb_attention_decode_clusters",
          [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _f, _i,
           _vp, _vp],
          _ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(line.k), _ptr(line.v),
          _ptr(line.page_table), line.max_pages, line.ring_pages, _ptr(step.tok_slot),
          _ptr(step.tok_pos), T, nh, nkv, hd, window, float(scale), splits, _ptr(error),
          _stream())


def attention_prefill(q: torch.Tensor, q_stride: int, out: torch.Tensor, step, line, nh, nkv,
                      hd, window: int, scale: float,
                      error: Optional[torch.Tensor] = None) -> None:
    """Causal attention of every sequence's new tokens over the paged cache on the tensor
    cores (the cache already holds their keys and values)."""
    _contig(out, "out")
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    _call("attention_mma", "mb_attention_prefill",
          [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f,
           _vp, _vp],
          _ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(line.k), _ptr(line.v),
          _ptr(line.page_table), line.max_pages, line.ring_pages, _ptr(step.seq_start),
          _ptr(step.seq_past), _ptr(step.seq_slot), step.B, step.max_new, nh, nkv, hd, window,
          float(scale), _ptr(error), _stream())


def attention_prefill_tc(q: torch.Tensor, q_stride: int, out: torch.Tensor, step, line, nh, nkv,
                         hd, window: int, scale: float, error: torch.Tensor) -> None:
    """The prefill attention on tcgen05 (heads of 128 values): S and O in tensor memory, Q, K
    and V tiles by TMA."""
    _contig(out, "out")
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and q.stride(1) == 1
    pool_rows = line.k.shape[0] * line.k.shape[1] * line.k.shape[2]
    _call("attention_tc", "mb_attention_prefill_tc",
          [_vp, _i, _i, _vp, _i, _vp, _vp, _ll, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i,
           _i, _i, _f, _vp, _vp],
          _ptr(q), q_stride, nh * hd, _ptr(out), out.stride(0), _ptr(line.k), _ptr(line.v),
          pool_rows, _ptr(line.page_table), line.max_pages, line.ring_pages,
          _ptr(step.seq_start), _ptr(step.seq_past), _ptr(step.seq_slot), step.B, q.shape[0],
          step.max_new, nh, nkv, hd, window, float(scale), _ptr(error), _stream())
