"""Each kernel alone against its plain reference, at other sizes than the engine's tests use:
head sizes in steps of 16, numbers of heads and groups, widths and vocabularies that are no
power of two, windows, rings of pages. Where random numbers would hide a fault (a far key
among hundreds, a window's edge, a page of the cache), the inputs are made so that it shows."""
import math

import numpy as np
import pytest
import torch

from mormot2_ai_b200 import kernels as K
from mormot2_ai_b200.engine.runtime import Runtime
from tests.gpu_helpers import DEV, fill_line, make_line, make_step, read_line
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rel(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.abs(got - want).max() / max(1.0, np.abs(want).max()))


@pytest.fixture(scope="module")
def rt():
    return Runtime(torch.bfloat16)


@pytest.mark.parametrize("table_dtype", ["float32", "bfloat16"])
def test_embed(table_dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(509, 96, generator=g).to(DT[table_dtype])
    ids = torch.tensor([0, 508, 17, 17, 3], dtype=torch.int32)
    x = torch.empty(5, 96, device=DEV)
    K.embed(table.to(DEV), ids.to(DEV), x)
    assert torch.equal(x.cpu(), table.float()[ids.long()])


@pytest.mark.parametrize("H", [16, 96, 1000, 4096, 5120 + 8])
@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
def test_rmsnorm(H, out_dtype):
    g = torch.Generator().manual_seed(H)
    x = torch.randn(7, H, generator=g) * 3
    w = 1 + 0.1 * torch.randn(H, generator=g)
    want = plain.rms_norm(x.numpy(), w.numpy(), 1e-5)
    out = torch.empty(7, H, dtype=DT[out_dtype], device=DEV)
    K.rmsnorm(x.to(DEV), w.to(DEV), 1e-5, out)
    assert rel(out.float().cpu(), want) <= (2e-6 if out_dtype == "float32" else 8e-3)
    # gathered rows, a bfloat16 weight
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    wb = w.to(torch.bfloat16)
    out = torch.empty(3, H, dtype=DT[out_dtype], device=DEV)
    K.rmsnorm(x.to(DEV), wb.to(DEV), 1e-5, out, rows)
    want = plain.rms_norm(x.numpy()[[6, 0, 3]], wb.float().numpy(), 1e-5)
    assert rel(out.float().cpu(), want) <= (2e-6 if out_dtype == "float32" else 8e-3)


@pytest.mark.parametrize("H", [1000, 2048, 4096, 5128, 16384, 20000])
def test_rmsnorm_many_rows(H):
    """More rows than a decode step has: the variants with 256 threads a row, the wide rows
    that go to 1024 threads, and a row beyond the vector kernels; with partial sums too."""
    g = torch.Generator().manual_seed(H)
    x = torch.randn(300, H, generator=g) * 3
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    parts = torch.randn(2, 300, H, generator=g)
    out = torch.empty(300, H, dtype=torch.bfloat16, device=DEV)
    K.rmsnorm(x.to(DEV), w.to(DEV), 1e-6, out)
    assert rel(out.float().cpu(), plain.rms_norm(x.numpy(), w.float().numpy(), 1e-6)) <= 8e-3
    xd = x.to(DEV)
    K.rmsnorm(xd, w.to(DEV), 1e-6, out, partial=parts.to(DEV))
    total = (x + parts[0]) + parts[1]
    assert torch.equal(xd.cpu(), total)
    assert rel(out.float().cpu(), plain.rms_norm(total.numpy(), w.float().numpy(), 1e-6)) <= 8e-3


@pytest.mark.parametrize("H,n_parts", [(320, 3), (2048, 9), (4096, 8), (5120, 1)])
def test_rmsnorm_adds_split_partials(H, n_parts):
    """Few rows, as a decode step has them: narrow and wide rows, up to nine partial sums."""
    g = torch.Generator().manual_seed(1)
    x = torch.randn(5, H, generator=g)
    parts = torch.randn(n_parts, 5, H, generator=g)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    xd = x.to(DEV)
    out = torch.empty(5, H, device=DEV)
    K.rmsnorm(xd, w.to(DEV), 1e-6, out, partial=parts.to(DEV))
    total = x.clone()
    for p in parts:                                            # in split order
        total = total + p
    assert torch.equal(xd.cpu(), total)
    assert rel(out.cpu(), plain.rms_norm(total.numpy(), w.numpy(), 1e-6)) <= 2e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu(dtype):
    g = torch.Generator().manual_seed(2)
    gu = (torch.randn(9, 2 * 330, generator=g) * 3).to(DT[dtype])
    out = torch.empty(9, 330, dtype=DT[dtype], device=DEV)
    K.swiglu(gu.to(DEV), out)
    want = plain.swiglu(gu.float().numpy()[:, :330], gu.float().numpy()[:, 330:])
    assert rel(out.float().cpu(), want) <= (2e-6 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("M,N,Kd", [(1, 7, 5), (3, 509, 96), (70, 65, 33), (130, 200, 320),
                                    (12, 131, 200), (16, 64, 1028), (17, 37, 132)])
@pytest.mark.parametrize("a_dt,w_dt,c_dt", [("float32", "float32", "float32"),
                                            ("bfloat16", "bfloat16", "bfloat16"),
                                            ("bfloat16", "float32", "float32"),
                                            ("float32", "bfloat16", "bfloat16")])
def test_gemm_simt(M, N, Kd, a_dt, w_dt, c_dt):
    g = torch.Generator().manual_seed(M * N)
    a = torch.randn(M, Kd, generator=g).to(DT[a_dt])
    w = (torch.randn(N, Kd, generator=g) * 0.2).to(DT[w_dt])
    want = a.double() @ w.double().T
    tol = 2e-6 if c_dt == "float32" else 8e-3
    c = torch.empty(M, N, dtype=DT[c_dt], device=DEV)
    K.gemm_simt(a.to(DEV), w.to(DEV), c)
    assert rel(c.float().cpu(), want) <= tol
    if c_dt == "float32":
        r = torch.randn(M, N, generator=g)
        c = r.to(DEV)
        K.gemm_simt(a.to(DEV), w.to(DEV), c, K.EPI_ADD)
        assert rel(c.cpu(), want + r.double()) <= tol
    w2 = (torch.randn(2 * N, Kd, generator=g) * 0.2).to(DT[w_dt])
    c = torch.empty(M, N, dtype=DT[c_dt], device=DEV)
    K.gemm_simt(a.to(DEV), w2.to(DEV), c, K.EPI_SWIGLU)
    gu = (a.double() @ w2.double().T).float().numpy()
    assert rel(c.float().cpu(), plain.swiglu(gu[:, :N], gu[:, N:])) <= tol
    c = torch.empty(M, N, dtype=DT[c_dt], device=DEV)         # rows alternating gate, up
    K.gemm_simt(a.to(DEV), w2.to(DEV), c, K.EPI_SWIGLU_PAIRS)
    assert rel(c.float().cpu(), plain.swiglu(gu[:, 0::2], gu[:, 1::2])) <= tol


@pytest.mark.parametrize("M,N,Kd", [(1, 96, 64), (5, 509, 96), (16, 130, 328), (17, 256, 200),
                                    (64, 1000, 1024), (65, 77, 72), (128, 384, 192),
                                    (300, 509, 320), (1030, 264, 520), (9, 4096, 2048),
                                    (8, 19000, 256), (40, 40000, 128), (3, 150, 64),
                                    (448, 778, 200), (512, 512, 2048), (256, 256, 64),
                                    (2048, 4096, 64), (1024, 6144, 72), (2048, 2304, 64)])
def test_gemm_tensor_cores(rt, M, N, Kd):
    """The forms of csrc/gemm_tc.cu (weight rows on the TMEM lanes for few tokens, tokens on the
    lanes of one CTA, 256 tokens on the lanes of a CTA pair with its tile widths), tails in every
    dimension, the split of K, all epilogues."""
    g = torch.Generator().manual_seed(M + N + Kd)
    a = torch.randn(M, Kd, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, Kd, generator=g) * 0.1).to(torch.bfloat16)
    want = a.double() @ w.double().T
    for c_dt, tol in ((torch.bfloat16, 8e-3), (torch.float32, 2e-5)):
        c = torch.full((M, N), 3.0, dtype=c_dt, device=DEV)
        K.gemm_tc(a.to(DEV), w.to(DEV), c, False, rt.workspace, rt.error_word, rt.sms)
        assert rel(c.float().cpu(), want) <= tol
    r = torch.randn(M, N, generator=g)
    c = r.to(DEV)
    K.gemm_tc(a.to(DEV), w.to(DEV), c, True, rt.workspace, rt.error_word, rt.sms)
    assert rel(c.cpu(), want + r.double()) <= 2e-5
    c = r.to(DEV)                                                 # without scratch: no split
    K.gemm_tc(a.to(DEV), w.to(DEV), c, True, None, rt.error_word, rt.sms)
    assert rel(c.cpu(), want + r.double()) <= 2e-5
    if N % 2 == 0:                                # SwiGLU over rows that alternate gate, up
        c = torch.full((M, N // 2), 3.0, dtype=torch.bfloat16, device=DEV)
        K.gemm_tc(a.to(DEV), w.to(DEV), c, False, rt.workspace, rt.error_word, rt.sms, swiglu=True)
        y = want.float().numpy()
        assert rel(c.float().cpu(), plain.swiglu(y[:, 0::2], y[:, 1::2])) <= 8e-3
    rt.check()


def test_gemm_tensor_cores_row_strides_and_refusals(rt):
    g = torch.Generator().manual_seed(5)
    buf = torch.randn(40, 104, generator=g).to(torch.bfloat16).to(DEV)
    a = buf[:, :96]                                               # rows 104 apart
    w = (torch.randn(50, 96, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    out = torch.zeros(40, 64, dtype=torch.bfloat16, device=DEV)
    K.gemm_tc(a, w, out[:, 8:58], False, rt.workspace, rt.error_word, rt.sms)
    want = a.double().cpu() @ w.double().cpu().T
    assert rel(out[:, 8:58].float().cpu(), want) <= 8e-3
    assert float(out[:, :8].abs().max()) == 0 and float(out[:, 58:].abs().max()) == 0
    assert not K.gemm_tc_supported(buf[:, :50], w[:, :50].contiguous())    # K no multiple of 8
    assert not K.gemm_tc_supported(buf[:, 1:97], w)                         # misaligned rows


def attention_reference(q, keys, values, nh, nkv, hd, pos, window, scale):
    """One query row at position pos over keys[0..pos] (float64)."""
    lo = max(0, pos + 1 - window) if window else 0
    out = np.zeros((nh, hd))
    for h in range(nh):
        g = h // (nh // nkv)
        s = keys[lo:pos + 1, g].astype(np.float64) @ q[h].astype(np.float64) * scale
        p = np.exp(s - s.max())
        out[h] = (p @ values[lo:pos + 1, g].astype(np.float64)) / p.sum()
    return out


def run_attention(kind, q, out, step, line, nh, nkv, hd, window, scale, splits=None):
    """The general kernel ("simt") or the tensor-core kernel for single tokens ("decode", with
    the sequence's pages shared out over `splits` CTAs; "decode_clusters": the same with the
    splits merged inside a thread-block cluster)."""
    if kind == "simt":
        K.attention_simt(q, nh * hd, out, step, line, nh, nkv, hd, window, scale)
        return
    if kind == "prefill":
        K.attention_prefill(q, nh * hd, out, step, line, nh, nkv, hd, window, scale)
        return
    if kind == "prefill_tc":
        error = torch.zeros(1, dtype=torch.int32, device=DEV)
        K.attention_prefill_tc(q, nh * hd, out, step, line, nh, nkv, hd, window, scale, error)
        assert int(error.item()) == 0
        return
    splits = splits or 3
    if kind == "decode_clusters":
        error = torch.zeros(1, dtype=torch.int32, device=DEV)
        K.attention_decode_clusters(q, nh * hd, out, step, line, nh, nkv, hd, window, scale,
                                    splits, error)
        assert int(error.item()) == 0
        return
    scratch = torch.empty(out.shape[0] * nh * splits * (hd + 2) + 5, device=DEV)
    error = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.attention_decode(q, nh * hd, out, step, line, nh, nkv, hd, window, scale, splits, scratch,
                       error)
    assert int(error.item()) == 0


ATTENTION_CASES = [("simt", 4, 2, 16, "float32"), ("simt", 6, 1, 48, "float32"),
                   ("simt", 3, 3, 80, "bfloat16"), ("simt", 8, 2, 128, "float32"),
                   ("simt", 16, 2, 64, "bfloat16"), ("simt", 2, 1, 256, "bfloat16"),
                   ("simt", 4, 2, 16, "bfloat16"),
                   ("decode", 8, 2, 128, "bfloat16"), ("decode", 16, 2, 64, "bfloat16"),
                   ("decode", 3, 3, 64, "bfloat16"), ("decode", 40, 2, 128, "bfloat16"),
                   ("decode", 7, 1, 128, "bfloat16"),
                   ("decode_clusters", 8, 2, 128, "bfloat16"),
                   ("decode_clusters", 16, 2, 64, "bfloat16"),
                   ("decode_clusters", 3, 3, 64, "bfloat16"),
                   ("decode_clusters", 40, 2, 128, "bfloat16"),
                   ("decode_clusters", 7, 1, 128, "bfloat16"),
                   ("prefill", 8, 2, 128, "bfloat16"), ("prefill", 16, 2, 64, "bfloat16"),
                   ("prefill", 3, 3, 64, "bfloat16"), ("prefill", 7, 1, 128, "bfloat16"),
                   ("prefill_tc", 8, 2, 128, "bfloat16"), ("prefill_tc", 7, 1, 128, "bfloat16"),
                   ("prefill_tc", 3, 3, 128, "bfloat16")]


@pytest.mark.parametrize("kind,nh,nkv,hd,dtype", ATTENTION_CASES)
def test_attention_over_the_paged_cache(kind, nh, nkv, hd, dtype):
    """Rows of three sequences of unequal lengths in one launch (the last rows of a long
    sequence, a sequence of one token, a whole prompt), over scrambled pages, with and without a
    window; for the tensor-core kernel also with the pages shared out in different ways."""
    rng = np.random.default_rng(nh * hd)
    lens = [200, 1, 77]           # positions already in the cache after this step
    new = [5, 1, 77]              # the last `new` of them are this step's rows
    dt = DT[dtype]
    tol = 2e-6 if dtype == "float32" else 1.2e-2
    for window in (0, 33):
        line = make_line(4, 256, nkv, hd, dt, window=window, seed=hd)
        kv = []
        for slot, n in zip((2, 0, 3), lens):
            k = torch.tensor(rng.standard_normal((n, nkv, hd)), dtype=torch.float32).to(dt).float()
            v = torch.tensor(rng.standard_normal((n, nkv, hd)), dtype=torch.float32).to(dt).float()
            fill_line(line, slot, k, v)
            kv.append((k.numpy(), v.numpy()))
        step = make_step([(slot, n - m, [0] * m, []) for slot, n, m in zip((2, 0, 3), lens, new)])
        T = sum(new)
        q = torch.tensor(rng.standard_normal((T, nh * hd)), dtype=torch.float32).to(dt)
        out = torch.empty(T, nh * hd, dtype=dt, device=DEV)
        scale = 1.0 / math.sqrt(hd)
        # more splits than a sequence has pages, and more than a cluster holds (scratch form)
        many = (18, 32) if kind == "decode" else ()
        for splits in ((1, 3, 4, 7, 8) + many if kind.startswith("decode") else (None,)):
            out.zero_()
            run_attention(kind, q.to(DEV), out, step, line, nh, nkv, hd, window, scale, splits)
            got = out.float().cpu().numpy().reshape(T, nh, hd)
            row = 0
            for (k, v), n, m in zip(kv, lens, new):
                for pos in range(n - m, n):
                    want = attention_reference(q[row].float().numpy().reshape(nh, hd), k, v, nh,
                                               nkv, hd, pos, window, scale)
                    assert rel(got[row], want) <= tol, (window, splits, pos)
                    row += 1


@pytest.mark.parametrize("kind,hd,dtype", [("simt", 32, "float32"), ("simt", 32, "bfloat16"),
                                           ("decode", 64, "bfloat16"), ("decode", 128, "bfloat16"),
                                           ("decode_clusters", 64, "bfloat16"),
                                           ("decode_clusters", 128, "bfloat16"),
                                           ("prefill", 64, "bfloat16"), ("prefill", 128, "bfloat16"),
                                           ("prefill_tc", 128, "bfloat16")])
def test_attention_finds_a_far_key_and_respects_the_windows_edge(kind, hd, dtype):
    """One key among 700 matches the query: the output must be that key's value. With a window,
    the matching key just inside the edge is found and the one just outside is not."""
    nh, nkv, n = 2, 1, 700
    dt = DT[dtype]
    rng = np.random.default_rng(3)
    q = rng.standard_normal((nh, hd)).astype(np.float32)
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    k = (rng.standard_normal((n, nkv, hd)) * 0.05).astype(np.float32)
    v = rng.standard_normal((n, nkv, hd)).astype(np.float32)
    pos = n - 1
    for window, far, seen in ((0, 3, True), (100, pos - 99, True), (100, pos - 100, False)):
        kk = k.copy()
        kk[far, 0] = 40.0 * (q[0] + q[1])       # both heads score this key far above the rest
        # with a window the line keeps a ring of pages: the key just outside the window is
        # still stored there and must be left out by its position
        line = make_line(2, n, nkv, hd, dt, window=window, ring_pages=3 if window else 0,
                         seed=window + far)
        fill_line(line, 1, torch.tensor(kk), torch.tensor(v))
        step = make_step([(1, pos, [0], [])])
        qd = torch.tensor((q * 8.0).reshape(1, nh * hd)).to(dt).to(DEV)
        out = torch.empty(1, nh * hd, dtype=dt, device=DEV)
        run_attention(kind, qd, out, step, line, nh, nkv, hd, window, 1.0, 5)
        got = out.float().cpu().numpy().reshape(nh, hd)
        target = torch.tensor(v[far, 0]).to(dt).float().numpy()
        hit = np.abs(got - target).max() < 2e-2
        assert hit == seen, (window, far, np.abs(got - target).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,rot", [(4, 2, 16, 16), (6, 1, 32, 32), (3, 3, 80, 40),
                                           (2, 2, 128, 128), (2, 1, 256, 0)])
def test_qk_norm_rope_store(dtype, nh, nkv, hd, rot):
    """q in place, k and v into the right page and row of the cache (and nowhere else), angles
    in float32 as the reference forms them, at positions up to 4095, for a ring of pages too."""
    dt = DT[dtype]
    rng = np.random.default_rng(hd + rot)
    seqs = [(1, 4090, [0] * 6, []), (0, 0, [0] * 3, []), (2, 63, [0] * 2, [])]
    T = 11
    for ring in (0, 2):
        line = make_line(3, 4096, nkv, hd, dt, ring_pages=ring, seed=ring)
        step = make_step(seqs)
        width = (nh + 2 * nkv) * hd
        qkv = torch.tensor(rng.standard_normal((T, width)), dtype=torch.float32).to(dt)
        qn = torch.tensor(1 + 0.1 * rng.standard_normal(hd), dtype=torch.float32)
        kn = torch.tensor(1 + 0.1 * rng.standard_normal(hd), dtype=torch.float32)
        inv = plain.inverse_frequencies(1e6, rot) if rot else None
        dev = qkv.to(DEV)
        K.qk_norm_rope_store(dev, qn.to(DEV), kn.to(DEV), 1e-6,
                             torch.tensor(inv).to(DEV) if rot else None, rot, step, line,
                             nh, nkv, hd, True)
        src = qkv.float().numpy()
        positions = [4090 + i for i in range(6)] + [0, 1, 2] + [63, 64]
        slots = [1] * 6 + [0] * 3 + [2] * 2
        tol = 3e-6 if dtype == "float32" else 1.6e-2
        for t in range(T):
            def normed(x, w, heads):
                y = plain.rms_norm(x.reshape(heads, hd), w.numpy(), 1e-6)
                if rot:
                    cos, sin = plain.rotary_tables(inv, [positions[t]])
                    y = y.copy()
                    y[:, :rot] = plain.rope(y[:, :rot].reshape(1, heads * rot), heads, rot,
                                            cos, sin).reshape(heads, rot)
                return y
            q_want = normed(src[t, :nh * hd], qn, nh)
            k_want = normed(src[t, nh * hd:(nh + nkv) * hd], kn, nkv)
            v_want = src[t, (nh + nkv) * hd:].reshape(nkv, hd)
            assert rel(dev[t, :nh * hd].float().cpu().numpy().reshape(nh, hd), q_want) <= tol
            k_got, v_got = read_line(line, slots[t], positions[t])
            assert rel(k_got.numpy(), k_want) <= tol, (t, ring)
            assert np.array_equal(v_got.numpy(), v_want)
        written = int((line.k.float().abs().sum(dim=(1, 3)) > 0).sum())
        assert written == T                      # no other row of any page was touched
        # write_kv off (a layer that reads another layer's cache): q only
        line2 = make_line(3, 4096, nkv, hd, dt, ring_pages=ring)
        q_only = qkv[:, :nh * hd].contiguous().to(DEV)
        K.qk_norm_rope_store(q_only, qn.to(DEV), kn.to(DEV), 1e-6,
                             torch.tensor(inv).to(DEV) if rot else None, rot, step, line2,
                             nh, 0, hd, False)
        assert torch.equal(q_only, dev[:, :nh * hd])
        assert float(line2.k.float().abs().sum()) == 0


def test_qk_norm_rope_store_many_tokens():
    """With many tokens in a step a warp takes several heads one after another and forms the
    sines and cosines of its token once: every head of every token, q, k and v, in bfloat16."""
    nh, nkv, hd, T = 5, 2, 128, 520
    rng = np.random.default_rng(7)
    line = make_line(1, 1024, nkv, hd, torch.bfloat16, seed=3)
    step = make_step([(0, 100, [0] * T, [])])
    qkv = torch.tensor(rng.standard_normal((T, (nh + 2 * nkv) * hd)),
                       dtype=torch.float32).to(torch.bfloat16)
    qn = torch.tensor(1 + 0.1 * rng.standard_normal(hd), dtype=torch.float32)
    kn = torch.tensor(1 + 0.1 * rng.standard_normal(hd), dtype=torch.float32)
    inv = plain.inverse_frequencies(1e6, hd)
    dev = qkv.to(DEV)
    K.qk_norm_rope_store(dev, qn.to(DEV), kn.to(DEV), 1e-6, torch.tensor(inv).to(DEV), hd, step,
                         line, nh, nkv, hd, True)
    src = qkv.float().numpy()
    got_q = dev[:, :nh * hd].float().cpu().numpy()
    for t in range(0, T, 7):
        cos, sin = plain.rotary_tables(inv, [100 + t])

        def normed(x, w, heads):
            y = plain.rms_norm(x.reshape(heads, hd), w.numpy(), 1e-6)
            return plain.rope(y.reshape(1, heads * hd), heads, hd, cos, sin).reshape(heads, hd)
        assert rel(got_q[t].reshape(nh, hd), normed(src[t, :nh * hd], qn, nh)) <= 1.6e-2
        k_got, v_got = read_line(line, 0, 100 + t)
        assert rel(k_got.numpy(), normed(src[t, nh * hd:(nh + nkv) * hd], kn, nkv)) <= 1.6e-2
        assert np.array_equal(v_got.numpy(), src[t, (nh + nkv) * hd:].reshape(nkv, hd))
    assert int((line.k.float().abs().sum(dim=(1, 3)) > 0).sum()) == T


def test_argmax_ties_nan_and_wide_rows():
    nan, inf = float("nan"), float("inf")
    rows = [[1.0, 3.0, 3.0, 2.0], [nan, -inf, nan, -inf], [nan, nan, nan, nan],
            [-0.0, 0.0, -1.0, -2.0], [-5.0, nan, -1.0, -1.0]]
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    K.argmax(torch.tensor(rows, device=DEV), out)
    assert out.tolist() == [1, 1, 0, 0, 2]
    g = torch.Generator().manual_seed(0)
    big = torch.randn(6, 151936 + 5, generator=g)
    big[2, 150000] = big[2, 77] = 9.0                     # a tie far apart: the lower id
    view = big.to(DEV)[:, :151936 + 3]                    # rows wider than the vocabulary
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    K.argmax(view, out)
    want = [plain.arg_max(r.numpy()) for r in big[:, :151936 + 3]]
    assert out.tolist() == want and want[2] == 77
    # the two-stage form: ties across chunks, a chunk of NaN only, the last short chunk
    big[3, 4096:6144] = float("nan")
    big[4, :] = float("nan")
    big[5, 151936 + 2] = 50.0
    want = [plain.arg_max(r.numpy()) for r in big[:, :151936 + 3]]
    scratch = torch.empty(6 * 80, dtype=torch.int64, device=DEV)
    out.fill_(-1)
    K.argmax(big.to(DEV)[:, :151936 + 3], out, scratch)
    assert out.tolist() == want and want[2] == 77 and want[4] == 0 and want[5] == 151936 + 2


@pytest.mark.parametrize("settings", [dict(temperature=1.0), dict(temperature=0.7),
                                      dict(temperature=1.0, top_k=5),
                                      dict(temperature=0.9, top_p=0.8),
                                      dict(temperature=1.3, min_p=0.05),
                                      dict(temperature=0.8, top_k=40, top_p=0.9, min_p=0.02)])
def test_device_sampler_draws_what_the_plain_sampler_draws(settings):
    from mormot2_ai_b200.sampling import DeviceSampler, Sampling
    V, rows, steps = 1000, 5, 40
    g = torch.Generator().manual_seed(11)
    sampler = DeviceSampler(torch.device(DEV), 8, V)
    plain_samplers = [plain.PlainSampler(seed=100 + r, **settings) for r in range(rows)]
    slots = torch.tensor([3, 0, 7, 1, 5], dtype=torch.int32, device=DEV)
    for r in range(rows):
        sampler.start(int(slots[r]), 100 + r)
    same = total = 0
    for _ in range(steps):
        logits = torch.randn(rows, V, generator=g) * 2.5
        logits[:, 10] = logits[:, 11]                      # ties
        logits[0, 5] = float("nan")
        logits[1, 6] = float("-inf")
        got = sampler.pick(logits.to(DEV), slots, Sampling(**settings)).tolist()
        want = [plain_samplers[r].next(logits[r].numpy()) for r in range(rows)]
        same += sum(int(a == b) for a, b in zip(got, want))
        total += rows
    assert same == total


@pytest.mark.parametrize("settings", [dict(temperature=0.9), dict(temperature=1.0, top_k=7),
                                      dict(temperature=0.8, top_p=0.85),
                                      dict(temperature=1.2, min_p=0.03),
                                      dict(temperature=0.8, top_k=50, top_p=0.9, min_p=0.01)])
def test_draws_over_a_wide_vocabulary(settings):
    """Wide rows are shared by a cluster of CTAs: the same draws as the plain sampler, with NaN,
    infinities and ties in the row, a width that the CTAs do not share evenly, and a row without
    any finite value (nothing is drawn and the stream does not move)."""
    from mormot2_ai_b200.sampling import DeviceSampler, Sampling
    V, rows, steps = 40003, 3, 12
    g = torch.Generator().manual_seed(5)
    sampler = DeviceSampler(torch.device(DEV), 4, V)
    plain_samplers = [plain.PlainSampler(seed=7 + r, **settings) for r in range(rows)]
    slots = torch.tensor([2, 0, 3], dtype=torch.int32, device=DEV)
    for r in range(rows):
        sampler.start(int(slots[r]), 7 + r)
    for step in range(steps):
        logits = torch.randn(rows, V, generator=g) * 3
        logits[:, 20000] = logits[:, 20001]
        logits[0, 5] = float("nan")
        logits[1, 39999:] = float("-inf")
        if step == 4:
            logits[2, :] = float("-inf")
            logits[2, 17] = float("nan")
        got = sampler.pick(logits.to(DEV), slots, Sampling(**settings)).tolist()
        want = [plain_samplers[r].next(logits[r].numpy()) for r in range(rows)]
        assert got == want, step


@pytest.mark.parametrize("settings", [dict(temperature=1.0, top_p=0.9),
                                      dict(temperature=0.7, min_p=0.5),
                                      dict(temperature=1.0, top_k=3000, top_p=0.99)])
def test_filtered_draws_from_a_flat_distribution(settings):
    """Nearly equal logits, as a model of random weights gives them: most of the vocabulary is
    a candidate, so the sort runs over tens of thousands of keys (its steps in shared memory
    and the far ones in global memory)."""
    from mormot2_ai_b200.sampling import DeviceSampler, Sampling
    V, rows, steps = 40003, 2, 6
    g = torch.Generator().manual_seed(9)
    sampler = DeviceSampler(torch.device(DEV), 2, V)
    plain_samplers = [plain.PlainSampler(seed=3 + r, **settings) for r in range(rows)]
    slots = torch.tensor([1, 0], dtype=torch.int32, device=DEV)
    for r in range(rows):
        sampler.start(int(slots[r]), 3 + r)
    for step in range(steps):
        logits = torch.randn(rows, V, generator=g) * 0.05
        got = sampler.pick(logits.to(DEV), slots, Sampling(**settings)).tolist()
        want = [plain_samplers[r].next(logits[r].numpy()) for r in range(rows)]
        assert got == want, step


def test_vocab_limit_is_never_crossed():
    from mormot2_ai_b200.sampling import DeviceSampler, Sampling
    sampler = DeviceSampler(torch.device(DEV), 2, 64)
    logits = torch.zeros(2, 64)
    logits[:, 50:] = 20.0                                   # the best ids are beyond the limit
    slots = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    for s in (Sampling(), Sampling(temperature=1.0), Sampling(temperature=1.0, top_k=3)):
        for _ in range(10):
            assert all(t < 50 for t in sampler.pick(logits.to(DEV), slots, s, 50).tolist())


@pytest.mark.parametrize("kind", ["prefill", "prefill_tc"])
@pytest.mark.parametrize("window", [0, 150])
def test_prefill_attention_of_long_unequal_prompts(window, kind):
    """The tensor-core prefill kernel over whole prompts of unequal lengths that cross several
    pages (65, 300, 1 and 129 tokens; the second one continues 70 cached positions)."""
    nh, nkv, hd = 4, 2, 128
    rng = np.random.default_rng(window)
    past = [0, 70, 0, 0]
    new = [65, 300, 1, 129]
    line = make_line(4, 512, nkv, hd, torch.bfloat16, window=window, seed=4)
    kv = []
    for slot, (p, n) in enumerate(zip(past, new)):
        k = torch.tensor(rng.standard_normal((p + n, nkv, hd)), dtype=torch.float32).bfloat16().float()
        v = torch.tensor(rng.standard_normal((p + n, nkv, hd)), dtype=torch.float32).bfloat16().float()
        fill_line(line, slot, k, v)
        kv.append((k.numpy(), v.numpy()))
    step = make_step([(slot, p, [0] * n, []) for slot, (p, n) in enumerate(zip(past, new))])
    T = sum(new)
    q = torch.tensor(rng.standard_normal((T, nh * hd)), dtype=torch.float32).bfloat16()
    out = torch.zeros(T, nh * hd, dtype=torch.bfloat16, device=DEV)
    scale = 1 / math.sqrt(hd)
    run_attention(kind, q.to(DEV), out, step, line, nh, nkv, hd, window, scale)
    got = out.float().cpu().numpy().reshape(T, nh, hd)
    row = 0
    for (k, v), p, n in zip(kv, past, new):
        for i in list(range(0, n, 7)) + [n - 1]:
            want = attention_reference(q[row + i].float().numpy().reshape(nh, hd), k, v, nh, nkv,
                                       hd, p + i, window, scale)
            assert rel(got[row + i], want) <= 1.2e-2, (window, p, i)
        row += n


def test_a_wait_that_nothing_ends_gives_up_and_reports(rt):
    """Every wait of the kernels has an iteration limit, after which the kernel records a code
    in the runtime's error word and goes on to its end. Here the limit is short (2,048 polls of
    a barrier that nothing completes): the kernel returns, the code is in the word, the
    runtime raises it and clears it, and the next kernels run as always."""
    from mormot2_ai_b200 import KernelError
    assert K.wait_selftest(rt.error_word, 17, tries=2048)
    with pytest.raises(KernelError, match="code 17"):
        rt.check()
    rt.check()                                                    # cleared
    a = torch.randn(8, 64).to(torch.bfloat16).to(DEV)
    w = torch.randn(24, 64).to(torch.bfloat16).to(DEV)
    c = torch.empty(8, 24, dtype=torch.float32, device=DEV)
    K.gemm_tc(a, w, c, False, rt.workspace, rt.error_word, rt.sms)
    assert rel(c.cpu(), a.double().cpu() @ w.double().cpu().T) <= 2e-5
    rt.check()
