"""Each CUDA kernel alone against its plain torch version, at sizes other than the engine tests use:
widths and vocabularies that are no power of two, head sizes in steps of 16, odd head counts and groups.
Where random inputs would hide a fault the inputs are made so that it shows (a far key, a window's edge,
a page boundary)."""
import math

import pytest
import torch

from tests.emu_kernels import EmuKernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": dict(atol=2e-6, rtol=1e-5), "bfloat16": dict(atol=2e-2, rtol=2e-2)}


@pytest.fixture(scope="module")
def K():
    from serve_b200.kernels import load_kernels

    return load_kernels(DEV, head_dims=(16, 48, 64, 80, 128, 256))


E = EmuKernels(DEV)


class Shape:
    def __init__(self, rows, tokens, max_q, max_kv, pure_decode=False, min_q=1):
        self.rows, self.tokens, self.max_q, self.max_kv, self.pure_decode, self.min_q = rows, tokens, max_q, max_kv, pure_decode, min_q


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("vocab,dim", [(331, 120), (1000, 2048), (77, 5)])
def test_embedding(K, dtype, vocab, dim):
    table = torch.randn(vocab, dim, device=DEV).to(DT[dtype])
    tokens = torch.randint(0, vocab, (37,), device=DEV, dtype=torch.int32)
    tokens[0], tokens[1] = 0, vocab - 1
    out, ref = torch.empty(37, dim, device=DEV), torch.empty(37, dim, device=DEV)
    K.embedding(tokens, table, out)
    E.embedding(tokens, table, ref)
    assert torch.equal(out, ref)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("wdtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,dim,eps", [(5, 120, 1e-6), (33, 2048, 1e-5), (2, 7, 3e-3), (3, 8192, 1e-5)])
def test_add_rmsnorm(K, dtype, wdtype, rows, dim, eps):
    if dtype == "float32" and wdtype == "bfloat16":
        pytest.skip("a 32-bit model keeps 32-bit norm weights")
    x = torch.randn(rows, dim, device=DEV) * 3
    delta = torch.randn(rows, dim, device=DEV).to(DT[dtype])
    w = (1 + 0.1 * torch.randn(dim, device=DEV)).to(DT[wdtype])
    x1, x2 = x.clone(), x.clone()
    out, ref = torch.empty(rows, dim, device=DEV, dtype=DT[dtype]), torch.empty(rows, dim, device=DEV, dtype=DT[dtype])
    K.add_rmsnorm(x1, delta, w, eps, out)
    E.add_rmsnorm(x2, delta, w, eps, ref)
    assert torch.equal(x1, x2)                       # the residual sum is exact float32 in both
    torch.testing.assert_close(out.float(), ref.float(), **TOL[dtype])
    # without a delta x stays as it is; with rows only those are normalised and x is not written
    x3 = x.clone()
    K.add_rmsnorm(x3, None, w, eps, out)
    assert torch.equal(x3, x)
    sel = torch.tensor([rows - 1, 0], device=DEV, dtype=torch.int32)
    o2, r2 = torch.empty(2, dim, device=DEV, dtype=DT[dtype]), torch.empty(2, dim, device=DEV, dtype=DT[dtype])
    K.add_rmsnorm_rows(x3, delta, sel, w, eps, o2)
    E.add_rmsnorm_rows(x, delta, sel, w, eps, r2)
    assert torch.equal(x3, x)
    torch.testing.assert_close(o2.float(), r2.float(), **TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("m,n,k", [(1, 331, 120), (7, 200, 120), (64, 1000, 72), (300, 8, 264)])
def test_linear(K, dtype, m, n, k):
    a = torch.randn(m, k, device=DEV).to(DT[dtype])
    w = torch.randn(n, k, device=DEV).to(DT[dtype])
    for out_dtype in {DT[dtype], torch.float32}:
        out = torch.empty(m, n, device=DEV, dtype=out_dtype)
        K.linear(a, w, out)
        ref = a.double() @ w.double().T
        tol = dict(atol=1e-4, rtol=1e-5) if out_dtype == torch.float32 else dict(atol=0.15, rtol=1e-2)
        torch.testing.assert_close(out.double(), ref, **tol)


def test_linear_float32_is_not_a_reduced_precision_mode(K):
    """TF32 would keep 10 bits of mantissa of the inputs: an error of ~1e-3 here; true float32 gives ~1e-6."""
    a = torch.full((4, 256), 1.0, device=DEV) + torch.rand(4, 256, device=DEV) * 1e-3
    w = torch.full((16, 256), 1.0, device=DEV) + torch.rand(16, 256, device=DEV) * 1e-3
    out = torch.empty(4, 16, device=DEV)
    K.linear(a, w, out)
    ref = (a.double() @ w.double().T)
    assert float((out.double() - ref).abs().max()) < 2e-4


@pytest.mark.parametrize("m", [1, 7, 8, 9, 17, 32, 33])
@pytest.mark.parametrize("n,k", [(2048, 2048), (331, 72), (5, 4), (1000, 8192), (128256, 256)])
def test_few_rows_product_in_true_float32(K, m, n, k):
    """Up to 32 rows in float32 run on the engine's own plain-arithmetic kernel (33 go to the library): against
    float64, with a bound that a reduced-precision matrix mode would miss by orders of magnitude, and row by row
    the same bits whatever the number of rows."""
    g = torch.Generator(device="cpu").manual_seed(m * 1000 + k)
    a = torch.randn(m, k, generator=g).to(DEV)
    w = torch.randn(n, k, generator=g).to(DEV)
    out = torch.full((m, n), float("nan"), device=DEV)
    before = K.launches
    K.linear(a, w, out)
    assert (K.launches == before + 1) == (m <= 32)
    ref = a.double() @ w.double().T
    assert float((out.double() - ref).abs().max()) <= 3e-7 * math.sqrt(k) * float(ref.abs().max())
    if 1 < m <= 32:
        alone = torch.empty(1, n, device=DEV)
        K.linear(a[m - 1:m].contiguous(), w, alone)
        assert torch.equal(alone[0], out[m - 1])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("t,inter", [(3, 200), (17, 8192), (1, 1)])
def test_swiglu(K, dtype, t, inter):
    gu = (torch.randn(t, 2 * inter, device=DEV) * 4).to(DT[dtype])
    out, ref = torch.empty(t, inter, device=DEV, dtype=DT[dtype]), torch.empty(t, inter, device=DEV, dtype=DT[dtype])
    K.swiglu(gu, out)
    E.swiglu(gu, ref)
    torch.testing.assert_close(out.float(), ref.float(), **TOL[dtype])


def _paged_setup(dtype, heads, kv_heads, d, page, q_lens, kv_lens, num_pages=None, seed=0):
    """Random qkv for a step, caches pre-filled for earlier positions, scrambled block tables."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    r = len(q_lens)
    t = sum(q_lens)
    blocks = [-(-n // page) for n in kv_lens]
    num_pages = num_pages or sum(blocks) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    width = max(blocks)
    bt = torch.full((r, width), -1, dtype=torch.int32)
    for i, nb in enumerate(blocks):
        for b in range(nb):
            bt[i, b] = perm.pop()
    qkv = torch.randn(t, (heads + 2 * kv_heads) * d, generator=g).to(DT[dtype])
    kc = torch.randn(num_pages, kv_heads, page, d, generator=g).to(DT[dtype])
    vc = torch.randn(num_pages, kv_heads, page, d, generator=g).to(DT[dtype])
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    pos = torch.cat([torch.arange(kv - q, kv) for q, kv in zip(q_lens, kv_lens)]).to(torch.int32)
    row = torch.cat([torch.full((q,), i) for i, q in enumerate(q_lens)]).to(torch.int32)
    to = lambda x: x.to(DEV)
    return dict(qkv=to(qkv), kc=to(kc), vc=to(vc), bt=to(bt), cu=to(cu), kv=to(torch.tensor(kv_lens, dtype=torch.int32)),
                pos=to(pos), row=to(row), shape=Shape(r, t, max(q_lens), max(kv_lens), all(q == 1 for q in q_lens), min(q_lens)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,d,rot,pairing,page", [
    (5, 1, 48, 48, 0, 16), (6, 3, 32, 32, 1, 8), (4, 4, 80, 40, 0, 5), (8, 2, 64, 64, 0, 64), (3, 3, 16, 0, 0, 4)])
def test_rope_cache_write(K, dtype, heads, kv_heads, d, rot, pairing, page):
    s = _paged_setup(dtype, heads, kv_heads, d, page, q_lens=[7, 1, 20], kv_lens=[7, 33, 52])
    inv = (1.0 / (10000.0 ** (torch.arange(0, max(rot, 2), 2).float() / max(rot, 2)))).to(DEV)
    a = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in s.items()}
    b = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in s.items()}
    K.rope_cache_write(a["qkv"], a["pos"], a["row"], inv, pairing, rot, heads, kv_heads, d, a["kc"], a["vc"], a["bt"], page, True)
    E.rope_cache_write(b["qkv"], b["pos"], b["row"], inv, pairing, rot, heads, kv_heads, d, b["kc"], b["vc"], b["bt"], page, True)
    K.check_errors()
    tol = dict(atol=3e-6, rtol=1e-5) if dtype == "float32" else dict(atol=4e-2, rtol=2e-2)
    torch.testing.assert_close(a["qkv"].float(), b["qkv"].float(), **tol)
    torch.testing.assert_close(a["kc"].float(), b["kc"].float(), **tol)
    assert torch.equal(a["vc"], b["vc"])
    # an execution that only reads another's cache rotates queries and leaves the pages alone
    c = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in s.items()}
    K.rope_cache_write(c["qkv"], c["pos"], c["row"], inv, pairing, rot, heads, kv_heads, d, c["kc"], c["vc"], c["bt"], page, False)
    assert torch.equal(c["kc"], s["kc"]) and torch.equal(c["vc"], s["vc"])
    torch.testing.assert_close(c["qkv"].float(), b["qkv"].float(), **tol)


@pytest.mark.parametrize("heads,kv_heads,d,rot,page", [(8, 2, 64, 64, 64), (5, 1, 48, 32, 16), (4, 4, 128, 128, 8)])
def test_rope_cache_write_many_tokens(K, heads, kv_heads, d, rot, page):
    """Prompt portions with adjacent pairs take a vectorised kernel (8 elements per thread)."""
    s = _paged_setup("bfloat16", heads, kv_heads, d, page, q_lens=[70, 1, 129], kv_lens=[70, 33, 300])
    inv = (1.0 / (10000.0 ** (torch.arange(0, rot, 2).float() / rot))).to(DEV)
    a = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in s.items()}
    b = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in s.items()}
    K.rope_cache_write(a["qkv"], a["pos"], a["row"], inv, 1, rot, heads, kv_heads, d, a["kc"], a["vc"], a["bt"], page, True)
    E.rope_cache_write(b["qkv"], b["pos"], b["row"], inv, 1, rot, heads, kv_heads, d, b["kc"], b["vc"], b["bt"], page, True)
    K.check_errors()
    q_cols = heads * d
    torch.testing.assert_close(a["qkv"][:, :q_cols].float(), b["qkv"][:, :q_cols].float(), atol=4e-2, rtol=2e-2)
    torch.testing.assert_close(a["kc"].float(), b["kc"].float(), atol=4e-2, rtol=2e-2)
    assert torch.equal(a["vc"], b["vc"])


def test_rotation_at_large_positions(K):
    """Angles are float32 products of position and frequency; at position 100000 a lost bit would show."""
    heads, kv_heads, d = 2, 1, 64
    s = _paged_setup("float32", heads, kv_heads, d, 64, q_lens=[4], kv_lens=[4])
    pos = torch.tensor([0, 8191, 65537, 100_000], dtype=torch.int32, device=DEV)
    inv = (1.0 / (500000.0 ** (torch.arange(0, d, 2).float() / d))).to(DEV)
    q0 = s["qkv"].clone()
    K.rope_cache_write(s["qkv"], pos, s["row"], inv, 0, d, heads, kv_heads, d, s["kc"], s["vc"], s["bt"], 64, False)
    ang = (pos.float()[:, None] * inv[None]).double()
    x = q0.view(4, 4, d)[:, :2].double()
    ref = torch.cat([x[..., :32] * ang.cos()[:, None] - x[..., 32:] * ang.sin()[:, None],
                     x[..., 32:] * ang.cos()[:, None] + x[..., :32] * ang.sin()[:, None]], -1)
    torch.testing.assert_close(s["qkv"].view(4, 4, d)[:, :2].double(), ref, atol=2e-6, rtol=0)


ATT_CASES = [
    # heads, kv, d, page, q_lens, kv_lens, window
    (5, 1, 48, 16, [7, 1, 20], [7, 33, 52], 0),
    (6, 3, 16, 4, [1, 1, 1, 1], [1, 9, 64, 130], 0),
    (8, 2, 64, 64, [40, 3], [200, 64], 0),
    (4, 4, 80, 8, [17, 2], [17, 90], 0),
    (2, 1, 128, 32, [33], [97], 0),
    (3, 1, 256, 16, [5, 1], [37, 50], 0),
    (4, 2, 64, 8, [30, 1, 6], [30, 77, 100], 11),
    (4, 2, 64, 16, [1, 1], [300, 17], 16),
    # page sizes that are no power of two, or larger than a tile of keys: a tile then crosses pages at odd places
    (8, 2, 64, 24, [40, 3, 1], [200, 75, 333], 0),
    (6, 2, 32, 48, [1, 1, 50], [500, 49, 97], 0),
    (8, 4, 64, 128, [130, 1, 2], [300, 1000, 129], 0),
    (4, 2, 128, 24, [1, 30], [700, 100], 50),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ATT_CASES, ids=[f"h{c[0]}kv{c[1]}d{c[2]}p{c[3]}w{c[6]}" for c in ATT_CASES])
def test_attention(K, dtype, case):
    heads, kv_heads, d, page, q_lens, kv_lens, window = case
    s = _paged_setup(dtype, heads, kv_heads, d, page, q_lens, kv_lens)
    t = sum(q_lens)
    out = torch.zeros(t, heads * d, device=DEV, dtype=DT[dtype])
    ref = torch.zeros(t, heads * d, device=DEV, dtype=DT[dtype])
    scale = 1.0 / math.sqrt(d)
    K.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page, scale, window, out, s["shape"])
    E.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page, scale, window, ref, s["shape"])
    tol = dict(atol=5e-6, rtol=1e-5) if dtype == "float32" else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(out.float(), ref.float(), **tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far_key", [0, 63, 64, 255, 256, 511])
def test_attention_finds_one_far_key(K, dtype, far_key):
    """One key among 600 is made to match the query (large score), its value is a marker: the output must be
    the marker. A fault at a page's edge, in a tile's mask or in the block table would lose it."""
    heads, kv_heads, d, page = 4, 2, 64, 64
    L = 600
    s = _paged_setup(dtype, heads, kv_heads, d, page, q_lens=[1], kv_lens=[L], seed=far_key)
    s["qkv"].mul_(0.05)
    s["kc"].mul_(0.05)
    blk, off = far_key // page, far_key % page
    pg = int(s["bt"][0, blk])
    for kvh in range(kv_heads):
        s["kc"][pg, kvh, off] = 0
        s["kc"][pg, kvh, off, :8] = 20.0
        s["vc"][pg, kvh, off] = 7.0
    q = s["qkv"].view(1, heads + 2 * kv_heads, d)
    q[0, :heads, :8] = 20.0
    out = torch.zeros(1, heads * d, device=DEV, dtype=DT[dtype])
    K.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page,
                1.0 / math.sqrt(d), 0, out, s["shape"])
    torch.testing.assert_close(out.float(), torch.full_like(out, 7.0).float(), atol=1e-2, rtol=0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_window_edge(K, dtype):
    """Window 16: the key 16 back is outside, the key 15 back is inside. Both are given huge scores in turn."""
    heads, kv_heads, d, page, window, L = 2, 1, 32, 8, 16, 100
    for back, inside in ((16, False), (15, True)):
        s = _paged_setup(dtype, heads, kv_heads, d, page, q_lens=[1], kv_lens=[L], seed=back)
        s["qkv"].mul_(0.05); s["kc"].mul_(0.05)
        key = L - 1 - back
        pg = int(s["bt"][0, key // page])
        s["kc"][pg, 0, key % page] = 0
        s["kc"][pg, 0, key % page, :8] = 20.0
        s["vc"][pg, 0, key % page] = 7.0
        s["qkv"].view(1, heads + 2, d)[0, :heads, :8] = 20.0
        out = torch.zeros(1, heads * d, device=DEV, dtype=DT[dtype])
        K.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page,
                    1.0 / math.sqrt(d), window, out, s["shape"])
        hit = bool((out.float() - 7.0).abs().max() < 1e-2)
        assert hit == inside, f"key {back} back: inside={inside}, output max {float(out.float().abs().max()):.3f}"


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("window,length", [(512, 513), (4096, 5000), (4096, 4097), (1000, 1301)])
def test_decode_attention_with_a_window_over_several_splits_keeps_the_newest_key(K, d, window, length):
    """Decoding with a window that spans several key splits: only the newest key (the token's own) matches the
    query, its value is a marker. Splits sized from a first key that lies on no boundary would end before it."""
    heads, kv_heads, page = 8, 2, 64
    s = _paged_setup("bfloat16", heads, kv_heads, d, page, q_lens=[1], kv_lens=[length], seed=window)
    s["qkv"].mul_(0.05); s["kc"].mul_(0.05)
    for key, marker in ((length - 1, 7.0), (length - window, -3.0), (length - window - 1, 100.0)):
        pg = int(s["bt"][0, key // page])
        for kvh in range(kv_heads):
            s["kc"][pg, kvh, key % page] = 0
            # the newest key matches strongly, the oldest key inside the window weakly, the first one outside strongly
            s["kc"][pg, kvh, key % page, :8] = 20.0 if marker != -3.0 else 2.0
            s["vc"][pg, kvh, key % page] = marker
    s["qkv"].view(1, heads + 2 * kv_heads, d)[0, :heads, :8] = 20.0
    out = torch.zeros(1, heads * d, device=DEV, dtype=torch.bfloat16)
    ref = torch.zeros_like(out)
    scale = 1.0 / math.sqrt(d)
    assert K.split_plan(1, kv_heads, length) > 1
    K.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page, scale, window, out, s["shape"])
    E.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page, scale, window, ref, s["shape"])
    torch.testing.assert_close(out.float(), ref.float(), atol=2e-2, rtol=2e-2)
    assert float((out.float() - 7.0).abs().max()) < 0.1


def test_refused_sizes(K):
    from serve_b200.kernels import KernelError

    for bad in (8, 24, 272, 100):
        with pytest.raises(KernelError, match="head_dim"):
            K.check_attention_shape(4, 2, bad)
    with pytest.raises(KernelError, match="multiple"):
        K.check_attention_shape(6, 4, 64)


@pytest.mark.parametrize("vocab", [331, 128256, 1000])
def test_sampling(K, vocab):
    from tests.plain.llama_plain import sample_token

    rows = 6
    logits = torch.randn(rows, vocab, device=DEV) * 3
    logits[0, 17] = logits[0, 200] = 50.0          # a tie: the lowest index wins
    temps = torch.tensor([0.0, 0.0, 0.8, 0.8, 1.5, 0.3], device=DEV)
    req = torch.tensor([0, 1, 2, 2, 5, 9], dtype=torch.int32, device=DEV)
    tok = torch.tensor([0, 3, 4, 5, 0, 7], dtype=torch.int32, device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    K.sample(logits, temps, req, tok, 1234567890123, out)
    got = out.tolist()
    assert got[0] == 17 and got[1] == int(logits[1].argmax())
    want = [sample_token(logits[i].cpu(), float(temps[i]), 1234567890123, int(req[i]), int(tok[i])) for i in range(rows)]
    assert got == want
    assert got[2] != got[3] or vocab < 10      # other token index, other draw (equal only by chance)


def test_sampling_distribution(K):
    logits = torch.tensor([[0.0, 1.0, 2.0, -1.0, 0.5]], device=DEV).repeat(4000, 1)
    temps = torch.full((4000,), 0.7, device=DEV)
    req = torch.zeros(4000, dtype=torch.int32, device=DEV)
    tok = torch.arange(4000, dtype=torch.int32, device=DEV)
    out = torch.empty(4000, dtype=torch.int32, device=DEV)
    K.sample(logits, temps, req, tok, 5, out)
    freq = torch.bincount(out.long(), minlength=5).float() / 4000
    want = torch.softmax(logits[0] / 0.7, -1)
    assert float((freq - want).abs().max()) < 0.03


MMA_CASES = [
    # heads, kv, d, page, q_lens, kv_lens, window : shapes that reach both block shapes, the split of keys and its merge
    (32, 8, 64, 64, [1] * 8, [2176, 100, 64, 65, 1, 4000, 513, 128], 0),       # decoding, long contexts, many splits
    (32, 8, 64, 64, [1], [3000], 0),                                          # batch 1
    (32, 8, 64, 16, [300, 1, 2, 4, 5, 64], [300, 700, 50, 4, 900, 1000], 0),  # portions beside decoded tokens
    (24, 8, 128, 32, [130, 1, 3], [130, 260, 131], 0),
    (5, 1, 48, 16, [40, 1, 3, 4], [41, 99, 200, 4], 0),                       # group of 5: 3 tokens fit the deep shape, 4 do not
    (40, 2, 32, 8, [1, 9], [77, 30], 0),                                      # group of 20: wide shape only
    (6, 6, 80, 8, [1, 16, 17], [500, 16, 300], 0),                            # no grouping
    (4, 2, 256, 16, [70, 1], [70, 333], 0),
    (8, 4, 16, 4, [3, 129], [1000, 129], 0),
    (8, 2, 64, 8, [60, 1, 2], [200, 400, 90], 37),                            # windows
    (8, 2, 64, 64, [1, 1], [1000, 40], 128),
    # a window over several key splits whose first key lies on no unit boundary of the splits
    (8, 2, 64, 64, [1, 1], [5000, 4097], 4096),
    (8, 2, 128, 64, [1, 1], [5000, 4097], 4096),
    (32, 8, 64, 64, [1], [513], 512),
    (8, 2, 64, 32, [2, 1, 1], [2000, 1500, 777], 700),
    # page sizes that are no power of two, or larger than a tile of keys
    (32, 8, 64, 24, [1, 1, 1, 70], [2176, 100, 25, 300], 0),
    (32, 8, 64, 48, [1, 300, 2], [3000, 300, 95], 0),
    (32, 8, 64, 128, [1, 1, 200, 3], [2176, 129, 1000, 128], 0),
    (16, 4, 128, 128, [1, 150], [1500, 150], 0),
    (8, 2, 64, 24, [1, 1], [1000, 40], 100),
]


@pytest.mark.parametrize("case", MMA_CASES, ids=[f"h{c[0]}kv{c[1]}d{c[2]}p{c[3]}w{c[6]}n{len(c[4])}" for c in MMA_CASES])
def test_attention_tensor_cores_against_plain_arithmetic(K, case):
    """bfloat16: the tensor-core kernel against the plain-arithmetic kernel and the torch version."""
    heads, kv_heads, d, page, q_lens, kv_lens, window = case
    s = _paged_setup("bfloat16", heads, kv_heads, d, page, q_lens, kv_lens)
    t = sum(q_lens)
    scale = 1.0 / math.sqrt(d)
    outs = {}
    for name in ("mma", "simt", "torch"):
        out = torch.full((t, heads * d), float("nan"), device=DEV, dtype=torch.bfloat16)
        if name == "torch":
            E.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page, scale, window, out, s["shape"])
        else:
            K.force_simt_attention = name == "simt"
            try:
                K.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page, scale, window, out, s["shape"])
            finally:
                K.force_simt_attention = False
        outs[name] = out.float()
    assert bool(torch.isfinite(outs["mma"]).all()), "a row was not written, or NaN"
    torch.testing.assert_close(outs["simt"], outs["torch"], atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(outs["mma"], outs["torch"], atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("heads,kv_heads,d,page,rows,max_q", [(32, 8, 64, 64, 150, 1), (16, 4, 128, 16, 300, 1), (24, 2, 64, 32, 520, 1),
                                                               (8, 8, 64, 64, 140, 2), (12, 4, 32, 8, 260, 3), (32, 8, 64, 64, 100, 1),
                                                               (32, 8, 64, 64, 60, 1), (16, 8, 128, 16, 45, 2), (6, 2, 256, 32, 170, 1)])
def test_decode_attention_for_a_crowd_of_short_requests(K, heads, kv_heads, d, page, rows, max_q):
    """Hundreds to thousands of (request, kv head) pairs in one step: blocks of one warp (a thousand and more pairs of
    short sequences, or when two-warp blocks would leave a thin last round) or of two warps (more pairs than four-warp
    blocks hold at once). Short sequences of very different lengths, one to three new tokens each, groups of 1 to 12
    query heads; unwritten cache rows hold NaN."""
    assert rows * kv_heads >= 300
    g = torch.Generator().manual_seed(rows)
    q_lens = torch.randint(1, max_q + 1, (rows,), generator=g).tolist()
    kv_lens = [q + int(x) for q, x in zip(q_lens, torch.randint(0, 330, (rows,), generator=g).tolist())]
    s = _paged_setup("bfloat16", heads, kv_heads, d, page, q_lens, kv_lens)
    for r, L in enumerate(kv_lens):
        b = (L - 1) // page
        if L % page:
            s["kc"][int(s["bt"][r, b]), :, L % page:] = float("nan")
            s["vc"][int(s["bt"][r, b]), :, L % page:] = float("nan")
    t = sum(q_lens)
    scale = 1.0 / math.sqrt(d)
    out = torch.full((t, heads * d), float("nan"), device=DEV, dtype=torch.bfloat16)
    ref = torch.empty_like(out)
    K.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page, scale, 0, out, s["shape"])
    K.check_errors()
    E.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page, scale, 0, ref, s["shape"])
    assert bool(torch.isfinite(out.float()).all()), "a row was not written, or NaN"
    torch.testing.assert_close(out.float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_attention_unwritten_cache_does_not_leak(K):
    """Pages hold NaN wherever nothing was written (beyond each request's length): outputs stay finite."""
    heads, kv_heads, d, page = 8, 2, 64, 16
    q_lens, kv_lens = [1, 5, 40], [70, 21, 40]
    s = _paged_setup("bfloat16", heads, kv_heads, d, page, q_lens, kv_lens)
    for r, L in enumerate(kv_lens):
        for b in range(-(-L // page)):
            pg = int(s["bt"][r, b])
            lo = max(0, L - b * page)
            if lo < page:
                s["kc"][pg, :, lo:] = float("nan")
                s["vc"][pg, :, lo:] = float("nan")
    used = set(int(x) for x in s["bt"].flatten().tolist() if x >= 0)
    for pg in range(s["kc"].shape[0]):
        if pg not in used:
            s["kc"][pg] = float("nan"); s["vc"][pg] = float("nan")
    out = torch.zeros(sum(q_lens), heads * d, device=DEV, dtype=torch.bfloat16)
    ref = torch.zeros_like(out)
    K.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page, 0.125, 0, out, s["shape"])
    E.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page, 0.125, 0, ref, s["shape"])
    assert bool(torch.isfinite(out.float()).all())
    torch.testing.assert_close(out.float(), ref.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("m", [1, 3, 8, 9, 12, 16])
@pytest.mark.parametrize("n,k", [(2048, 2048), (100, 64), (331, 96), (16, 8192), (4000, 32)])
def test_skinny_linear(K, m, n, k):
    """The few-rows product against float64, bfloat16 and float outputs; and a row's result must not depend on
    how many other rows there are."""
    a = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = torch.randn(n, k, device=DEV).to(torch.bfloat16)
    ref = a.double() @ w.double().T
    assert K._core.sb_skinny_linear_supports(m, n, k, 0) == 1
    before = K.launches
    for out_dtype in (torch.float32, torch.bfloat16):
        out = torch.full((m, n), float("nan"), device=DEV, dtype=out_dtype)
        K.linear(a, w, out)
        tol = dict(atol=2e-3 * math.sqrt(k / 64), rtol=1e-4) if out_dtype == torch.float32 else dict(atol=0.1 * math.sqrt(k / 64), rtol=1e-2)
        torch.testing.assert_close(out.double(), ref, **tol)
    assert K.launches == before + 2, "these sizes must take the hand-written kernel"
    one = torch.empty(1, n, device=DEV)
    K.linear(a[m - 1:m].contiguous(), w, one)
    full = torch.empty(m, n, device=DEV)
    K.linear(a, w, full)
    assert torch.equal(one[0], full[m - 1])


@pytest.mark.parametrize("m", [1, 5, 8, 16])
@pytest.mark.parametrize("inter,k", [(8192, 2048), (200, 96), (320, 192)])
def test_fused_gate_up_equals_unfused(K, m, inter, k):
    h = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, device=DEV) * 0.05).to(torch.bfloat16)
    fused = torch.full((m, inter), float("nan"), device=DEV, dtype=torch.bfloat16)
    K.gate_up_swiglu(h, w, fused)
    K.use_skinny_linear = False
    try:
        plain = torch.empty_like(fused)
        K.gate_up_swiglu(h, w, plain)
    finally:
        K.use_skinny_linear = True
    ref = torch.empty_like(fused)
    E.gate_up_swiglu(h, w, ref)
    scale = float(ref.float().abs().max())
    torch.testing.assert_close(fused.float(), ref.float(), atol=scale * 2.0 ** -6, rtol=0)
    torch.testing.assert_close(plain.float(), ref.float(), atol=scale * 2.0 ** -6, rtol=0)


def test_sizes_the_skinny_kernel_leaves_to_the_library(K):
    for m, n, k in [(17, 64, 64), (33, 64, 64), (4, 64, 120), (4, 64, 16)]:
        assert K._core.sb_skinny_linear_supports(m, n, k, 0) == 0
        a = torch.randn(m, k, device=DEV).to(torch.bfloat16)
        w = torch.randn(n, k, device=DEV).to(torch.bfloat16)
        out = torch.empty(m, n, device=DEV)
        K.linear(a, w, out)
        torch.testing.assert_close(out.double(), a.double() @ w.double().T, atol=1e-2, rtol=1e-3)


TC_SHAPES = [(128, 128, 64), (256, 256, 256), (2048, 3072, 2048), (300, 264, 200), (64, 136, 72), (1000, 2048, 8192), (129, 8, 8)]


@pytest.fixture(params=["pairs", "single"])
def cta_mode(K, request):
    """Tiles of more than 128 rows run on CTA pairs (cta_group::2) by default; "single" keeps them on the one-CTA kernel."""
    K._core.sb_gemm_tcgen05_use_pairs(2 if request.param == "pairs" else 0)
    K.tcgen05_for_plain_products = True      # (plain products are the library's unless asked for: these tests ask)
    yield request.param
    K._core.sb_gemm_tcgen05_use_pairs(1)
    del K.tcgen05_for_plain_products


@pytest.mark.parametrize("m,n,k", TC_SHAPES + [(257, 520, 136), (4096, 512, 64), (777, 2048, 1000)])
def test_tcgen05_product(K, m, n, k, cta_mode):
    """The tensor-memory product (TMA in, tcgen05.mma, tcgen05.ld out) against float64: full tiles, ragged edges in every
    dimension, k not a multiple of the stage, a single partial tile."""
    a = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    out = torch.full((m, n), float("nan"), device=DEV, dtype=torch.bfloat16)
    assert K._core.sb_gemm_tcgen05_supports(m, n, k, 0) == 1
    before = K.launches
    K.TCGEN05_MIN_TILES = 1            # small cases too go to the kernel under test
    try:
        K.linear(a, w, out)
    finally:
        K.TCGEN05_MIN_TILES = type(K).TCGEN05_MIN_TILES
    assert K.launches == before + 1, "these sizes must take the hand-written kernel"
    K.check_errors()
    ref = a.double() @ w.double().T
    assert bool(torch.isfinite(out.float()).all()), "a tile was not written"
    torch.testing.assert_close(out.double(), ref, atol=float(ref.abs().max()) * 2.0 ** -7, rtol=0)
    # the library agrees, and a row's result does not depend on the other rows of the step
    K.use_tcgen05 = False
    try:
        lib = torch.empty_like(out)
        K.linear(a, w, lib)
    finally:
        K.use_tcgen05 = True
    torch.testing.assert_close(out.float(), lib.float(), atol=float(ref.abs().max()) * 2.0 ** -7, rtol=0)
    if m > 64:
        part = torch.empty(64, n, device=DEV, dtype=torch.bfloat16)
        K.TCGEN05_MIN_TILES = 1
        try:
            K.linear(a[m - 64:].contiguous(), w, part)
        finally:
            K.TCGEN05_MIN_TILES = type(K).TCGEN05_MIN_TILES
        assert torch.equal(part, out[m - 64:])


@pytest.mark.parametrize("width", [96, 128, 160, 224, 256])
def test_tcgen05_product_at_every_tile_width(K, width, cta_mode):
    """The tile plan picks the accumulator width per product (a multiple of 32 columns); every width gives the same
    numbers, since the order of the k-values in a sum does not depend on it."""
    m, n, k = 390, 712, 200
    a = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    outs = []
    K.TCGEN05_MIN_TILES = 1
    try:
        for bn in (0, width):
            K._core.sb_gemm_tcgen05_force_width(bn)
            out = torch.full((m, n), float("nan"), device=DEV, dtype=torch.bfloat16)
            before = K.launches
            K.linear(a, w, out)
            assert K.launches == before + 1
            outs.append(out)
    finally:
        K._core.sb_gemm_tcgen05_force_width(0)
        K.TCGEN05_MIN_TILES = type(K).TCGEN05_MIN_TILES
    K.check_errors()
    ref = a.double() @ w.double().T
    torch.testing.assert_close(outs[1].double(), ref, atol=float(ref.abs().max()) * 2.0 ** -7, rtol=0)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("m,inter,k", [(128, 128, 64), (2048, 8192, 2048), (300, 384, 200), (130, 128, 72), (64, 256, 96)])
def test_tcgen05_gate_up_with_swiglu(K, m, inter, k, cta_mode):
    h = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, device=DEV) * 0.05).to(torch.bfloat16)
    fused = torch.full((m, inter), float("nan"), device=DEV, dtype=torch.bfloat16)
    assert K._core.sb_gemm_tcgen05_supports(m, inter, k, 1) == 1
    before = K.launches
    K.TCGEN05_MIN_TILES = 1
    try:
        K.gate_up_swiglu(h, w, fused)
    finally:
        K.TCGEN05_MIN_TILES = type(K).TCGEN05_MIN_TILES
    assert K.launches == before + 1
    K.check_errors()
    ref = torch.empty_like(fused)
    E.gate_up_swiglu(h, w, ref)
    scale = float(ref.float().abs().max())
    assert bool(torch.isfinite(fused.float()).all())
    torch.testing.assert_close(fused.float(), ref.float(), atol=scale * 2.0 ** -6, rtol=0)


@pytest.mark.parametrize("heads,kv_heads,d,rot,page,k,q_lens,kv_lens", [
    (8, 2, 64, 64, 64, 512, [300, 1, 129], [300, 33, 400]),        # whole tiles and a ragged last one
    (5, 1, 96, 64, 16, 200, [70, 200], [70, 333]),                 # partial rotation, 3 chunks of 32 a head, ragged k
    (3, 3, 128, 128, 8, 136, [257], [1000]),                       # as many k/v heads as q heads, tiny pages
    (2, 1, 32, 32, 32, 64, [64], [64])])                           # a tile wider than all the columns
def test_tcgen05_qkv_product_with_rotation(K, heads, kv_heads, d, rot, page, k, q_lens, kv_lens, cta_mode):
    """The q/k/v product whose epilogue rotates and writes the cache against the product followed by the rotary kernel:
    same rounding points, so they agree to the last bit of bfloat16 except where the compiler contracted differently."""
    s = _paged_setup("bfloat16", heads, kv_heads, d, page, q_lens=q_lens, kv_lens=kv_lens, seed=5)
    t, n = s["qkv"].shape
    h = torch.randn(t, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    inv = (1.0 / (500000.0 ** (torch.arange(0, rot, 2).float() / rot))).to(DEV)
    assert K._core.sb_gemm_tcgen05_qkv_rope_supports(t, k, rot, heads, kv_heads, d) == 1
    a = {key: (v.clone() if torch.is_tensor(v) else v) for key, v in s.items()}
    b = {key: (v.clone() if torch.is_tensor(v) else v) for key, v in s.items()}
    a["qkv"].fill_(float("nan"))
    K.TCGEN05_MIN_TILES = 1
    try:
        before = K.launches
        memo = {}
        K.qkv_rope_cache(h, w, a["qkv"], a["pos"], a["row"], inv, 1, rot, heads, kv_heads, d, a["kc"], a["vc"], a["bt"], page, True,
                         memo=memo)
        assert K.launches == before + 2, "the step's table of cosines and sines, and one kernel for the rest"
        # a later layer of the step finds the table; one that reads another layer's cache rotates its queries and
        # writes no page
        c = {key: (v.clone() if torch.is_tensor(v) else v) for key, v in s.items()}
        K.qkv_rope_cache(h, w, c["qkv"], a["pos"], c["row"], inv, 1, rot, heads, kv_heads, d, c["kc"], c["vc"], c["bt"], page, False,
                         memo=memo)
        assert K.launches == before + 3
        K.fuse_rope = False
        K.qkv_rope_cache(h, w, b["qkv"], b["pos"], b["row"], inv, 1, rot, heads, kv_heads, d, b["kc"], b["vc"], b["bt"], page, True)
        assert K.launches == before + 5
    finally:
        K.fuse_rope = True
        K.TCGEN05_MIN_TILES = type(K).TCGEN05_MIN_TILES
    K.check_errors()
    q_cols = heads * d
    assert bool(torch.isfinite(a["qkv"][:, :q_cols].float()).all()), "a query tile was not written"
    ulp = dict(atol=2.0 ** -7 * float(b["qkv"][:, :q_cols].float().abs().max()), rtol=0)
    torch.testing.assert_close(a["qkv"][:, :q_cols].float(), b["qkv"][:, :q_cols].float(), **ulp)
    torch.testing.assert_close(a["kc"].float(), b["kc"].float(), **ulp)
    assert torch.equal(a["vc"], b["vc"])
    assert not torch.equal(a["kc"], s["kc"]) and not torch.equal(a["vc"], s["vc"])
    assert torch.equal(c["kc"], s["kc"]) and torch.equal(c["vc"], s["vc"])
    assert torch.equal(c["qkv"][:, :q_cols], a["qkv"][:, :q_cols])
    # against float64 from the definition: the product, then pairs (2j, 2j+1) turned by position * inv_freq[j]
    full = (h.double() @ w.double().T).view(t, heads + 2 * kv_heads, d)
    ang = s["pos"].double()[:, None] * inv.double()[None]
    x, y = full[:, :heads + kv_heads, 0:rot:2], full[:, :heads + kv_heads, 1:rot:2]
    turned = full.clone()
    turned[:, :heads + kv_heads, 0:rot:2] = x * ang.cos()[:, None] - y * ang.sin()[:, None]
    turned[:, :heads + kv_heads, 1:rot:2] = y * ang.cos()[:, None] + x * ang.sin()[:, None]
    tol = dict(atol=float(turned.abs().max()) * 2.0 ** -6, rtol=0)
    torch.testing.assert_close(a["qkv"][:, :q_cols].double().view(t, heads, d), turned[:, :heads], **tol)
    pos, row = s["pos"].long(), s["row"].long()
    pages = s["bt"].long()[row, pos // page]
    got_k = a["kc"][pages, :, pos % page].double()            # [t, kv_heads, d]
    got_v = a["vc"][pages, :, pos % page].double()
    torch.testing.assert_close(got_k, turned[:, heads:heads + kv_heads], **tol)
    torch.testing.assert_close(got_v, turned[:, heads + kv_heads:], **tol)


def test_sizes_the_tcgen05_product_leaves_to_the_library(K):
    assert K._core.sb_gemm_tcgen05_supports(128, 100, 64, 0) == 0      # output rows must be 16-byte multiples
    assert K._core.sb_gemm_tcgen05_supports(128, 128, 60, 0) == 0      # so must input rows (TMA pitch)
    assert K._core.sb_gemm_tcgen05_supports(128, 192, 64, 1) == 0      # gate tile would reach into the up rows
    assert K._core.sb_gemm_tcgen05_qkv_rope_supports(128, 64, 48, 4, 2, 48) == 0   # heads of 48: a 32-column chunk would span two
    assert K._core.sb_gemm_tcgen05_qkv_rope_supports(128, 64, 31, 4, 2, 64) == 0   # pairs need an even rotary width
    a = torch.randn(128, 60, device=DEV).to(torch.bfloat16)
    w = torch.randn(100, 60, device=DEV).to(torch.bfloat16)
    out = torch.empty(128, 100, device=DEV, dtype=torch.bfloat16)
    K.linear(a, w, out)
    torch.testing.assert_close(out.double(), a.double() @ w.double().T, atol=0.3, rtol=2e-2)


TC_ATT_CASES = [
    # heads, kv, page, q_lens, kv_lens
    (4, 1, 64, [128], [128]),                              # one full tile of rows, one page
    (4, 1, 64, [33], [33]),                                # a ragged tile
    (32, 8, 64, [2048], [2048]),                           # the benchmark's shape
    (32, 8, 16, [300, 1, 70], [300, 700, 500]),            # portions with a cached prefix beside a decoded token
    (8, 8, 32, [130, 40], [130, 1000]),                    # no grouping
    (16, 2, 8, [65, 17], [400, 17]),                       # group of 8, small pages
    (64, 1, 64, [50], [777]),                              # group of 64: two tokens to a tile
    (24, 8, 64, [300, 45], [300, 700]),                    # group of 3: 42 tokens (126 rows) to a tile, two rows unused
    (10, 2, 32, [129, 90], [129, 500]),                    # group of 5
    (12, 1, 16, [70], [333]),                              # group of 12: ten tokens to a tile
    (100, 1, 64, [40], [40]),                              # group of 100: one token to a tile
    (32, 8, 128, [300, 1, 70], [300, 700, 500]),           # pages of two key tiles
    (6, 2, 256, [513, 40], [513, 1000]),                   # pages of four key tiles, sequences that end inside one
]


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("case", TC_ATT_CASES, ids=[f"h{c[0]}kv{c[1]}p{c[2]}n{len(c[3])}" for c in TC_ATT_CASES])
def test_attention_tensor_memory_path(K, case, d):
    """Prompt portions at head_dim 64 and 128 run on tcgen05 (TMA in, scores and output in tensor memory): against the
    mma.sync kernel and the torch version, with unwritten cache rows poisoned. At 128 every operand row is two
    swizzle atoms."""
    heads, kv_heads, page, q_lens, kv_lens = case
    lib = K._attention_lib(d)
    assert lib.sb_attention_tc_supports(heads, kv_heads, page, 0, (heads + 2 * kv_heads) * d) == 1
    s = _paged_setup("bfloat16", heads, kv_heads, d, page, q_lens, kv_lens)
    for r, L in enumerate(kv_lens):                        # rows of the last page beyond the sequence: NaN
        b = (L - 1) // page
        if L % page:
            s["kc"][int(s["bt"][r, b]), :, L % page:] = float("nan")
            s["vc"][int(s["bt"][r, b]), :, L % page:] = float("nan")
    t = sum(q_lens)
    scale = 1.0 / math.sqrt(d)
    outs = {}
    for name in ("tc", "legacy", "torch"):
        out = torch.full((t, heads * d), float("nan"), device=DEV, dtype=torch.bfloat16)
        if name == "torch":
            E.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page, scale, 0, out, s["shape"])
        else:
            K.use_tcgen05_attention = name == "tc"
            try:
                K.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page, scale, 0, out, s["shape"])
            finally:
                K.use_tcgen05_attention = True
            K.check_errors()
        outs[name] = out.float()
    assert bool(torch.isfinite(outs["tc"]).all()), "a row was not written, or NaN"
    torch.testing.assert_close(outs["tc"], outs["torch"], atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(outs["legacy"], outs["torch"], atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("d", [64, 128])
def test_attention_tensor_memory_path_rescales_when_the_maximum_runs_ahead(K, d):
    """The tcgen05 kernel keeps its output in tensor memory and rescales it only when a row's maximum has moved by
    more than a factor 2^8. Here later keys score far higher than earlier ones, several times in a row."""
    heads, kv_heads, page = 4, 1, 64
    L = 512
    s = _paged_setup("bfloat16", heads, kv_heads, d, page, [L], [L], seed=7)
    s["qkv"].mul_(0.1)
    q = s["qkv"].view(L, heads + 2, d)
    q[:, :heads, :4] = 3.0
    for key in range(L):                                   # keys grow with their position: maxima keep moving
        blk, off = key // page, key % page
        s["kc"][int(s["bt"][0, blk]), 0, off, :4] = 0.02 * key
    out = torch.full((L, heads * d), float("nan"), device=DEV, dtype=torch.bfloat16)
    ref = torch.empty_like(out)
    K.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page, 1.0, 0, out, s["shape"])
    K.check_errors()
    E.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], s["row"], s["pos"], heads, kv_heads, d, page, 1.0, 0, ref, s["shape"])
    torch.testing.assert_close(out.float(), ref.float(), atol=3e-2, rtol=3e-2)
