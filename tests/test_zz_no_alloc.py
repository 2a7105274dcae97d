"""The attention entry point that brings its own scratch memory (csrc/attention_noalloc.h).

Some users of this library cannot allocate device memory when they need attention: their process gave out the
whole device at start-up, or they run inside another runtime's callback where allocators are off limits. For them
the library has one exported C function that uses a fixed array linked into the library instead of caller-provided
scratch. This test calls it through its C symbol, twice in a row (the second call finds the first call's leftovers in
the array), and checks both results against attention in plain float arithmetic (torch) and against the regular
entry point's: one token per request and up to three (nine to twelve rows: the second kernel instantiation), head
sizes 64 and 128, with and without key splits, and with a window longer than a split.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _setup(q_lens, heads, kv_heads, d, page, kv_lens, seed):
    g = torch.Generator().manual_seed(seed)
    batch = len(kv_lens)
    blocks = [-(-n // page) for n in kv_lens]
    pages = sum(blocks) + 2
    perm = torch.randperm(pages, generator=g).tolist()
    bt = torch.full((batch, max(blocks)), -1, dtype=torch.int32)
    for i, nb in enumerate(blocks):
        for b in range(nb):
            bt[i, b] = perm.pop()
    to = lambda x: x.to(DEV)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    return dict(
        qkv=to(torch.randn(sum(q_lens), (heads + 2 * kv_heads) * d, generator=g).to(torch.bfloat16)),
        kc=to(torch.randn(pages, kv_heads, page, d, generator=g).to(torch.bfloat16)),
        vc=to(torch.randn(pages, kv_heads, page, d, generator=g).to(torch.bfloat16)),
        bt=to(bt), cu=to(cu), kv=to(torch.tensor(kv_lens, dtype=torch.int32)))


class _Shape:
    def __init__(self, rows, tokens, max_q, max_kv):
        self.rows, self.tokens, self.max_q, self.min_q, self.max_kv, self.pure_decode = rows, tokens, max_q, 1, max_kv, max_q == 1


# head_dim, page, tokens per request, lengths after the step, key splits, window: two calls in a row each, so that the
# second call's scratch starts out full of the first call's partial results
CASES = {
    "one token each, several splits": (64, 64, [[1, 1, 1, 1], [1, 1, 1, 1]], [[2176, 900, 64, 1500], [333, 4000, 17, 2048]], [5, 9], 0),
    "up to three tokens of four heads each (9 to 12 rows), head_dim 128": (128, 32, [[3, 1, 2, 3], [2, 3, 3]], [[700, 50, 1303, 4], [90, 2048, 515]], [4, 7], 0),
    "no split: no scratch used": (64, 16, [[1, 3, 2], [3, 1]], [[300, 77, 1000], [640, 129]], [1, 1], 0),
    "a window longer than a split": (64, 64, [[1, 1, 2], [1, 1]], [[5000, 4097, 1301], [513, 3000]], [6, 3], 1000),
}


@pytest.mark.parametrize("case", list(CASES), ids=[c.split(":")[0].replace(" ", "_").replace(",", "") for c in CASES])
def test_no_alloc_entry_point_equals_plain_attention_and_the_regular_one_twice_in_a_row(case):
    from serve_b200.kernels import load_kernels
    from tests.emu_kernels import EmuKernels

    d, page, q_lens_all, kv_lens_all, splits_all, window = CASES[case]
    K = load_kernels(DEV, head_dims=(d,))
    lib = ctypes.CDLL(K.paths[f"sb_attention_hd{d}"])      # the exported C symbols of the built library
    fn = lib.sb_attention_decode_noalloc
    fn.restype = ctypes.c_int
    assert lib.sb_attention_decode_noalloc_max_tiles() == 512
    heads, kv_heads = 32, 8
    scale = 1.0 / math.sqrt(d)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    plain_attention = EmuKernels(DEV).attention           # float arithmetic in torch: shares nothing with the kernels
    for call, (q_lens, kv_lens, splits) in enumerate(zip(q_lens_all, kv_lens_all, splits_all)):
        s = _setup(q_lens, heads, kv_heads, d, page, kv_lens, seed=call)
        t = sum(q_lens)
        shape = _Shape(len(kv_lens), t, max(q_lens), max(kv_lens))
        plain = torch.zeros(t, heads * d, device=DEV, dtype=torch.float32)
        plain_attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], None, None, heads, kv_heads, d, page, scale, window, plain, shape)
        regular = torch.zeros(t, heads * d, device=DEV, dtype=torch.bfloat16)
        K.attention(s["qkv"], s["kc"], s["vc"], s["bt"], s["cu"], s["kv"], None, None, heads, kv_heads, d, page, scale, window, regular, shape)
        got = torch.full_like(regular, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(DEV)
        rc = fn(ptr(s["qkv"]), s["qkv"].shape[1], ptr(s["kc"]), ptr(s["vc"]), ptr(s["bt"]), s["bt"].shape[1], ptr(s["cu"]), ptr(s["kv"]),
                heads, kv_heads, page, s["kc"].shape[0], ctypes.c_float(scale), window, ptr(got), len(kv_lens), max(q_lens), splits,
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert rc == 0, f"call {call}: return code {rc}"
        assert torch.cuda.memory_allocated(DEV) == before
        assert bool(torch.isfinite(got.float()).all()), f"call {call}: a row was not written"
        torch.testing.assert_close(got.float(), plain, atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(got.float(), regular.float(), atol=2e-2, rtol=2e-2)


def test_no_alloc_entry_point_refuses_what_exceeds_its_array():
    from serve_b200.kernels import load_kernels

    K = load_kernels(DEV, head_dims=(64,))
    lib = ctypes.CDLL(K.paths["sb_attention_hd64"])
    fn = lib.sb_attention_decode_noalloc
    fn.restype = ctypes.c_int
    s = _setup([1] * 9, 32, 8, 64, 64, [100] * 9, seed=3)
    out = torch.zeros(9, 32 * 64, device=DEV, dtype=torch.bfloat16)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    args = lambda n_splits, max_q: (ptr(s["qkv"]), s["qkv"].shape[1], ptr(s["kc"]), ptr(s["vc"]), ptr(s["bt"]), s["bt"].shape[1],
                                    ptr(s["cu"]), ptr(s["kv"]), 32, 8, 64, s["kc"].shape[0], ctypes.c_float(0.125), 0, ptr(out), 9,
                                    max_q, n_splits, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert fn(*args(8, 1)) == -4          # 9 * 8 * 8 = 576 triples: more than the array holds
    assert fn(*args(7, 1)) == 0           # 504: fits
    assert fn(*args(40, 1)) == -2         # more splits than the merge takes
    assert fn(*args(2, 5)) == -2          # 5 tokens x group of 4 = 20 rows: not a decoding step
    torch.cuda.synchronize()
