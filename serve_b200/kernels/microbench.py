"""Run one kernel of the engine by itself a few times and print its time (CUDA events) and bandwidth or FLOP rate.

    python -m serve_b200.kernels.microbench linear --m 8 --n 2048 --k 8192
    python -m serve_b200.kernels.microbench gate_up --m 8 --n 8192 --k 2048
    python -m serve_b200.kernels.microbench qkv_rope --m 2048 --k 2048 [--unfused]
    python -m serve_b200.kernels.microbench decode_attention --batch 64 --context 2176
    python -m serve_b200.kernels.microbench prefill_attention --tokens 2048

Each repetition uses another copy of the weights or of the cache (``--copies``), so that data comes from HBM and
not from the L2 cache; with ``--graph`` the repetitions are captured in one CUDA graph, as decoding steps are.
This is also the program the summaries under profiles/ were captured from (ncu -k ... python -m ...).
"""
from __future__ import annotations

import argparse
import math
import sys

import torch


class _Shape:
    def __init__(self, rows, tokens, max_q, min_q, max_kv):
        self.rows, self.tokens, self.max_q, self.min_q, self.max_kv = rows, tokens, max_q, min_q, max_kv
        self.pure_decode = max_q == 1


def _time(fn, reps, graph):
    fn()
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        run = g.replay
        run()
        torch.cuda.synchronize()
    else:
        run = fn
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps     # microseconds per call of fn


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m serve_b200.kernels.microbench")
    ap.add_argument("kernel", choices=["linear", "gate_up", "qkv_rope", "decode_attention", "prefill_attention"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2176)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--copies", type=int, default=8)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--graph", action="store_true")
    ap.add_argument("--legacy-attention", action="store_true", help="prompt attention on the mma.sync kernel instead of tcgen05")
    ap.add_argument("--unfused", action="store_true", help="qkv_rope: the product, then the rotary kernel")
    ap.add_argument("--library", action="store_true", help="send products to the library (cuBLAS) instead of this engine's kernels")
    ap.add_argument("--device", default="cuda:0")
    a = ap.parse_args(argv)
    from .cuda import load_kernels

    dev = a.device
    K = load_kernels(dev, head_dims=(a.head_dim,))
    if a.library:
        K.use_tcgen05 = K.use_skinny_linear = False
    if a.legacy_attention:
        K.use_tcgen05_attention = False
    bf = torch.bfloat16
    if a.kernel == "qkv_rope":
        # the q/k/v product of a prompt of --m tokens with rotation and cache write (--heads, --kv-heads, --head-dim)
        n = (a.heads + 2 * a.kv_heads) * a.head_dim
        ws = [torch.randn(n, a.k, device=dev, dtype=bf) * 0.02 for _ in range(a.copies)]
        x = torch.randn(a.m, a.k, device=dev, dtype=bf)
        qkv = torch.empty(a.m, n, device=dev, dtype=bf)
        nblk = -(-a.m // a.page_size)
        kc = torch.zeros(nblk, a.kv_heads, a.page_size, a.head_dim, device=dev, dtype=bf)
        vc = torch.zeros_like(kc)
        bt = torch.randperm(nblk, device=dev, dtype=torch.int32).view(1, nblk).contiguous()
        pos = torch.arange(a.m, device=dev, dtype=torch.int32)
        row = torch.zeros(a.m, device=dev, dtype=torch.int32)
        inv = (1.0 / (500000.0 ** (torch.arange(0, a.head_dim, 2).float() / a.head_dim))).to(dev)
        K.fuse_rope = not a.unfused
        memo = {}

        def fn():
            for w in ws:
                K.qkv_rope_cache(x, w, qkv, pos, row, inv, 1, a.head_dim, a.heads, a.kv_heads, a.head_dim, kc, vc, bt, a.page_size,
                                 True, memo=memo)

        us = _time(fn, a.reps, a.graph) / a.copies
        flops = 2.0 * a.m * n * a.k
        print(f"qkv_rope m={a.m} n={n} k={a.k}{' unfused' if a.unfused else ''}: {us:.2f} us, {flops / us / 1e6:.1f} TFLOP/s")
    elif a.kernel in ("linear", "gate_up"):
        rows = 2 * a.n if a.kernel == "gate_up" else a.n
        ws = [torch.randn(rows, a.k, device=dev, dtype=bf) * 0.02 for _ in range(a.copies)]
        x = torch.randn(a.m, a.k, device=dev, dtype=bf)
        out = torch.empty(a.m, a.n, device=dev, dtype=bf)

        def fn():
            for w in ws:
                if a.kernel == "gate_up":
                    K.gate_up_swiglu(x, w, out)
                else:
                    K.linear(x, w, out)

        us = _time(fn, a.reps, a.graph) / a.copies
        nbytes, flops = rows * a.k * 2, 2.0 * a.m * rows * a.k
        print(f"{a.kernel} m={a.m} n={a.n} k={a.k}: {us:.2f} us, {nbytes / us / 1e6:.2f} TB/s of weights, {flops / us / 1e6:.1f} TFLOP/s")
    else:
        decode = a.kernel == "decode_attention"
        r = a.batch if decode else 1
        q = 1 if decode else a.tokens
        ctx = a.context if decode else a.tokens
        nblk = -(-ctx // a.page_size)
        pages = r * nblk
        kcs = [torch.randn(pages, a.kv_heads, a.page_size, a.head_dim, device=dev, dtype=bf) for _ in range(a.copies)]
        vcs = [torch.randn(pages, a.kv_heads, a.page_size, a.head_dim, device=dev, dtype=bf) for _ in range(a.copies)]
        bt = torch.randperm(pages, device=dev, dtype=torch.int32).view(r, nblk).contiguous()
        t = r * q
        qkv = torch.randn(t, (a.heads + 2 * a.kv_heads) * a.head_dim, device=dev, dtype=bf)
        cu = torch.arange(0, t + 1, q, device=dev, dtype=torch.int32)
        kv = torch.full((r,), ctx, device=dev, dtype=torch.int32)
        out = torch.empty(t, a.heads * a.head_dim, device=dev, dtype=bf)
        shape = _Shape(r, t, q, q, ctx)

        def fn():
            for kc, vc in zip(kcs, vcs):
                K.attention(qkv, kc, vc, bt, cu, kv, None, None, a.heads, a.kv_heads, a.head_dim, a.page_size,
                            1.0 / math.sqrt(a.head_dim), 0, out, shape)

        us = _time(fn, a.reps, a.graph) / a.copies
        nbytes = r * ctx * a.kv_heads * a.head_dim * 2 * 2
        flops = 4.0 * a.head_dim * a.heads * (r * ctx if decode else q * (q + 1) / 2)
        print(f"{a.kernel} batch={r} tokens={q} context={ctx}: {us:.2f} us, {nbytes / us / 1e6:.2f} TB/s of cache, "
              f"{flops / us / 1e6:.1f} TFLOP/s")
    K.check_errors()
    return 0


if __name__ == "__main__":
    sys.exit(main())
