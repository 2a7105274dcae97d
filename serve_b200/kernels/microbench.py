"""Run one kernel of the engine by itself a few times and print its time (CUDA events) and bandwidth or FLOP rate.

    python -m serve_b200.kernels.microbench linear --m 8 --n 2048 --k 8192
    python -m serve_b200.kernels.microbench gate_up --m 8 --n 8192 --k 2048
    python -m serve_b200.kernels.microbench qkv_rope --m 2048 --k 2048 [--unfused]
    python -m serve_b200.kernels.microbench decode_attention --batch 64 --context 2176
    python -m serve_b200.kernels.microbench prefill_attention --tokens 2048
    python -m serve_b200.kernels.microbench step --preset llama-3.2-3b --layers 8 --batches 1,8,32 --context 2048 --tokens 2048
    python -m serve_b200.kernels.microbench layer_run --preset llama-3.2-1b --batches 8,1 --context 2048
    python -m serve_b200.kernels.microbench marginal --preset llama-3.2-1b --batches 8,1 --context 2048
    python -m serve_b200.kernels.microbench long_prompt --preset llama-3.2-1b --context 32768 --tokens 8192

Each repetition uses another copy of the weights or of the cache (``--copies``), so that data comes from HBM and
not from the L2 cache; with ``--graph`` the repetitions are captured in one CUDA graph, as decoding steps are.
``step`` measures whole decoding steps (step function + sampling, from CUDA graphs) and a prompt step of a preset's
shape with random weights, with fewer layers if asked, against the bytes and flops they need: the way to see how the
engine does at other sizes, batches and contexts than the benchmark's.
``marginal`` times the same decoding steps with one kind of kernel left out at a time (the step's results are then
wrong; only its time is read): what each kernel costs inside the chain, hand-overs included, against its bytes.
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


def _step_bench(a) -> int:
    """Decoding steps at several batch sizes and one prompt step, through the engine, for a preset's shape."""
    import dataclasses
    import json
    import os

    from ..config import EngineConfig, load_preset
    from ..engine import Engine, StepEntry
    from ..sampling import Sampler

    hbm, flops_peak = 6540.5e9, 1669.7e12
    peaks = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.isfile(peaks):
        with open(peaks) as f:
            d = json.load(f)
        hbm, flops_peak = float(d["hbm_gbs"]) * 1e9, float(d["bf16_tflops"]) * 1e12
    full = load_preset(a.preset)
    cfg = dataclasses.replace(full, num_hidden_layers=a.layers or full.num_hidden_layers)
    h, nl, nh, nkv, d_, inter, v = (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads,
                                    cfg.head_dim, cfg.intermediate_size, cfg.vocab_size)
    per_layer = (nh + 2 * nkv) * d_ * h + h * nh * d_ + 3 * inter * h
    weights, kv_per_token = (nl * per_layer + v * h) * 2, nl * 2 * nkv * d_ * 2
    batches = [int(b) for b in a.batches.split(",")]
    ctx, page = a.context, a.page_size
    ec = EngineConfig(dtype="bfloat16", page_size=page, num_pages=max(batches) * (ctx + 256) // page + 64, max_slots=max(batches) + 2,
                      max_tokens_per_step=max(min(ctx, 8192), a.tokens, max(batches)), max_context=ctx + 512, device=a.device)
    out = {}
    with torch.inference_mode():
        eng = Engine.from_config(cfg, seed=0, engine_config=ec)
        sampler = Sampler(eng.kernels, eng.rt.device, 0)
        g = torch.Generator().manual_seed(1)
        for b in batches:
            rids = [f"b{b}-{i}" for i in range(b)]
            for rid in rids:
                done = 0
                while done < ctx:
                    n = min(ctx - done, ec.max_tokens_per_step)
                    eng.step([StepEntry(rid, torch.randint(0, v, (n,), generator=g).tolist(), [])])
                    done += n

            def one():
                logits = eng.step([StepEntry(rid, [7], [0]) for rid in rids])
                return sampler.sample(logits, [0.0] * b, list(range(b)), [0] * b)

            for _ in range(6):
                one()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.reps * 4):
                one()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / (a.reps * 4)
            frac = (weights + b * (ctx + 6 + a.reps * 2) * kv_per_token) / (ms * 1e-3) / hbm
            out[f"decode_b{b}"] = {"ms": round(ms, 3), "tokens_per_s": round(b * 1000 / ms, 1), "of_copy_bandwidth": round(frac, 3)}
            for rid in rids:
                eng.end(rid)
        times = []
        for _ in range(5):
            toks = torch.randint(0, v, (a.tokens,), generator=g).tolist()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.step([StepEntry("p", toks, [a.tokens - 1])])
            e1.record()
            torch.cuda.synchronize()
            eng.end("p")
            times.append(e0.elapsed_time(e1))
        ms = sorted(times[1:])[2]
        t = a.tokens
        flops = 2 * t * nl * per_layer + nl * 4 * d_ * nh * t * (t + 1) // 2 + 2 * v * h
        out[f"prefill_{t}"] = {"ms": round(ms, 3), "tokens_per_s": round(t * 1000 / ms, 1),
                               "of_cublas_burst": round(flops / (ms * 1e-3) / flops_peak, 3)}
        eng.kernels.check_errors()
    print(json.dumps({"preset": a.preset, "layers": nl, "layers_full": full.num_hidden_layers, "context": ctx, **out}))
    return 0


def _marginal_times(a) -> int:
    """Decoding steps with one kind of kernel left out at a time: the difference to the whole step is what that kernel
    costs where it stands, between its neighbours."""
    import dataclasses
    import json

    from ..config import EngineConfig, load_preset
    from ..engine import Engine, StepEntry
    from ..sampling import Sampler

    full = load_preset(a.preset)
    cfg = dataclasses.replace(full, num_hidden_layers=a.layers or full.num_hidden_layers)
    v, hidden = cfg.vocab_size, cfg.hidden_size
    batches = [int(b) for b in a.batches.split(",")]
    ctx, page = a.context, a.page_size

    def leave_out(kernels, what):
        """Shadow one method of the kernels object (which engines share) by a do-nothing; returns the shadowed name."""
        nothing = lambda *args, **kw: None
        name = {"norm": "add_rmsnorm", "attention": "attention", "q/k/v": "qkv_rope_cache", "gate/up": "gate_up_swiglu"}.get(what, "linear")
        if name == "linear":
            whole = kernels.linear

            def linear(x, w, out):
                kind = "head" if w.shape[0] == v else ("down projection" if x.shape[1] > hidden else "output projection")
                return None if kind == what else whole(x, w, out)

            nothing = linear
        setattr(kernels, name, nothing)
        return name

    out = {}
    kinds = ["nothing", "norm", "q/k/v", "attention", "output projection", "gate/up", "down projection", "head"]
    with torch.inference_mode():
        for what in kinds:
            ec = EngineConfig(dtype="bfloat16", page_size=page, num_pages=max(batches) * (ctx + 256) // page + 64,
                              max_slots=max(batches) + 2, max_tokens_per_step=max(min(ctx, 8192), max(batches)), max_context=ctx + 512,
                              device=a.device)
            eng = Engine.from_config(cfg, seed=0, engine_config=ec)
            sampler = Sampler(eng.kernels, eng.rt.device, 0)
            g = torch.Generator().manual_seed(1)
            for b in batches:
                rids = [f"b{b}-{i}" for i in range(b)]
                for rid in rids:
                    eng.step([StepEntry(rid, torch.randint(0, v, (ctx,), generator=g).tolist(), [])])
                shadowed = leave_out(eng.kernels, what) if what != "nothing" else None

                def one():
                    logits = eng.step([StepEntry(rid, [7], [0]) for rid in rids])
                    return sampler.sample(logits, [0.0] * b, list(range(b)), [0] * b)

                try:
                    ms = _time(lambda: [one() for _ in range(4)], a.reps, False) / 4e3
                finally:
                    if shadowed:
                        delattr(eng.kernels, shadowed)       # the class's method shows again
                out.setdefault(f"b{b}", {})[what] = round(ms, 4)
                for rid in rids:
                    eng.end(rid)
            eng.kernels.check_errors()
            del eng, sampler
    for b, row in out.items():
        whole = row["nothing"]
        print(f"{a.preset}, {cfg.num_hidden_layers} layers, context {ctx}, {b}: whole step {whole * 1e3:.1f} us; left out -> us less a step "
              f"(a layer): " + ", ".join(f"{k} {(whole - t) * 1e3:.1f}" + ("" if k == "head" else f" ({(whole - t) * 1e3 / cfg.num_hidden_layers:.2f})")
                                       for k, t in row.items() if k != "nothing"))
    print(json.dumps(out))
    return 0


def _long_prompt(a) -> int:
    """One prompt of --context tokens in portions of --tokens: the time of every portion as the cached part grows."""
    import dataclasses

    from ..config import EngineConfig, load_preset
    from ..engine import Engine, StepEntry

    full = load_preset(a.preset)
    cfg = dataclasses.replace(full, num_hidden_layers=a.layers or full.num_hidden_layers)
    total, chunk = a.context, a.tokens
    ec = EngineConfig(dtype="bfloat16", page_size=a.page_size, num_pages=2 * (total // a.page_size + 8), max_slots=4,
                      max_tokens_per_step=chunk, max_context=total, device=a.device)
    with torch.inference_mode():
        eng = Engine.from_config(cfg, seed=0, engine_config=ec)
        toks = torch.randint(0, cfg.vocab_size, (total,), generator=torch.Generator().manual_seed(0)).tolist()
        for rep in range(2):                     # the second pass is the one reported
            events = []
            for i in range(0, total, chunk):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                eng.step([StepEntry(f"r{rep}", toks[i:i + chunk], [])])
                e1.record()
                events.append((e0, e1))
            torch.cuda.synchronize()
            ms = [x.elapsed_time(y) for x, y in events]
            eng.end(f"r{rep}")
        eng.kernels.check_errors()
    flops = 4.0 * cfg.head_dim * cfg.num_attention_heads * chunk * (total - chunk / 2) * cfg.num_hidden_layers
    more = (ms[-1] - ms[0]) * 1e-3
    print(f"{a.preset}, {cfg.num_hidden_layers} layers: {total} tokens in portions of {chunk}: {sum(ms):.1f} ms = "
          f"{total / sum(ms):.0f} k tokens/s; portions (ms): " + " ".join(f"{m:.1f}" for m in ms))
    if more > 0:
        print(f"attention of the last portion over the cached part: {flops / 1e12:.1f} TFLOP in {more * 1e3:.1f} ms more than the "
              f"first portion = {flops / more / 1e12:.0f} TFLOP/s")
    return 0


def _layer_run_phases(a) -> int:
    """The persistent all-layers kernel (csrc/decode_stack.cu) on decoding steps of a preset's shape: what block 0's clock
    says after every phase and every barrier of three of the layers."""
    import dataclasses

    from ..config import EngineConfig, load_preset
    from ..engine import Engine, StepEntry

    full = load_preset(a.preset)
    cfg = dataclasses.replace(full, num_hidden_layers=a.layers or full.num_hidden_layers)
    nl = cfg.num_hidden_layers
    names = ["q/k/v", "barrier", "attention", "barrier", "o", "barrier", "gate/up", "barrier", "down", "barrier"]
    with torch.inference_mode():
        for batch in [int(b) for b in a.batches.split(",")]:
            ec = EngineConfig(dtype="bfloat16", page_size=a.page_size, num_pages=batch * (a.context + 256) // a.page_size + 8,
                              max_slots=batch + 1, max_tokens_per_step=max(2048, batch), max_context=a.context + 512,
                              use_cuda_graphs=False, device=a.device)
            eng = Engine.from_config(cfg, seed=0, engine_config=ec)
            eng.kernels.use_layer_runs = True
            g = torch.Generator().manual_seed(1)
            rids = [f"r{i}" for i in range(batch)]
            for rid in rids:
                done = 0
                while done < a.context:
                    n = min(a.context - done, 2048)
                    eng.step([StepEntry(rid, torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist(), [])])
                    done += n
            timing = torch.zeros(nl * 10, dtype=torch.int64, device=a.device)
            eng.kernels.layer_run_timing = timing
            for i in range(6):
                eng.step([StepEntry(rid, [5 + i], [0]) for rid in rids])
            torch.cuda.synchronize()
            eng.kernels.layer_run_timing = None
            eng.kernels.use_layer_runs = False
            eng.kernels.check_errors()
            t = timing.view(nl, 10).cpu()
            for layer in sorted({1, nl // 2, nl - 2} & set(range(1, nl))):
                base = int(t[layer - 1, 9])
                row = [int(t[layer, k]) for k in range(10)]
                spans = [row[0] - base] + [row[k] - row[k - 1] for k in range(1, 10)]
                print(f"batch {batch}, layer {layer}: {(row[9] - base) / 1000:.1f} us: " +
                      ", ".join(f"{n} {s / 1000:.1f}" for n, s in zip(names, spans)))
            del eng
            torch.cuda.empty_cache()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m serve_b200.kernels.microbench")
    ap.add_argument("kernel", choices=["linear", "gate_up", "qkv_rope", "decode_attention", "prefill_attention", "step", "layer_run", "marginal", "long_prompt"])
    ap.add_argument("--preset", default="llama-3.2-1b", help="step: the shape")
    ap.add_argument("--layers", type=int, default=None, help="step: fewer layers than the preset has")
    ap.add_argument("--batches", default="1,8,32", help="step: decoding batch sizes, comma separated")
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
    ap.add_argument("--tiles", action="store_true", help="send products of more than 16 rows to the tcgen05 tiles whatever their size")
    ap.add_argument("--device", default="cuda:0")
    a = ap.parse_args(argv)
    if a.kernel == "step":
        return _step_bench(a)
    if a.kernel == "layer_run":
        return _layer_run_phases(a)
    if a.kernel == "marginal":
        return _marginal_times(a)
    if a.kernel == "long_prompt":
        return _long_prompt(a)
    from .cuda import load_kernels

    dev = a.device
    K = load_kernels(dev, head_dims=(a.head_dim,))
    if a.library:
        K.use_tcgen05 = K.use_skinny_linear = False
    if a.tiles:
        K.TCGEN05_MIN_TILES = 1
        K.tcgen05_for_plain_products = True
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
