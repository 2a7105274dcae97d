"""Decode and prefill throughput of the engine at the Llama-3.2-1B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line. ``value`` is decoded tokens per second at batch 8 (2,048-token prompts, context limit
4,096), timed on the device with CUDA events over K decode steps after W warm-up steps; ``e2e`` is generated
tokens per second of whole ``serve_b200.generate`` calls (8 requests of 2,048 prompt tokens and 256 new tokens; token
ids come from and go back to the host every step; wall clock between synchronisations, one untimed call, the median
of three: the way the reference's own benchmark times its generate()); ``prefill`` is one 2,048-token prompt;
``points`` holds decode at batch 1 and 64; ``float32`` the decode step and the prefill in true 32-bit; ``roofline``
compares the decode step with the bytes it has to read (every weight once, and the cache of the live requests).
The weights (2.47 GB) are larger than the L2 cache, so no flush is needed between steps.

``--impl reference`` runs limei1221/serve itself, unmodified, from baseline/_ref at the same configuration and prints
the same line (baseline/reference_arm.py); it imports nothing of serve_b200.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
ROOT = os.path.dirname(os.path.abspath(__file__))

PROMPT_LEN = 2048
CONTEXT = 4096
PREFILL_TOKENS = 2048
E2E_NEW_TOKENS = 256      # tokens each request generates in the end-to-end runs (both arms)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    "sm_max_mhz": float(d.get("sm_max_mhz", 1965.0)), "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "sm_max_mhz": 1965.0, "source": "fallback"}


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.path, self.gpu = None, None, None

    @staticmethod
    def gpu_in_use():
        """The UUID of CUDA device 0 of this process ("GPU-..."): nvidia-smi numbers the machine's GPUs its own way,
        and the visible device need not be its index 0."""
        try:
            import torch

            uuid = str(torch.cuda.get_device_properties(0).uuid)
            return uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:
            return None

    def start(self):
        try:
            self.gpu = self.gpu_in_use()
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.gpu or "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "gpu": self.gpu or "index 0"}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        try:
            with open(self.path) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) >= 7 and parts[0].isdigit():
                        rows.append(parts)
            os.remove(self.path)
        except Exception:
            pass
        if rows:
            sm = sorted(int(r[0]) for r in rows)
            out["sm_mhz"] = sm[len(sm) // 2]
            out["sm_max_mhz"] = int(rows[0][1])
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            out["reasons"] = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
            out["samples"] = len(rows)
        return out


def model_bytes_and_flops(cfg, dtype_bytes):
    h, L, H, Hkv, D, I, V = (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads,
                             cfg.head_dim, cfg.intermediate_size, cfg.vocab_size)
    per_layer = (H + 2 * Hkv) * D * h + h * H * D + 2 * I * h + h * I
    weights = (L * per_layer + V * h) * dtype_bytes                   # every weight a decode step uses, once
    kv_per_token = L * 2 * Hkv * D * dtype_bytes
    def prefill_flops(t):
        return 2 * t * L * per_layer + L * 4 * D * H * t * (t + 1) // 2 + 2 * V * h
    return weights, kv_per_token, prefill_flops


def decode_bench(eng, sampler, batch, steps, warmup, vocab, seed, cuda_profiler=False):
    """Prefill ``batch`` prompts of PROMPT_LEN tokens, then time ``steps`` decode steps on the device."""
    import torch
    from serve_b200.engine import StepEntry

    g = torch.Generator().manual_seed(seed)
    rids = [f"b{batch}-{i}" for i in range(batch)]
    for rid in rids:
        toks = torch.randint(0, vocab, (PROMPT_LEN,), generator=g).tolist()
        eng.step([StepEntry(rid, toks, [])])
    feed = torch.randint(0, vocab, (warmup + steps, batch), generator=g).tolist()
    temps, tok_idx = [0.0] * batch, [0] * batch

    def one(i):
        logits = eng.step([StepEntry(rid, [feed[i][j]], [0]) for j, rid in enumerate(rids)])
        return sampler.sample(logits, temps, list(range(batch)), tok_idx)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    k = eng.kernels
    l0, c0 = k.launches, k.library_calls
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if cuda_profiler:
        torch.cuda.profiler.start()
    ev0.record()
    for i in range(warmup, warmup + steps):
        one(i)
    ev1.record()
    torch.cuda.synchronize()
    if cuda_profiler:
        torch.cuda.profiler.stop()
    ms = ev0.elapsed_time(ev1) / steps
    ctx_mid = PROMPT_LEN + warmup + steps / 2.0
    for rid in rids:
        eng.end(rid)
    return ms, ctx_mid, k.launches - l0, k.library_calls - c0


def decode_timeline(eng, batch, vocab):
    """One decoding step as it runs inside its graph: when each kernel starts (relative to the step's first kernel),
    how long it runs, and how far its start lies before (-) or after (+) the end of everything launched before it.
    With dependent launches a kernel's length includes the time it waits for its predecessor."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    from serve_b200 import Request, generate

    g = torch.Generator().manual_seed(1)
    # prompts enter one a step and every request decodes batch + 24 tokens, so for 24 steps all of them decode together;
    # batch + 5 steps before the end is one of those
    reqs = [Request(torch.randint(0, vocab, (PROMPT_LEN,), generator=g), PROMPT_LEN, batch + 24) for _ in range(batch)]
    generate(eng, reqs, temperature=0.0, eos_token_id=None)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        generate(eng, reqs, temperature=0.0, eos_token_id=None)
    evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda e: e.time_range.start)
    firsts = [i for i, e in enumerate(evs) if "embedding" in e.name]
    step = evs[firsts[-(batch + 5)]:firsts[-(batch + 4)]]
    t0, prev_end = step[0].time_range.start, step[0].time_range.start
    print(f"decoding step, batch {batch}: {evs[firsts[-(batch + 4)]].time_range.start - t0:.1f} us from first kernel to the next step's first kernel")
    print(f"{'start us':>9} {'length us':>9} {'vs end of earlier':>17}  kernel")
    for e in step:
        name = e.name.replace("(anonymous namespace)::", "").replace("void ", "")
        print(f"{e.time_range.start - t0:9.2f} {e.time_range.end - e.time_range.start:9.2f} {e.time_range.start - prev_end:17.2f}  {name[:70]}")
        prev_end = max(prev_end, e.time_range.end)
    return 0


def prefill_timeline(eng, vocab):
    """The kernels of one prompt step of PREFILL_TOKENS tokens, as decode_timeline prints them (first 40)."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    from serve_b200.engine import StepEntry

    g = torch.Generator().manual_seed(3)
    for rep in range(3):
        toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=g).tolist()
        if rep == 2:
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                eng.step([StepEntry("tl", toks, [PREFILL_TOKENS - 1])])
                torch.cuda.synchronize()
        else:
            eng.step([StepEntry("tl", toks, [PREFILL_TOKENS - 1])])
        eng.end("tl")
    evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda e: e.time_range.start)
    first = next(i for i, e in enumerate(evs) if "embedding" in e.name)
    step = evs[first:]
    t0, prev_end = step[0].time_range.start, step[0].time_range.start
    print(f"prompt step of {PREFILL_TOKENS} tokens: {step[-1].time_range.end - t0:.1f} us from the first kernel's start to the last one's end")
    print(f"{'start us':>9} {'length us':>9} {'vs end of earlier':>17}  kernel")
    for e in step[:40]:
        name = e.name.replace("(anonymous namespace)::", "").replace("void ", "")
        print(f"{e.time_range.start - t0:9.2f} {e.time_range.end - e.time_range.start:9.2f} {e.time_range.start - prev_end:17.2f}  {name[:70]}")
        prev_end = max(prev_end, e.time_range.end)
    return 0


def prefill_bench(eng, vocab, reps, seed, cuda_profiler=False):
    import torch
    from serve_b200.engine import StepEntry

    g = torch.Generator().manual_seed(seed)
    times = []
    for i in range(reps + 2):
        toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=g).tolist()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if cuda_profiler and i == reps + 1:
            torch.cuda.profiler.start()
        ev0.record()
        eng.step([StepEntry(f"p{i}", toks, [PREFILL_TOKENS - 1])])
        ev1.record()
        torch.cuda.synchronize()
        if cuda_profiler and i == reps + 1:
            torch.cuda.profiler.stop()
        eng.end(f"p{i}")
        if i >= 2:
            times.append(ev0.elapsed_time(ev1))
    times.sort()
    return times[len(times) // 2]


def e2e_bench(eng, batch, new_tokens, vocab, seed, runs=3):
    """Generated tokens per second of whole serve_b200.generate() calls: host token ids in, host token ids out, every
    step, the prompts' prefill included. Timed by the wall clock between device synchronisations, as the reference's own
    benchmark times its generate() (serve/benchmark.py:63-80); one untimed call first, then the median of ``runs`` calls.
    ``decode_window`` is the rate inside the pure-decode steps of the median call (from one step's end to the last step's)."""
    import torch
    from serve_b200 import Request, generate

    g = torch.Generator().manual_seed(seed)
    reqs = [Request(torch.randint(0, vocab, (PROMPT_LEN,), generator=g), PROMPT_LEN, new_tokens) for _ in range(batch)]
    generate(eng, reqs, temperature=0.0, eos_token_id=None)
    results = []
    for _ in range(runs):
        timeline = []
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = generate(eng, reqs, temperature=0.0, eos_token_id=None, timeline=timeline)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        results.append((sum(len(r.generated_tokens) for r in out) / dt, timeline))
    results.sort(key=lambda x: x[0])
    rate, timeline = results[len(results) // 2]
    dec = [(t, nd, b) for t, npf, nd, b in timeline if nd == batch and npf == 0]
    rec = {"value": round(rate, 1), "unit": "tokens/s", "what": "whole generate() calls, wall clock, median",
           "runs": runs, "new_tokens": new_tokens, "slowest_run": round(results[0][0], 1), "fastest_run": round(results[-1][0], 1)}
    if len(dec) > 4:
        rec["decode_window"] = round(batch * (len(dec) - 4) / (dec[-1][0] - dec[3][0]), 1)
        rec["h2d_bytes_per_step"] = int(dec[-1][2])
        rec["d2h_bytes_per_step"] = 4 * batch
    return rec


def reference_arm(args):
    """limei1221/serve itself at the same configuration (baseline/reference_arm.py); nothing of serve_b200 is imported."""
    from baseline import reference_arm as arm

    args.warmup = max(args.warmup, 3)
    return arm.main(args, ClockSampler(), peaks(), {"PROMPT_LEN": PROMPT_LEN, "CONTEXT": CONTEXT, "PREFILL_TOKENS": PREFILL_TOKENS,
                                                    "E2E_NEW_TOKENS": E2E_NEW_TOKENS})


def float32_points(cfg, args, pk):
    """The same decode step (batch 8) and prefill (2,048 tokens) in true 32-bit: every byte doubles, the products run on
    the plain FMA units (no tensor-core mode), so the prefill is compared with the FMA peak of the SMs."""
    import torch

    from serve_b200.config import EngineConfig
    from serve_b200.engine import Engine
    from serve_b200.sampling import Sampler

    page, batch = 64, args.batch
    ec = EngineConfig(dtype="float32", page_size=page, num_pages=(batch + 1) * CONTEXT // page, max_slots=batch + 2,
                      max_tokens_per_step=max(PROMPT_LEN, PREFILL_TOKENS), max_context=CONTEXT, use_cuda_graphs=not args.no_graphs)
    eng = Engine.from_config(cfg, seed=0, engine_config=ec)
    sampler = Sampler(eng.kernels, eng.rt.device, seed=0)
    weights, kv_per_token, prefill_flops = model_bytes_and_flops(cfg, 4)
    steps = max(16, args.steps // 4)
    ms, ctx_mid, _, _ = decode_bench(eng, sampler, batch, steps, args.warmup, cfg.vocab_size, seed=21)
    achieved = (weights + batch * ctx_mid * kv_per_token) / (ms * 1e-3) / 1e9
    pre_ms = prefill_bench(eng, cfg.vocab_size, reps=3, seed=27)
    props = torch.cuda.get_device_properties(0)
    fma_tflops = props.multi_processor_count * 128 * 2 * pk.get("sm_max_mhz", 1965.0) * 1e6 / 1e12
    return {"decode_b%d" % batch: round(batch * 1000.0 / ms, 1), "ms_per_step": round(ms, 4), "steps": steps,
            "roofline_frac": round(achieved / pk["hbm_gbs"], 4), "achieved_gbs": round(achieved, 1),
            "prefill": {"value": round(PREFILL_TOKENS / (pre_ms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                        "frac": round(prefill_flops(PREFILL_TOKENS) / (pre_ms * 1e-3) / (fma_tflops * 1e12), 4),
                        "peak_tflops": round(fma_tflops, 1), "peak": "SMs x 128 FMA x 2 x max SM clock"}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (named in the record)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode kernels one by one (for per-kernel profiles)")
    ap.add_argument("--cuda-profiler", action="store_true",
                    help="bracket the timed region with cudaProfilerStart/Stop (ncu --profile-from-start off)")
    ap.add_argument("--only", choices=["decode", "prefill", "timeline", "timeline-prefill"], default=None,
                    help="measure just this part (for profiles); timeline: start and length of every kernel of one decoding "
                         "step as it runs inside its CUDA graph (torch.profiler), printed as a table")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)

    import dataclasses

    import torch

    from serve_b200.config import EngineConfig, load_preset
    from serve_b200.engine import Engine
    from serve_b200.sampling import Sampler

    cfg_full = load_preset("llama-3.2-1b")
    cfg = cfg_full if args.layers is None else dataclasses.replace(cfg_full, num_hidden_layers=args.layers)
    pk = peaks()
    page = 64
    max_batch = max(64, args.batch)
    # the scheduler's token budget per step: all prompts of the end-to-end batch in one step (8 x 2,048), as a server sized
    # for this load would be set; the 2,048-token prompt step and the decoding steps are what they are under any budget
    step_tokens = max(args.batch * PROMPT_LEN, PREFILL_TOKENS)
    ec = EngineConfig(dtype="bfloat16", page_size=page, num_pages=max_batch * CONTEXT // page + 64, max_slots=max_batch + 2,
                      max_tokens_per_step=step_tokens, max_context=CONTEXT,
                      use_cuda_graphs=not args.no_graphs)
    with torch.inference_mode():
        eng = Engine.from_config(cfg, seed=0, engine_config=ec)
        sampler = Sampler(eng.kernels, eng.rt.device, seed=0)
        weights, kv_per_token, prefill_flops = model_bytes_and_flops(cfg, 2)

        if args.only == "timeline":
            return decode_timeline(eng, args.batch, cfg.vocab_size)
        if args.only == "timeline-prefill":
            return prefill_timeline(eng, cfg.vocab_size)
        if args.only == "prefill":
            pre_ms = prefill_bench(eng, cfg.vocab_size, reps=2, seed=7, cuda_profiler=args.cuda_profiler)
            print(json.dumps({"only": "prefill", "ms": round(pre_ms, 3), "tokens": PREFILL_TOKENS}))
            return 0
        clocks = ClockSampler()
        clocks.start()
        ms, ctx_mid, launches, lib_calls = decode_bench(eng, sampler, args.batch, args.steps, args.warmup, cfg.vocab_size, seed=1,
                                                        cuda_profiler=args.cuda_profiler)
        clock_rec = clocks.stop()
        if args.only == "decode":
            print(json.dumps({"only": "decode", "batch": args.batch, "ms_per_step": round(ms, 4), "graphs": not args.no_graphs}))
            return 0
        value = args.batch * 1000.0 / ms
        step_bytes = weights + args.batch * ctx_mid * kv_per_token
        achieved = step_bytes / (ms * 1e-3) / 1e9

        points = {}
        if not args.skip_points:
            for b in (1, 64):
                pms, _, _, _ = decode_bench(eng, sampler, b, max(16, args.steps // 2), args.warmup, cfg.vocab_size, seed=2 + b)
                points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)

        pre_ms = prefill_bench(eng, cfg.vocab_size, reps=5, seed=7)
        pre_frac = prefill_flops(PREFILL_TOKENS) / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)

        e2e = e2e_bench(eng, args.batch, E2E_NEW_TOKENS, cfg.vocab_size, seed=9)

        fp32 = None
        if not args.skip_points:
            del eng, sampler
            torch.cuda.empty_cache()
            fp32 = float32_points(cfg, args, pk)

    rec = {
        "metric": "decode tok/s at batch 8 (Llama-3.2-1B shape, 2048-token prompts, context 4096)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, seeded random weights N(0,0.02)",
        "impl": "ours",
        "config": {"model": "llama-3.2-1b-shape", "layers": cfg.num_hidden_layers, "layers_full": cfg_full.num_hidden_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "page_size": page, "step_tokens": step_tokens,
                   "parallelism": "single-gpu", "l2": "inputs larger than L2: 2.47 GB of weights read per step",
                   "peaks": pk["source"]},
        "e2e": e2e,
        "gpu_launches": int(launches),
        "library_gemm_calls": int(lib_calls),
        "prefill": {"value": round(PREFILL_TOKENS / (pre_ms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                    "frac": round(pre_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "float32": fp32,
        "clocks": clock_rec,
    }
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
