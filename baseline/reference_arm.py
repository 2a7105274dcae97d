"""The reference arm of bench.py: limei1221/serve itself, unmodified, timed at the benchmark's configuration.

Nothing of serve_b200 is imported here. The reference package lies under
baseline/_ref/serve (a plain copy of the project's ``serve`` folder: it is
pure Python plus Triton kernels, so a copy is everything a wheel of it would
hold). What runs is its stock code path:

- weights: a state dict with the reference's own tensor names, random
  N(0, 0.02) with norm weights of one and the output matrix tied to the
  embedding as its converter does for the 1B model
  (serve/hf_utils/convert_hf_checkpoint.py:146-147), written to a file and
  loaded by ``serve.utils._load_model`` (serve/utils.py:61-78) with
  ``serve.utils.config_1b`` and a context limit of 4,096;
- ``e2e``: generated tokens per second of whole ``serve.run.generate`` calls
  (serve/run.py:238-308), timed by the wall clock between synchronisations as
  the reference's own benchmark does (serve/benchmark.py:63-80), after one
  untimed call;
- ``value``, ``points``: CUDA-event time of K calls of
  ``serve.run.decode_one_token`` (run.py:164-209) after ``serve.run.prefill``
  (run.py:109-161) of each prompt;
- ``prefill``: one 2,048-token prompt through ``serve.run.prefill``.
"""
import json
import os
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def available():
    """None if the reference can be run from baseline/_ref, else the reason as one line."""
    if not os.path.isfile(os.path.join(REF, "serve", "run.py")):
        return ("baseline/_ref/serve is missing: pip cannot build limei1221/serve offline (its build backend 'hatchling' is "
                "neither installed nor in /opt/wheelhouse), and no copy of its serve/ folder was put there")
    try:
        import triton  # noqa: F401
    except Exception as e:  # pragma: no cover
        return f"triton cannot be imported: {type(e).__name__}: {e}"
    return None


def _write_state_dict(path, config, dtype, seed):
    """Random weights under the reference's own tensor names, one tensor at a time (made on the GPU, stored on the CPU)."""
    import torch

    from serve.model import LlamaModel, ModelArgs

    with torch.device("meta"):
        shapes = {k: tuple(v.shape) for k, v in LlamaModel(ModelArgs(**config), dtype=dtype).state_dict().items()}
    g = torch.Generator(device="cuda").manual_seed(seed)
    sd = {}
    for name, shape in shapes.items():
        if name == "output.weight":
            continue
        if name.endswith("norm.weight"):
            sd[name] = torch.ones(shape, dtype=dtype)
        else:
            sd[name] = (torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(dtype).cpu()
    sd["output.weight"] = sd["tok_embeddings.weight"].clone()
    torch.save(sd, path)


def load_reference_model(config, dtype, seed=0):
    import torch

    from serve.utils import _load_model

    fd, path = tempfile.mkstemp(suffix=".pth")
    os.close(fd)
    try:
        _write_state_dict(path, config, dtype, seed)
        model = _load_model(dict(config), path, "cuda", dtype)
    finally:
        os.remove(path)
    torch.cuda.synchronize()
    return model


def _requests(run, batch, prompt_len, vocab, seed, tag):
    import torch

    g = torch.Generator().manual_seed(seed)
    return [run.RequestData(request_id=tag * 100000 + i, input_ids=torch.randint(0, vocab, (prompt_len,), generator=g, dtype=torch.long),
                            generated_tokens=[], input_length=prompt_len, max_new_tokens=1 << 30) for i in range(batch)]


def decode_bench(run, model, batch, steps, warmup, prompt_len, vocab, seed):
    """Milliseconds per call of serve.run.decode_one_token at ``batch`` requests (CUDA events around ``steps`` calls)."""
    import torch

    reqs = _requests(run, batch, prompt_len, vocab, seed, tag=batch)
    for r in reqs:
        run.prefill(model, [r], model.kv_caches, model.kv_cache_ix, 0.0)
    for _ in range(warmup):
        run.decode_one_token(model, reqs, model.kv_caches, model.kv_cache_ix, 0.0)
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        run.decode_one_token(model, reqs, model.kv_caches, model.kv_cache_ix, 0.0)
    ev1.record()
    torch.cuda.synchronize()
    for r in reqs:
        model.kv_cache_ix.free_request(r.request_id)
    return ev0.elapsed_time(ev1) / steps


def prefill_bench(run, model, tokens, vocab, reps, seed):
    import torch

    times = []
    for i in range(reps + 2):
        (r,) = _requests(run, 1, tokens, vocab, seed + i, tag=7000 + i)
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        run.prefill(model, [r], model.kv_caches, model.kv_cache_ix, 0.0)
        ev1.record()
        torch.cuda.synchronize()
        model.kv_cache_ix.free_request(r.request_id)
        if i >= 2:
            times.append(ev0.elapsed_time(ev1))
    times.sort()
    return times[len(times) // 2]


def e2e_bench(run, model, batch, prompt_len, new_tokens, vocab, seed, runs):
    """Generated tokens per second of whole generate() calls: the median of ``runs`` calls after one untimed call."""
    import torch

    g = torch.Generator().manual_seed(seed)
    reqs = [run.Request(input_ids=torch.randint(0, vocab, (prompt_len,), generator=g, dtype=torch.long), input_length=prompt_len,
                        max_new_tokens=new_tokens) for _ in range(batch)]
    run.generate(model, reqs, 0.0)
    rates = []
    for _ in range(runs):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = run.generate(model, reqs, 0.0)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        rates.append(sum(len(r.generated_tokens) for r in out) / dt)
    rates.sort()
    return {"value": round(rates[len(rates) // 2], 1), "unit": "tokens/s", "what": "whole generate() calls, wall clock, median",
            "runs": runs, "new_tokens": new_tokens, "slowest_run": round(rates[0], 1), "fastest_run": round(rates[-1], 1),
            "h2d_bytes_per_step": 4 * batch + 4 * batch + 4 * batch, "d2h_bytes_per_step": 8 * batch}


def main(args, clock_sampler, peaks, consts):
    """Runs the arm and prints its JSON line. ``consts``: PROMPT_LEN, CONTEXT, PREFILL_TOKENS, E2E_NEW_TOKENS of bench.py."""
    why = available()
    if why is not None:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    sys.path.insert(0, REF)
    sys.dont_write_bytecode = True
    try:
        import torch

        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        import serve.run as run
        from serve.utils import config_1b
    except Exception as e:
        print(json.dumps({"impl": "reference", "unavailable": f"the reference cannot be imported: {type(e).__name__}: {e}"}))
        return 0
    prompt_len, context, prefill_tokens = consts["PROMPT_LEN"], consts["CONTEXT"], consts["PREFILL_TOKENS"]
    config = dict(config_1b, max_seq_len=context)
    vocab = config["vocab_size"]
    try:
        with torch.inference_mode():
            model = load_reference_model(config, torch.bfloat16, seed=0)
            model.create_kv_cache(blocksize_k=64, max_batch_size=run.MAX_ALLOWED_BATCH_SIZE, device="cuda")
            # the first calls compile and tune the Triton kernels
            decode_bench(run, model, 2, 2, 1, 128, vocab, seed=99)
            clock_sampler.start()
            ms = decode_bench(run, model, args.batch, args.steps, args.warmup, prompt_len, vocab, seed=1)
            clocks = clock_sampler.stop()
            points = {}
            if not args.skip_points:
                for b in (1, 64):
                    pms = decode_bench(run, model, b, max(16, args.steps // 2), args.warmup, prompt_len, vocab, seed=2 + b)
                    points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
            pre_ms = prefill_bench(run, model, prefill_tokens, vocab, reps=5, seed=7)
            e2e = e2e_bench(run, model, args.batch, prompt_len, consts["E2E_NEW_TOKENS"], vocab, seed=9, runs=3)
    except Exception as e:
        msg = " ".join(f"{type(e).__name__}: {e}".split())[:400]
        print(json.dumps({"impl": "reference", "unavailable": f"the reference failed on this GPU: {msg}"}))
        return 0
    n_layers, dim = config["n_layers"], config["dim"]
    head_dim = dim // config["n_heads"]
    inter = model.layers[0].mlp.w1.weight.shape[0]
    per_layer = (config["n_heads"] + 2 * config["n_kv_heads"]) * head_dim * dim + dim * dim + 3 * inter * dim
    weights = (n_layers * per_layer + vocab * dim) * 2
    kv_per_token = n_layers * 2 * config["n_kv_heads"] * head_dim * 2
    ctx_mid = prompt_len + args.warmup + args.steps / 2.0
    achieved = (weights + args.batch * ctx_mid * kv_per_token) / (ms * 1e-3) / 1e9
    flops = 2 * prefill_tokens * n_layers * per_layer + n_layers * 4 * head_dim * config["n_heads"] * prefill_tokens * (prefill_tokens + 1) // 2 \
        + 2 * vocab * dim
    rec = {
        "metric": "decode tok/s at batch 8 (Llama-3.2-1B shape, 2048-token prompts, context 4096)",
        "value": round(args.batch * 1000.0 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, seeded random weights N(0,0.02)",
        "impl": "reference",
        "config": {"model": "llama-3.2-1b-shape", "layers": n_layers, "layers_full": n_layers, "hidden": dim,
                   "heads": config["n_heads"], "kv_heads": config["n_kv_heads"], "head_dim": head_dim, "intermediate": inter,
                   "vocab": vocab, "global_batch": args.batch, "seq_len": context, "prompt_len": prompt_len, "page_size": 64,
                   "parallelism": "single-gpu", "l2": "inputs larger than L2: 2.47 GB of weights read per step",
                   "peaks": peaks["source"], "path": "serve.run.decode_one_token / prefill / generate, stock, eager"},
        "e2e": e2e,
        "prefill": {"value": round(prefill_tokens / (pre_ms * 1e-3), 1), "tokens": prefill_tokens, "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks,
    }
    print(json.dumps(rec))
    return 0


def offline_load(which: str, num_sequences: int = 2000) -> int:
    """The reference's own benchmark load (serve/benchmark.py:12-24: lengths uniform in 1..256, seeds 1352, temperature
    0.6) on random weights of its 1B or 8B configuration: one untimed run, then the timed run, as its benchmark does
    (benchmark.py:63-80). The model is built on the GPU directly (no checkpoint file of 16 GB is written)."""
    sys.path.insert(0, REF)
    sys.dont_write_bytecode = True
    import torch

    import serve.run as run
    from serve.model import LlamaModel, ModelArgs
    from serve.utils import config_1b, config_8b

    import random       # (serve/benchmark.py itself is not imported: its module body loads a checkpoint from the hub)

    config = dict(config_1b if which == "1b" else config_8b)
    with torch.device("cuda"):
        model = LlamaModel(ModelArgs(**config), dtype=torch.bfloat16).to(torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(0)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith("norm.weight"):
                p.fill_(1.0)
            else:
                p.copy_((torch.randn(p.shape, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(p.dtype))
    model.compute_freqs_cis("cuda")
    model = model.eval()
    random.seed(1352)
    torch.manual_seed(1352)
    reqs = []
    for _ in range(num_sequences):                       # serve/benchmark.py:12-24
        n_in, n_out = random.randint(1, 256), random.randint(1, 256)
        reqs.append(run.Request(input_ids=torch.randint(0, 10000, (n_in,), dtype=torch.long), input_length=n_in, max_new_tokens=n_out))
    t0 = time.perf_counter()
    run.generate(model, reqs, 0.6)
    print(f"Warmup time: {time.perf_counter() - t0:.4f} seconds")
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = run.generate(model, reqs, 0.6)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    total = sum(len(r.generated_tokens) for r in out)
    print(f"Time taken: {dt:.4f} seconds")
    print(f"Throughput: {total / dt:.2f} tokens/second")
    return 0


if __name__ == "__main__":
    if len(sys.argv) >= 3 and sys.argv[1] == "--offline":
        sys.exit(offline_load(sys.argv[2], int(sys.argv[3]) if len(sys.argv) > 3 else 2000))
    sys.exit("usage: python baseline/reference_arm.py --offline 1b|8b [requests]   (bench.py --impl reference runs the benchmark arm)")
