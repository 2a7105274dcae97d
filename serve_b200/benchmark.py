"""Offline-batch benchmark in the manner of the reference's serve/benchmark.py.

    python -m serve_b200.benchmark --random llama-3.2-1b [--fixed-lengths] [--profile] [--profile-only]

Seeded synthetic requests (prompt and output lengths uniform in 1..256, token ids below 10000, seeds 1352:
serve/benchmark.py:12-24), one untimed warm-up run of the whole load, then a timed run between device
synchronisations; prints the time taken and generated tokens per second (benchmark.py:63-80). ``--profile``
adds a run under torch.profiler and writes a chrome trace (benchmark.py:82-101); ``--profile-only`` skips the
timed run.
"""
from __future__ import annotations

import argparse
import os
import random
import sys
import time

import torch

from .run import Request, add_engine_args, build_engine_from_args, generate


def generate_requests(input_length: int, output_length: int, num_sequences: int, vocab_limit: int = 10000, fixed_lengths: bool = False):
    """``fixed_lengths``: every request has exactly input_length prompt tokens and output_length new tokens (the form the
    reference's benchmark keeps commented out, serve/benchmark.py:19-20) instead of lengths drawn from 1..n."""
    random.seed(1352)
    torch.manual_seed(1352)
    reqs = []
    for _ in range(num_sequences):
        n_in = input_length if fixed_lengths else random.randint(1, input_length)
        n_out = output_length if fixed_lengths else random.randint(1, output_length)
        reqs.append(Request(torch.randint(0, vocab_limit, (n_in,), dtype=torch.long), n_in, n_out))
    return reqs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m serve_b200.benchmark")
    add_engine_args(ap)
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--profile-only", action="store_true")
    ap.add_argument("--input-length", type=int, default=256)
    ap.add_argument("--output-length", type=int, default=256)
    ap.add_argument("--num-sequences", type=int, default=2000)
    ap.add_argument("--temperature", type=float, default=0.6)
    ap.add_argument("--fixed-lengths", action="store_true",
                    help="every request has exactly --input-length prompt tokens and --output-length new tokens")
    # the load is 2000 requests at once: more live requests mean fewer, fuller steps (the reference admits up to 4000,
    # serve/run.py:13)
    ap.set_defaults(max_slots=1024)
    args = ap.parse_args(argv)
    engine = build_engine_from_args(args)
    reqs = generate_requests(args.input_length, args.output_length, args.num_sequences,
                             min(10000, engine.spec.vocab_size), fixed_lengths=args.fixed_lengths)

    def fn():
        return generate(engine, reqs, args.temperature, seed=args.seed, eos_token_id=None)   # by length only, as the reference

    print("doing first run")
    st = time.perf_counter()
    fn()
    print(f"Warmup time: {time.perf_counter() - st:.4f} seconds")
    if not args.profile_only:
        torch.cuda.synchronize()
        st = time.perf_counter()
        responses = fn()
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - st
        total = sum(len(r.generated_tokens) for r in responses)
        print(f"Time taken: {elapsed:.4f} seconds")
        print(f"Throughput: {total / elapsed:.2f} tokens/second")
        s = engine.last_stats
        print(f"steps {s.steps}, prompt tokens {s.prefill_tokens}, decoded tokens {s.decode_tokens}, "
              f"evictions {s.preemptions}, most requests at once {s.max_running}")
    if args.profile:
        name = f"generate_{args.input_length}_{args.output_length}_{args.num_sequences}"
        with torch.profiler.profile() as prof:
            with torch.autograd.profiler.record_function(name):
                fn()
        os.makedirs("/tmp/traces", exist_ok=True)
        path = f"/tmp/traces/trace_{name}_{time.strftime('%H%M')}.json"
        prof.export_chrome_trace(path)
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=15))
        print(f"Trace saved to {path}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
