"""The Python entry point, in the manner of the reference's serve/run.py, and a command line.

    model, tokenizer = load_model("path/to/folder", device="cuda", dtype=torch.bfloat16)
    requests = [Request(input_ids=torch.tensor([...]), input_length=n, max_new_tokens=64)]
    finished = generate(model, requests, temperature=0.0, return_logits=False)

``Request`` has the reference's fields (serve/run.py:16-22), ``generate`` its
signature and meaning (run.py:238-308): it returns the requests in the order
given, each with ``generated_tokens`` and, if asked, the logits of its final
step. Stopping is by ``max_new_tokens`` as in the reference (run.py:222), and
by the end-of-sequence ids of the model's config.json if it names any (or by
the ids passed as ``eos_token_id``; ``None`` switches that off, which is the
reference's behaviour).

Command line:  python -m serve_b200.run --model DIR --prompt-ids 1,2,3 --max-new-tokens 16
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import sys
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .config import EngineConfig, load_preset, normalize_dtype
from .engine import Engine, StepEntry
from .engine.scheduler import SchedRequest, Scheduler
from .sampling import Sampler


@dataclass
class Request:
    input_ids: torch.Tensor
    input_length: int
    max_new_tokens: int
    generated_tokens: torch.Tensor = field(default_factory=lambda: torch.tensor([], dtype=torch.long))
    logits: Optional[torch.Tensor] = None


def load_model(model_name, device: str = "cuda", dtype=torch.bfloat16, **engine_options):
    """An engine for the model folder ``model_name`` and its tokenizer (None if the folder has none).

    The reference resolves a hub name and downloads (serve/utils.py:41-58); here the name is a local
    folder with config.json and model.safetensors. ``engine_options`` are fields of EngineConfig."""
    dev = "cuda:0" if device == "cuda" else device
    ec = EngineConfig(dtype=normalize_dtype(dtype), device=dev, **engine_options)
    print(f"loading model {model_name}...")
    engine = Engine.from_folder(str(model_name), ec)
    tokenizer = None
    if os.path.isfile(os.path.join(str(model_name), "tokenizer.json")) or os.path.isfile(os.path.join(str(model_name), "tokenizer.model")):
        try:
            from transformers import AutoTokenizer  # text <-> ids only; no model code

            tokenizer = AutoTokenizer.from_pretrained(str(model_name))
        except Exception as e:  # the engine works on token ids; a tokenizer is optional
            print(f"tokenizer not loaded ({e})")
    print("Model finished loading")
    return engine, tokenizer


@torch.inference_mode()
def generate(model: Engine, requests: Sequence[Request], temperature: float = 0.0, return_logits: bool = False,
             seed: int = 0, eos_token_id="config", timeline: Optional[list] = None) -> List[Request]:
    """Run all requests to the end; token ids come from the host and go back to the host every step.

    ``eos_token_id``: an id or several that end a request when generated; "config" (the default) takes the ids the
    model's configuration names, None stops by length only.

    ``timeline``, if a list, receives one record per step after its tokens have reached the host:
    (time.perf_counter(), prompt tokens in the step, decoded tokens in the step, bytes copied to the device)."""
    ec = model.engine_config
    sched = Scheduler(model.cache, ec.max_tokens_per_step, ec.prefill_chunk, ec.reserve_full, ec.admission_fraction,
                      model.max_context)
    sampler = Sampler(model.kernels, model.rt.device, seed)
    if isinstance(eos_token_id, str):
        if eos_token_id != "config":
            raise ValueError('eos_token_id must be an id, a list of ids, None or "config"')
        eos_token_id = getattr(model.config, "eos_token_id", None)
    if eos_token_id is None:
        stop = ()
    elif isinstance(eos_token_id, (list, tuple)):
        stop = tuple(int(e) for e in eos_token_id)
    else:
        stop = (int(eos_token_id),)
    for i, r in enumerate(requests):
        ids = r.input_ids.tolist() if isinstance(r.input_ids, torch.Tensor) else list(r.input_ids)
        sched.add(SchedRequest(i, ids[: r.input_length], r.max_new_tokens, temperature, stop))
    model.last_stats = sched.stats
    # The loop below makes many short-lived lists in every step, none of them part of a reference cycle; what costs is
    # the cyclic collector walking the long-lived objects (thousands of requests, the engine) again and again: 12 % of
    # the reference's 2,000-request load at the 1B shape. They are set aside while the call lasts; what the loop drops
    # is still freed at once by reference counting, and young cycles are still collected.
    gc.freeze()
    try:
        return _generate_loop(model, requests, sched, sampler, stop, return_logits, timeline)
    finally:
        gc.unfreeze()


def _generate_loop(model, requests, sched, sampler, stop, return_logits, timeline):
    import time

    # Steps are launched one ahead of the host's knowledge of their tokens: step N+1 takes the tokens step N sampled
    # straight from the device (FROM_DEVICE), and the host reads step N's tokens while step N+1 runs. A stop id is
    # therefore found one step late (that step's work for the request is dropped). With return_logits and a stop id
    # the logits of the last step must still be there when the stop is found, so that case runs step by step.
    pipelined = not (return_logits and stop)
    on_cuda = model.rt.device.type == "cuda"
    staging = [None, None]
    turn = 0
    inflight = None          # (requests, indices of their new tokens, host tensor, event, step record)
    ended = set()

    def end(r):
        if r.rid not in ended:
            ended.add(r.rid)
            model.end(r.rid)

    def resolve(rec):
        reqs, idxs, host, event, stamp, step_logits = rec
        if event is not None:
            event.synchronize()
        toks = host[: len(reqs)].tolist()        # device -> host: the step's result
        if not stop:
            for r, i, tok in zip(reqs, idxs, toks):      # nothing can end a request here: the tokens take their places
                if i < len(r.generated):
                    r.generated[i] = tok
        else:
            for row, (r, i, tok) in enumerate(zip(reqs, idxs, toks)):
                if sched.resolve(r, i, tok):
                    if return_logits and step_logits is not None:
                        r.last_logits = step_logits[row].clone()
                    end(r)
        if timeline is not None:
            timeline.append((time.perf_counter(),) + stamp)

    while sched.has_work() or inflight is not None:
        launched = None
        if sched.has_work():
            planned = sched.plan()
            if sched.evicted and inflight is not None:
                resolve(inflight)                # an evicted request is recomputed from tokens the host must know
                inflight = None
                if not sched.has_work():
                    continue
                planned = [p for p in planned if not p.request.finished]
            for victim in sched.evicted:
                if not victim.finished:
                    model.end(victim.rid)
            if not planned:
                if inflight is not None:
                    resolve(inflight)
                    inflight = None
                    continue
                raise RuntimeError("the scheduler found nothing to run although requests are waiting")
            # one pass over the step's requests (a thousand of them in a full step) for everything that is per request
            entries, sampling, temps, sampled_rids, idxs = [], [], [], [], []
            n_dec = n_tok = 0
            for p in planned:
                r, toks = p.request, p.tokens
                n = len(toks)
                n_tok += n
                if p.samples:
                    entries.append(StepEntry(r.rid, toks, [n - 1]))
                    sampling.append(r)
                    temps.append(r.temperature)
                    sampled_rids.append(r.rid)
                    made = len(r.generated)
                    idxs.append(made)
                    if n == 1 and made:
                        n_dec += 1
                else:
                    entries.append(StepEntry(r.rid, toks, []))
            logits = model.step(entries)
            host = event = None
            if sampling:
                turn ^= 1
                if staging[turn] is None or staging[turn].numel() < len(sampling):
                    staging[turn] = torch.empty(max(64, 1 << (len(sampling) - 1).bit_length()), dtype=torch.int32, pin_memory=on_cuda)
                host = staging[turn]
                # on a GPU the sampling kernel writes the tokens straight into this pinned host buffer
                out = sampler.sample(logits, temps, sampled_rids, idxs, model.cache.lengths_and_slots(sampled_rids)[1],
                                     model.stepper.last_token, out=host if on_cuda else None)
                if on_cuda:
                    event = torch.cuda.Event()
                    event.record()
                else:
                    host[: len(sampling)].copy_(out)
            stamp = (n_tok - n_dec, n_dec, model.stepper.last_h2d_bytes + 16 * len(sampling))
            done = sched.update(planned, [None] * len(sampling))
            if done:
                rows = {id(r): i for i, r in enumerate(sampling)}
                for r in done:
                    if return_logits:
                        r.last_logits = logits[rows[id(r)]].clone()
                    end(r)
            launched = (sampling, idxs, host, event, stamp, logits if (return_logits and not pipelined) else None)
        if inflight is not None:
            resolve(inflight)                    # the previous step's tokens, read while this step runs
        inflight = launched if (launched is not None and launched[0]) else None
        if launched is not None and not launched[0] and timeline is not None:
            timeline.append((time.perf_counter(),) + launched[4])
        if inflight is not None and not pipelined:
            resolve(inflight)
            inflight = None
    by_id = {r.rid: r for r in sched.finished}
    out_requests = []
    for i, r in enumerate(requests):
        f = by_id[i]
        out_requests.append(Request(input_ids=r.input_ids, input_length=r.input_length, max_new_tokens=r.max_new_tokens,
                                    generated_tokens=torch.tensor(f.generated, dtype=torch.long),
                                    logits=f.last_logits if return_logits else None))
    return out_requests


# ---- command line ---------------------------------------------------------------
def _parse_ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def build_engine_from_args(args) -> Engine:
    ec = EngineConfig(dtype=normalize_dtype(args.dtype), device=args.device, page_size=args.page_size, num_pages=args.num_pages,
                      max_tokens_per_step=args.max_tokens_per_step, max_slots=args.max_slots, max_context=args.max_context,
                      prefill_chunk=args.prefill_chunk, memory_fraction=args.memory_fraction,
                      use_cuda_graphs=not args.no_graphs)
    if args.model:
        return Engine.from_folder(args.model, ec)
    return Engine.from_config(load_preset(args.random), args.seed, ec)


def add_engine_args(ap: argparse.ArgumentParser) -> None:
    src = ap.add_mutually_exclusive_group(required=True)
    src.add_argument("--model", help="model folder (config.json + model.safetensors)")
    src.add_argument("--random", metavar="PRESET", help="random weights for a named configuration (e.g. llama-3.2-1b, tiny-a)")
    ap.add_argument("--seed", type=int, default=0, help="seed of the random weights and of sampling")
    ap.add_argument("--dtype", default="bfloat16", help="bfloat16 | float32")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--num-pages", type=int, default=None, help="cache pages (default: from --memory-fraction)")
    ap.add_argument("--memory-fraction", type=float, default=0.6)
    ap.add_argument("--max-slots", type=int, default=256)
    ap.add_argument("--max-context", type=int, default=None)
    ap.add_argument("--max-tokens-per-step", type=int, default=2048)
    ap.add_argument("--prefill-chunk", type=int, default=None)
    ap.add_argument("--no-graphs", action="store_true")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m serve_b200.run", description="Generate token ids with the engine.")
    add_engine_args(ap)
    ap.add_argument("--prompt-ids", action="append", default=[], help="token ids of one prompt, comma or space separated (repeatable)")
    ap.add_argument("--prompt-file", help="file with one prompt per line (token ids), or a JSON list of lists")
    ap.add_argument("--prompt", action="append", default=[], help="text prompt (needs a tokenizer in the model folder)")
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--eos-token-id", type=int, action="append", default=None,
                    help="id that ends a request (repeatable); default: the ids config.json names")
    ap.add_argument("--ignore-eos", action="store_true", help="stop by length only")
    ap.add_argument("--return-logits", action="store_true")
    args = ap.parse_args(argv)

    prompts = [_parse_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            text = f.read()
        try:
            prompts += [list(map(int, p)) for p in json.loads(text)]
        except json.JSONDecodeError:
            prompts += [_parse_ids(line) for line in text.splitlines() if line.strip()]
    engine = build_engine_from_args(args)
    tokenizer = None
    if args.prompt:
        from transformers import AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(args.model)
        prompts += [tokenizer.encode(p) for p in args.prompt]
    if not prompts:
        ap.error("no prompt given (--prompt-ids, --prompt-file or --prompt)")
    reqs = [Request(torch.tensor(p, dtype=torch.long), len(p), args.max_new_tokens) for p in prompts]
    out = generate(engine, reqs, temperature=args.temperature, return_logits=args.return_logits, seed=args.seed,
                   eos_token_id=None if args.ignore_eos else (args.eos_token_id or "config"))
    for i, r in enumerate(out):
        rec = {"request": i, "generated_tokens": r.generated_tokens.tolist()}
        if tokenizer is not None:
            rec["text"] = tokenizer.decode(r.generated_tokens.tolist())
        print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
