"""Shared by the tests: tiny configurations, model folders, traces and their replay."""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List, Sequence

import torch

# Two tiny configurations that differ in every size and option, plus a third with sizes that are
# no power of two anywhere (odd head count, group of 5, head_dim 48, vocabulary 331).
TINY = {
    "a": dict(architectures=["LlamaForCausalLM"], hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256, rms_norm_eps=1e-5,
              rope_theta=10000.0, rope_scaling=None, tie_word_embeddings=True, max_position_embeddings=2048),
    "b": dict(architectures=["LlamaForCausalLM"], hidden_size=192, num_hidden_layers=3, num_attention_heads=6,
              num_key_value_heads=3, head_dim=32, intermediate_size=320, vocab_size=384, rms_norm_eps=1e-6,
              rope_theta=500000.0,
              rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=64),
              tie_word_embeddings=False, max_position_embeddings=2048),
    "c": dict(architectures=["LlamaForCausalLM"], hidden_size=120, num_hidden_layers=4, num_attention_heads=5,
              num_key_value_heads=1, head_dim=48, intermediate_size=200, vocab_size=331, rms_norm_eps=3e-6,
              rope_theta=25000.0,
              rope_scaling=dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=8.0,
                                original_max_position_embeddings=32),
              tie_word_embeddings=True, max_position_embeddings=1024),
}
NORM_STD = {"a": 0.0, "b": 0.1, "c": 0.2}
# random weights N(0, 0.02) give logits near zero; a larger std makes attention and logits matter
WEIGHT_STD = {"a": 0.02, "b": 0.02, "c": 0.05}


def make_folder(path: str, name: str, seed: int = 0, dtype=torch.float32, std=None) -> str:
    from serve_b200.config import config_from_dict
    from serve_b200.weights import write_random_model

    cfg = config_from_dict(TINY[name])
    write_random_model(path, cfg, seed, std=WEIGHT_STD[name] if std is None else std, norm_std=NORM_STD[name], dtype=dtype)
    return path


def read_folder(path: str):
    """(config dict, weights as float32 by name) through the safetensors package, not the engine's reader."""
    from safetensors.torch import load_file

    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    w = {k: v.float() for k, v in load_file(os.path.join(path, "model.safetensors")).items()}
    return cfg, w


# A shape the reference's own Triton kernels take (pages of 64, head_dim 64): the golden outputs made on a GPU use it.
GOLDEN_GPU = dict(architectures=["LlamaForCausalLM"], hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=64, intermediate_size=768, vocab_size=512, rms_norm_eps=1e-5,
                  rope_theta=500000.0,
                  rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                    original_max_position_embeddings=64),
                  tie_word_embeddings=False, max_position_embeddings=256)


def llama_tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Tensor names of a Llama weight file (the left column of serve/hf_utils/convert_hf_checkpoint.py:98-112) and shapes."""
    h, d = cfg["hidden_size"], cfg["head_dim"]
    nh, nkv, inter, v = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"], cfg["vocab_size"]
    shapes = {"model.embed_tokens.weight": (v, h), "model.norm.weight": (h,)}
    if not cfg["tie_word_embeddings"]:
        shapes["lm_head.weight"] = (v, h)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        shapes.update({p + "self_attn.q_proj.weight": (nh * d, h), p + "self_attn.k_proj.weight": (nkv * d, h),
                       p + "self_attn.v_proj.weight": (nkv * d, h), p + "self_attn.o_proj.weight": (h, nh * d),
                       p + "mlp.gate_proj.weight": (inter, h), p + "mlp.up_proj.weight": (inter, h),
                       p + "mlp.down_proj.weight": (h, inter), p + "input_layernorm.weight": (h,),
                       p + "post_attention_layernorm.weight": (h,)})
    return shapes


def counted_weights(cfg: dict, seed: int, std: float = 0.05, norm_spread: float = 0.1) -> Dict[str, torch.Tensor]:
    """Weights that are the same numbers on every machine and under every version of torch and numpy: uniform values
    from the raw 64-bit stream of numpy's PCG64 (whose stream is fixed by its definition), one stream per tensor name.
    Matrices are uniform with standard deviation ``std``; norm weights uniform in 1 +- norm_spread."""
    import hashlib

    import numpy as np

    out = {}
    for name, shape in llama_tensor_shapes(cfg).items():
        key = int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")
        n = 1
        for s in shape:
            n *= s
        raw = np.random.PCG64(key).random_raw(n)
        u = (raw >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0) * 2.0 - 1.0     # [-1, 1)
        if len(shape) == 1:
            vals = 1.0 + norm_spread * u
        else:
            vals = u * (std * 3.0 ** 0.5)
        out[name] = torch.from_numpy(vals.astype(np.float32).reshape(shape))
    return out


def counted_tokens(vocab: int, n: int, seed: int) -> List[int]:
    """Token ids from the same fixed stream."""
    import numpy as np

    return (np.random.PCG64(seed).random_raw(n) % np.uint64(vocab)).astype(np.int64).tolist()


def write_folder(path: str, cfg: dict, weights: Dict[str, torch.Tensor], dtype=torch.float32) -> str:
    """A model folder from a config dict and weights by name (through the safetensors package)."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(dict(cfg, torch_dtype=str(dtype).replace("torch.", "")), f)
    save_file({k: v.to(dtype).contiguous() for k, v in weights.items()}, os.path.join(path, "model.safetensors"))
    return path


def random_tokens(vocab: int, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ---- traces -------------------------------------------------------------------
# A trace is a list of steps {"step": i, "entries": [{"id", "tokens", "want"}], "end": [ids]}.

def _step(i, entries, end=()):
    return {"step": i, "entries": entries, "end": list(end)}


def trace_whole(requests: Dict[str, List[int]]):
    """Each request alone and whole, every position wanted."""
    steps = []
    for rid, toks in requests.items():
        steps.append(_step(len(steps), [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], [rid]))
    return steps


def trace_tail_decode(requests: Dict[str, List[int]], tail: int = 32):
    """Most of each request in one step, then its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append(_step(len(steps), [{"id": rid, "tokens": toks[:head], "want": list(range(head))}]))
        for j in range(head, len(toks)):
            steps.append(_step(len(steps), [{"id": rid, "tokens": [toks[j]], "want": [0]}],
                               [rid] if j == len(toks) - 1 else []))
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: Dict[str, List[int]], sizes: Sequence[int] = (7, 2, 19, 3, 2, 33, 5, 64, 2, 11)):
    """Each request alone, cut into portions of changing size, down to two tokens."""
    steps = []
    k = 0
    for rid, toks in requests.items():
        at = 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            last = at + n == len(toks)
            steps.append(_step(len(steps), [{"id": rid, "tokens": toks[at:at + n], "want": list(range(n))}], [rid] if last else []))
            at += n
    return steps


def trace_mixed(requests: Dict[str, List[int]], live: int = 4, seed: int = 0, decode_tail: int = 6, budget: int = 48):
    """Up to ``live`` requests at a time: portions of some beside single tokens of others;
    a request's last ``decode_tail`` tokens come one by one; now and then a request sits a step out."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    running: List[list] = []   # [rid, toks, at]
    steps = []
    while waiting or running:
        while waiting and len(running) < live:
            rid, toks = waiting.pop(0)
            running.append([rid, toks, 0])
        entries, end, left = [], [], budget
        for slot in running:
            rid, toks, at = slot
            if len(running) > 1 and rng.random() < 0.15:
                continue  # left out of this step; goes on later
            remaining = len(toks) - at
            if remaining <= decode_tail:
                n = 1
            else:
                n = min(rng.choice([2, 3, 5, 8, 13, 21]), remaining - decode_tail, max(left, 1))
            if n > left:
                continue
            entries.append({"id": rid, "tokens": toks[at:at + n], "want": list(range(n))})
            left -= n
            slot[2] = at + n
            if slot[2] == len(toks):
                end.append(rid)
        if not entries:
            continue
        steps.append(_step(len(steps), entries, end))
        running = [s for s in running if s[0] not in end]
    return steps


def tokens_needed(steps, page: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``page``."""
    held: Dict[str, int] = {}
    worst = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // page) * page for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return worst


def replay(engine, steps):
    """Drive an Engine through a trace; returns {(rid, position): logits row (cpu float32)}."""
    from serve_b200.engine import StepEntry

    got = {}
    at: Dict[str, int] = {}
    for st in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]]
        logits = engine.step(entries)
        if logits is not None:
            logits = logits.detach().float().cpu().clone()
        i = 0
        for e in st["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = logits[i]
                i += 1
            at[e["id"]] = base + len(e["tokens"])
        for rid in st["end"]:
            engine.end(rid)
            at.pop(rid, None)
    return got


def compare_with_plain(got, plain: Dict[str, torch.Tensor], atol: float, rtol: float = 0.0):
    """Every collected row against the plain logits; reports the first wrong token by request and position."""
    worst = 0.0
    for (rid, pos), row in sorted(got.items(), key=lambda kv: (str(kv[0][0]), kv[0][1])):
        ref = plain[rid][pos]
        diff = (row - ref).abs()
        tol = atol + rtol * ref.abs()
        if not bool((diff <= tol).all()) or not bool(torch.isfinite(row).all()):
            raise AssertionError(f"first wrong token: request {rid!r} position {pos}: max |diff| {float(diff.max()):.3e} "
                                 f"(allowed {atol:.1e} + {rtol:.1e}*|ref|), logits scale {float(ref.abs().max()):.3f}")
        worst = max(worst, float(diff.max()))
    return worst
