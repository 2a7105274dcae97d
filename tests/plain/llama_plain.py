"""A plain, slow Llama: whole sequences, no cache, float32 (or float64), one function per part.

Written from the formulas of limei1221/serve, cited per function by file:line
within that project. It shares no code with ``serve_b200``: weights are a dict
from the weight file's tensor names to torch tensors, the configuration is the
parsed config.json dict. The reference keeps q/k rows permuted for interleaved
rotation (serve/hf_utils/convert_hf_checkpoint.py:115-118); with the file's own
row order the same rotation pairs element j with j + D/2, which is what
``rotate`` does here (checked against the reference's own code on tiny models,
see tests/golden/).
"""
from __future__ import annotations

import math

import torch


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None, dtype=torch.float32) -> torch.Tensor:
    """serve/model.py:276 (freq_j = 1/base^(2j/D)) and :247-266 (llama3 scaling per frequency)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    if scaling is not None and scaling.get("rope_type", scaling.get("type", "llama3")) not in (None, "default"):
        factor = scaling["factor"]
        low = scaling["low_freq_factor"]
        high = scaling["high_freq_factor"]
        old = scaling["original_max_position_embeddings"]
        wavelen = 2 * math.pi / inv
        smooth = (old / wavelen - low) / (high - low)
        mid = (1 - smooth) * inv / factor + smooth * inv
        inv = torch.where(wavelen < old / high, inv, torch.where(wavelen > old / low, inv / factor, mid))
    return inv.to(dtype)


def rotate(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """serve/model.py:234-244 on unpermuted rows: x [T, heads, D], pairs (j, j + D/2). Below 32-bit the rotation
    itself is done in float32 and cast back, as the reference does (model.py:235,244)."""
    d = x.shape[-1]
    wide = torch.float32 if x.dtype in (torch.bfloat16, torch.float16) else x.dtype
    ang = positions.to(inv_freq.dtype if wide != torch.float32 else torch.float32)[:, None] * inv_freq.to(wide)[None, :]      # [T, D/2]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., : d // 2].to(wide), x[..., d // 2:].to(wide)
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """serve/model.py:63-68: the mean square and the scaling in float32 (or wider), cast back, then times the weight."""
    wide = x.float() if x.dtype in (torch.bfloat16, torch.float16) else x
    return (wide * torch.rsqrt(wide.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


def swiglu(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """serve/model.py:85: w2(silu(w1 x) * w3 x)."""
    g = x @ gate.T
    return ((g * torch.sigmoid(g)) * (x @ up.T)) @ down.T


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int | None = None,
                     q_positions: torch.Tensor | None = None) -> torch.Tensor:
    """serve/kernels/attn_prefill.py:56-72 without tiling: softmax(q k^T * scale + causal mask) v.

    q [Tq, H, D]; k, v [Tk, Hkv, D]; head h reads kv head h // (H / Hkv) (attn_prefill.py:265).
    Query i sits at position q_positions[i] (default: Tk - Tq + i) and sees keys
    0..position (or the last ``window`` of them)."""
    tq, h, d = q.shape
    tk, hkv, _ = k.shape
    g = h // hkv
    if q_positions is None:
        q_positions = torch.arange(tk - tq, tk, device=q.device)
    kk = k.repeat_interleave(g, dim=1)
    vv = v.repeat_interleave(g, dim=1)
    s = torch.einsum("thd,shd->hts", q, kk) * scale
    key_pos = torch.arange(tk, device=q.device)[None, :]
    mask = key_pos > q_positions[:, None]
    if window:
        mask = mask | (key_pos <= q_positions[:, None] - window)
    s = s.masked_fill(mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hts,shd->thd", p, vv)


def attention_layer(x, w, prefix, cfg, positions, inv_freq, window=None, kv_override=None):
    """serve/model.py:103-134 with separate q/k/v matrices; returns (out, (k, v))."""
    t = x.shape[0]
    h, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    q = (x @ w[prefix + "q_proj.weight"].T).view(t, h, d)
    q = rotate(q, positions, inv_freq)
    if kv_override is None:
        k = rotate((x @ w[prefix + "k_proj.weight"].T).view(t, hkv, d), positions, inv_freq)
        v = (x @ w[prefix + "v_proj.weight"].T).view(t, hkv, d)
    else:
        k, v = kv_override
    a = causal_attention(q, k, v, 1.0 / math.sqrt(d), window, positions)
    return a.reshape(t, h * d) @ w[prefix + "o_proj.weight"].T, (k, v)


def normalise_config(cfg: dict) -> dict:
    c = dict(cfg)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    if c.get("head_dim") is None:
        c["head_dim"] = c["hidden_size"] // c["num_attention_heads"]
    c.setdefault("rms_norm_eps", 1e-5)
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("rope_scaling", None)
    c.setdefault("tie_word_embeddings", False)
    return c


def llama_forward(weights: dict, cfg: dict, tokens, dtype=torch.float32, schedule=None, window=None, device=None,
                  rows=None) -> torch.Tensor:
    """serve/model.py:196-231 for one whole sequence from position 0: logits [T, V] at every position.

    ``schedule``: list of (layer, cache_of) pairs; default one run of each layer in order.
    ``device``: where to compute (the weights must lie there already; on a GPU the caller switches TF32 off).
    ``rows``: positions whose logits are wanted (default all): the head is applied to these only."""
    cfg = normalise_config(cfg)
    w = weights if all(v.dtype == dtype for v in weights.values()) else {k: v.to(dtype) for k, v in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long, device=device)
    t = tokens.shape[0]
    positions = torch.arange(t, device=device)
    # frequencies stay 32-bit below 32-bit too: the reference keeps its table of cosines and sines in float32 (model.py:279-283)
    inv_freq = rope_inv_freq(cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"]).to(
        torch.float32 if dtype in (torch.bfloat16, torch.float16) else dtype).to(tokens.device)
    eps = cfg["rms_norm_eps"]
    x = w["model.embed_tokens.weight"][tokens]                                           # model.py:220
    if schedule is None:
        schedule = [(i, None) for i in range(cfg["num_hidden_layers"])]
    kvs = []
    for layer, cache_of in schedule:
        p = f"model.layers.{layer}."
        hn = rms_norm(x, w[p + "input_layernorm.weight"], eps)
        a, kv = attention_layer(hn, w, p + "self_attn.", cfg, positions, inv_freq, window,
                                kv_override=None if cache_of is None else kvs[cache_of])
        kvs.append(kv)
        x = x + a                                                                        # model.py:147
        hn = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + swiglu(hn, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])  # :148
    x = rms_norm(x, w["model.norm.weight"], eps)                                         # model.py:223
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long, device=x.device)]
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return x @ head.T                                                                    # model.py:227


# ---- sampling (serve/run.py:47-60) ------------------------------------------------
def _mix32(x: int) -> int:
    x &= 0xFFFFFFFF
    x ^= x >> 16
    x = (x * 0x7FEB352D) & 0xFFFFFFFF
    x ^= x >> 15
    x = (x * 0x846CA68B) & 0xFFFFFFFF
    x ^= x >> 16
    return x


def counter_uniforms(seed: int, req: int, tok: int, vocab: int):
    """The engine's counter-based uniforms for one (request, token index): numpy float32 [vocab]."""
    import numpy as np

    h = _mix32((seed & 0xFFFFFFFF) ^ 0x9E3779B9)
    h = _mix32(h ^ ((seed >> 32) & 0xFFFFFFFF))
    h = _mix32((h + req * 0x85EBCA6B) & 0xFFFFFFFF)
    h = _mix32(h ^ ((tok * 0xC2B2AE35) & 0xFFFFFFFF))
    i = np.arange(vocab, dtype=np.uint64)
    x = (np.uint64(h) + i) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(16)
    x = (x * np.uint64(0x7FEB352D)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(15)
    x = (x * np.uint64(0x846CA68B)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(16)
    return ((x >> np.uint64(8)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)


def sample_token(logits_row: torch.Tensor, temperature: float, seed: int = 0, req: int = 0, tok: int = 0) -> int:
    """run.py:56-60: argmax for temperature 0, else argmax(softmax(l/T) / q), q ~ Exp(1), as argmax(l/T - log q)."""
    import numpy as np

    l = logits_row.detach().cpu().numpy().astype(np.float32)
    if temperature == 0:
        return int(np.argmax(l))
    u = counter_uniforms(seed, req, tok, l.shape[0])
    q = -np.log(u)
    return int(np.argmax(l / np.float32(temperature) - np.log(q)))
