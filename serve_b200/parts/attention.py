"""Grouped-query causal attention over a paged key/value cache.

Per token: fused q/k/v projection (serve/model.py:104-112), rotation of q and k
(model.py:118), write of the new k and v rows into the request's pages before
attention (model.py:120-124), softmax(q k^T * scale) v over all cached keys up
to the token's own position (serve/kernels/attn_prefill.py:56-72,
serve/kernels/attn_decode.py:99-111), output projection (model.py:132-133).
Query head h reads key/value head h // (heads / kv_heads)
(attn_prefill.py:265). A window, if given, limits a query at position p to
keys p-window+1 .. p; the reference has none.
"""
from __future__ import annotations

import math

import torch

from .base import CacheNeed, Mixer, TensorDecl, build_part, register_part
from .rotary import PAIRING_HALF, PAIRING_INTERLEAVED


@register_part("mixer", "attention")
class Attention(Mixer):
    """params: hidden, heads, kv_heads, head_dim, scale (None: head_dim**-0.5),
    window (None: all keys), position (PartSpec), names (q/k/v/o relative to prefix)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.kv_heads = int(p["kv_heads"])
        self.head_dim = int(p["head_dim"])
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        self.window = int(p["window"]) if p.get("window") else None
        self.position = build_part("position", p["position"], runtime)
        if self.position.rotary_dim > self.head_dim:
            raise ValueError("rotary_dim exceeds head_dim")
        names = p.get("names", {})
        self.q_name = self.prefix + names.get("q", "q_proj.weight")
        self.k_name = self.prefix + names.get("k", "k_proj.weight")
        self.v_name = self.prefix + names.get("v", "v_proj.weight")
        self.o_name = self.prefix + names.get("o", "o_proj.weight")
        self.q_size = self.heads * self.head_dim
        self.kv_size = self.kv_heads * self.head_dim
        self.w_qkv = None
        self.w_o = None
        runtime.kernels.check_attention_shape(self.heads, self.kv_heads, self.head_dim)

    def tensor_decls(self):
        return [
            TensorDecl(self.q_name, (self.q_size, self.hidden)),
            TensorDecl(self.k_name, (self.kv_size, self.hidden)),
            TensorDecl(self.v_name, (self.kv_size, self.hidden)),
            TensorDecl(self.o_name, (self.hidden, self.q_size)),
        ]

    def ignorable_tensors(self):
        return [self.prefix + "rotary_emb.inv_freq"]

    def _adjacent_pairs(self, w: torch.Tensor, n_heads: int) -> torch.Tensor:
        """Rows of a q or k projection reordered inside every head so that the two elements of a rotary pair
        (j, j + rot/2) become neighbours (2j, 2j+1). Scores q.k do not notice a reordering of the head's elements
        that queries and keys share; the rotation can then be done wherever two neighbouring columns meet, e.g. in
        the epilogue of the product. (The reference stores its weights in this order too,
        serve/hf_utils/convert_hf_checkpoint.py:115-118.)"""
        rot, d = self.position.rotary_dim, self.head_dim
        idx = torch.arange(d)
        idx[:rot] = torch.stack([torch.arange(rot // 2), torch.arange(rot // 2) + rot // 2], dim=1).reshape(-1)
        return w.view(n_heads, d, -1)[:, idx.to(w.device)].reshape(n_heads * d, -1)

    def load(self, tensors):
        wq, wk = tensors[self.q_name], tensors[self.k_name]
        self.pairing = self.position.pairing
        if self.position.rotary_dim > 0 and self.position.pairing == PAIRING_HALF:
            wq, wk = self._adjacent_pairs(wq, self.heads), self._adjacent_pairs(wk, self.kv_heads)
            self.pairing = PAIRING_INTERLEAVED
        self.w_qkv = torch.cat([wq, wk, tensors[self.v_name]], dim=0).contiguous()
        self.w_o = tensors[self.o_name].contiguous()

    def cache_need(self):
        return CacheNeed(kv_heads=self.kv_heads, head_dim=self.head_dim, window=self.window)

    def fused_description(self, cache):
        """What a kernel that runs whole layers at once needs to know of this mixer (tensors and constants)."""
        return dict(kind="attention", hidden=self.hidden, heads=self.heads, kv_heads=self.kv_heads, head_dim=self.head_dim,
                    w_qkv=self.w_qkv, w_o=self.w_o, rotary_dim=self.position.rotary_dim, pairing=self.pairing,
                    inv_freq=self.position.inv_freq, scale=self.scale, window=self.window or 0, k=cache.k, v=cache.v,
                    group=cache.group, writes=cache.writes, page_size=cache.page_size)

    def forward(self, h, ctx, cache):
        rt = self.rt
        t = h.shape[0]
        qkv = rt.empty_act((t, self.q_size + 2 * self.kv_size))
        block_table = ctx.block_tables[cache.group]
        rt.kernels.qkv_rope_cache(
            h, self.w_qkv, qkv, ctx.positions, ctx.token_row, self.position.inv_freq, self.pairing,
            self.position.rotary_dim, self.heads, self.kv_heads, self.head_dim,
            cache.k, cache.v, block_table, cache.page_size, cache.writes, memo=getattr(ctx, "memo", None),
        )
        attn = rt.empty_act((t, self.q_size))
        rt.kernels.attention(
            qkv, cache.k, cache.v, block_table, ctx.cu_q, ctx.kv_len, ctx.token_row, ctx.positions,
            self.heads, self.kv_heads, self.head_dim, cache.page_size,
            self.scale, self.window or 0, attn, ctx.shape,
        )
        out = rt.empty_act((t, self.hidden))
        rt.kernels.linear(attn, self.w_o, out)
        return out
