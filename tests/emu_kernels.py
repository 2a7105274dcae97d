"""Plain torch versions of every kernel, with the call signatures of ``CudaKernels``.

Two uses, both in tests only: (1) the reference each CUDA kernel is compared
with on the GPU; (2) a stand-in that lets the step function, the cache manager
and the scheduler be exercised on a machine without a GPU. It is not a product
path: the engine itself has no CPU fallback. All arithmetic is float32 (float64
if asked), outputs are rounded once to the output tensor's dtype.
"""
from __future__ import annotations

import torch


class EmuKernels:
    def __init__(self, device="cpu", math_dtype=torch.float32):
        self.device = torch.device(device)
        self.math = math_dtype
        self.launches = 0

    @staticmethod
    def check_attention_shape(heads, kv_heads, head_dim):
        if head_dim % 2 or heads % kv_heads:
            raise ValueError("bad attention shape")

    def check_errors(self):
        return None

    def on_current_stream(self):
        import contextlib

        return contextlib.nullcontext()

    def fetch_ints(self, host, dev, n):
        dev.view(-1)[:n].copy_(host.view(-1)[:n])

    def embedding(self, tokens, table, out, last_token=None):
        ids = tokens.long()
        if last_token is not None:
            neg = ids < 0
            ids = torch.where(neg, last_token.long()[(-ids - 1).clamp(min=0)], ids)
        out.copy_(table[ids].to(out.dtype))

    def _norm(self, v, weight, eps):
        v = v.to(self.math)
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight.to(self.math)

    def add_rmsnorm(self, x, delta, weight, eps, out):
        if delta is not None:
            x.add_(delta.to(x.dtype))
        out.copy_(self._norm(x, weight, eps).to(out.dtype))

    def add_rmsnorm_rows(self, x, delta, rows, weight, eps, out):
        v = x[rows.long()]
        if delta is not None:
            v = v + delta[rows.long()].to(x.dtype)
        out.copy_(self._norm(v, weight, eps).to(out.dtype))

    def linear(self, a, w, out):
        out.copy_((a.to(self.math) @ w.to(self.math).T).to(out.dtype))

    def swiglu(self, gate_up, out):
        inter = out.shape[1]
        g = gate_up[:, :inter].to(self.math)
        u = gate_up[:, inter:].to(self.math)
        out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))

    def gate_up_swiglu(self, h, w_gate_up, out):
        gate_up = torch.empty((h.shape[0], w_gate_up.shape[0]), dtype=h.dtype, device=h.device)
        self.linear(h, w_gate_up, gate_up)
        self.swiglu(gate_up, out)

    def qkv_rope_cache(self, h, w_qkv, qkv, positions, token_row, inv_freq, pairing, rotary_dim, heads, kv_heads, head_dim,
                       k_cache, v_cache, block_table, page_size, write_cache, memo=None):
        self.linear(h, w_qkv, qkv)
        self.rope_cache_write(qkv, positions, token_row, inv_freq, pairing, rotary_dim, heads, kv_heads, head_dim,
                              k_cache, v_cache, block_table, page_size, write_cache)

    def rope_cache_write(self, qkv, positions, token_row, inv_freq, pairing, rotary_dim, heads, kv_heads, head_dim,
                         k_cache, v_cache, block_table, page_size, write_cache):
        t = qkv.shape[0]
        d = head_dim
        x = qkv.view(t, heads + 2 * kv_heads, d)
        qk = x[:, : heads + kv_heads].to(self.math)
        if rotary_dim > 0:
            ang = positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, : rotary_dim // 2]
            cos, sin = ang.cos().to(self.math)[:, None, :], ang.sin().to(self.math)[:, None, :]
            if pairing == 0:
                a, b = qk[..., : rotary_dim // 2], qk[..., rotary_dim // 2: rotary_dim]
                rot = torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
            else:
                a, b = qk[..., 0:rotary_dim:2], qk[..., 1:rotary_dim:2]
                rot = torch.stack([a * cos - b * sin, b * cos + a * sin], -1).flatten(-2)
            qk = torch.cat([rot, qk[..., rotary_dim:]], -1)
        qk = qk.to(qkv.dtype)
        x[:, :heads] = qk[:, :heads]
        if write_cache:
            pos = positions.long()
            pages = block_table.long()[token_row.long(), pos // page_size]
            assert bool((pages >= 0).all()), "cache write to a missing page"
            k_cache[pages, :, pos % page_size] = qk[:, heads:]          # caches are [pages, kv_heads, page_size, D]
            v_cache[pages, :, pos % page_size] = x[:, heads + kv_heads:]

    def attention(self, qkv, k_cache, v_cache, block_table, cu_q, kv_len, token_row, positions, heads, kv_heads, head_dim,
                  page_size, scale, window, out, shape):
        d = head_dim
        g = heads // kv_heads
        cu = cu_q.tolist()
        lens = kv_len.tolist()
        for r in range(len(lens)):
            q0, q1 = cu[r], cu[r + 1]
            n, L = q1 - q0, lens[r]
            if n == 0:
                continue
            q = qkv[q0:q1, : heads * d].view(n, heads, d).to(self.math)
            key_pos = torch.arange(L, device=qkv.device)
            lo = max(0, (L - n) - window + 1) if window else 0
            pages = block_table[r].long()[key_pos[lo:] // page_size]
            assert bool((pages >= 0).all()), "attention reads a missing page"
            k = k_cache[pages, :, key_pos[lo:] % page_size].to(self.math)
            v = v_cache[pages, :, key_pos[lo:] % page_size].to(self.math)
            kk, vv = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
            s = torch.einsum("thd,shd->hts", q, kk) * scale
            qp = torch.arange(L - n, L, device=qkv.device)[:, None]
            kp = key_pos[lo:][None, :]
            mask = kp > qp
            if window:
                mask = mask | (kp <= qp - window)
            s = s.masked_fill(mask[None], float("-inf"))
            o = torch.einsum("hts,shd->thd", torch.softmax(s, -1), vv)
            out[q0:q1] = o.reshape(n, heads * d).to(out.dtype)

    def sample(self, logits, temperature, req_ids, tok_index, seed, out, slots=None, last_token=None):
        from tests.plain.llama_plain import sample_token

        for r in range(logits.shape[0]):
            out[r] = sample_token(logits[r], float(temperature[r]), seed, int(req_ids[r]), int(tok_index[r]))
            if slots is not None and last_token is not None:
                last_token[int(slots[r])] = out[r]
