"""Makes tests/golden/reference_<name>.npz: logits of limei1221/serve's own model code on CPU.

The reference's LlamaModel, LlamaRMSNorm, LlamaMLP, rotary code and its paged
cache index (serve/model.py, serve/kv_cache_paged.py) import and run on the
CPU; only its four Triton entry points cannot, so this script replaces exactly
those four names with dense torch stand-ins (page writes by loop, softmax
attention over the gathered pages). Weights are the tiny configurations of
tests/helpers.py with values from a fixed integer stream
(``helpers.counted_weights``: the same numbers on every machine), passed
through the reference's own conversion rules
(serve/hf_utils/convert_hf_checkpoint.py:115-118 permute, :156 fuse, :146-147
tie). The run is: prefill of the first 5 tokens (its logits are those of
position 4), then the remaining tokens fed one by one through its decode path.

Usage (needs the reference checkout):  python tests/golden/make_golden.py /path/to/limei1221-serve
tests/test_plain.py compares the plain implementation with the stored outputs.
"""
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from tests import helpers  # noqa: E402


WEIGHT_SEED = 3


def install_standins(M):
    def write_multi(cache, x, seqlens, btd):
        start = 0
        for b, n in enumerate(seqlens.tolist()):
            slot = int(btd.block_table_index[b])
            for h in range(x.shape[1]):
                for p in range(n):
                    cache[btd.block_table[slot, h, p // btd.block_table_size], p % btd.block_table_size] = x[start + p, h]
            start += n

    def write_single(cache, x, seqlens, btd):
        for b, n in enumerate(seqlens.tolist()):
            slot, p = int(btd.block_table_index[b]), n - 1
            for h in range(x.shape[1]):
                cache[btd.block_table[slot, h, p // btd.block_table_size], p % btd.block_table_size] = x[b, h, 0]

    def gather(cache, btd, slot, h, n):
        bs = btd.block_table_size
        return torch.stack([cache[btd.block_table[slot, h, p // bs], p % bs] for p in range(n)])

    def attend(q, kc, vc, btd, slot, n, qpos, g):
        out = torch.empty_like(q)
        for hq in range(q.shape[1]):
            k, v = gather(kc, btd, slot, hq // g, n), gather(vc, btd, slot, hq // g, n)
            s = (q[:, hq] @ k.T) / math.sqrt(q.shape[-1])
            s = s.masked_fill(torch.arange(n)[None, :] > qpos[:, None], float("-inf"))
            out[:, hq] = torch.softmax(s, -1) @ v
        return out

    def prefill(q, kc, vc, btd, seqlens, max_seqlen, cfg):
        g, o, start = cfg.n_heads // cfg.n_kv_heads, torch.empty_like(q), 0
        for b, n in enumerate(seqlens.tolist()):
            o[start:start + n] = attend(q[start:start + n], kc, vc, btd, int(btd.block_table_index[b]), n, torch.arange(n), g)
            start += n
        return o

    def decode(q, kc, vc, btd, seqlens, max_seqlen, cfg):
        g, o = cfg.n_heads // cfg.n_kv_heads, torch.empty_like(q)
        for b, n in enumerate(seqlens.tolist()):
            o[b, :, 0] = attend(q[b, :, 0][None], kc, vc, btd, int(btd.block_table_index[b]), n, torch.tensor([n - 1]), g)[0]
        return o

    M.write_multiple_positions_triton, M.write_single_position_triton = write_multi, write_single
    M.attn_prefill_triton, M.attn_decode_triton = prefill, decode


def run(name, M, KVIndex, page, n_tokens=24, prefill=5):
    cfg = helpers.TINY[name]
    hf = helpers.counted_weights(cfg, WEIGHT_SEED, std=helpers.WEIGHT_STD[name], norm_spread=helpers.NORM_STD[name])
    dim, L, H, Hkv, D = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    inter, V = cfg["intermediate_size"], cfg["vocab_size"]
    assert D == dim // H, "the reference derives head_dim from dim // n_heads"
    scaling = None
    if cfg["rope_scaling"]:
        scaling = {k: cfg["rope_scaling"][k] for k in ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")}
    args = M.ModelArgs(dim=dim, n_layers=L, n_heads=H, n_kv_heads=Hkv, vocab_size=V, multiple_of=1,
                       ffn_dim_multiplier=inter / int(8 * dim / 3), norm_eps=cfg["rms_norm_eps"], rope_base=cfg["rope_theta"],
                       max_seq_len=128, rope_scaling=scaling)
    m = M.LlamaModel(args, torch.float32).eval()
    assert m.layers[0].mlp.w1.weight.shape[0] == inter

    def permute(w, nh):
        return w.view(nh, 2, D // 2, dim).transpose(1, 2).reshape(D * nh, dim)

    sd = {"tok_embeddings.weight": hf["model.embed_tokens.weight"], "norm.weight": hf["model.norm.weight"],
          "output.weight": hf["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else hf["lm_head.weight"]}
    for i in range(L):
        p, r = f"model.layers.{i}.", f"layers.{i}."
        sd[r + "attn.wqkv.weight"] = torch.cat([permute(hf[p + "self_attn.q_proj.weight"], H), permute(hf[p + "self_attn.k_proj.weight"], Hkv),
                                                hf[p + "self_attn.v_proj.weight"]])
        sd[r + "attn.wo.weight"] = hf[p + "self_attn.o_proj.weight"]
        sd[r + "mlp.w1.weight"], sd[r + "mlp.w3.weight"], sd[r + "mlp.w2.weight"] = (
            hf[p + "mlp.gate_proj.weight"], hf[p + "mlp.up_proj.weight"], hf[p + "mlp.down_proj.weight"])
        sd[r + "attention_norm.weight"], sd[r + "ffn_norm.weight"] = hf[p + "input_layernorm.weight"], hf[p + "post_attention_layernorm.weight"]
    m.load_state_dict(sd)
    m.compute_freqs_cis("cpu")
    kv = [(torch.zeros(256, page, D), torch.zeros(256, page, D)) for _ in range(L)]
    ix = KVIndex(256, page, Hkv, L, 128, 4, "cpu")
    toks = helpers.counted_tokens(V, n_tokens, seed=77)
    rows = []
    with torch.no_grad():
        ix.allocate_requests_batched([0], [prefill])
        lg = m(torch.tensor(toks[:prefill]), kv, torch.arange(prefill), torch.tensor([prefill], dtype=torch.int32),
               ix.get_block_table_data([0]), prefill, "prefill")
        rows.append(lg[0])
        for j in range(prefill, n_tokens):
            ix.allocate_requests_batched([0], [j + 1])
            sl = torch.tensor([j + 1], dtype=torch.int32)
            lg = m(torch.tensor([[toks[j]]]), kv, (sl - 1).unsqueeze(1).long(), sl, ix.get_block_table_data([0]), 1, "decode")
            rows.append(lg[0, 0])
    out = os.path.join(HERE, f"reference_{name}.npz")
    np.savez_compressed(out, tokens=np.array(toks), first_position=prefill - 1, logits=torch.stack(rows).numpy(), weight_seed=WEIGHT_SEED,
                        embed_checksum=float(hf["model.embed_tokens.weight"].double().abs().sum()))
    print("wrote", out, torch.stack(rows).shape)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of limei1221/serve>")
    ref = sys.argv[1]
    sys.path.insert(0, ref)
    sys.dont_write_bytecode = True
    import serve.model as M
    from serve.kv_cache_paged import KVCacheIndexPaged

    install_standins(M)
    run("a", M, KVCacheIndexPaged, page=4)
    run("b", M, KVCacheIndexPaged, page=8)
