"""Makes tests/golden/reference_gpu_<dtype>.npz: logits of limei1221/serve's own, unmodified code on a GPU.

Unlike make_golden.py nothing is replaced here: the reference's model
(serve/model.py), its paged cache index (serve/kv_cache_paged.py), its Triton
kernels for cache writes, prompt attention and decoding attention
(serve/kernels/*.py) and its ``prefill`` / ``decode_one_token`` functions
(serve/run.py:109-209) run as they are. So these files pin what its attention
kernels compute (scale, causal mask, head mapping, paging), which the CPU
golden files cannot.

The model is the small shape ``helpers.GOLDEN_GPU`` (pages of 64 and head_dim
64, which the reference's kernels take), with weights and prompts from a fixed
integer stream (``helpers.counted_weights``), so the test can make the same
numbers again on any machine. Weights pass through the reference's conversion
rules (serve/hf_utils/convert_hf_checkpoint.py:115-118 permute, :156 fuse).
The run: one prefill step of three prompts (5, 60 and 130 tokens; the logits
of each prompt's last token), then eight greedy decode steps of all three (the
second request grows across a page edge). Stored: prompts, generated tokens,
logits [3 requests, 9 rows, vocabulary] as float32.

Usage (on a machine with a GPU and Triton):
    python tests/golden/make_golden_gpu.py <folder that holds the reference's serve/ package> [out folder]
tests/test_plain.py compares the plain implementation with the stored outputs.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from tests import helpers  # noqa: E402

PROMPT_LENGTHS = (5, 60, 130)
DECODE_STEPS = 8
WEIGHT_SEED = 11


def reference_state_dict(cfg, hf):
    dim, L, H, Hkv, D = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

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
    return sd


def run(dtype, out_dir):
    import serve.model as M
    import serve.run as R
    from serve.kv_cache_paged import setup_kv_cache_paged

    cfg = helpers.GOLDEN_GPU
    hf = helpers.counted_weights(cfg, WEIGHT_SEED)
    if dtype == torch.bfloat16:
        hf = {k: v.to(torch.bfloat16).float() for k, v in hf.items()}
    dim, H, inter = cfg["hidden_size"], cfg["num_attention_heads"], cfg["intermediate_size"]
    sc = cfg["rope_scaling"]
    args = M.ModelArgs(dim=dim, n_layers=cfg["num_hidden_layers"], n_heads=H, n_kv_heads=cfg["num_key_value_heads"],
                       vocab_size=cfg["vocab_size"], multiple_of=1, ffn_dim_multiplier=inter / int(8 * dim / 3),
                       norm_eps=cfg["rms_norm_eps"], rope_base=cfg["rope_theta"], max_seq_len=cfg["max_position_embeddings"],
                       rope_scaling={k: sc[k] for k in ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")})
    model = M.LlamaModel(args, dtype).eval()
    assert model.layers[0].mlp.w1.weight.shape[0] == inter
    model.load_state_dict(reference_state_dict(cfg, hf))
    model = model.to(device="cuda", dtype=dtype)
    model.compute_freqs_cis("cuda")
    kv_caches, kv_ix = setup_kv_cache_paged(64, 64, args.n_layers, args.n_kv_heads, cfg["head_dim"], dtype, "cuda",
                                            args.max_seq_len, 8)
    for k, v in kv_caches:
        k.fill_(float("nan"))        # a page read before it is written would show
        v.fill_(float("nan"))
    prompts = [helpers.counted_tokens(cfg["vocab_size"], n, seed=100 + i) for i, n in enumerate(PROMPT_LENGTHS)]
    reqs = [R.RequestData(request_id=i, input_ids=torch.tensor(p, dtype=torch.long), generated_tokens=[], input_length=len(p),
                          max_new_tokens=DECODE_STEPS + 1) for i, p in enumerate(prompts)]
    rows = []
    with torch.inference_mode():
        rows.append(R.prefill(model, reqs, kv_caches, kv_ix, 0.0).float().cpu())                  # [3, V]
        for _ in range(DECODE_STEPS):
            rows.append(R.decode_one_token(model, reqs, kv_caches, kv_ix, 0.0)[:, 0].float().cpu())   # [3, V]
    logits = torch.stack(rows, dim=1).numpy()                                                      # [3, 9, V]
    assert np.isfinite(logits).all()
    name = "float32" if dtype == torch.float32 else "bfloat16"
    out = os.path.join(out_dir, f"reference_gpu_{name}.npz")
    np.savez_compressed(out, prompt_lengths=np.array(PROMPT_LENGTHS), weight_seed=WEIGHT_SEED,
                        prompts=np.concatenate([np.array(p) for p in prompts]),
                        generated=np.array([r.generated_tokens for r in reqs]), logits=logits,
                        embed_checksum=float(hf["model.embed_tokens.weight"].double().abs().sum()),
                        made_with=f"torch {torch.__version__}, {torch.cuda.get_device_name(0)}")
    print("wrote", out, logits.shape, "generated", [r.generated_tokens for r in reqs])


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        sys.exit("usage: python tests/golden/make_golden_gpu.py <folder holding the reference's serve/ package> [out folder]")
    sys.path.insert(0, sys.argv[1])
    sys.dont_write_bytecode = True
    out_dir = sys.argv[2] if len(sys.argv) == 3 else HERE
    os.makedirs(out_dir, exist_ok=True)
    run(torch.float32, out_dir)
    run(torch.bfloat16, out_dir)
