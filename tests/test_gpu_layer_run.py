"""Decoding steps of at most 16 requests can run all layers in one launch (csrc/decode_stack.cu; off by default, since
the chain of separate kernels measured faster). These tests switch it on and drive that kernel through the engine at sizes it takes (widths that are multiples of 128, head sizes 64 and 128) and compare with
the plain implementation and with the same engine running part by part: batches of 1 to 16, lengths that cross pages
and key splits, a window, a layer that runs twice, untied and tied heads, with and without graphs."""
import pytest
import torch

from tests import helpers
from tests.plain.llama_plain import llama_forward

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["LlamaForCausalLM"], rms_norm_eps=1e-5, rope_theta=500000.0,
            rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                              original_max_position_embeddings=64),
            max_position_embeddings=4096)
CONFIGS = {
    "d64": dict(BASE, hidden_size=256, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                intermediate_size=512, vocab_size=512, tie_word_embeddings=False),
    "d128": dict(BASE, hidden_size=384, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=1, head_dim=128,
                 intermediate_size=640, vocab_size=331, tie_word_embeddings=True, rope_scaling=None, rope_theta=10000.0,
                 rms_norm_eps=3e-6),
    "wide": dict(BASE, hidden_size=2048, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
                 intermediate_size=8192, vocab_size=1024, tie_word_embeddings=True),
}


def _folder(tmp_path_factory, name):
    from serve_b200.config import config_from_dict
    from serve_b200.weights import write_random_model

    folder = str(tmp_path_factory.mktemp(name))
    write_random_model(folder, config_from_dict(CONFIGS[name]), seed=21, std=0.05 if name != "wide" else 0.02, norm_std=0.1,
                       dtype=torch.bfloat16)
    return folder


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: _folder(tmp_path_factory, name) for name in CONFIGS}


def _engine(folder, page, num_pages, slots, graphs, context=4096):
    from serve_b200.config import EngineConfig
    from serve_b200.engine import Engine

    return Engine.from_folder(folder, EngineConfig(dtype="bfloat16", page_size=page, num_pages=num_pages, max_slots=slots,
                                                   max_tokens_per_step=16384, max_context=context, use_cuda_graphs=graphs))


def _decode_trace(reqs, decoded):
    """All prompts in one step, then ``decoded`` steps in which every request brings one token."""
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": t[:-decoded], "want": [len(t) - decoded - 1]} for rid, t in reqs.items()], "end": []}]
    for d in range(decoded):
        steps.append({"step": d + 1, "entries": [{"id": rid, "tokens": [t[len(t) - decoded + d]], "want": [0]} for rid, t in reqs.items()],
                      "end": list(reqs) if d == decoded - 1 else []})
    return steps


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name,page,batch", [("d64", 16, 1), ("d64", 16, 8), ("d64", 64, 9), ("d64", 8, 16), ("d128", 16, 5),
                                             ("d128", 32, 13), ("wide", 64, 8), ("wide", 64, 16)])
def test_layer_run_equals_plain_and_the_parts(folders, name, page, batch, graphs):
    folder = folders[name]
    cfg, w = helpers.read_folder(folder)
    decoded = 6
    lengths = [3 + (i * 97) % 700 + decoded for i in range(batch)]
    lengths[0] = 1030 + decoded                               # one long request: several key splits at small batches
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab_size"], n, seed=300 + i) for i, n in enumerate(lengths)}
    torch.backends.cuda.matmul.allow_tf32 = False
    wd = {k: v.to("cuda:0") for k, v in w.items()}
    with torch.no_grad():
        plain = {rid: llama_forward(wd, cfg, t, device="cuda:0").cpu() for rid, t in reqs.items()}
    del wd
    steps = _decode_trace(reqs, decoded)
    pages = sum(-(-n // page) for n in lengths) + 2
    got = {}
    for fused in (True, False):
        eng = _engine(folder, page, pages, batch, graphs)
        eng.kernels.use_layer_runs = fused
        for view in eng.stepper.views:
            view.k.fill_(float("nan"))
            view.v.fill_(float("nan"))
        before = eng.kernels.layer_runs
        try:
            with torch.inference_mode():
                got[fused] = helpers.replay(eng, steps)
            eng.kernels.check_errors()
        finally:
            eng.kernels.use_layer_runs = False
        ran = eng.kernels.layer_runs - before
        assert (ran > 0) == fused, "decoding steps of up to 16 requests go through the one-launch kernel, and only when it is on"
        if fused and graphs:
            assert eng.stepper.launched_graphs >= decoded - 1
    scale = max(float(p.abs().max()) for p in plain.values())
    helpers.compare_with_plain(got[True], plain, atol=scale * 2.0 ** -6)
    helpers.compare_with_plain(got[False], plain, atol=scale * 2.0 ** -6)
    # against the same engine part by part: the same rounding points, but sums in another order, so a value near the
    # middle between two bfloat16 numbers may round the other way; the two lie as close to one another as each to plain
    worst = max(float((got[True][k] - got[False][k]).abs().max()) for k in got[True])
    assert worst <= scale * 2.0 ** -6, f"one launch against part by part: {worst:.3e} at logit scale {scale:.2f}"


def test_layer_run_with_a_window_a_repeated_layer_and_reused_pages(folders):
    """A model described by hand: layer 0 with a window of 100 keys, layer 1 with all keys, layer 0 once more (its own
    cache): two cache groups in one launch. Requests come and go, so pages are used again."""
    from serve_b200.config import EngineConfig, ModelSpec, PartSpec, ScheduleEntry, config_from_dict
    from serve_b200.config.base import build_spec
    from serve_b200.engine import Engine

    folder = folders["d64"]
    cfg, w = helpers.read_folder(folder)
    spec = build_spec(config_from_dict(CONFIGS["d64"]))
    layers = list(spec.layers[:2])
    parts0 = dict(layers[0].parts)
    parts0["mixer"] = PartSpec("attention", dict(parts0["mixer"].params, window=100), prefix=parts0["mixer"].prefix)
    layers[0] = type(layers[0])(layers[0].block, parts0)
    spec2 = ModelSpec(spec.architecture, spec.hidden_size, spec.vocab_size, spec.embedding, layers,
                      [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)], spec.final_norm, spec.head, spec.max_position)

    def plain_forward(tokens):
        # layer 0 (window 100), layer 1, layer 0 again: the plain implementation takes a schedule and one window for all
        # layers, so the two kinds of layer are put together here from its parts
        from tests.plain import llama_plain as P

        c = P.normalise_config(cfg)
        x = w["model.embed_tokens.weight"][torch.tensor(tokens)]
        pos = torch.arange(len(tokens))
        inv = P.rope_inv_freq(c["head_dim"], c["rope_theta"], c["rope_scaling"])
        for layer, window in ((0, 100), (1, None), (0, 100)):
            p = f"model.layers.{layer}."
            a, _ = P.attention_layer(P.rms_norm(x, w[p + "input_layernorm.weight"], c["rms_norm_eps"]), w, p + "self_attn.", c, pos, inv, window)
            x = x + a
            x = x + P.swiglu(P.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["rms_norm_eps"]), w[p + "mlp.gate_proj.weight"],
                             w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        return P.rms_norm(x, w["model.norm.weight"], c["rms_norm_eps"]) @ w["lm_head.weight"].T

    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab_size"], n, seed=700 + i) for i, n in enumerate([260, 40, 131, 90, 17, 200])}
    with torch.no_grad():
        plain = {rid: plain_forward(t) for rid, t in reqs.items()}
    steps = helpers.trace_mixed(reqs, live=3, seed=11, decode_tail=60, budget=300)
    eng = Engine(config_from_dict(CONFIGS["d64"]), EngineConfig(dtype="bfloat16", page_size=16, num_pages=40, max_slots=4,
                                                                max_tokens_per_step=512, max_context=512, use_cuda_graphs=True), spec=spec2)
    from serve_b200.weights.loader import load_from_source

    # (the folder holds a third layer that this model does not have: the tensors are handed over by name instead)
    load_from_source(eng.model, lambda d: w[d.name], eng.dtype, eng.rt.device)
    eng._make_cache()
    assert len(eng.cache.groups) == 2
    eng.kernels.use_layer_runs = True
    try:
        with torch.inference_mode():
            got = helpers.replay(eng, steps)
        eng.kernels.check_errors()
    finally:
        eng.kernels.use_layer_runs = False
    assert eng.kernels.layer_runs > 50
    scale = max(float(p.abs().max()) for p in plain.values())
    helpers.compare_with_plain(got, plain, atol=scale * 2.0 ** -6)
    eng.cache.check()
    assert eng.cache.live == 0
