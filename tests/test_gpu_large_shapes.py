"""The engine at the benchmark's layer sizes (Llama-3.2-1B widths, two layers, a smaller vocabulary) against the plain
implementation: only at these sizes do prompt portions run on the tcgen05 kernels (products with >= 96 tiles,
attention at head_dim 64) and decoding on the fused few-rows kernels with their real widths. A second shape has the
head size of the larger models (128: two swizzle atoms per operand row in the tcgen05 attention) and 3 query heads
per key/value head."""
import pytest
import torch

from tests import helpers
from tests.plain.llama_plain import llama_forward

pytestmark = pytest.mark.gpu

CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, num_hidden_layers=2, num_attention_heads=32,
           num_key_value_heads=8, head_dim=64, intermediate_size=8192, vocab_size=8192, rms_norm_eps=1e-5, rope_theta=500000.0,
           rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                             original_max_position_embeddings=8192),
           tie_word_embeddings=True, max_position_embeddings=131072)
CFG128 = dict(CFG, hidden_size=1536, num_attention_heads=12, num_key_value_heads=4, head_dim=128, intermediate_size=8192,
              vocab_size=4096, tie_word_embeddings=False,
              rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=8192))


@pytest.fixture(scope="module", params=["head_dim_64", "head_dim_128"])
def big(tmp_path_factory, request):
    from serve_b200.config import config_from_dict
    from serve_b200.weights import write_random_model

    folder = str(tmp_path_factory.mktemp("big"))
    cfg_dict = CFG if request.param == "head_dim_64" else CFG128
    write_random_model(folder, config_from_dict(cfg_dict), seed=11, std=0.02, norm_std=0.05, dtype=torch.bfloat16)
    cfg, w = helpers.read_folder(folder)
    reqs = {"long": helpers.random_tokens(cfg["vocab_size"], 1600, seed=1), "short": helpers.random_tokens(cfg["vocab_size"], 300, seed=2)}
    with torch.no_grad():
        plain = {rid: llama_forward(w, cfg, toks) for rid, toks in reqs.items()}
    return folder, reqs, plain


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_benchmark_widths_match_plain(big, dtype):
    from serve_b200.config import EngineConfig
    from serve_b200.engine import Engine

    folder, reqs, plain = big
    eng = Engine.from_folder(folder, EngineConfig(dtype=dtype, page_size=64, num_pages=64, max_slots=4, max_tokens_per_step=2048,
                                                  max_context=2048, use_cuda_graphs=True))
    # the long prompt whole (tcgen05 products and attention in bfloat16), then the short one in portions beside
    # decoded tokens of the long one, then both decoding from graphs
    steps = [{"step": 0, "entries": [{"id": "long", "tokens": reqs["long"][:1500], "want": [0, 700, 1499]}], "end": []}]
    at_long, at_short = 1500, 0
    for n in (130, 64, 90, 16):
        take = min(n, 300 - at_short)
        steps.append({"step": len(steps), "entries": [
            {"id": "long", "tokens": [reqs["long"][at_long]], "want": [0]},
            {"id": "short", "tokens": reqs["short"][at_short:at_short + take], "want": [take - 1]}], "end": []})
        at_long += 1
        at_short += take
    assert at_short == 300
    for _ in range(12):
        steps.append({"step": len(steps), "entries": [{"id": "long", "tokens": [reqs["long"][at_long]], "want": [0]}], "end": []})
        at_long += 1
    launches_before = eng.kernels.launches
    library_before = eng.kernels.library_calls
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    eng.kernels.check_errors()
    scale = max(float(p.abs().max()) for p in plain.values())
    helpers.compare_with_plain(got, plain, atol=scale * 2.0 ** -6 if dtype == "bfloat16" else 2e-4)
    if dtype == "bfloat16":
        assert eng.stepper.launched_graphs >= 10
        assert eng.kernels.launches > launches_before
        # the whole-prompt step keeps its fused products (q/k/v with rotation, gate/up with SwiGLU) on this engine's
        # kernels and sends the two plain ones of a layer to the library; the four mixed steps' 17..131-row products are
        # all the library's; decoding steps use none
        layers = CFG["num_hidden_layers"]
        assert 2 * layers <= eng.kernels.library_calls - library_before <= (2 + 4 * 4) * layers


SMALL = dict(CFG, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=512, vocab_size=512)


def test_many_rows_decoding_from_graphs_through_the_tensor_memory_products(tmp_path):
    """Forty requests decode together from CUDA graphs, with every product of more than 32 rows sent to the tcgen05
    kernels (as happens by itself from about nine hundred rows on): the q/k/v product then takes its cosines and sines
    from a table made once per step, and a replayed graph must make that table again for its own positions."""
    from serve_b200.config import EngineConfig, config_from_dict
    from serve_b200.engine import Engine
    from serve_b200.weights import write_random_model

    folder = str(tmp_path)
    write_random_model(folder, config_from_dict(SMALL), seed=3, std=0.05, norm_std=0.1, dtype=torch.bfloat16)
    cfg, w = helpers.read_folder(folder)
    n_req, decoded = 40, 5
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab_size"], 3 + (i * 7) % 23 + decoded, seed=100 + i) for i in range(n_req)}
    with torch.no_grad():
        plain = {rid: llama_forward(w, cfg, toks) for rid, toks in reqs.items()}
    eng = Engine.from_folder(folder, EngineConfig(dtype="bfloat16", page_size=16, num_pages=n_req * 3, max_slots=n_req,
                                                  max_tokens_per_step=1024, max_context=64, use_cuda_graphs=True))
    eng.kernels.TCGEN05_MIN_TILES = 1
    eng.kernels.tcgen05_for_plain_products = True
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": toks[:-decoded], "want": [len(toks) - decoded - 1]} for rid, toks in reqs.items()],
              "end": []}]
    for d in range(decoded):
        steps.append({"step": d + 1, "entries": [{"id": rid, "tokens": [toks[len(toks) - decoded + d]], "want": [0]}
                                                  for rid, toks in reqs.items()], "end": []})
    try:
        with torch.inference_mode():
            got = helpers.replay(eng, steps)
    finally:
        del eng.kernels.TCGEN05_MIN_TILES, eng.kernels.tcgen05_for_plain_products     # (engines share the kernels object)
        eng.kernels._routes.clear()
    eng.kernels.check_errors()
    assert eng.stepper.launched_graphs >= decoded - 1
    scale = max(float(p.abs().max()) for p in plain.values())
    helpers.compare_with_plain(got, plain, atol=scale * 2.0 ** -6)
