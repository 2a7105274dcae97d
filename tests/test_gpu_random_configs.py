"""Random configurations of the architecture (head sizes in steps of 16, odd numbers of heads and groups, widths and
vocabularies that are no power of two, with and without llama3 scaling, tied and untied) through the engine, whole,
with a decoded tail and mixed with few pages, against the plain implementation, in 32-bit and in bfloat16. Once as the
engine routes its products by itself and once with every product of more than 32 rows on the tcgen05 kernels, which
small models would otherwise never reach."""
import random

import pytest
import torch

from tests import helpers
from tests.plain.llama_plain import llama_forward

pytestmark = pytest.mark.gpu


def random_config(rng: random.Random) -> dict:
    d = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 160, 192, 256])
    kv = rng.choice([1, 1, 2, 3, 4])
    heads = kv * rng.choice([1, 2, 3, 4, 5, 7, 8])
    hidden = rng.choice([heads * d, 72, 100, 136, 50, 264, 66, 96])
    scaling = None
    if rng.random() < 0.5:
        scaling = dict(rope_type="llama3", factor=rng.choice([2.0, 8.0, 32.0]), low_freq_factor=1.0,
                       high_freq_factor=rng.choice([2.0, 4.0]), original_max_position_embeddings=rng.choice([16, 64, 8192]))
    return dict(architectures=["LlamaForCausalLM"], hidden_size=hidden, num_hidden_layers=rng.choice([1, 2, 3]),
                num_attention_heads=heads, num_key_value_heads=kv, head_dim=d,
                intermediate_size=rng.choice([90, 128, 200, 333, 512, 77]), vocab_size=rng.choice([257, 331, 500, 1000, 2049, 64]),
                rms_norm_eps=rng.choice([1e-5, 1e-6, 3e-4]), rope_theta=rng.choice([10000.0, 500000.0, 1e6]),
                rope_scaling=scaling, tie_word_embeddings=rng.random() < 0.5, max_position_embeddings=4096)


@pytest.mark.parametrize("tensor_memory_products", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [3, 5, 7, 11, 12, 21])
def test_random_configuration(tmp_path, seed, dtype, tensor_memory_products):
    from serve_b200.config import EngineConfig, config_from_dict
    from serve_b200.engine import Engine
    from serve_b200.weights import write_random_model

    if tensor_memory_products and dtype == "float32":
        pytest.skip("the tcgen05 products are bfloat16 kernels")
    rng = random.Random(seed)
    cfg = config_from_dict(random_config(rng))
    folder = str(tmp_path)
    write_random_model(folder, cfg, seed, std=0.05, norm_std=0.1, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    cj, w = helpers.read_folder(folder)
    lens = [rng.choice([3, 17, 64, 65, 130, 200, 257]) for _ in range(5)]
    reqs = {f"r{i}": helpers.random_tokens(cj["vocab_size"], n, seed=seed * 10 + i) for i, n in enumerate(lens)}
    with torch.no_grad():
        plain = {rid: llama_forward(w, cj, t) for rid, t in reqs.items()}
    scale = max(float(p.abs().max()) for p in plain.values())
    atol = 3e-5 * max(1.0, scale) if dtype == "float32" else scale * 2.0 ** -6
    cuts = {"whole": helpers.trace_whole, "tail": helpers.trace_tail_decode, "mixed": lambda r: helpers.trace_mixed(r, live=4, seed=seed)}
    for cut, make in cuts.items():
        steps = make(reqs)
        pages = helpers.tokens_needed(steps, 64) // 64
        eng = Engine.from_folder(folder, EngineConfig(dtype=dtype, page_size=64, num_pages=pages, max_slots=8,
                                                      max_tokens_per_step=max(512, pages * 64), max_context=pages * 64,
                                                      use_cuda_graphs=True))
        if tensor_memory_products:
            eng.kernels.TCGEN05_MIN_TILES = 1
            eng.kernels.tcgen05_for_plain_products = True
        eng.kernels._routes.clear()
        try:
            for v in eng.stepper.views:          # a page that is read before it is written shows
                v.k.fill_(float("nan"))
                v.v.fill_(float("nan"))
            with torch.inference_mode():
                got = helpers.replay(eng, steps)
            eng.kernels.check_errors()
            try:
                helpers.compare_with_plain(got, plain, atol=atol)
            except AssertionError as e:
                raise AssertionError(f"{cut}: {e}") from None
        finally:
            if tensor_memory_products:
                del eng.kernels.TCGEN05_MIN_TILES
                del eng.kernels.tcgen05_for_plain_products
            eng.kernels._routes.clear()
