"""A context of several thousand tokens (a hundred pages, split keys in decoding, many key tiles per query tile in the
prompt kernels): the same sequence whole, in portions, and with its tail decoded token by token from CUDA graphs,
against the plain implementation, in 32-bit and in bfloat16. One key far back is made to stand out for the last
queries, so that a fault in a far page or split shows."""
import pytest
import torch

from tests import helpers
from tests.plain.llama_plain import llama_forward

pytestmark = pytest.mark.gpu

CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=64, intermediate_size=512, vocab_size=512, rms_norm_eps=1e-5, rope_theta=500000.0,
           rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                             original_max_position_embeddings=8192),
           tie_word_embeddings=True, max_position_embeddings=131072)
LENGTH, TAIL = 5000, 24


@pytest.fixture(scope="module")
def long_model(tmp_path_factory):
    from serve_b200.config import config_from_dict
    from serve_b200.weights import write_random_model

    folder = str(tmp_path_factory.mktemp("long"))
    write_random_model(folder, config_from_dict(CFG), seed=5, std=0.05, norm_std=0.1, dtype=torch.bfloat16)
    cfg, w = helpers.read_folder(folder)
    toks = helpers.random_tokens(cfg["vocab_size"], LENGTH, seed=9)
    toks[137] = toks[LENGTH - 1]          # the same token far back and at the end: its key matches the last query best
    with torch.no_grad():
        plain = llama_forward(w, cfg, toks)
    return folder, toks, plain


def _engine(folder, dtype, budget, graphs):
    from serve_b200.config import EngineConfig
    from serve_b200.engine import Engine

    return Engine.from_folder(folder, EngineConfig(dtype=dtype, page_size=64, num_pages=-(-LENGTH // 64) + 1, max_slots=2,
                                                   max_tokens_per_step=budget, max_context=LENGTH + 64, use_cuda_graphs=graphs))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_sequence_whole_in_portions_and_decoded(long_model, dtype):
    folder, toks, plain = long_model
    want = list(range(LENGTH - TAIL, LENGTH)) + [0, 63, 64, 137, 2047, 2048, 4095, 4096]
    scale = float(plain.abs().max())
    atol = scale * 2.0 ** -6 if dtype == "bfloat16" else 3e-4
    results = {}
    # whole, in one step
    eng = _engine(folder, dtype, LENGTH, False)
    with torch.inference_mode():
        results["whole"] = helpers.replay(eng, [{"step": 0, "entries": [{"id": "s", "tokens": toks, "want": sorted(want)}], "end": ["s"]}])
    eng.kernels.check_errors()
    # portions of changing size, then the tail token by token (graphs)
    eng = _engine(folder, dtype, 1024, True)
    steps, at, sizes, k = [], 0, [1000, 64, 333, 1024, 2, 700], 0
    while at < LENGTH - TAIL:
        n = min(sizes[k % len(sizes)], LENGTH - TAIL - at)
        k += 1
        steps.append({"step": len(steps), "entries": [{"id": "s", "tokens": toks[at:at + n], "want": [w - at for w in want if at <= w < at + n]}], "end": []})
        at += n
    for j in range(LENGTH - TAIL, LENGTH):
        steps.append({"step": len(steps), "entries": [{"id": "s", "tokens": [toks[j]], "want": [0]}], "end": ["s"] if j == LENGTH - 1 else []})
    with torch.inference_mode():
        results["cut"] = helpers.replay(eng, steps)
    eng.kernels.check_errors()
    if dtype == "bfloat16":
        assert eng.stepper.launched_graphs >= TAIL - 2
    for name, got in results.items():
        assert len(got) == len(want), name
        helpers.compare_with_plain(got, {"s": plain}, atol=atol)
    # the two ways agree with each other more closely than either needs to agree with plain
    worst = max(float((results["whole"][key] - results["cut"][key]).abs().max()) for key in results["whole"])
    assert worst <= atol
