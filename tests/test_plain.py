"""The plain implementation itself: each part against a closed form, the whole against the stored
outputs of the reference's own model code (tests/golden/), and the sampler's counter-based draws."""
import math
import os

import numpy as np
import pytest
import torch

from tests import helpers
from tests.plain import llama_plain as P

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["a", "b"])
def test_whole_model_equals_the_reference_code(name):
    g = np.load(os.path.join(GOLDEN, f"reference_{name}.npz"))
    cfg = helpers.TINY[name]
    w = helpers.counted_weights(cfg, int(g["weight_seed"]), std=helpers.WEIGHT_STD[name], norm_spread=helpers.NORM_STD[name])
    assert abs(float(w["model.embed_tokens.weight"].double().abs().sum()) - float(g["embed_checksum"])) < 1e-6, \
        "the weights are not the ones the golden file was made with"
    logits = P.llama_forward(w, cfg, g["tokens"].tolist())
    first = int(g["first_position"])
    ref = torch.from_numpy(g["logits"])
    assert ref.shape[0] == logits.shape[0] - first
    torch.testing.assert_close(logits[first:], ref, atol=3e-6, rtol=0)


def golden_gpu_case(dtype_name):
    """(config, weights, [(prompt, generated tokens, reference logits [9, V])]) of tests/golden/reference_gpu_<dtype>.npz."""
    g = np.load(os.path.join(GOLDEN, f"reference_gpu_{dtype_name}.npz"))      # a missing file fails the test
    cfg = helpers.GOLDEN_GPU
    w = helpers.counted_weights(cfg, int(g["weight_seed"]))
    if dtype_name == "bfloat16":
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    assert abs(float(w["model.embed_tokens.weight"].double().abs().sum()) - float(g["embed_checksum"])) < 1e-6, \
        "the counted weights are not the ones the golden file was made with"
    lengths = g["prompt_lengths"].tolist()
    prompts = np.split(g["prompts"], np.cumsum(lengths)[:-1])
    return cfg, w, [(p.tolist(), gen.tolist(), torch.from_numpy(lg)) for p, gen, lg in zip(prompts, g["generated"], g["logits"])]


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
def test_whole_model_equals_the_reference_run_on_a_gpu(dtype_name):
    """The reference's unmodified code, its Triton attention and cache-write kernels included, ran on a B200
    (tests/golden/make_golden_gpu.py): a prefill step of three prompts, then eight greedy decode steps. The plain
    implementation, fed the same tokens, must give the same logits: within the TF32 rounding of the reference's
    products of scores and values in its 32-bit run (2e-3 of the logit scale), within bfloat16 rounding (2^-6 of the
    scale; the reference's own test allows 2e-2 on logits of size one, test/test_model.py:90) in its bfloat16 run.
    Every greedy token of the reference is the plain implementation's argmax too."""
    cfg, w, cases = golden_gpu_case(dtype_name)
    for prompt, generated, ref in cases:
        logits = P.llama_forward(w, cfg, prompt + generated[:-1])[len(prompt) - 1:]
        assert logits.shape == ref.shape
        scale = float(ref.abs().max())
        atol = scale * (2e-3 if dtype_name == "float32" else 2.0 ** -6)
        torch.testing.assert_close(logits, ref, atol=atol, rtol=0)
        assert logits.argmax(-1).tolist() == generated


def test_rms_norm_closed_form():
    x = torch.tensor([[3.0, -4.0, 0.0, 0.0]])
    y = P.rms_norm(x, torch.tensor([1.0, 2.0, 1.0, 1.0]), 0.0)
    torch.testing.assert_close(y, torch.tensor([[3 / 2.5, -8 / 2.5, 0.0, 0.0]]))
    assert float(P.rms_norm(torch.zeros(1, 4), torch.ones(4), 1e-6).abs().max()) == 0.0


def test_swiglu_closed_form():
    x = torch.tensor([[1.0, 2.0]])
    gate, up, down = torch.tensor([[1.0, 0.0], [0.0, 1.0]]), torch.tensor([[2.0, 0.0], [0.0, 3.0]]), torch.tensor([[1.0, 1.0]])
    want = 1 / (1 + math.exp(-1)) * 2 + 2 / (1 + math.exp(-2)) * 6
    torch.testing.assert_close(P.swiglu(x, gate, up, down), torch.tensor([[want]]))


def test_rotation_properties():
    inv = P.rope_inv_freq(8, 10000.0, None)
    torch.testing.assert_close(inv, torch.tensor([1.0, 0.1, 0.01, 0.001]))
    x = torch.randn(5, 2, 8)
    pos = torch.arange(5)
    y = P.rotate(x, pos, inv)
    torch.testing.assert_close(y[0], x[0])                                       # position 0: no rotation
    torch.testing.assert_close(y.norm(dim=-1), x.norm(dim=-1))                    # rotations keep lengths
    # the score of a rotated pair depends on the distance only
    q, k = torch.randn(1, 1, 8), torch.randn(1, 1, 8)
    s = lambda a, b: float((P.rotate(q, torch.tensor([a]), inv) * P.rotate(k, torch.tensor([b]), inv)).sum())
    assert abs(s(7, 3) - s(104, 100)) < 1e-4


def test_llama3_scaling_branches():
    sc = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=64)
    base = P.rope_inv_freq(32, 500000.0, None)
    inv = P.rope_inv_freq(32, 500000.0, sc)
    wavelen = 2 * math.pi / base
    assert torch.equal(inv[wavelen < 16], base[wavelen < 16])                     # short waves kept
    torch.testing.assert_close(inv[wavelen > 64], base[wavelen > 64] / 8)         # long waves slowed by the factor
    mid = (wavelen >= 16) & (wavelen <= 64)
    assert mid.any() and bool(((inv[mid] < base[mid]) & (inv[mid] > base[mid] / 8)).all())


def test_attention_masks():
    torch.manual_seed(0)
    q, k, v = torch.randn(4, 2, 8), torch.randn(4, 1, 8), torch.randn(4, 1, 8)
    out = P.causal_attention(q, k, v, 0.5)
    torch.testing.assert_close(out[0], v[0].expand(2, 8))                         # the first token sees only itself
    k2, v2 = k.clone(), v.clone()
    k2[3], v2[3] = 100.0, -100.0                                                   # the future must not matter
    torch.testing.assert_close(P.causal_attention(q, k2, v2, 0.5)[:3], out[:3])
    w = P.causal_attention(q, k, v, 0.5, window=1)
    torch.testing.assert_close(w, v.expand(4, 2, 8))                               # window 1: each token sees itself
    # queries at given positions against a longer history equal the tail of the whole computation
    tail = P.causal_attention(q[2:], k, v, 0.5)
    torch.testing.assert_close(tail, out[2:])


def test_counter_uniforms_are_uniform_and_keyed():
    u = P.counter_uniforms(1, 2, 3, 200_000)
    assert u.min() > 0 and u.max() < 1 and abs(float(u.mean()) - 0.5) < 5e-3
    hist = np.histogram(u, bins=20, range=(0, 1))[0]
    assert hist.min() > 9_000 and hist.max() < 11_000
    assert not np.array_equal(u[:100], P.counter_uniforms(1, 2, 4, 100))
    assert not np.array_equal(u[:100], P.counter_uniforms(1, 3, 3, 100))
    assert not np.array_equal(u[:100], P.counter_uniforms(2, 2, 3, 100))
    assert np.array_equal(u[:100], P.counter_uniforms(1, 2, 3, 100))


def test_sampling_follows_the_softmax():
    logits = torch.tensor([0.0, 1.0, 2.0, -1.0])
    assert P.sample_token(logits, 0.0) == 2
    counts = np.zeros(4)
    for t in range(4000):
        counts[P.sample_token(logits, 0.7, seed=9, req=1, tok=t)] += 1
    want = torch.softmax(logits / 0.7, -1).numpy()
    assert np.abs(counts / 4000 - want).max() < 0.03
