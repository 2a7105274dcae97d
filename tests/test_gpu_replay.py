"""The engine on the GPU against the plain implementation, under every way of cutting the work,
in 32-bit and in bfloat16, for three tiny configurations."""
import pytest
import torch

from tests import helpers
from tests.plain.llama_plain import llama_forward

pytestmark = pytest.mark.gpu

LENGTHS = {"a": [5, 9, 13, 70, 100], "b": [1, 17, 40, 70, 129, 52], "c": [3, 64, 65, 37, 90, 128]}
PAGE = {"a": 4, "b": 8, "c": 16}
# float32: every reduction is float32, so differences are rounding of sums of a few hundred terms.
# bfloat16: activations are rounded to 8 bits of mantissa (2^-9 relative) several times a layer; logits of
# these models are of size ~1, and the bound below is 2^-6 of the largest logit of the sequence.
F32_ATOL = 3e-5


def _tolerance(dtype, plain):
    if dtype == "float32":
        return F32_ATOL
    scale = max(float(p.abs().max()) for p in plain.values())
    return scale * 2.0 ** -6


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name in ("a", "b", "c"):
        for dtype in ("float32", "bfloat16"):
            folder = helpers.make_folder(str(tmp_path_factory.mktemp(f"{name}-{dtype}")), name, seed=3,
                                         dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
            cfg, w = helpers.read_folder(folder)
            reqs = {f"r{i}": helpers.random_tokens(cfg["vocab_size"], n, seed=10 + i) for i, n in enumerate(LENGTHS[name])}
            plain = {rid: llama_forward(w, cfg, toks) for rid, toks in reqs.items()}
            out[(name, dtype)] = (folder, reqs, plain)
    return out


def _engine(folder, dtype, page, num_pages, graphs=False):
    from serve_b200.config import EngineConfig
    from serve_b200.engine import Engine

    ec = EngineConfig(dtype=dtype, page_size=page, num_pages=num_pages, max_slots=4, max_tokens_per_step=512,
                      max_context=256, use_cuda_graphs=graphs)
    return Engine.from_folder(folder, ec)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions"])
def test_cuts_match_plain(models, name, dtype, cut):
    folder, reqs, plain = models[(name, dtype)]
    page = PAGE[name]
    eng = _engine(folder, dtype, page, num_pages=-(-4 * 160 // page), graphs=(cut == "tail_decode"))
    make = {"whole": helpers.trace_whole, "tail_decode": helpers.trace_tail_decode, "portions": helpers.trace_portions}[cut]
    with torch.inference_mode():
        got = helpers.replay(eng, make(reqs))
    eng.kernels.check_errors()
    assert len(got) == sum(len(t) for t in reqs.values())
    helpers.compare_with_plain(got, plain, atol=_tolerance(dtype, plain))
    eng.cache.check()
    assert eng.cache.live == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_mixed_batches_with_reused_pages(models, name, dtype):
    folder, reqs, plain = models[(name, dtype)]
    page = PAGE[name]
    steps = helpers.trace_mixed(reqs, live=4, seed=5)
    need = helpers.tokens_needed(steps, page) // page
    assert need < sum(-(-len(t) // page) for t in reqs.values())
    eng = _engine(folder, dtype, page, num_pages=need)
    # freed pages keep what they held; poison the pool first so that a read of a page never written shows
    for view in eng.stepper.views:
        view.k.fill_(float("nan"))
        view.v.fill_(float("nan"))
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    eng.kernels.check_errors()
    helpers.compare_with_plain(got, plain, atol=_tolerance(dtype, plain))
    assert eng.cache.groups[0].pool.high_water == need
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_graphs(models, dtype):
    """200 tokens one by one after a short prompt, two requests side by side, replayed from CUDA graphs."""
    folder, reqs, plain = models[("b", dtype)]
    cfg, w = helpers.read_folder(folder)
    seqs = {f"d{i}": helpers.random_tokens(cfg["vocab_size"], 230, seed=40 + i) for i in range(2)}
    plain = {rid: llama_forward(w, cfg, toks) for rid, toks in seqs.items()}
    eng = _engine(folder, dtype, 8, num_pages=64, graphs=True)
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": t[:30 - 7 * i], "want": [29 - 7 * i]} for i, (rid, t) in enumerate(seqs.items())], "end": []}]
    at = {rid: 30 - 7 * i for i, rid in enumerate(seqs)}
    while any(at[rid] < 230 for rid in seqs):
        entries = []
        for rid, t in seqs.items():
            if at[rid] < 230:
                entries.append({"id": rid, "tokens": [t[at[rid]]], "want": [0]})
                at[rid] += 1
        steps.append({"step": len(steps), "entries": entries, "end": []})
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    eng.kernels.check_errors()
    assert eng.stepper.launched_graphs > 150
    helpers.compare_with_plain(got, plain, atol=_tolerance(dtype, plain))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens(models, dtype):
    """Position 0 alone, then position 1 alone: the smallest caches there are."""
    folder, reqs, plain = models[("c", dtype)]
    eng = _engine(folder, dtype, 16, num_pages=8)
    toks = reqs["r1"]
    steps = [{"step": i, "entries": [{"id": "f", "tokens": [toks[i]], "want": [0]}], "end": []} for i in range(3)]
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    helpers.compare_with_plain(got, {"f": plain["r1"]}, atol=_tolerance(dtype, plain))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page", [("b", 24), ("c", 48), ("b", 128), ("c", 3)])
def test_page_sizes_that_are_no_power_of_two_or_exceed_a_tile(models, name, dtype, page):
    """Pages of 24, 48 and 3 tokens (a tile of keys then crosses pages at odd places, and the page index is a
    division, not a shift) and of 128 (larger than a tile): mixed batches with reused pages, and decoded tails from graphs."""
    folder, reqs, plain = models[(name, dtype)]
    steps = helpers.trace_mixed(reqs, live=4, seed=7)
    need = helpers.tokens_needed(steps, page) // page
    eng = _engine(folder, dtype, page, num_pages=need)
    for view in eng.stepper.views:
        view.k.fill_(float("nan"))
        view.v.fill_(float("nan"))
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    eng.kernels.check_errors()
    helpers.compare_with_plain(got, plain, atol=_tolerance(dtype, plain))
    eng.cache.check()
    eng = _engine(folder, dtype, page, num_pages=-(-4 * 256 // page), graphs=True)
    with torch.inference_mode():
        got = helpers.replay(eng, helpers.trace_tail_decode(reqs, tail=20))
    eng.kernels.check_errors()
    helpers.compare_with_plain(got, plain, atol=_tolerance(dtype, plain))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_more_than_five_hundred_requests_decode_together(tmp_path, dtype):
    """530 live requests: their prompts come in over a few mixed steps, then all decode together for four steps. That is
    more rows than decoding graphs are kept for, so the steps launch kernel by kernel, and in bfloat16 more than a
    thousand (request, kv head) pairs, which the decoding attention runs one warp per pair."""
    from serve_b200.config import EngineConfig
    from serve_b200.engine import Engine

    folder = helpers.make_folder(str(tmp_path / "a"), "a", seed=3, std=0.08,
                                 dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    cfg, w = helpers.read_folder(folder)
    n_req, decoded = 530, 4
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab_size"], 1 + (i * 11) % 29 + decoded, seed=500 + i) for i in range(n_req)}
    plain = {rid: llama_forward(w, cfg, t) for rid, t in reqs.items()}
    eng = Engine.from_folder(folder, EngineConfig(dtype=dtype, page_size=8, num_pages=n_req * 5, max_slots=n_req + 2,
                                                  max_tokens_per_step=4096, max_context=64, use_cuda_graphs=True))
    items = list(reqs.items())
    steps = []
    for lo in range(0, n_req, 120):
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": t[:-decoded], "want": [len(t) - decoded - 1]}
                                                       for rid, t in items[lo:lo + 120]], "end": []})
    for d in range(decoded):
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [t[len(t) - decoded + d]], "want": [0]} for rid, t in items],
                      "end": [rid for rid, _ in items] if d == decoded - 1 else []})
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    eng.kernels.check_errors()
    assert eng.stepper.launched_graphs == 0
    assert len(got) == n_req * (decoded + 1)
    helpers.compare_with_plain(got, plain, atol=_tolerance(dtype, plain))
    eng.cache.check()
    assert eng.cache.live == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_equals_the_reference_run_on_a_gpu(tmp_path, dtype):
    """The engine against the logits that the reference's unmodified code (its Triton kernels included) gave on a B200
    (tests/golden/reference_gpu_*.npz): three prompts in one step, then eight steps of their decoded tokens."""
    from serve_b200.config import EngineConfig
    from serve_b200.engine import Engine, StepEntry
    from tests.test_plain import golden_gpu_case

    cfg, w, cases = golden_gpu_case(dtype)
    folder = helpers.write_folder(str(tmp_path / "g"), cfg, w, torch.float32 if dtype == "float32" else torch.bfloat16)
    eng = Engine.from_folder(folder, EngineConfig(dtype=dtype, page_size=64, num_pages=8, max_slots=4, max_tokens_per_step=256,
                                                  max_context=192, use_cuda_graphs=True))
    with torch.inference_mode():
        rows = [eng.step([StepEntry(i, p, [len(p) - 1]) for i, (p, _g, _l) in enumerate(cases)]).float().cpu().clone()]
        for j in range(8):
            rows.append(eng.step([StepEntry(i, [g[j]], [0]) for i, (_p, g, _l) in enumerate(cases)]).float().cpu().clone())
    eng.kernels.check_errors()
    got = torch.stack(rows, dim=1)                      # [3, 9, V]
    for i, (_p, g, ref) in enumerate(cases):
        scale = float(ref.abs().max())
        # float32: the reference's attention products are TF32 (2e-3 of the scale). bfloat16: both sides round to
        # bfloat16, each within 2^-6 of the scale of the exact result, so they lie within 2^-5 of one another.
        torch.testing.assert_close(got[i], ref, atol=scale * (2e-3 if dtype == "float32" else 2.0 ** -5), rtol=0)
        if dtype == "float32":
            assert got[i].argmax(-1).tolist() == g
