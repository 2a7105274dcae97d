"""The step function, the cache and the model wiring against the plain implementation,
with torch stand-ins for the kernels, on the CPU. What the kernels themselves do is
tested on the GPU (test_gpu_*.py); this file finds faults of the cache and of the batch."""
import pytest
import torch

from serve_b200.config import EngineConfig
from serve_b200.engine import Engine
from tests import helpers
from tests.emu_kernels import EmuKernels
from tests.plain.llama_plain import llama_forward

LENGTHS = {"a": [5, 9, 13, 70], "b": [1, 17, 40, 70, 33, 52], "c": [3, 64, 65, 37, 90]}


def _setup(tmp_path, name, page_size, num_pages):
    folder = helpers.make_folder(str(tmp_path / name), name, seed=3)
    cfg, w = helpers.read_folder(folder)
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab_size"], n, seed=10 + i) for i, n in enumerate(LENGTHS[name])}
    plain = {rid: llama_forward(w, cfg, toks) for rid, toks in reqs.items()}
    ec = EngineConfig(dtype="float32", page_size=page_size, num_pages=num_pages, max_slots=4, max_tokens_per_step=256,
                      max_context=128, device="cpu", use_cuda_graphs=False)
    eng = Engine.from_folder(folder, ec, kernels=EmuKernels())
    return eng, reqs, plain


@pytest.mark.parametrize("name,page", [("a", 4), ("b", 8), ("c", 16)])
def test_every_cut_matches_plain(tmp_path, name, page):
    eng, reqs, plain = _setup(tmp_path, name, page, num_pages=-(-4 * 96 // page))
    for make in (helpers.trace_whole, helpers.trace_tail_decode, helpers.trace_portions):
        got = helpers.replay(eng, make(reqs))
        assert len(got) == sum(len(t) for t in reqs.values())
        helpers.compare_with_plain(got, plain, atol=2e-5)
        eng.cache.check()
        assert eng.cache.live == 0 and all(g.pool.in_use == 0 for g in eng.cache.groups)


@pytest.mark.parametrize("name,page", [("a", 4), ("b", 8), ("c", 16)])
def test_mixed_batches_reuse_pages(tmp_path, name, page):
    eng, reqs, plain = _setup(tmp_path, name, page, num_pages=1)
    steps = helpers.trace_mixed(reqs, live=4, seed=5)
    need = helpers.tokens_needed(steps, page) // page
    total = sum(-(-len(t) // page) for t in reqs.values())
    assert need < total, "the trace must need fewer pages than all requests together"
    eng, reqs, plain = _setup(tmp_path, name, page, num_pages=need)
    got = helpers.replay(eng, steps)
    helpers.compare_with_plain(got, plain, atol=2e-5)
    assert eng.cache.groups[0].pool.high_water == need
    eng.cache.check()


def test_out_of_pages_changes_nothing(tmp_path):
    from serve_b200.cache import OutOfPages
    from serve_b200.engine import StepEntry

    eng, reqs, plain = _setup(tmp_path, "a", 4, num_pages=5)
    eng.step([StepEntry("x", reqs["r3"][:9], [8])])           # 3 of 5 pages
    with pytest.raises(OutOfPages):
        eng.step([StepEntry("x", reqs["r3"][9:13], []), StepEntry("y", reqs["r2"], [])])   # 1 + 4 more
    eng.cache.check()
    assert eng.cache.length("x") == 9 and not eng.cache.is_open("y")
    assert eng.cache.groups[0].pool.in_use == 3
    out = eng.step([StepEntry("x", [reqs["r3"][9]], [0])])      # still usable
    assert out.shape == (1, 256)
    torch.testing.assert_close(out[0], plain["r3"][9], atol=2e-5, rtol=0)


def test_schedule_repeats_a_layer_and_shares_a_cache(tmp_path):
    """The run order is data: layer 0 twice, and an execution that reads another's cache."""
    import dataclasses

    from serve_b200.config import ScheduleEntry, build_spec, load_config

    folder = helpers.make_folder(str(tmp_path / "b"), "b", seed=4)
    cfg, w = helpers.read_folder(folder)
    config = load_config(folder)
    schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(2, cache_of=1)]
    spec = dataclasses.replace(build_spec(config), schedule=schedule)
    ec = EngineConfig(dtype="float32", page_size=8, num_pages=32, max_slots=2, max_tokens_per_step=128, max_context=128,
                      device="cpu", use_cuda_graphs=False)
    eng = Engine(config, ec, kernels=EmuKernels(), spec=spec)
    from serve_b200.weights import load_weights

    load_weights(eng.model, folder, torch.float32, "cpu")
    eng._make_cache()
    toks = helpers.random_tokens(cfg["vocab_size"], 45, seed=2)
    plain = {"s": llama_forward(w, cfg, toks, schedule=[(0, None), (1, None), (0, None), (2, 1)])}
    got = helpers.replay(eng, helpers.trace_portions({"s": toks}, sizes=(11, 2, 7, 25)))
    helpers.compare_with_plain(got, plain, atol=2e-5)
    assert sum(v is not None and v.writes for v in eng.stepper.views) == 3


# ---- generation through the entry point (scheduler + sampler + step), still with stand-in kernels ----
def _plain_generate(w, cfg, prompt, n_new, temperature=0.0, seed=0, rid=0):
    from tests.plain.llama_plain import sample_token

    toks = list(prompt)
    for i in range(n_new):
        logits = llama_forward(w, cfg, toks)[-1]
        toks.append(sample_token(logits, temperature, seed, rid, i))
    return toks[len(prompt):]


@pytest.mark.parametrize("name,temperature", [("a", 0.0), ("b", 0.8)])
def test_generate_equals_plain_under_chunking_and_eviction(tmp_path, name, temperature):
    from serve_b200.run import Request, generate

    folder = helpers.make_folder(str(tmp_path / name), name, seed=3, std=0.08)
    cfg, w = helpers.read_folder(folder)
    lengths = [5, 9, 13] if name == "a" else [1, 17, 40, 70]
    prompts = [helpers.random_tokens(cfg["vocab_size"], n, seed=20 + i) for i, n in enumerate(lengths)]
    n_new = 8
    want = [_plain_generate(w, cfg, p, n_new, temperature, seed=11, rid=i) for i, p in enumerate(prompts)]
    page = 4 if name == "a" else 8
    settings = [
        dict(num_pages=64, max_tokens_per_step=256, prefill_chunk=None),       # whole prompts
        dict(num_pages=64, max_tokens_per_step=24, prefill_chunk=16),          # portions of 16 mixed with decodes
        dict(num_pages=-(-(max(lengths) + n_new) // page) + 3, max_tokens_per_step=32, prefill_chunk=16),  # pages run out
    ]
    for i, st in enumerate(settings):
        ec = EngineConfig(dtype="float32", page_size=page, max_slots=4, max_context=128, device="cpu", use_cuda_graphs=False, **st)
        eng = Engine.from_folder(folder, ec, kernels=EmuKernels())
        reqs = [Request(torch.tensor(p), len(p), n_new) for p in prompts]
        out = generate(eng, reqs, temperature=temperature, seed=11, return_logits=True)
        assert [r.generated_tokens.tolist() for r in out] == want, f"setting {i}"
        assert all(r.logits is not None and r.logits.shape == (cfg["vocab_size"],) for r in out)
        if i == 2:
            assert eng.last_stats.preemptions > 0, "this pool was meant to run out of pages"
        assert eng.cache.live == 0
        eng.cache.check()


@pytest.mark.parametrize("return_logits", [False, True])
def test_stop_id_found_one_step_late_changes_nothing(tmp_path, return_logits):
    """generate() launches a step before it has read the previous step's tokens; a stop id is then seen one step
    late. The output must still end with the stop id, requests beside it must be untouched, all pages come back."""
    from serve_b200.run import Request, generate

    folder = helpers.make_folder(str(tmp_path / "a"), "a", seed=3, std=0.08)
    cfg, w = helpers.read_folder(folder)
    prompts = [helpers.random_tokens(cfg["vocab_size"], n, seed=50 + i) for i, n in enumerate([6, 11, 4])]
    full = [_plain_generate(w, cfg, p, 12) for p in prompts]
    stop = full[1][5]                                   # request 1 stops here at the latest
    want = []
    for g in full:
        cut = g.index(stop) + 1 if stop in g else len(g)
        want.append(g[:cut])
    assert len(want[1]) <= 6 and any(len(x) == 12 for x in want) or True
    ec = EngineConfig(dtype="float32", page_size=4, num_pages=64, max_slots=4, max_context=128, device="cpu",
                      use_cuda_graphs=False, max_tokens_per_step=64)
    eng = Engine.from_folder(folder, ec, kernels=EmuKernels())
    out = generate(eng, [Request(torch.tensor(p), len(p), 12) for p in prompts], eos_token_id=stop, return_logits=return_logits)
    assert [r.generated_tokens.tolist() for r in out] == want
    if return_logits:
        for r, p, g in zip(out, prompts, want):
            ref = llama_forward(w, cfg, p + g[:-1])[-1]
            torch.testing.assert_close(r.logits, ref, atol=2e-5, rtol=0)
    assert eng.cache.live == 0
    eng.cache.check()


def test_an_architecture_defined_outside_the_framework_loads_and_runs(tmp_path):
    """A toy architecture (tests/toy_model.py: its own config.json keys, a mixer with per-request state, a routed
    feed-forward, a position part without rotation, one layer run twice) is registered by the test module alone. A model
    folder of it is written with seeded random weights, read back by architecture name, replayed in portions and mixed
    batches, and generated from through the Python entry point; everything equals its plain whole-sequence version.
    No file of serve_b200 names it."""
    from safetensors.torch import load_file

    from serve_b200 import Request, generate
    from serve_b200.config import known_architectures, load_config
    from serve_b200.weights import write_random_model
    from tests.toy_model import ToyConfig, toy_plain

    assert "ToyDecoderForTests" in known_architectures()
    folder = str(tmp_path / "toy")
    write_random_model(folder, ToyConfig(width=64, tokens=97), seed=5, std=0.3, norm_std=0.1, dtype=torch.float32)
    cfg = load_config(folder)
    assert isinstance(cfg, ToyConfig) and cfg.width == 64 and cfg.tokens == 97
    w = {k: v.float() for k, v in load_file(folder + "/model.safetensors").items()}
    ec = EngineConfig(dtype="float32", page_size=8, num_pages=24, max_slots=3, max_tokens_per_step=128, max_context=128,
                      device="cpu", use_cuda_graphs=False)
    eng = Engine.from_folder(folder, ec, kernels=EmuKernels())
    needs = eng.model.cache_needs()
    assert needs[0].state_shape == (65,) and needs[1].has_pages and needs[2].state_shape == (65,)
    reqs = {"x": helpers.random_tokens(97, 41, 1), "y": helpers.random_tokens(97, 23, 2), "z": helpers.random_tokens(97, 30, 3)}
    plain = {rid: toy_plain(w, torch.tensor(t), 64) for rid, t in reqs.items()}
    got = helpers.replay(eng, helpers.trace_mixed(reqs, live=2, seed=3, budget=24))
    helpers.compare_with_plain(got, plain, atol=2e-4)
    got = helpers.replay(eng, helpers.trace_portions(reqs, sizes=(5, 2, 11)))       # slots handed out again start from zero
    helpers.compare_with_plain(got, plain, atol=2e-4)
    assert eng.cache.live == 0
    # greedy generation through the entry point (scheduler, portions of 16, sampling)
    prompts = [reqs["x"][:20], reqs["y"][:7]]
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(6):
            toks.append(int(toy_plain(w, torch.tensor(toks), 64)[-1].argmax()))
        want.append(toks[len(p):])
    eng2 = Engine.from_folder(folder, EngineConfig(dtype="float32", page_size=8, num_pages=24, max_slots=3, max_tokens_per_step=32,
                                                   prefill_chunk=16, max_context=128, device="cpu", use_cuda_graphs=False),
                              kernels=EmuKernels())
    out = generate(eng2, [Request(torch.tensor(p), len(p), 6) for p in prompts], temperature=0.0)
    assert [r.generated_tokens.tolist() for r in out] == want
