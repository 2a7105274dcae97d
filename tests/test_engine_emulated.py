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
