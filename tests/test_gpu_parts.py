"""Each part of a layer alone on the GPU against the plain implementation's function for it, and parts
defined here (outside the framework) registered, built and stepped: a mixer with state of its own,
a feed-forward with routing, another position encoding."""
import math

import pytest
import torch

from serve_b200.cache import CacheManager
from serve_b200.config import EngineConfig, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from serve_b200.engine import Engine, StepEntry
from serve_b200.engine.runtime import Runtime
from serve_b200.engine.step import BatchShape, StepContext
from serve_b200.parts import Block, CacheNeed, FeedForward, Mixer, PositionEncoding, TensorDecl, build_part, register_part
from tests import helpers
from tests.plain import llama_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _rt(dtype):
    from serve_b200.kernels import load_kernels

    return Runtime(load_kernels(DEV), DEV, DT[dtype])


def _ctx(rt, q_lens, starts, mgr=None, rids=None):
    t = sum(q_lens)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    pos = [s + j for q, s in zip(q_lens, starts) for j in range(q)]
    row = [i for i, q in enumerate(q_lens) for _ in range(q)]
    cu = [0]
    for q in q_lens:
        cu.append(cu[-1] + q)
    kv = [s + q for q, s in zip(q_lens, starts)]
    tables = []
    if mgr is not None:
        tables = [torch.from_numpy(mgr.table_rows(g, rids)).to(DEV) for g in range(len(mgr.groups))]
    return StepContext(rt=rt, shape=BatchShape(len(q_lens), t, max(q_lens), min(q_lens), max(kv), all(q == 1 for q in q_lens)),
                       tokens=i32([0] * t), positions=i32(pos), token_row=i32(row), cu_q=i32(cu), kv_len=i32(kv),
                       slots=i32(list(range(len(q_lens)))), logit_rows=i32([]), block_tables=tables, rids=rids or [])


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-6), ("bfloat16", 3e-2)])
def test_norm_part(dtype, tol):
    rt = _rt(dtype)
    norm = build_part("norm", PartSpec("rms", {"size": 200, "eps": 3e-4}, prefix="n."), rt)
    assert [d.name for d in norm.tensor_decls()] == ["n.weight"] and norm.tensor_decls()[0].role == "vector"
    w = (1 + 0.2 * torch.randn(200)).to(DEV)
    norm.load({"n.weight": w})
    x = torch.randn(9, 200, device=DEV) * 2
    delta = torch.randn(9, 200, device=DEV).to(DT[dtype])
    want = P.rms_norm(x + delta.float(), w, 3e-4)
    x_in = x.clone()
    got = norm.forward(x_in, delta, None)
    torch.testing.assert_close(x_in, x + delta.float())
    torch.testing.assert_close(got.float(), want, atol=tol, rtol=tol)


def _bf16_tol(want):
    """bfloat16 keeps 8 bits: the bound is 2^-6 of the largest value, the rule the replay tests use for logits."""
    return float(want.abs().max()) * 2.0 ** -6


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", None)])
def test_feed_forward_part(dtype, tol):
    rt = _rt(dtype)
    ff = build_part("feed_forward", PartSpec("swiglu", {"hidden": 120, "intermediate": 200}, prefix="m."), rt)
    w = {d.name: (torch.randn(d.shape) * 0.2).to(DEV).to(DT[dtype]) for d in ff.tensor_decls()}
    ff.load(w)
    h = torch.randn(13, 120, device=DEV).to(DT[dtype])
    want = P.swiglu(h.float(), w["m.gate_proj.weight"].float(), w["m.up_proj.weight"].float(), w["m.down_proj.weight"].float())
    tol = tol or _bf16_tol(want)
    torch.testing.assert_close(ff.forward(h, None).float(), want, atol=tol, rtol=0)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", None)])
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_in_two_portions(dtype, tol, window):
    """The mixer alone: 21 tokens in one go, then 9 more; against whole-sequence attention of the plain code."""
    rt = _rt(dtype)
    heads, kv_heads, d, hidden = 6, 2, 48, 120
    scaling = dict(factor=4.0, low_freq_factor=1.0, high_freq_factor=8.0, original_max_position_embeddings=32)
    spec = PartSpec("attention", {"hidden": hidden, "heads": heads, "kv_heads": kv_heads, "head_dim": d, "scale": None, "window": window,
                                  "position": PartSpec("rotary", {"rotary_dim": d, "theta": 25000.0, "scaling": scaling, "pairing": "half"})},
                    prefix="a.")
    att = build_part("mixer", spec, rt)
    w = {dcl.name: (torch.randn(dcl.shape) * 0.15).to(DEV).to(DT[dtype]) for dcl in att.tensor_decls()}
    att.load(w)
    need = att.cache_need()
    assert need == CacheNeed(kv_heads, d, window)
    mgr = CacheManager([need], [None], 8, 16, 2, 128, device=DEV, kv_dtype=DT[dtype])
    view = mgr.views()[0]
    x = torch.randn(30, hidden, device=DEV).to(DT[dtype])
    cfg = dict(num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=d)
    inv = P.rope_inv_freq(d, 25000.0, dict(rope_type="llama3", **scaling))
    want, _ = P.attention_layer(x.float().cpu(), {k: v.float().cpu() for k, v in w.items()}, "a.", cfg, torch.arange(30), inv, window)
    mgr.open("r")
    outs = []
    for start, n in ((0, 21), (21, 9)):
        mgr.reserve([("r", start + n)])
        outs.append(att.forward(x[start:start + n], _ctx(rt, [n], [start], mgr, ["r"]), view))
        mgr.commit("r", start + n)
    rt.kernels.check_errors()
    tol = tol or _bf16_tol(want)
    torch.testing.assert_close(torch.cat(outs).float().cpu(), want, atol=tol, rtol=0)
    if window:
        assert mgr.groups[0].pool.in_use < mgr.blocks_for(30), "pages the window has passed go back to the pool"


def test_position_part_matches_plain_frequencies():
    rt = _rt("float32")
    sc = dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=64)
    rot = build_part("position", PartSpec("rotary", {"rotary_dim": 32, "theta": 500000.0, "scaling": sc}), rt)
    torch.testing.assert_close(rot.inv_freq.cpu(), P.rope_inv_freq(32, 500000.0, dict(rope_type="llama3", **sc)), atol=0, rtol=2e-7)


from tests.toy_model import toy_plain as _toy_plain, toy_spec as _toy_spec  # noqa: E402  (also registers the toy parts)


def test_toy_parts_are_registered_built_and_stepped():
    """A model made of parts defined in this file runs through the engine's step function, cut in portions and
    mixed with another request, and equals its plain whole-sequence version. No framework file knows these parts."""
    from serve_b200.weights.loader import load_from_source
    from serve_b200.weights.random_init import random_tensor

    hidden, vocab = 64, 97
    spec = _toy_spec(hidden, vocab)
    ec = EngineConfig(dtype="float32", page_size=8, num_pages=24, max_slots=3, max_tokens_per_step=128, max_context=128, use_cuda_graphs=False)
    eng = Engine(config=None, engine_config=ec, spec=spec)
    made = {}
    def source(decl):
        made[decl.name] = random_tensor(decl, seed=5, std=0.3, norm_std=0.1)
        return made[decl.name]
    load_from_source(eng.model, source, torch.float32, DEV)
    eng._make_cache()
    needs = eng.model.cache_needs()
    assert needs[0].state_shape == (hidden + 1,) and needs[1].has_pages and needs[2].state_shape == (hidden + 1,)
    assert eng.stepper.views[0].state is not eng.stepper.views[2].state     # the layer run twice has a state per run
    reqs = {"x": helpers.random_tokens(vocab, 41, 1), "y": helpers.random_tokens(vocab, 23, 2), "z": helpers.random_tokens(vocab, 30, 3)}
    plain = {rid: _toy_plain(made, torch.tensor(t), hidden) for rid, t in reqs.items()}
    with torch.inference_mode():
        got = helpers.replay(eng, helpers.trace_mixed(reqs, live=2, seed=3, budget=24))
    helpers.compare_with_plain(got, plain, atol=2e-4)
    assert eng.cache.live == 0
    # a slot handed out again starts from zeroed state: replay once more on the used engine
    with torch.inference_mode():
        got = helpers.replay(eng, helpers.trace_portions(reqs, sizes=(5, 2, 11)))
    helpers.compare_with_plain(got, plain, atol=2e-4)


def test_a_mixer_with_state_decodes_from_graphs():
    """The toy model decodes its last tokens from CUDA graphs. The first step of a kind runs eagerly and is then
    captured; if capture or a warm-up ran the step's kernels a second time, the running-mean mixer would count that
    token twice and every later logit would be off."""
    from serve_b200.weights.loader import load_from_source
    from serve_b200.weights.random_init import random_tensor

    hidden, vocab = 64, 97
    ec = EngineConfig(dtype="float32", page_size=8, num_pages=48, max_slots=3, max_tokens_per_step=128, max_context=128, use_cuda_graphs=True)
    eng = Engine(config=None, engine_config=ec, spec=_toy_spec(hidden, vocab))
    made = {}
    def source(decl):
        made[decl.name] = random_tensor(decl, seed=6, std=0.3, norm_std=0.1)
        return made[decl.name]
    load_from_source(eng.model, source, torch.float32, DEV)
    eng._make_cache()
    reqs = {"x": helpers.random_tokens(vocab, 41, 4), "y": helpers.random_tokens(vocab, 23, 5)}
    plain = {rid: _toy_plain(made, torch.tensor(t), hidden) for rid, t in reqs.items()}
    with torch.inference_mode():
        got = helpers.replay(eng, helpers.trace_tail_decode(reqs, tail=12))
    assert eng.stepper.launched_graphs >= 20
    helpers.compare_with_plain(got, plain, atol=2e-4)
    # two requests decoding side by side are another kind of step (another graph): first sight again
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": t[:10], "want": [9]} for rid, t in reqs.items()], "end": []}]
    for j in range(10, 23):
        steps.append({"step": j, "entries": [{"id": rid, "tokens": [t[j]], "want": [0]} for rid, t in reqs.items()], "end": []})
    with torch.inference_mode():
        got = helpers.replay(eng, steps)
    helpers.compare_with_plain(got, plain, atol=2e-4)


@register_part("block", "test_sandwich")
class SandwichBlock(Block):
    """Another arrangement: every sub-layer has a norm before it and a norm after it (on its output, before the
    residual sum), and the output of the second is scaled by a constant of the arrangement's own."""

    wants = {"pre_mixer": "norm", "mixer": "mixer", "post_mixer": "norm", "pre_ff": "norm", "feed_forward": "feed_forward",
             "post_ff": "norm"}

    def __init__(self, spec, runtime, parts=None):
        super().__init__(spec, runtime, parts)
        self.ff_scale = float(spec.params.get("ff_scale", 1.0))

    def forward(self, x, pending, ctx, cache):
        h = self.pre_mixer.forward(x, pending, ctx)
        a = self.post_mixer.forward(self.mixer.forward(h, ctx, cache).float(), None, ctx)
        h = self.pre_ff.forward(x, a, ctx)
        f = self.post_ff.forward(self.feed_forward.forward(h, ctx).float(), None, ctx)
        return x, f * self.ff_scale


WINDOW = 10


def _two_kinds_spec(hidden, vocab):
    norm = lambda p: PartSpec("rms", {"size": hidden, "eps": 1e-5}, prefix=p)
    rope = PartSpec("rotary", {"rotary_dim": 16, "theta": 10000.0, "scaling": None, "pairing": "half"})
    att = lambda p, window: PartSpec("attention", {"hidden": hidden, "heads": 4, "kv_heads": 2, "head_dim": 16, "scale": None,
                                                   "window": window, "position": rope}, prefix=p)
    ff = lambda p: PartSpec("swiglu", {"hidden": hidden, "intermediate": 96}, prefix=p)
    layers = [
        LayerSpec(PartSpec("test_sandwich", {"ff_scale": 0.5}),
                  {"pre_mixer": norm("l0.n1."), "mixer": att("l0.att.", WINDOW), "post_mixer": norm("l0.n2."),
                   "pre_ff": norm("l0.n3."), "feed_forward": ff("l0.mlp."), "post_ff": norm("l0.n4.")}),
        LayerSpec.pre_norm(att("l1.att.", None), ff("l1.mlp."), norm("l1.n1."), norm("l1.n2.")),
    ]
    return ModelSpec("TwoKindsForTests", hidden, vocab, PartSpec("table", {"vocab": vocab, "hidden": hidden, "name": "emb.weight"}),
                     layers, [ScheduleEntry(0), ScheduleEntry(1)], norm("final."),
                     PartSpec("linear", {"vocab": vocab, "hidden": hidden, "name": "head.weight", "tied_to": None}), 512)


def _two_kinds_plain(w, tokens):
    cfg = dict(num_attention_heads=4, num_key_value_heads=2, head_dim=16)
    inv = P.rope_inv_freq(16, 10000.0, None)
    t = len(tokens)
    pos = torch.arange(t)
    n = lambda v, name: P.rms_norm(v, w[name], 1e-5)
    x = w["emb.weight"][torch.tensor(tokens)]
    a, _ = P.attention_layer(n(x, "l0.n1.weight"), w, "l0.att.", cfg, pos, inv, WINDOW)
    x = x + n(a, "l0.n2.weight")
    f = P.swiglu(n(x, "l0.n3.weight"), w["l0.mlp.gate_proj.weight"], w["l0.mlp.up_proj.weight"], w["l0.mlp.down_proj.weight"])
    x = x + 0.5 * n(f, "l0.n4.weight")
    a, _ = P.attention_layer(n(x, "l1.n1.weight"), w, "l1.att.", cfg, pos, inv, None)
    x = x + a
    x = x + P.swiglu(n(x, "l1.n2.weight"), w["l1.mlp.gate_proj.weight"], w["l1.mlp.up_proj.weight"], w["l1.mlp.down_proj.weight"])
    return n(x, "final.weight") @ w["head.weight"].T


def test_another_arrangement_and_a_windowed_layer_beside_a_full_one_generate_with_evictions():
    """A layer of another arrangement (norms after the sub-layers too, defined above) whose attention has a window,
    beside an ordinary layer with all keys: two cache groups with pools of their own, the windowed one giving pages
    back while requests run. Greedy generation through the entry point, with portions of 16 tokens and a pool so small
    that requests are evicted, equals the plain whole-sequence computation token by token; replay in portions and mixed
    equals it logit by logit."""
    from serve_b200 import Request, generate
    from serve_b200.weights.loader import load_from_source
    from serve_b200.weights.random_init import random_tensor

    hidden, vocab, page = 64, 97, 4
    made = {}
    def source(decl):
        made[decl.name] = random_tensor(decl, seed=8, std=0.25, norm_std=0.1)
        return made[decl.name]
    def engine(num_pages, **kw):
        ec = EngineConfig(dtype="float32", page_size=page, num_pages=num_pages, max_slots=4, max_context=128, **kw)
        eng = Engine(config=None, engine_config=ec, spec=_two_kinds_spec(hidden, vocab))
        load_from_source(eng.model, source, torch.float32, DEV)
        eng._make_cache()
        return eng
    eng = engine([24, 30], max_tokens_per_step=128, use_cuda_graphs=False)
    assert len(eng.cache.groups) == 2 and {g.window for g in eng.cache.groups} == {WINDOW, None}
    assert eng.cache.pool_pages() == [24, 30]
    reqs = {"x": helpers.random_tokens(vocab, 41, 1), "y": helpers.random_tokens(vocab, 23, 2), "z": helpers.random_tokens(vocab, 30, 3)}
    plain = {rid: _two_kinds_plain(made, t) for rid, t in reqs.items()}
    with torch.inference_mode():
        got = helpers.replay(eng, helpers.trace_portions(reqs, sizes=(5, 2, 11, 17)))
        got2 = helpers.replay(eng, helpers.trace_mixed(reqs, live=3, seed=4, budget=24))
    eng.kernels.check_errors()
    helpers.compare_with_plain(got, plain, atol=2e-4)
    helpers.compare_with_plain(got2, plain, atol=2e-4)
    windowed = next(g for g in eng.cache.groups if g.window)
    assert windowed.pool.high_water < sum(-(-len(t) // page) for t in reqs.values()), "pages behind the window went back early"
    # generation, with so few pages of the full group that the scheduler evicts
    prompts = [reqs["x"][:25], reqs["y"][:9], reqs["z"][:17], reqs["x"][5:18]]
    n_new = 10
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(n_new):
            toks.append(int(_two_kinds_plain(made, toks)[-1].argmax()))
        want.append(toks[len(p):])
    order = [g.window for g in eng.cache.groups]
    full_pages = -(-(25 + n_new) // page) + 3
    eng = engine([full_pages if wdw is None else 12 for wdw in order], max_tokens_per_step=32, prefill_chunk=16)
    out = generate(eng, [Request(torch.tensor(p), len(p), n_new) for p in prompts], temperature=0.0)
    eng.kernels.check_errors()
    assert [r.generated_tokens.tolist() for r in out] == want
    assert eng.last_stats.preemptions > 0
    eng.cache.check()
    assert eng.cache.live == 0 and all(g.pool.in_use == 0 for g in eng.cache.groups)


def test_an_architecture_defined_in_the_tests_loads_from_a_folder_and_generates(tmp_path):
    """The toy architecture of tests/toy_model.py (registered by that module alone) goes the whole way on the GPU: a model
    folder written with seeded random weights, loaded by the architecture name in its config.json through the entry
    point, greedy generation with portions of 16 tokens, against its plain whole-sequence version."""
    from safetensors.torch import load_file

    from serve_b200 import Request, generate, load_model
    from serve_b200.weights import write_random_model
    from tests.toy_model import ToyConfig

    folder = str(tmp_path / "toy")
    write_random_model(folder, ToyConfig(width=64, tokens=97), seed=5, std=0.3, norm_std=0.1, dtype=torch.float32)
    w = {k: v.float() for k, v in load_file(folder + "/model.safetensors").items()}
    eng, _ = load_model(folder, device="cuda", dtype="float32", page_size=8, num_pages=24, max_slots=3, max_tokens_per_step=32,
                        prefill_chunk=16, max_context=128)
    prompts = [helpers.random_tokens(97, 20, 1), helpers.random_tokens(97, 7, 2), helpers.random_tokens(97, 33, 3)]
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(6):
            toks.append(int(_toy_plain(w, torch.tensor(toks), 64)[-1].argmax()))
        want.append(toks[len(p):])
    out = generate(eng, [Request(torch.tensor(p), len(p), 6) for p in prompts], temperature=0.0)
    eng.kernels.check_errors()
    assert [r.generated_tokens.tolist() for r in out] == want
    assert eng.cache.live == 0
