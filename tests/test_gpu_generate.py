"""Generation through the Python entry point and the command line on the GPU, against the plain implementation."""
import json
import os
import subprocess
import sys

import pytest
import torch

from tests import helpers
from tests.plain.llama_plain import llama_forward, sample_token

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _plain_generate(w, cfg, prompt, n_new, temperature=0.0, seed=0, rid=0):
    toks = list(prompt)
    for i in range(n_new):
        toks.append(sample_token(llama_forward(w, cfg, toks)[-1], temperature, seed, rid, i))
    return toks[len(prompt):]


@pytest.mark.parametrize("name,dtype,temperature", [("a", "float32", 0.0), ("b", "float32", 0.8), ("c", "float32", 0.0), ("b", "bfloat16", 0.0)])
def test_generate_equals_plain(tmp_path, name, dtype, temperature):
    from serve_b200 import Request, generate, load_model

    folder = helpers.make_folder(str(tmp_path / name), name, seed=3, std=0.08,
                                 dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    cfg, w = helpers.read_folder(folder)
    lengths = {"a": [5, 9, 13], "b": [1, 17, 40, 70], "c": [3, 33, 64]}[name]
    prompts = [helpers.random_tokens(cfg["vocab_size"], n, seed=20 + i) for i, n in enumerate(lengths)]
    n_new = 8 if dtype == "float32" else 6
    want = [_plain_generate(w, cfg, p, n_new, temperature, seed=11, rid=i) for i, p in enumerate(prompts)]
    page = {"a": 4, "b": 8, "c": 16}[name]
    settings = [dict(num_pages=64, max_tokens_per_step=256),
                dict(num_pages=64, max_tokens_per_step=24, prefill_chunk=16),
                dict(num_pages=-(-(max(lengths) + n_new) // page) + 3, max_tokens_per_step=32, prefill_chunk=16)]
    for i, st in enumerate(settings):
        eng, _tok = load_model(folder, device="cuda", dtype=dtype, page_size=page, max_slots=4, max_context=128, **st)
        reqs = [Request(torch.tensor(p), len(p), n_new) for p in prompts]
        out = generate(eng, reqs, temperature=temperature, seed=11, return_logits=True)
        eng.kernels.check_errors()
        got = [r.generated_tokens.tolist() for r in out]
        if dtype == "float32":
            assert got == want, f"setting {i}"
        else:
            # bfloat16 may flip a near-tie, after which the histories differ. So every generated token is judged against
            # plain's logits for the engine's own history: it must be plain's choice wherever plain's best two logits
            # lie further apart than the bfloat16 bound, and never lie further below plain's best than that bound.
            judged = 0
            for p, g_ in zip(prompts, got):
                assert len(g_) == n_new
                lg = llama_forward(w, cfg, p + g_[:-1])[len(p) - 1:]
                bound = 2 * float(lg.abs().max()) * 2.0 ** -6
                for j, tok in enumerate(g_):
                    top2 = torch.topk(lg[j], 2).values
                    assert float(top2[0] - lg[j][tok]) <= bound, f"setting {i}, token {j}"
                    if float(top2[0] - top2[1]) > bound:
                        assert tok == int(lg[j].argmax()), f"setting {i}, token {j}"
                        judged += 1
            assert judged >= n_new
        assert eng.cache.live == 0
        eng.cache.check()
        if i == 2:
            assert eng.last_stats.preemptions > 0


@pytest.mark.parametrize("return_logits", [False, True])
def test_stop_id_in_the_middle_of_a_run_with_evictions(tmp_path, return_logits):
    """A stop id that some requests meet after a few tokens, others never, under a pool so small that requests are
    evicted and recomputed: every request ends with plain's tokens up to and with its first stop id (found one step
    late by the pipelined loop, whose extra step is dropped), its last logits are those of the step that made its last
    token, and every page and slot comes back."""
    from serve_b200 import Request, generate, load_model

    folder = helpers.make_folder(str(tmp_path / "a"), "a", seed=3, std=0.08)
    cfg, w = helpers.read_folder(folder)
    lengths = [5, 9, 13, 21]
    n_new = 10
    prompts = [helpers.random_tokens(cfg["vocab_size"], n, seed=20 + i) for i, n in enumerate(lengths)]
    full = [_plain_generate(w, cfg, p, n_new) for p in prompts]
    stop = full[1][3]                                            # request 1 stops at its fourth token at the latest
    want = [g[: g.index(stop) + 1] if stop in g else g for g in full]
    assert any(len(x) < n_new for x in want) and any(len(x) == n_new for x in want)
    page = 4
    eng, _ = load_model(folder, device="cuda", dtype="float32", page_size=page, max_slots=4, max_context=128,
                        num_pages=-(-(max(lengths) + n_new) // page) + 3, max_tokens_per_step=32, prefill_chunk=16)
    out = generate(eng, [Request(torch.tensor(p), len(p), n_new) for p in prompts], temperature=0.0, eos_token_id=stop,
                   return_logits=return_logits)
    eng.kernels.check_errors()
    assert [r.generated_tokens.tolist() for r in out] == want
    assert eng.last_stats.preemptions > 0
    assert eng.cache.live == 0
    eng.cache.check()
    assert all(g.pool.in_use == 0 for g in eng.cache.groups)
    if return_logits:
        for p, g_, r in zip(prompts, want, out):
            ref = llama_forward(w, cfg, p + g_[:-1])[-1]
            torch.testing.assert_close(r.logits.float().cpu(), ref, atol=3e-5, rtol=0)
    else:
        assert all(r.logits is None for r in out)


def test_command_line(tmp_path):
    folder = helpers.make_folder(str(tmp_path / "a"), "a", seed=3, std=0.08)
    cfg, w = helpers.read_folder(folder)
    prompt = helpers.random_tokens(cfg["vocab_size"], 11, seed=4)
    want = _plain_generate(w, cfg, prompt, 5)
    out = subprocess.run([sys.executable, "-m", "serve_b200.run", "--model", folder, "--dtype", "float32", "--page-size", "4",
                          "--num-pages", "32", "--max-context", "64", "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "5"],
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    rec = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert rec["generated_tokens"] == want


def test_trace_run_program(tmp_path):
    """bin/trace_run as a user starts it: JSON lines in, <step>.f32 files and 'done <step>' lines out."""
    import numpy as np

    folder = helpers.make_folder(str(tmp_path / "b"), "b", seed=3, dtype=torch.bfloat16)
    cfg, w = helpers.read_folder(folder)
    reqs = {f"r{i}": helpers.random_tokens(cfg["vocab_size"], n, seed=30 + i) for i, n in enumerate([70, 130, 64, 90, 33])}
    plain = {rid: llama_forward(w, cfg, t) for rid, t in reqs.items()}
    steps = helpers.trace_mixed(reqs, live=4, seed=9)
    need = helpers.tokens_needed(steps, 64)
    assert need < sum(-(-len(t) // 64) * 64 for t in reqs.values())
    for dtype, atol in (("float32", 3e-5), ("bfloat16", max(float(p.abs().max()) for p in plain.values()) * 2.0 ** -6)):
        out_dir = tmp_path / f"out-{dtype}"
        proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out_dir),
                               "--max-tokens", str(need)], input="\n".join(json.dumps(s) for s in steps) + "\n",
                              capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-3000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
        got, at = {}, {}
        for s in steps:
            n_want = sum(len(e["want"]) for e in s["entries"])
            arr = np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(n_want, cfg["vocab_size"])
            i = 0
            for e in s["entries"]:
                base = at.get(e["id"], 0)
                for wi in e["want"]:
                    got[(e["id"], base + wi)] = torch.from_numpy(arr[i].copy())
                    i += 1
                at[e["id"]] = base + len(e["tokens"])
        helpers.compare_with_plain(got, plain, atol=atol)
