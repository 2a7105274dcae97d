"""Weights by name: reading, kept dtypes, the one error that lists everything, random-weights folders."""
import json
import os
import struct

import pytest
import torch

from serve_b200.config import build_spec, config_from_dict
from serve_b200.engine.runtime import Runtime
from serve_b200.models.decoder import DecoderModel
from serve_b200.weights import SafetensorsFile, WeightError, load_weights, write_random_model, write_safetensors
from tests import helpers


def _model(name):
    return DecoderModel(build_spec(config_from_dict(helpers.TINY[name])), Runtime.describe_only())


def test_writer_is_read_by_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file

    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
         "d": torch.tensor(2.5)}
    write_safetensors(str(tmp_path / "x.safetensors"), t)
    back = load_file(str(tmp_path / "x.safetensors"))
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])
    save_file(t, str(tmp_path / "y.safetensors"))
    f = SafetensorsFile(str(tmp_path / "y.safetensors"))
    for k in t:
        assert torch.equal(f.tensor(k), t[k])


def test_random_folder_loads_and_is_seeded(tmp_path):
    cfg = config_from_dict(helpers.TINY["b"])
    write_random_model(str(tmp_path / "m1"), cfg, seed=5, norm_std=0.1, dtype=torch.bfloat16)
    write_random_model(str(tmp_path / "m2"), cfg, seed=5, norm_std=0.1, dtype=torch.bfloat16)
    write_random_model(str(tmp_path / "m3"), cfg, seed=6, norm_std=0.1, dtype=torch.bfloat16)
    c1, w1 = helpers.read_folder(str(tmp_path / "m1"))
    _, w2 = helpers.read_folder(str(tmp_path / "m2"))
    _, w3 = helpers.read_folder(str(tmp_path / "m3"))
    assert c1["architectures"] == ["LlamaForCausalLM"] and c1["hidden_size"] == 192
    assert set(w1) == set(_model("b").tensor_decls()) and "lm_head.weight" in w1
    assert all(torch.equal(w1[k], w2[k]) for k in w1)
    assert not torch.equal(w1["model.embed_tokens.weight"], w3["model.embed_tokens.weight"])
    assert abs(float(w1["model.layers.0.mlp.up_proj.weight"].std()) - 0.02) < 2e-3
    assert abs(float(w1["model.norm.weight"].mean()) - 1.0) < 0.05
    m = _model("b")
    load_weights(m, str(tmp_path / "m1"), torch.float32, "cpu")
    att = m.blocks[2].mixer
    assert att.w_qkv.shape == ((6 + 2 * 3) * 32, 192) and att.w_qkv.dtype == torch.float32
    # fused rows: q heads, k heads, v heads; inside a q or k head the two elements of a rotary pair are neighbours
    wk = w1["model.layers.2.self_attn.k_proj.weight"]
    assert torch.equal(att.w_qkv[6 * 32: 6 * 32 + 32: 2], wk[:16]) and torch.equal(att.w_qkv[6 * 32 + 1: 6 * 32 + 32: 2], wk[16:32])
    assert torch.equal(att.w_qkv[9 * 32:], w1["model.layers.2.self_attn.v_proj.weight"])
    assert m.blocks[0].feed_forward.w_gate_up.shape == (640, 192)


def test_kept_dtypes(tmp_path):
    """Matrices become the compute dtype; a vector stored in 32-bit stays 32-bit; tied head shares the table."""
    cfg = config_from_dict(helpers.TINY["a"])
    write_random_model(str(tmp_path / "m"), cfg, seed=1, dtype=torch.bfloat16)
    from safetensors.torch import load_file, save_file

    w = load_file(str(tmp_path / "m" / "model.safetensors"))
    w["model.norm.weight"] = w["model.norm.weight"].float()
    save_file(w, str(tmp_path / "m" / "model.safetensors"))
    m = _model("a")
    load_weights(m, str(tmp_path / "m"), torch.bfloat16, "cpu")
    assert m.final_norm.weight.dtype == torch.float32
    assert m.blocks[0].mixer_norm.weight.dtype == torch.bfloat16
    assert m.blocks[0].mixer.w_qkv.dtype == torch.bfloat16
    assert m.head.weight.data_ptr() == m.embedding.table.data_ptr()
    m32 = _model("a")
    load_weights(m32, str(tmp_path / "m"), torch.float32, "cpu")
    assert m32.blocks[0].mixer.w_o.dtype == torch.float32 and m32.blocks[0].mixer_norm.weight.dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(helpers.TINY["b"])
    write_random_model(str(tmp_path / "m"), cfg, seed=1, dtype=torch.float32)
    from safetensors.torch import load_file, save_file

    w = load_file(str(tmp_path / "m" / "model.safetensors"))
    del w["model.layers.1.mlp.down_proj.weight"]
    del w["lm_head.weight"]
    w["model.layers.0.self_attn.q_norm.weight"] = torch.ones(32)
    w["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(64, 192)
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(16)      # ignored, as the reference drops it
    save_file(w, str(tmp_path / "m" / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_weights(_model("b"), str(tmp_path / "m"), torch.float32, "cpu")
    msg = str(e.value)
    assert "missing (2)" in msg and "model.layers.1.mlp.down_proj.weight" in msg and "lm_head.weight" in msg
    assert "unexpected (1)" in msg and "q_norm" in msg and "inv_freq" not in msg
    assert "wrong shape (1)" in msg and "[64, 192]" in msg and "[96, 192]" in msg


def test_tied_model_ignores_a_stored_head(tmp_path):
    cfg = config_from_dict(helpers.TINY["a"])
    write_random_model(str(tmp_path / "m"), cfg, seed=1, dtype=torch.float32)
    from safetensors.torch import load_file, save_file

    w = load_file(str(tmp_path / "m" / "model.safetensors"))
    assert "lm_head.weight" not in w
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    save_file(w, str(tmp_path / "m" / "model.safetensors"))
    load_weights(_model("a"), str(tmp_path / "m"), torch.float32, "cpu")


def test_sharded_folder_and_broken_files(tmp_path):
    cfg = config_from_dict(helpers.TINY["a"])
    write_random_model(str(tmp_path / "m"), cfg, seed=1, dtype=torch.float32)
    from safetensors.torch import load_file, save_file

    w = load_file(str(tmp_path / "m" / "model.safetensors"))
    os.remove(tmp_path / "m" / "model.safetensors")
    names = sorted(w)
    half = len(names) // 2
    save_file({k: w[k] for k in names[:half]}, str(tmp_path / "m" / "model-00001-of-00002.safetensors"))
    save_file({k: w[k] for k in names[half:]}, str(tmp_path / "m" / "model-00002-of-00002.safetensors"))
    index = {"weight_map": {k: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                            for i, k in enumerate(names)}}
    (tmp_path / "m" / "model.safetensors.index.json").write_text(json.dumps(index))
    m = _model("a")
    load_weights(m, str(tmp_path / "m"), torch.float32, "cpu")
    assert torch.equal(m.embedding.table, w["model.embed_tokens.weight"])
    # truncated header
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "config.json").write_text(json.dumps(helpers.TINY["a"]))
    (bad / "model.safetensors").write_bytes(struct.pack("<Q", 10_000) + b"{}")
    with pytest.raises(WeightError, match="truncated"):
        load_weights(_model("a"), str(bad), torch.float32, "cpu")
    os.remove(bad / "model.safetensors")
    with pytest.raises(WeightError, match="neither"):
        load_weights(_model("a"), str(bad), torch.float32, "cpu")
