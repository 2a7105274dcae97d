"""Typed configuration, architecture registry, presets."""
import json

import pytest

from serve_b200.config import ConfigError, build_spec, config_from_dict, known_architectures, load_config, load_preset
from serve_b200.config.llama import LlamaConfig
from tests.helpers import TINY


def test_reads_every_key_from_the_file(tmp_path):
    for name, d in TINY.items():
        (tmp_path / name).mkdir()
        (tmp_path / name / "config.json").write_text(json.dumps(d))
        cfg = load_config(str(tmp_path / name))
        assert isinstance(cfg, LlamaConfig)
        for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
                    "intermediate_size", "vocab_size", "rms_norm_eps", "rope_theta", "tie_word_embeddings"):
            assert getattr(cfg, key) == d[key], key
        if d["rope_scaling"] is None:
            assert cfg.rope_scaling is None
        else:
            assert cfg.rope_scaling.factor == d["rope_scaling"]["factor"]
            assert cfg.rope_scaling.original_max_position_embeddings == d["rope_scaling"]["original_max_position_embeddings"]
        assert config_from_dict(cfg.to_dict()) == cfg


def test_fallbacks_only_for_absent_keys():
    d = dict(architectures=["LlamaForCausalLM"], hidden_size=96, num_hidden_layers=1, num_attention_heads=6,
             intermediate_size=64, vocab_size=50)
    cfg = config_from_dict(d)
    assert cfg.num_key_value_heads == 6 and cfg.head_dim == 16
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0 and cfg.rope_scaling is None and not cfg.tie_word_embeddings


@pytest.mark.parametrize("patch,word", [
    ({"architectures": ["MysteryForCausalLM"]}, "unknown architecture"),
    ({"architectures": []}, "architectures"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "head_dim"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "rope_type"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "lacks keys"),
    ({"vocab_size": None}, "vocab_size"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
])
def test_refusals(patch, word):
    d = dict(TINY["a"])
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_registry_and_spec():
    assert "LlamaForCausalLM" in known_architectures()
    cfg = config_from_dict(TINY["b"])
    spec = build_spec(cfg)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    att = spec.layers[1].parts["mixer"]
    assert att.kind == "attention" and att.prefix == "model.layers.1.self_attn."
    assert att.params["heads"] == 6 and att.params["kv_heads"] == 3 and att.params["head_dim"] == 32
    assert att.params["position"].params["scaling"]["factor"] == 8.0
    assert spec.layers[0].parts["feed_forward"].params["intermediate"] == 320
    assert spec.head.params["tied_to"] is None
    assert build_spec(config_from_dict(TINY["a"])).head.params["tied_to"] == "model.embed_tokens.weight"


def test_presets():
    cfg = load_preset("llama-3.2-1b")
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
            cfg.intermediate_size, cfg.vocab_size) == (2048, 16, 32, 8, 64, 8192, 128256)
    assert cfg.rope_scaling.factor == 32.0 and cfg.tie_word_embeddings
    with pytest.raises(ConfigError, match="no preset"):
        load_preset("nope")


def test_schedule_validation():
    import dataclasses

    from serve_b200.config import ScheduleEntry

    spec = build_spec(config_from_dict(TINY["a"]))
    for bad in ([ScheduleEntry(5)], [ScheduleEntry(0, cache_of=0)], [ScheduleEntry(0), ScheduleEntry(1, 0), ScheduleEntry(0, 1)], []):
        with pytest.raises(ConfigError):
            dataclasses.replace(spec, schedule=bad).validate()


def test_rotary_parts_with_equal_parameters_share_their_frequencies():
    """What a step derives from the frequencies (the table of cosines and sines) is made once per step only if the
    layers' position parts hand out the same tensor; other parameters get a tensor of their own."""
    from serve_b200.config.spec import PartSpec
    from serve_b200.engine.runtime import Runtime
    from serve_b200.parts.base import build_part

    rt = Runtime.describe_only()
    scaling = dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)
    a = build_part("position", PartSpec("rotary", {"rotary_dim": 32, "theta": 10000.0, "scaling": scaling}), rt)
    b = build_part("position", PartSpec("rotary", {"rotary_dim": 32, "theta": 10000.0, "scaling": dict(scaling)}), rt)
    c = build_part("position", PartSpec("rotary", {"rotary_dim": 32, "theta": 500000.0, "scaling": scaling}), rt)
    d = build_part("position", PartSpec("rotary", {"rotary_dim": 32, "theta": 10000.0, "scaling": None}), rt)
    assert a.inv_freq is b.inv_freq
    assert c.inv_freq is not a.inv_freq and d.inv_freq is not a.inv_freq
    assert not bool((c.inv_freq == a.inv_freq).all()) and not bool((d.inv_freq == a.inv_freq).all())
    other = build_part("position", PartSpec("rotary", {"rotary_dim": 32, "theta": 10000.0, "scaling": scaling}), Runtime.describe_only())
    assert other.inv_freq is not a.inv_freq and bool((other.inv_freq == a.inv_freq).all())
