"""The Llama dense decoder as a layer description.

What the reference builds in code (serve/model.py:137-160: embedding, N equal
pre-norm blocks of attention + SwiGLU, final RMSNorm, output projection) is
written here as a ``ModelSpec``; tensor names are the weight file's own
(the left column of serve/hf_utils/convert_hf_checkpoint.py:98-112).
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.llama import LlamaConfig
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    scaling = None
    if cfg.rope_scaling is not None:
        s = cfg.rope_scaling
        scaling = {
            "factor": s.factor,
            "low_freq_factor": s.low_freq_factor,
            "high_freq_factor": s.high_freq_factor,
            "original_max_position_embeddings": s.original_max_position_embeddings,
        }
    position = PartSpec("rotary", {"rotary_dim": cfg.head_dim, "theta": cfg.rope_theta, "scaling": scaling, "pairing": "half"})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(
            LayerSpec.pre_norm(
                mixer=PartSpec(
                    "attention",
                    {
                        "hidden": cfg.hidden_size,
                        "heads": cfg.num_attention_heads,
                        "kv_heads": cfg.num_key_value_heads,
                        "head_dim": cfg.head_dim,
                        "scale": None,
                        "window": None,
                        "position": position,
                    },
                    prefix=p + "self_attn.",
                ),
                feed_forward=PartSpec("swiglu", {"hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size}, prefix=p + "mlp."),
                mixer_norm=PartSpec("rms", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, prefix=p + "input_layernorm."),
                feed_forward_norm=PartSpec("rms", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, prefix=p + "post_attention_layernorm."),
            )
        )
    embed_name = "model.embed_tokens.weight"
    spec = ModelSpec(
        architecture=LlamaConfig.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("table", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size, "name": embed_name}),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rms", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, prefix="model.norm."),
        head=PartSpec(
            "linear",
            {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size, "name": "lm_head.weight",
             "tied_to": embed_name if cfg.tie_word_embeddings else None},
        ),
        max_position=cfg.max_position_embeddings,
    )
    spec.validate()
    return spec


register_architecture(LlamaConfig.architecture, LlamaConfig, llama_spec)
