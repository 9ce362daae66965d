"""The Llama dense decoder as a model description.

Pre-norm residual layers of grouped-query attention with llama3-scaled rotate-half
rotary encoding and a SwiGLU feed-forward, RMSNorm, bias-free linears, a tied or
untied LM head: what upstream computes for Llama-3.2-1B
(base/src/engine.cu:639-890, tensor names base/src/model.cu:69-82).  Every number
comes from the configuration.
"""

from __future__ import annotations

from ..config.model_config import LlamaConfig
from ..registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def build_llama_spec(cfg: LlamaConfig) -> ModelSpec:
    rope = PartSpec("rope", {
        "head_dim": cfg.head_dim,
        "rotary_dim": cfg.head_dim,
        "theta": cfg.rope_theta,
        "scaling": cfg.rope_scaling.to_dict() if cfg.rope_scaling else None,
    })
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(block="prenorm", parts=dict(
            mixer=PartSpec("attention", {
                "hidden_size": cfg.hidden_size,
                "num_heads": cfg.num_attention_heads,
                "num_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim,
                "window": None,
                "position": rope,
            }, {
                "q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
                "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight",
            }),
            mixer_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                                {"weight": p + "input_layernorm.weight"}),
            feed_forward=PartSpec("swiglu", {
                "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
            }, {
                "gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
                "down": p + "mlp.down_proj.weight",
            }),
            ff_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                             {"weight": p + "post_attention_layernorm.weight"}),
        )))
    embed_name = "model.embed_tokens.weight"
    spec = ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size},
                           {"table": embed_name}),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                            {"weight": "model.norm.weight"}),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size},
                         {"weight": embed_name if cfg.tie_word_embeddings else "lm_head.weight"}),
        eos_token_ids=cfg.eos_token_ids,
    )
    spec.validate()
    return spec


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, build_llama_spec)
