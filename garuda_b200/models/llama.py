"""The dense Llama decoder (TinyLlama family) as a ``ModelSpec``.

garuda/src/llama/mod.rs: pre-norm blocks of grouped-query attention with rotary
positions and a SwiGLU feed-forward (:851-893), RMS norms (:733-738), a final
norm and an output head that is the embedding table itself when the checkpoint
has none (:563-572). Tensor names are those of a safetensors Llama folder; the
reference's GGUF names for the same tensors are at :562-621.
"""
from __future__ import annotations

from ..config.model_config import LlamaConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from ..parts.block import BlockSpec
from .decoder import ModelSpec, LayerCall


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    norm_init = ("ones",)
    std = float(cfg.extra.get("initializer_range", 0.02))
    position = {"name": "rotary",
                "params": {"theta": cfg.rope_theta, "head_dim": cfg.head_dim, "layout": cfg.rope_layout}}
    layers = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        layers.append(BlockSpec(
            mixer=PartSpec("paged_attention", dict(
                width=cfg.hidden_size, heads=cfg.num_attention_heads, kv_heads=cfg.num_key_value_heads,
                head_dim=cfg.head_dim, position=position, window=cfg.layer_window(l), init_std=std),
                prefix=p + "self_attn."),
            feed_forward=PartSpec("swiglu", dict(width=cfg.hidden_size, inner=cfg.intermediate_size,
                                                 init_std=std), prefix=p + "mlp."),
            mixer_norm=PartSpec("rms", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps,
                                            weight_init=norm_init), prefix=p + "input_layernorm."),
            feed_forward_norm=PartSpec("rms", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps,
                                                   weight_init=norm_init),
                                       prefix=p + "post_attention_layernorm."),
        ))
    return ModelSpec(
        architecture=cfg.architecture, width=cfg.hidden_size, vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings, embedding="model.embed_tokens.weight",
        layers=layers, order=[LayerCall(l) for l in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rms", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps,
                                        weight_init=norm_init), prefix="model.norm."),
        head=None if cfg.tie_word_embeddings else "lm_head.weight",
        embedding_init=("normal", std), eos_token_ids=cfg.eos_token_ids,
        ignored_tensors=("lm_head.weight",) if cfg.tie_word_embeddings else (),
    )


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_spec)
