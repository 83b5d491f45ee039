"""The Llama dense decoder as a description: which parts each layer has, with what
numbers, and what the checkpoint calls their tensors.

Tensor names are those the reference binds (thinruntime/gpu_runtime.py:3979-3991 per
layer; ``model.embed_tokens.weight``, ``model.norm.weight`` and ``lm_head.weight`` at
thinruntime/execution_plan.py:167-186), the layer is its ``separate_qkv_gated_dense``
schema (thinruntime/execution_plan.py:136-164) and the registry entry it replaces is
thinruntime/architectures.py:90-115.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run

EMBEDDING_NAME = "model.embed_tokens.weight"


def describe_llama(config: LlamaConfig) -> ModelSpec:
    rope = PartSpec("rope", {
        "head_dim": config.head_dim,
        "theta": config.rope_theta,
        "scaling": config.rope_scaling.to_dict() if config.rope_scaling else None,
    })
    layers = []
    for index in range(config.num_hidden_layers):
        prefix = f"model.layers.{index}."
        layers.append(LayerSpec("pre_norm", {
            "mixer_norm": PartSpec("rmsnorm", {"dim": config.hidden_size, "eps": config.rms_norm_eps}, prefix + "input_layernorm."),
            "mixer": PartSpec("attention", {
                "hidden": config.hidden_size,
                "heads": config.num_attention_heads,
                "kv_heads": config.num_key_value_heads,
                "head_dim": config.head_dim,
                "position": rope,
                "bias": config.attention_bias,
            }, prefix + "self_attn."),
            "ffn_norm": PartSpec("rmsnorm", {"dim": config.hidden_size, "eps": config.rms_norm_eps}, prefix + "post_attention_layernorm."),
            "ffn": PartSpec("swiglu", {"hidden": config.hidden_size, "inter": config.intermediate_size, "bias": config.mlp_bias}, prefix + "mlp."),
        }))
    return ModelSpec(
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        embedding=PartSpec("table", {"vocab": config.vocab_size, "hidden": config.hidden_size}, "model.embed_tokens."),
        layers=tuple(layers),
        schedule=tuple(Run(i) for i in range(config.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"dim": config.hidden_size, "eps": config.rms_norm_eps}, "model.norm."),
        head=PartSpec("linear", {
            "hidden": config.hidden_size,
            "vocab": config.vocab_size,
            "fallback": EMBEDDING_NAME,     # the reference uses the table when no head is stored
            "tied": config.tie_word_embeddings,
        }, "lm_head."),
    )


register_architecture(Architecture(
    name="LlamaForCausalLM",
    model_types=("llama", "tinyllama"),
    config_class=LlamaConfig,
    describe=describe_llama,
))
