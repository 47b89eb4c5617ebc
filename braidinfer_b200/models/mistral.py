"""The dense Mistral decoder as a description of parts.

token embedding -> L x [RMSNorm -> grouped-query attention (rotary, causal, optional
window) -> + -> RMSNorm -> SwiGLU -> +] -> RMSNorm -> output head.  Tensor names are the
ones Mistral model folders use (reference loader:
crates/braidinfer-runtime/src/model/model_load.rs:387-399 embedding, head, final norm;
:620-746 attention layer; layer order
crates/braidinfer-runtime/src/megakernel/megakernel_compile.rs:115-236).
"""
from __future__ import annotations

from ..config.mistral import MistralConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import Architecture, register_architecture


def build_mistral_spec(cfg: MistralConfig) -> ModelSpec:
    layers = []
    for i in range(cfg.num_hidden_layers):
        rope = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                 "rope_dim": cfg.rope_dim, "pairing": cfg.rope_pairing})
        mixer = PartSpec("gqa_attention", {
            "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "window": cfg.layer_window(i), "position_encoding": rope})
        ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
        layers.append(LayerSpec(
            block="prenorm_residual", prefix=f"model.layers.{i}.", mixer=mixer,
            mixer_norm=PartSpec("rmsnorm", {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                            "name": "input_layernorm.weight"}),
            feed_forward=ffn,
            feed_forward_norm=PartSpec("rmsnorm", {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                                   "name": "post_attention_layernorm.weight"})))
    return ModelSpec(
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                               "name": "model.embed_tokens.weight"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                        "name": "model.norm.weight"}),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                      "name": "lm_head.weight", "tied": cfg.tie_word_embeddings}),
        max_position=cfg.max_position_embeddings,
        eos_token_ids=tuple(cfg.eos_token_id or ()), bos_token_id=cfg.bos_token_id)


MISTRAL = register_architecture(Architecture(
    name="MistralForCausalLM", config_from_dict=MistralConfig.from_dict, build_spec=build_mistral_spec))
