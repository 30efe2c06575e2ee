"""Qwen3 dense decoder: from its typed config to a :class:`ModelSpec`.

The layer this builds is the one the reference's decoder recipe emits when every mixer
is `Attention{qk_norm: true, output_gate: false}` and the feed-forward is `Dense`
(crates/model/recipes/src/decoder.rs:93-154, :229-364, :467-502): pre-norm RMSNorm,
q/k/v projections, per-head q/k RMSNorm before RoPE, causal grouped-query attention,
output projection and residual, RMSNorm, SwiGLU and residual.  Tensor names are the
checkpoint's own (decoder.rs:55-64, :104-149); `lm_head.weight` lives at the file's
root, everything else under one of the prefixes the provider lists
(crates/model/package/src/providers/qwen/mod.rs:371-374).

Nothing below is Qwen-specific except the mapping itself: the parts are chosen by
`kind` and take every size and constant as a parameter.
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..config.registry import Architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec


def build_spec(cfg: Qwen3Config) -> ModelSpec:
    norm = PartSpec.make("rms", eps=cfg.rms_norm_eps)
    layers = []
    for i in range(cfg.num_hidden_layers):
        position = PartSpec.make(
            "rope_neox", theta=cfg.rope_theta, rotary_dim=cfg.rotary_dim,
            head_dim=cfg.head_dim)
        mixer = PartSpec.make(
            "gqa_attention",
            hidden_size=cfg.hidden_size,
            num_heads=cfg.num_attention_heads,
            num_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim,
            qk_norm=True,
            qk_norm_eps=cfg.rms_norm_eps,
            bias=cfg.attention_bias,
            window=cfg.layer_window(i),
            max_positions=cfg.max_position_embeddings,
            position=position,
        )
        ffn = PartSpec.make(
            "swiglu", hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size)
        layers.append(LayerSpec(
            prefix=f"layers.{i}.",
            block=PartSpec.make(
                "pre_norm", hidden_size=cfg.hidden_size,
                mixer_prefix="self_attn.", ffn_prefix="mlp.",
                mixer_norm="input_layernorm.", ffn_norm="post_attention_layernorm."),
            mixer=mixer, feed_forward=ffn, norm=norm))
    return ModelSpec(
        architecture="Qwen3ForCausalLM",
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_positions=cfg.max_position_embeddings,
        embedding_name="embed_tokens.weight",
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        final_norm_name="norm.weight",
        final_norm=norm,
        layers=tuple(layers),
        weight_prefixes=("model.language_model.", "model.", ""),
    )


ARCHITECTURE = Architecture(
    name="qwen3-dense",
    claims=("Qwen3ForCausalLM", "qwen3"),
    read_config=Qwen3Config.from_dict,
    build_spec=build_spec,
)
