"""Qwen2 dense decoder as a specification: the one architecture of this library.

Per layer: RMSNorm → grouped-query attention with bias on q, k, v only and rotate-half
RoPE → residual; RMSNorm → SwiGLU → residual; then a final RMSNorm and a linear head that
may be tied to the embedding.  This is what the reference computes when its loader sees
`general.architecture == "qwen2"` (src/gguf_loader.cpp:263-266, 423-425, 436-443;
src/forward.cpp:726-780, 849-853).  Tensor names are the checkpoint's own
(`model.layers.{i}.self_attn.q_proj.weight`, ...); the reference's container uses
`blk.{i}.attn_q.weight` and so on for the same tensors (src/gguf_loader.cpp:16-83).
"""
from __future__ import annotations

from ..config.model_config import ConfigError, ModelConfig
from ..config.registry import register_architecture
from ..config.specs import LayerSpec, ModelSpec, PartSpec, sequential_schedule

LAYER_NAMES = {
    "mixer_norm": "input_layernorm.",
    "mixer": "self_attn.",
    "feed_forward_norm": "post_attention_layernorm.",
    "feed_forward": "mlp.",
}


@register_architecture("Qwen2ForCausalLM")
def qwen2(config: ModelConfig) -> ModelSpec:
    if config.hidden_act != "silu":
        raise ConfigError(f"hidden_act {config.hidden_act!r} is not supported: the feed-forward is SwiGLU with SiLU (src/ops.cpp:94-107)")
    c = config
    norm = PartSpec("norm", "rmsnorm", dict(size=c.hidden_size, eps=c.rms_norm_eps))
    rope = PartSpec("position", "rope_neox", dict(head_dim=c.head_dim, theta=c.rope_theta,
                                                  max_positions=c.max_position_embeddings))
    ffn = PartSpec("feed_forward", "swiglu", dict(hidden_size=c.hidden_size, intermediate_size=c.intermediate_size,
                                                  activation=c.hidden_act))
    layers = []
    for i in range(c.num_hidden_layers):
        attn = PartSpec("mixer", "gqa_attention", dict(
            hidden_size=c.hidden_size, num_heads=c.num_attention_heads, num_kv_heads=c.num_key_value_heads,
            head_dim=c.head_dim, qkv_bias=c.attention_bias, position=rope, window=c.window_of_layer(i)))
        layers.append(LayerSpec(name=f"model.layers.{i}.", block="prenorm", mixer=attn, feed_forward=ffn,
                                mixer_norm=norm, feed_forward_norm=norm, names=LAYER_NAMES))
    return ModelSpec(
        config=c,
        embedding=PartSpec("embedding", "token_embedding", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size)),
        layers=tuple(layers),
        schedule=sequential_schedule(c.num_hidden_layers),
        final_norm=norm,
        head=PartSpec("head", "linear_head", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size,
                                                  tied_to="model.embed_tokens.weight" if c.tie_word_embeddings else None)),
    )
