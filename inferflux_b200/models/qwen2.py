"""``Qwen2ForCausalLM`` as a spec: the one file that knows this architecture.

What the reference's forward does for this model
(runtime/backends/cuda/native/transformer_forward.cu:1341-2202) and which
tensors it binds (runtime/backends/cuda/native/weight_map.cpp:21-58):
token embedding; per layer a pre-norm block of grouped-query attention with
q/k/v biases and no output bias, rotate-half rotary positions over the whole
head, and a SwiGLU feed-forward; a final RMSNorm; an output head that is the
embedding table when ``tie_word_embeddings`` is set.  Layers at or above
``max_window_layers`` attend within ``sliding_window`` when
``use_sliding_window`` is set (keys the reference never reads,
runtime/backends/cuda/inferflux_cuda_executor.cpp:524-604).
"""
from __future__ import annotations

from ..config.model_config import Qwen2Config
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, Run


def build_qwen2_spec(cfg: Qwen2Config) -> ModelSpec:
    h = cfg.hidden_size
    layers = []
    for i in range(cfg.num_hidden_layers):
        layers.append(LayerSpec(
            prefix=f"model.layers.{i}",
            arrangement="prenorm",
            parts=dict(
                mixer=PartSpec("gqa_attention", dict(
                    name="self_attn", hidden=h, n_heads=cfg.num_attention_heads,
                    n_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                    qkv_bias=True, o_bias=False, window=cfg.window_of_layer(i))),
                mixer_norm=PartSpec("rmsnorm", dict(name="input_layernorm", hidden=h, eps=cfg.rms_norm_eps)),
                feed_forward=PartSpec("swiglu", dict(name="mlp", hidden=h, intermediate=cfg.intermediate_size)),
                feed_forward_norm=PartSpec("rmsnorm", dict(name="post_attention_layernorm", hidden=h,
                                                           eps=cfg.rms_norm_eps))),
            position="rope",
        ))
    return ModelSpec(
        architecture=Qwen2Config.ARCHITECTURE,
        hidden_size=h,
        vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", dict(name="model.embed_tokens", vocab=cfg.vocab_size, hidden=h)),
        final_norm=PartSpec("rmsnorm", dict(name="model.norm", hidden=h, eps=cfg.rms_norm_eps)),
        lm_head=PartSpec("linear_head", dict(
            name="lm_head", vocab=cfg.vocab_size, hidden=h,
            tied_to="model.embed_tokens.weight" if cfg.tie_word_embeddings else None)),
        positions={"rope": PartSpec("rotary_half", dict(rotary_dim=cfg.head_dim, theta=cfg.rope_theta))},
        layers=layers,
        schedule=[Run(i) for i in range(cfg.num_hidden_layers)],
    )


register_architecture(Qwen2Config.ARCHITECTURE, Qwen2Config, build_qwen2_spec, model_type=Qwen2Config.MODEL_TYPE)
