"""Llama, as a description made of the library's parts.

Pre-norm decoder: x -> [RMSNorm -> causal grouped-query attention with RoPE -> +x]
-> [RMSNorm -> SwiGLU feed-forward -> +x] per layer, then RMSNorm and the
classifier (src/model.rs:1244-1366).  Tensor names are those of a checkpoint
with Hugging Face Llama naming; such checkpoints pair rotary dimensions
(j, j + head_dim/2), where the reference's own formats pair neighbours
(src/model.rs:1953-1991).
"""

from __future__ import annotations

from ..config.llama import ARCHITECTURE, LlamaConfig
from ..registry import Architecture, register_architecture
from ..spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def describe_llama(cfg: LlamaConfig) -> ModelSpec:
    position = PartSpec(
        "rotary",
        {
            "rotary_dim": cfg.head_dim,
            "theta": cfg.rope_theta,
            "scaling": cfg.rope_scaling,
            "interleaved": False,
        },
    )

    def norm(prefix: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, prefix)

    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(
            LayerSpec(
                block="prenorm",
                mixer=PartSpec(
                    "attention",
                    {
                        "hidden_size": cfg.hidden_size,
                        "num_heads": cfg.num_attention_heads,
                        "num_kv_heads": cfg.num_key_value_heads,
                        "head_dim": cfg.head_dim,
                        "window": 0,
                        "position": position,
                    },
                    p + "self_attn.",
                ),
                feed_forward=PartSpec(
                    "gated_mlp",
                    {
                        "hidden_size": cfg.hidden_size,
                        "intermediate_size": cfg.intermediate_size,
                        "activation": "silu",
                    },
                    p + "mlp.",
                ),
                norms={
                    "mixer": norm(p + "input_layernorm."),
                    "feed_forward": norm(p + "post_attention_layernorm."),
                },
            )
        )
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec(
            "token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}, "model.embed_tokens."
        ),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm("model.norm."),
        head=PartSpec(
            "linear_head",
            {
                "vocab_size": cfg.vocab_size,
                "hidden_size": cfg.hidden_size,
                # A tied model has no lm_head tensor: the classifier is a second
                # view of the embedding matrix (src/model.rs:469-473).
                "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None,
            },
            "lm_head.",
        ),
        stop_token_ids=cfg.eos_token_ids,
        stored_dtype=cfg.torch_dtype,
        # Llama folders often carry the rotary tables as buffers (they are recomputed here from theta and
        # the scaling) and, beside tied embeddings, a second copy of the matrix as lm_head.weight
        redundant_tensors=("*.rotary_emb.inv_freq",) + (("lm_head.weight",) if cfg.tie_word_embeddings else ()),
    )


register_architecture(Architecture(ARCHITECTURE, LlamaConfig.from_json, describe_llama), replace=True)
