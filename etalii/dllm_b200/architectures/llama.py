"""The Llama architecture as data: which parts each layer has, with sizes and constants from `LlamaConfig`, and the
checkpoint's tensor names (Hugging Face names, src/etalii_dllm/importing/importer.py:74-113). Every layer is
RMSNorm -> grouped-query attention with rotary positions -> RMSNorm -> SwiGLU, pre-norm arrangement, no biases
(src/etalii_dllm/transformer.py:493-562)."""
from __future__ import annotations

import math

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def build_spec(config: LlamaConfig) -> ModelSpec:
    hidden = config.hidden_size
    position = PartSpec("rotary", {
        "head_dim": config.head_dim, "theta": config.rope_theta,
        "scaling": None if config.rope_scaling is None else config.rope_scaling.to_hf(),
    })
    layers = []
    for index in range(config.num_hidden_layers):
        p = f"model.layers.{index}."
        layers.append(LayerSpec(
            mixer=PartSpec("attention", {
                "hidden_size": hidden, "num_heads": config.num_attention_heads,
                "num_kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
                "scale": 1.0 / math.sqrt(config.head_dim),  # src/etalii_dllm/architecture.py:310-312
                "window": None, "position": position,
            }, {"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
                "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight"}),
            feed_forward=PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": config.intermediate_size},
                                  {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
                                   "down": p + "mlp.down_proj.weight"}),
            mixer_norm=PartSpec("rmsnorm", {"hidden_size": hidden, "eps": config.rms_norm_eps},
                                {"weight": p + "input_layernorm.weight"}),
            feed_forward_norm=PartSpec("rmsnorm", {"hidden_size": hidden, "eps": config.rms_norm_eps},
                                       {"weight": p + "post_attention_layernorm.weight"}),
            block="pre_norm",
        ))
    tied = config.tie_word_embeddings
    return ModelSpec(
        vocab_size=config.vocab_size,
        hidden_size=hidden,
        max_position=config.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab_size, "hidden_size": hidden},
                           {"weight": "model.embed_tokens.weight"}),
        layers=tuple(layers),
        final_norm=PartSpec("rmsnorm", {"hidden_size": hidden, "eps": config.rms_norm_eps},
                            {"weight": "model.norm.weight"}),
        head=PartSpec("linear", {"vocab_size": config.vocab_size, "hidden_size": hidden},
                      {"weight": "model.embed_tokens.weight" if tied else "lm_head.weight"}),
        stop_token_ids=tuple(config.eos_token_ids),
        # a tied checkpoint may still store its head; it must then equal the embedding (importer.py:1279-1283)
        equal_if_present={"lm_head.weight": "model.embed_tokens.weight"} if tied else {},
        ignored_suffixes=("rotary_emb.inv_freq",),  # importer.py:534-535
    )


register_architecture("llama", LlamaConfig, build_spec)
