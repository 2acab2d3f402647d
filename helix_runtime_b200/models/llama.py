"""The Llama-style MHA decoder as a list of parts (src/model/cpu_llama.cpp:37-110).

Every layer is the same block: RMSNorm, attention with equal query and key/value
heads and adjacent-pair rotary encoding, RMSNorm, SwiGLU feed-forward, two
residuals.  Tensor names are the checkpoint's (tools/convert_hf_llama.py:400-510),
whose q/k rows are ordered for half-split rotation; the attention part permutes them
at load so that the kernel rotates adjacent pairs as the reference does.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..config.spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry


def build_llama_spec(config: LlamaConfig) -> ModelSpec:
    hidden = config.hidden_size
    position = PartSpec("rotary", {
        "theta": config.rope_theta,
        "head_dim": config.head_dim,
        "rotary_dim": config.head_dim,
        "pairing": "adjacent",
        "max_positions": config.max_position_embeddings,
    })
    blocks = []
    for layer in range(config.num_hidden_layers):
        prefix = f"model.layers.{layer}"
        blocks.append(BlockSpec(
            arrangement="pre_norm",
            mixer_norm=PartSpec("rms", {"eps": config.rms_norm_eps},
                                {"weight": f"{prefix}.input_layernorm.weight"}),
            mixer=PartSpec("paged_attention", {
                "num_heads": config.num_attention_heads,
                "num_kv_heads": config.num_key_value_heads,
                "head_dim": config.head_dim,
                "scale": None,
                "window": None,
                "position": position,
                "checkpoint_pairing": "half_split",
            }, {
                "q": f"{prefix}.self_attn.q_proj.weight",
                "k": f"{prefix}.self_attn.k_proj.weight",
                "v": f"{prefix}.self_attn.v_proj.weight",
                "o": f"{prefix}.self_attn.o_proj.weight",
            }),
            feed_forward_norm=PartSpec("rms", {"eps": config.rms_norm_eps},
                                       {"weight": f"{prefix}.post_attention_layernorm.weight"}),
            feed_forward=PartSpec("gated_mlp", {
                "intermediate_size": config.intermediate_size,
                "activation": "silu",
            }, {
                "gate": f"{prefix}.mlp.gate_proj.weight",
                "up": f"{prefix}.mlp.up_proj.weight",
                "down": f"{prefix}.mlp.down_proj.weight",
            }),
        ))
    return ModelSpec(
        architecture=config.architecture,
        hidden_size=hidden,
        vocab_size=config.vocab_size,
        max_positions=config.max_position_embeddings,
        embedding=PartSpec("token_table", {"vocab_size": config.vocab_size},
                           {"weight": "model.embed_tokens.weight"}),
        blocks=tuple(blocks),
        schedule=tuple(ScheduleEntry(block=layer) for layer in range(config.num_hidden_layers)),
        final_norm=PartSpec("rms", {"eps": config.rms_norm_eps}, {"weight": "model.norm.weight"}),
        lm_head=PartSpec("linear", {"vocab_size": config.vocab_size,
                                    "tied": config.tie_word_embeddings},
                         {"weight": "lm_head.weight", "tied_to": "model.embed_tokens.weight"}),
    )


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, build_llama_spec,
                      aliases=("llama",))
