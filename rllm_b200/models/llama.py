"""Llama (``LlamaForCausalLM``): the dense GQA decoder rLLM is centred on
(crates/rllm-model/src/llama.rs), as a ``ModelSpec``.

Every layer: pre-norm block, attention with rotary positions (rotate-half,
optionally llama3-rescaled frequencies), SiLU-gated feed-forward, RMSNorm.
Tensor names are the checkpoint's (llama.rs:169, 174, 192-204, 220-228,
234-238, 254).  The output head uses ``lm_head.weight`` if the file has it and
may fall back to the embedding table only when ``tie_word_embeddings`` is set.
"""
from __future__ import annotations

from ..config.model_config import LlamaConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    scaling = cfg.rope_scaling.to_json() if cfg.rope_scaling else None
    position = PartSpec.of("rotary", head_dim=cfg.head_dim, rotary_dim=cfg.head_dim,
                           theta=cfg.rope_theta, scaling=scaling,
                           ignored_tensors=("rotary_emb.inv_freq",))      # older checkpoints store the table
    mixer = PartSpec.of("attention", hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads,
                        num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, window=None,
                        scale=None, position=position, tensor_prefix="self_attn.",
                        tensor_names={"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight",
                                      "o": "o_proj.weight"})
    ffn = PartSpec.of("gated_mlp", hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                      tensor_prefix="mlp.",
                      tensor_names={"gate": "gate_proj.weight", "up": "up_proj.weight",
                                    "down": "down_proj.weight"})
    norms = (PartSpec.of("rmsnorm", size=cfg.hidden_size, eps=cfg.rms_norm_eps, name="input_layernorm.weight"),
             PartSpec.of("rmsnorm", size=cfg.hidden_size, eps=cfg.rms_norm_eps,
                         name="post_attention_layernorm.weight"))
    layers = tuple(LayerSpec(block="pre_norm", mixer=mixer, ffn=ffn, norms=norms,
                             prefix=f"model.layers.{i}.") for i in range(cfg.num_hidden_layers))
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec.of("token_embedding", vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                              name="model.embed_tokens.weight"),
        layers=layers,
        order=tuple(Run(layer=i, cache=i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec.of("rmsnorm", size=cfg.hidden_size, eps=cfg.rms_norm_eps, name="model.norm.weight"),
        head=PartSpec.of("lm_head", vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                         name="lm_head.weight",
                         tied_to="model.embed_tokens.weight" if cfg.tie_word_embeddings else None),
        max_positions=cfg.max_position_embeddings,
        eos_token_ids=cfg.eos_token_ids,
    )


register_architecture("LlamaForCausalLM", LlamaConfig.from_json, llama_spec)
