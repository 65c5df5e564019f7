"""The Llama 3 dense decoder, described from parts.

Tensor names are those of the checkpoint format that goes with config.json; the
reference's GGUF names map onto them one to one (internal/engine/engine.go:887-951:
token_embd -> model.embed_tokens, blk.N.attn_q -> model.layers.N.self_attn.q_proj,
attn_k, attn_v, attn_output -> o_proj, attn_norm -> input_layernorm, ffn_gate, ffn_up,
ffn_down -> mlp.*_proj, ffn_norm -> post_attention_layernorm, output_norm -> model.norm,
output -> lm_head).  The attention scale 1/sqrt(head_dim) is the reference's
(internal/device/kernels.metal:673), passed to the attention part as a parameter.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

EMBED = "model.embed_tokens.weight"


def describe(cfg: LlamaConfig) -> ModelSpec:
    position = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta, "scaling": cfg.rope_scaling})
    layers = []
    for i in range(cfg.num_hidden_layers):
        layers.append(LayerSpec(prefix=f"model.layers.{i}.", arrangement="pre_norm", parts=dict(
            norm1=PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                        "name": "input_layernorm.weight"}),
            mixer=PartSpec("attention", {
                "hidden_size": cfg.hidden_size, "n_heads": cfg.num_attention_heads,
                "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                "scale": cfg.head_dim ** -0.5, "position": position, "window": cfg.window_of_layer(i),
                "names": {"q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight",
                          "v": "self_attn.v_proj.weight", "o": "self_attn.o_proj.weight"}}),
            norm2=PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                        "name": "post_attention_layernorm.weight"}),
            ffn=PartSpec("gated_mlp", {
                "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size, "activation": "silu",
                "names": {"gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight",
                          "down": "mlp.down_proj.weight"}}))))
    return ModelSpec(
        name="LlamaForCausalLM",
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                               "name": EMBED}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i, cache=i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps, "name": "model.norm.weight"}),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                      "name": "lm_head.weight", "tied_to": EMBED, "tied": cfg.tie_word_embeddings}),
        max_positions=cfg.max_position_embeddings,
        stop_tokens=tuple(cfg.eos_token_id),
        bos_token=cfg.bos_token_id,
    )


register_architecture("LlamaForCausalLM", LlamaConfig.from_dict, describe)
