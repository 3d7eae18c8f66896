"""Recursive Flint MoE: from its typed configuration to the architecture-neutral ModelSpec.

Per layer (crates/engine/src/flint.rs:815-1075): RMSNorm, GQA self-attention (optional QK-norm,
RoPE per the layer's flag, sinks, full or sliding window per the layer's flag), RMSNorm, then a
dense SwiGLU MLP in the leading `first_k_dense_replace` layers and routed SwiGLU experts (with an
optional ungated shared expert) in the rest; a final RMSNorm and the LM head.  Tensor names are
the Hugging Face style ones listed in `tensor_names` below.
"""
from __future__ import annotations

import re
from typing import Optional

from ..config.flint import ARCHITECTURE, FlintConfig
from ..config.registry import register_architecture
from ..spec import LayerSpec, ModelSpec, PartSpec


# The reference's tensor names (GGUF, crates/engine/src/flint.rs:270-375) -> the names declared here.  Its expert
# tensors are stacked as [E*I, D] (gate, up) and [E*D, I] (down), which the loader takes for the declared
# [E, I, D] and [E, D, I].
_GGUF_TOP = {"token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight", "output.weight": "lm_head.weight"}
_GGUF_LAYER = {
    "attn_norm.weight": "input_layernorm.weight", "ffn_norm.weight": "post_attention_layernorm.weight",
    "attn_q.weight": "self_attn.q_proj.weight", "attn_k.weight": "self_attn.k_proj.weight", "attn_v.weight": "self_attn.v_proj.weight",
    "attn_output.weight": "self_attn.o_proj.weight", "attn_q_norm.weight": "self_attn.q_norm.weight",
    "attn_k_norm.weight": "self_attn.k_norm.weight", "attn_sinks.weight": "self_attn.sinks", "ffn_gate_inp.weight": "mlp.gate.weight",
    "ffn_gate_exps.weight": "mlp.experts.gate_proj.weight", "ffn_up_exps.weight": "mlp.experts.up_proj.weight",
    "ffn_down_exps.weight": "mlp.experts.down_proj.weight", "ffn_gate_shexp.weight": "mlp.shared_experts.gate_proj.weight",
    "ffn_up_shexp.weight": "mlp.shared_experts.up_proj.weight", "ffn_down_shexp.weight": "mlp.shared_experts.down_proj.weight",
    "ffn_gate.weight": "mlp.gate_proj.weight", "ffn_up.weight": "mlp.up_proj.weight", "ffn_down.weight": "mlp.down_proj.weight",
}
_GGUF_BLOCK = re.compile(r"^blk\.(\d+)\.(.+)$")
# experts stored one by one, as checkpoints of this family of models usually hold them
_ONE_EXPERT = re.compile(r"^(model\.layers\.\d+\.mlp\.experts)\.(\d+)\.((?:gate|up|down)_proj\.weight)$")


def gguf_alias(name: str):
    """The declared name of a tensor stored under another name, or None: the reference's GGUF
    names, and `...mlp.experts.{e}.{gate,up,down}_proj.weight` -> (the stacked tensor's name, e),
    which the loader stacks as it reads (the reference addresses its stacked expert tensors
    expert by expert the other way round, crates/engine/src/flint.rs:358-364)."""
    m = _ONE_EXPERT.match(name)
    if m:
        return f"{m.group(1)}.{m.group(3)}", int(m.group(2))
    if name in _GGUF_TOP:
        return _GGUF_TOP[name]
    m = _GGUF_BLOCK.match(name)
    if m and m.group(2) in _GGUF_LAYER:
        return f"model.layers.{m.group(1)}.{_GGUF_LAYER[m.group(2)]}"
    return None


def build_spec(cfg: FlintConfig, norm_init: str = "ones") -> ModelSpec:
    layers = []
    for i in range(cfg.num_hidden_layers):
        pos = (PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta}) if cfg.layer_has_rope(i)
               else PartSpec("none", {"head_dim": cfg.head_dim}))
        mixer = PartSpec("attention", {
            "num_heads": cfg.num_attention_heads, "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "eps": cfg.qk_norm_eps if cfg.qk_norm_eps is not None else cfg.rms_norm_eps, "pos": pos, "window": cfg.sliding_window if cfg.layer_is_sliding(i) else None,
            "sinks": cfg.attn_sinks, "qk_norm": cfg.qk_norm, "norm_init": norm_init})
        if cfg.layer_is_dense(i):
            ffn = PartSpec("dense", {"intermediate_size": cfg.intermediate_size})
        else:
            ffn = PartSpec("moe", {
                "num_experts": cfg.n_routed_experts, "top_k": cfg.num_experts_per_tok,
                "intermediate_size": cfg.moe_intermediate_size, "scoring": cfg.scoring_func,
                "renormalize": cfg.norm_topk_prob,
                "shared_intermediate_size": cfg.shared_expert_intermediate_size if cfg.n_shared_experts > 0 else 0})
        layers.append(LayerSpec(prefix=f"model.layers.{i}.", mixer=mixer, ffn=ffn,
                                norm=PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps, "init": norm_init})))
    return ModelSpec(hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, layers=layers,
                     order=cfg.execution_order(), kv_source=cfg.kv_sources(),
                     final_norm=PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps, "init": norm_init}),
                     head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
                     eos_token_ids=tuple(cfg.eos_token_id), name_alias=gguf_alias)


register_architecture(ARCHITECTURE, FlintConfig, build_spec, aliases=("flint",))
