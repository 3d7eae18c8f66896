"""Typed configuration of the Recursive Flint MoE decoder, read from config.json.

The reference fixes every Flint size at compile time (crates/engine/src/flint.rs:17-34) and checks
them against GGUF metadata (crates/engine/src/flint.rs:219-259); its only dynamic inputs are the
per-layer sliding/rope patterns and the leading dense layer count.  Here every one of those sizes
and switches is a config.json key, nothing is compiled in.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional

ARCHITECTURE = "FlintForCausalLM"


class ConfigError(ValueError):
    """config.json is missing a key, or a key has an impossible value."""


_REQUIRED = (
    "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
    "vocab_size", "n_routed_experts", "num_experts_per_tok", "moe_intermediate_size",
    "rms_norm_eps", "rope_theta",
)


@dataclass
class FlintConfig:
    # sizes: all required, config.json is the only source
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    n_routed_experts: int
    num_experts_per_tok: int
    moe_intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    # options; the default of each is "off" (the plain decoder)
    tie_word_embeddings: bool = False
    scoring_func: str = "softmax"            # "softmax" | "sigmoid" (reference: flint.cu:829-868)
    norm_topk_prob: bool = True              # divide chosen weights by their sum
    qk_norm: bool = False                    # per-head RMSNorm of q and k before RoPE
    qk_norm_eps: Optional[float] = None      # eps of that norm; None: rms_norm_eps (the reference's is the literal 1e-6, flint.cu:139)
    attn_sinks: bool = False                 # learned per-head logit in the softmax denominator
    sliding_window: Optional[int] = None     # keys visible to a sliding layer (reference: 513)
    sliding_window_pattern: Optional[List[bool]] = None   # per layer: True = sliding
    rope_pattern: Optional[List[bool]] = None             # per layer: True = RoPE applied
    n_shared_experts: int = 0
    shared_expert_intermediate_size: int = 0
    first_k_dense_replace: int = 0           # leading layers with a dense SwiGLU MLP
    intermediate_size: int = 0               # width of that dense MLP
    eos_token_id: List[int] = field(default_factory=list)
    torch_dtype: str = "bfloat16"
    # execution order: weight-layer index per executed position; kv_source[p] names an earlier
    # position whose cache position p reads instead of writing its own (None: own cache)
    layer_order: Optional[List[int]] = None
    kv_source: Optional[List[Optional[int]]] = None
    # engine-side hint, not a model size
    kv_page_size: Optional[int] = None
    architectures: List[str] = field(default_factory=lambda: [ARCHITECTURE])

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FlintConfig":
        missing = [k for k in _REQUIRED if k not in d]
        if missing:
            raise ConfigError("config.json lacks required keys: " + ", ".join(missing))
        known = {f.name for f in fields(cls)}
        kw = {k: v for k, v in d.items() if k in known}
        eos = kw.get("eos_token_id", [])
        if eos is None:
            eos = []
        if isinstance(eos, int):
            eos = [eos]
        kw["eos_token_id"] = [int(x) for x in eos]
        cfg = cls(**kw)
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "FlintConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        out = {}
        for f in fields(self):
            out[f.name] = getattr(self, f.name)
        return out

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(self.to_dict(), f, indent=1)

    # ------------------------------------------------------------------ checking
    def validate(self) -> None:
        def need(cond: bool, msg: str) -> None:
            if not cond:
                raise ConfigError(msg)

        L = self.num_hidden_layers
        for k in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                  "head_dim", "vocab_size", "n_routed_experts", "num_experts_per_tok",
                  "moe_intermediate_size"):
            v = getattr(self, k)
            need(isinstance(v, int) and not isinstance(v, bool) and v > 0, f"{k} must be a positive integer, got {v!r}")
        need(self.num_attention_heads % self.num_key_value_heads == 0,
             f"num_attention_heads {self.num_attention_heads} is not a multiple of num_key_value_heads {self.num_key_value_heads}")
        need(self.head_dim % 16 == 0 and self.head_dim <= 256,
             f"head_dim {self.head_dim}: the attention kernels take multiples of 16 up to 256")
        need(self.num_experts_per_tok <= self.n_routed_experts,
             f"num_experts_per_tok {self.num_experts_per_tok} exceeds n_routed_experts {self.n_routed_experts}")
        need(self.rms_norm_eps > 0, "rms_norm_eps must be positive")
        need(self.qk_norm_eps is None or self.qk_norm_eps > 0, "qk_norm_eps must be positive")
        need(self.rope_theta > 0, "rope_theta must be positive")
        need(self.scoring_func in ("softmax", "sigmoid"), f"scoring_func {self.scoring_func!r} is neither 'softmax' nor 'sigmoid'")
        need(self.torch_dtype in ("bfloat16", "float32"), f"torch_dtype {self.torch_dtype!r} is neither 'bfloat16' nor 'float32'")
        need(self.architectures and isinstance(self.architectures, list), "architectures must be a non-empty list")
        for name in ("sliding_window_pattern", "rope_pattern"):
            p = getattr(self, name)
            if p is not None:
                need(len(p) == L, f"{name} has {len(p)} entries for {L} layers")
                setattr(self, name, [bool(x) for x in p])
        if self.sliding_window_pattern is not None and any(self.sliding_window_pattern):
            need(isinstance(self.sliding_window, int) and self.sliding_window > 0,
                 "sliding_window_pattern marks sliding layers but sliding_window is not a positive integer")
        need(0 <= self.first_k_dense_replace <= L, f"first_k_dense_replace {self.first_k_dense_replace} outside 0..{L}")
        if self.first_k_dense_replace > 0:
            need(self.intermediate_size > 0, "first_k_dense_replace > 0 needs intermediate_size")
        need(self.n_shared_experts in (0, 1),
             f"n_shared_experts {self.n_shared_experts}: one ungated shared expert (of shared_expert_intermediate_size) or none is built")
        if self.n_shared_experts > 0:
            need(self.shared_expert_intermediate_size > 0, "n_shared_experts > 0 needs shared_expert_intermediate_size")
        for t in self.eos_token_id:
            need(0 <= t < self.vocab_size, f"eos_token_id {t} outside the vocabulary")
        order = self.execution_order()
        need(len(order) > 0, "layer_order is empty")
        for i in order:
            need(isinstance(i, int) and 0 <= i < L, f"layer_order names layer {i!r}; there are {L}")
        src = self.kv_sources()
        need(len(src) == len(order), f"kv_source has {len(src)} entries for {len(order)} executed layers")
        for p, s in enumerate(src):
            if s is None:
                continue
            need(isinstance(s, int) and 0 <= s < p, f"kv_source[{p}] = {s!r} must name an earlier position")
            need(src[s] is None, f"kv_source[{p}] = {s} names a position that itself borrows a cache")
            need(self.layer_is_sliding(order[p]) == self.layer_is_sliding(order[s]),
                 f"kv_source[{p}] = {s}: a sliding layer and a full layer cannot share a cache")
        if self.kv_page_size is not None:
            need(isinstance(self.kv_page_size, int) and self.kv_page_size > 0, "kv_page_size must be a positive integer")

    # ------------------------------------------------------------------ derived
    def execution_order(self) -> List[int]:
        return list(self.layer_order) if self.layer_order is not None else list(range(self.num_hidden_layers))

    def kv_sources(self) -> List[Optional[int]]:
        n = len(self.execution_order())
        return list(self.kv_source) if self.kv_source is not None else [None] * n

    def layer_is_sliding(self, layer: int) -> bool:
        return bool(self.sliding_window_pattern[layer]) if self.sliding_window_pattern is not None else False

    def layer_has_rope(self, layer: int) -> bool:
        return bool(self.rope_pattern[layer]) if self.rope_pattern is not None else True

    def layer_is_dense(self, layer: int) -> bool:
        return layer < self.first_k_dense_replace
