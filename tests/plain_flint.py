"""Plain, slow implementation of the Recursive Flint MoE decoder: the yardstick of the tests.

It rests on the reference's formulas only (file:line given at each function; paths are those of
lkarlslund/quench6k).  The reference's own Flint code could not be run here: its host is Rust
(no cargo/rustc in this environment), its kernels are CUDA for sm_120a with NVFP4 weights and
sizes fixed at compile time, and its Python oracle (tools/ref/ref.py) covers another architecture
and hard-codes a CUDA device.  So there is no golden output of the reference itself.

Whole sequences, no cache, one function per part, plain tensor arithmetic in float64 by default,
on the CPU unless a test with large layers asks for the device its weights are on.  It shares
no code with quench6k_b200: it reads config.json as a plain dict and the weights as a dict of
tensors by name.

`emulate_bf16=True` rounds to bfloat16 at the places where the reference's arithmetic does
(normed activations, q, cached k and v, softmax probabilities, attention output, the SwiGLU
activation; weights are bfloat16 already), so that a bfloat16 engine can be compared tightly.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np
import torch


def _r(x: torch.Tensor, emulate: bool) -> torch.Tensor:
    """Round to bfloat16 and back when emulating the reference's storage precision."""
    return x.to(torch.bfloat16).to(x.dtype) if emulate else x


# --------------------------------------------------------------------------- parts
def embed(tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """h[t] = f32(table[tok[t]]), no scaling.  crates/cuda/kernels/flint.cu:89-95"""
    return table[tokens.long()]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w with the plain weight (not 1 + w), mean over the last axis.
    crates/cuda/kernels/flint.cu:97-122 (rows of the stream), :138-140 (per head, for q and k)"""
    return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def rope_neox(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half RoPE over the full head: i = d mod hd/2, inv = theta^(-2i/hd), a = pos * inv;
    d < hd/2: x[d] cos a - x[d+hd/2] sin a; else x[d] cos a + x[d-hd/2] sin a.
    x: [T, H, hd].  crates/cuda/kernels/flint.cu:141-149

    The angle is a 32-bit quantity there (inv and the product pos * inv are floats) and so it is
    here: inv is rounded to float32, and so is its product with the position (an angle of
    thousands of radians carries a rounding of 1e-4 rad that way, which is part of what is
    computed); the cosine and sine of that angle and the rotation are in x's precision.  (The
    reference gets inv from exp2f(-(2i/hd) * log2(theta)) on the device, which differs from the
    rounded exact value by an ulp in half of the dimensions; no output of it exists to compare with.)"""
    hd = x.shape[-1]
    half = hd // 2
    i = torch.arange(half, dtype=torch.float64, device=x.device)
    inv = (theta ** (-(2.0 * i) / hd)).to(torch.float32)
    a = (positions.to(torch.float32)[:, None] * inv[None, :]).to(x.dtype)       # [T, half], a float32 product
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    lo, hi = x[..., :half], x[..., half:]
    return torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int],
              sinks: Optional[torch.Tensor], emulate: bool) -> torch.Tensor:
    """Grouped-query causal attention over one whole sequence.
    q: [T, Hq, hd], k, v: [T, Hkv, hd].  Query head h uses KV head h // (Hq/Hkv)
    (flint.cu:225-245); score = q.k / sqrt(hd) (:325); key j is visible to the query at position p
    iff j <= p and, with a window W, j > p - W (:178, :315-322, :370-374); a sink adds
    exp(sink_h - m) to the denominator only (:505-526, :549-560); probabilities are rounded to
    bfloat16 before they are summed (:409-415) when emulating."""
    T, Hq, hd = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    pos = torch.arange(T, device=q.device)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= pos[None, :] > pos[:, None] - window
    out = torch.empty_like(q)
    for h in range(Hq):
        kh = h // G
        s = (q[:, h, :] @ k[:, kh, :].T) / math.sqrt(hd)
        s = s.masked_fill(~visible, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        if sinks is not None:
            m = torch.maximum(m, sinks[h].expand_as(m))
        p = _r(torch.exp(s - m), emulate)
        den = p.sum(dim=-1, keepdim=True)
        if sinks is not None:
            den = den + torch.exp(sinks[h] - m)
        out[:, h, :] = (p @ v[:, kh, :]) / den
    return out


_last_route_margin = None      # set by route(): per token, (k-th logit - (k+1)-th logit) / rms of the token's router logits


_last_router = None            # set by route(): (the router logits [T, E], this router's own choice [T, k])


def route(logits: torch.Tensor, scoring: str, top_k: int, renorm: bool, forced: Optional[torch.Tensor] = None):
    """Router scores, the top-k experts (ties -> lower expert index) and their weights.
    sigmoid: score = 1/(1+exp(-z)), weights = score / (sum of chosen + 1e-20)
    (crates/cuda/kernels/flint.cu:829-864).  softmax: softmax over all experts, top-k, divided by
    the chosen sum (crates/cuda/kernels/moe.cu:19-71).  Without renormalisation the scores stand.
    forced [T, k]: the experts to use instead of the router's own choice, in this slot order; the
    weights are still this function's scores of those experts."""
    if scoring == "sigmoid":
        score = 1.0 / (1.0 + torch.exp(-logits))
    elif scoring == "softmax":
        score = torch.softmax(logits, dim=-1)
    else:
        raise ValueError(scoring)
    ranked = torch.sort(score, dim=-1, descending=True, stable=True)
    order = ranked.indices[:, :top_k]
    global _last_route_margin, _last_router
    _last_router = (logits, order)
    if forced is not None:
        order = forced.to(device=order.device, dtype=order.dtype)
    w = torch.gather(score, 1, order)
    if score.shape[-1] > top_k:
        # both scorings are monotone in the logit, so the choice is the order of the logits
        z = torch.sort(logits, dim=-1, descending=True).values
        _last_route_margin = (z[:, top_k - 1] - z[:, top_k]) / logits.pow(2).mean(dim=-1).sqrt()
    else:
        _last_route_margin = torch.full((score.shape[0],), float("inf"), dtype=score.dtype, device=score.device)
    if renorm:
        s = w.sum(dim=-1, keepdim=True)
        w = w / (s + 1e-20) if scoring == "sigmoid" else w / s
    return order, w


def silu(x: torch.Tensor) -> torch.Tensor:
    """x / (1 + exp(-x)).  crates/cuda/kernels/common.cuh:13"""
    return x / (1.0 + torch.exp(-x))


def swiglu_mlp(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor, emulate: bool) -> torch.Tensor:
    """Wd . (silu(Wg x) * (Wu x)); the activation is rounded to bfloat16 when emulating
    (crates/cuda/kernels/flint.cu:1221-1226).  Weights are [out, in]."""
    act = _r(silu(x @ wg.T) * (x @ wu.T), emulate)
    return act @ wd.T


def moe(x: torch.Tensor, router_w: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor,
        scoring: str, top_k: int, renorm: bool, emulate: bool, forced: Optional[torch.Tensor] = None) -> torch.Tensor:
    """sum over the chosen experts, in slot order, of w_r * expert_r(x).
    crates/cuda/kernels/flint.cu:1228-1239 (combine), :829-868 (route).  wg, wu: [E, I, D], wd: [E, D, I]."""
    sel, w = route(x @ router_w.T, scoring, top_k, renorm, forced)
    out = torch.zeros_like(x)
    chosen = sel.tolist()
    for t in range(x.shape[0]):
        acc = torch.zeros_like(x[t])
        for r in range(top_k):
            e = chosen[t][r]
            acc = acc + w[t, r] * swiglu_mlp(x[t:t + 1], wg[e], wu[e], wd[e], emulate)[0]
        out[t] = acc
    return out


# --------------------------------------------------------------------------- whole model
def forward(cfg: Dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            emulate_bf16: bool = False, return_margins: bool = False, forced_routing: Optional[Dict[int, torch.Tensor]] = None,
            logit_positions: Optional[List[int]] = None, device=None):
    """Logits [T, V] of one whole sequence (with return_margins also, per position, the smallest
    gap over the MoE layers between the last chosen and the first rejected router logit, relative to
    the rms of the token's router logits:
    where it is tiny, rounding may legitimately choose another expert); the layer loop of crates/engine/src/flint.rs:775-1117
    (embed, per layer: norm, q/k/v, qk-norm, RoPE, attention, o-proj + residual, norm, router +
    experts (+ shared expert) or dense MLP + residual; final norm and LM head).

    forced_routing: executed position -> experts [T, k] to use there instead of the router's own
    choice (another implementation's selection, so that two implementations can be compared on the
    same experts); the second result is then a dict: executed position -> (this implementation's
    router logits [T, E], its own choice [T, k]) for the routed layers.
    logit_positions: only these positions' logits are computed ([len, V]).  device: where the
    arithmetic runs (default: where the weights are); weights are converted as they are used, so
    that a large model is never held twice."""
    dev = torch.device(device) if device is not None else next(iter(weights.values())).device
    W = lambda name: weights[name].to(device=dev, dtype=dtype)
    em = emulate_bf16
    L = cfg["num_hidden_layers"]
    Hq, Hkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    qk_eps = cfg.get("qk_norm_eps") or eps
    order = cfg.get("layer_order") or list(range(L))
    kv_source = cfg.get("kv_source") or [None] * len(order)
    sliding = cfg.get("sliding_window_pattern") or [False] * L
    roped = cfg.get("rope_pattern") or [True] * L
    T = len(tokens)
    pos = torch.arange(T, device=dev)
    h = embed(torch.tensor(tokens, device=dev), W("model.embed_tokens.weight"))
    kept = {}
    margins = torch.full((T,), float("inf"), dtype=dtype, device=dev)
    routers = {}
    for p, i in enumerate(order):
        pre = f"model.layers.{i}."
        xn = _r(rmsnorm(h, W(pre + "input_layernorm.weight"), eps), em)
        q = (xn @ W(pre + "self_attn.q_proj.weight").T).view(T, Hq, hd)
        if kv_source[p] is None:
            k = (xn @ W(pre + "self_attn.k_proj.weight").T).view(T, Hkv, hd)
            v = (xn @ W(pre + "self_attn.v_proj.weight").T).view(T, Hkv, hd)
        if cfg.get("qk_norm"):
            q = rmsnorm(q, W(pre + "self_attn.q_norm.weight"), qk_eps)
            if kv_source[p] is None:
                k = rmsnorm(k, W(pre + "self_attn.k_norm.weight"), qk_eps)
        if roped[i]:
            q = rope_neox(q, pos, cfg["rope_theta"])
            if kv_source[p] is None:
                k = rope_neox(k, pos, cfg["rope_theta"])
        q = _r(q, em)
        if kv_source[p] is None:
            k, v = _r(k, em), _r(v, em)
            kept[p] = (k, v)
        else:
            k, v = kept[kv_source[p]]
        a = attention(q, k, v, cfg["sliding_window"] if sliding[i] else None,
                      W(pre + "self_attn.sinks") if cfg.get("attn_sinks") else None, em)
        a = _r(a, em).reshape(T, Hq * hd)
        h = h + a @ W(pre + "self_attn.o_proj.weight").T
        xn = _r(rmsnorm(h, W(pre + "post_attention_layernorm.weight"), eps), em)
        if i < cfg.get("first_k_dense_replace", 0):
            f = swiglu_mlp(xn, W(pre + "mlp.gate_proj.weight"), W(pre + "mlp.up_proj.weight"),
                           W(pre + "mlp.down_proj.weight"), em)
        else:
            forced = forced_routing.get(p) if forced_routing is not None else None
            f = moe(xn, W(pre + "mlp.gate.weight"), W(pre + "mlp.experts.gate_proj.weight"),
                    W(pre + "mlp.experts.up_proj.weight"), W(pre + "mlp.experts.down_proj.weight"),
                    cfg.get("scoring_func", "softmax"), cfg["num_experts_per_tok"],
                    cfg.get("norm_topk_prob", True), em, forced)
            margins = torch.minimum(margins, _last_route_margin)
            routers[p] = _last_router
            if cfg.get("n_shared_experts", 0) > 0:
                f = f + swiglu_mlp(xn, W(pre + "mlp.shared_experts.gate_proj.weight"),
                                   W(pre + "mlp.shared_experts.up_proj.weight"),
                                   W(pre + "mlp.shared_experts.down_proj.weight"), em)
        h = h + f
    if logit_positions is not None:
        h = h[torch.tensor(list(logit_positions), dtype=torch.long, device=dev)]
    xn = _r(rmsnorm(h, W("model.norm.weight"), eps), em)
    head = W("model.embed_tokens.weight") if cfg.get("tie_word_embeddings") else W("lm_head.weight")
    logits = xn @ head.T
    if forced_routing is not None:
        return logits, routers
    return (logits, margins) if return_margins else logits


# --------------------------------------------------------------------------- sampling
def splitmix64_uniform(seed: int, n: int) -> float:
    """The n-th (1-based) uniform of the splitmix64 stream started at `seed`.
    crates/cli/src/flint.rs:318-325"""
    mask = (1 << 64) - 1
    z = (seed + n * 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z ^= z >> 31
    return (z >> 11) / float(1 << 53)


def pick(logits: List[float], temperature: float, top_k: int, top_p: float, min_p: float, u: float, pool: int = 256) -> int:
    """The reference's host sampler without penalties: candidates sorted by (logit desc, id asc),
    greedy when temperature <= 0 or top_k == 1; p_i = exp((l_i - l_0)/T) in double; min-p drops
    p_i < min_p; top-p keeps the shortest prefix with mass >= top_p; inverse CDF with u * total.
    The candidate pool is the top `pool` (256) logits, or top_k if smaller.
    crates/cli/src/flint.rs:385-430, pool :303,:339-347"""
    ids = sorted(range(len(logits)), key=lambda i: (-logits[i], i))
    if temperature <= 0.0 or top_k == 1:
        return ids[0]
    keep = min(pool, len(ids)) if top_k == 0 else min(top_k, pool, len(ids))
    ids = ids[:keep]
    top = logits[ids[0]]
    # the reference divides in single precision, then exponentiates in double
    f32 = np.float32
    probs = [math.exp(float(f32(f32(logits[i]) - f32(top)) / f32(temperature))) for i in ids]
    if min_p > 0.0:
        probs = [q if q >= min_p else 0.0 for q in probs]
    total = sum(probs)
    cut = len(probs)
    if top_p < 1.0:
        acc = 0.0
        for i, q in enumerate(probs):
            acc += q / total
            if acc >= top_p:
                cut = i + 1
                break
    total = sum(probs[:cut])
    r = u * total
    for i, q in enumerate(probs[:cut]):
        r -= q
        if r <= 0.0:
            return ids[i]
    return ids[cut - 1]
