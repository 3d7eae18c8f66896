"""A second plain implementation of the Recursive Flint MoE decoder, in NumPy, written from the
reference's formulas without reusing tests/plain_flint.py (another reading of the same sources:
the two must agree before either is trusted; tests/test_plain.py compares them).  Token by token
and head by head, with explicit loops; float64; whole sequences, no cache.

Formulas (paths of lkarlslund/quench6k):
  embedding              h[t] = table[token[t]], no scaling                    crates/cuda/kernels/flint.cu:89-95
  RMSNorm                x * rsqrt(mean(x^2) + eps) * w, plain weight           flint.cu:97-122
  QK-norm                the same per head of q and k, before the rotation      flint.cu:138-140,155
  rotation               pair (d, d + hd/2) turned by pos * theta^(-2d/hd),
                         the angle a float32 product                            flint.cu:141-149
  attention              head h reads KV head h // (Hq/Hkv); score q.k/sqrt(hd);
                         key j seen from p iff j <= p and j > p - window;
                         sink: one more term exp(sink_h - max) in the denominator flint.cu:225-245,315-325,505-526
  router                 sigmoid(z) or softmax(z); top-k, ties to the lower index;
                         sigmoid weights / (sum + 1e-20), softmax weights / sum  flint.cu:829-864, crates/cuda/kernels/moe.cu:19-71
  expert                 Wd (silu(Wg x) * (Wu x)), silu(x) = x / (1 + exp(-x))   flint.cu:1221-1239, common.cuh:13
  shared expert, dense   the same SwiGLU, weight 1                              flint.cu:865-878
  layer                  h += attn(norm(h)); h += ffn(norm(h)); final norm; head crates/engine/src/flint.rs:775-1117
"""
import math

import numpy as np


def _f64(t):
    return t.detach().to("cpu").double().numpy() if hasattr(t, "detach") else np.asarray(t, dtype=np.float64)


def _rms(x, w, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def _rotate(x, theta):
    """x: [T, heads, hd]; position t is row t."""
    T, _, hd = x.shape
    half = hd // 2
    inv = (theta ** (-(2.0 * np.arange(half, dtype=np.float64)) / hd)).astype(np.float32)
    out = np.empty_like(x)
    for t in range(T):
        a = (np.float32(t) * inv).astype(np.float64)              # a float32 product, then exact
        c, s = np.cos(a), np.sin(a)
        out[t, :, :half] = x[t, :, :half] * c - x[t, :, half:] * s
        out[t, :, half:] = x[t, :, half:] * c + x[t, :, :half] * s
    return out


def _attend(q, k, v, window, sinks):
    T, Hq, hd = q.shape
    G = Hq // k.shape[1]
    out = np.zeros_like(q)
    for t in range(T):
        first = 0 if window is None else max(0, t - window + 1)
        for h in range(Hq):
            kh = h // G
            s = k[first:t + 1, kh] @ q[t, h] / math.sqrt(hd)
            m = s.max() if sinks is None else max(s.max(), sinks[h])
            e = np.exp(s - m)
            den = e.sum() + (0.0 if sinks is None else math.exp(sinks[h] - m))
            out[t, h] = (e @ v[first:t + 1, kh]) / den
    return out


def _swiglu(x, wg, wu, wd):
    g = wg @ x
    return wd @ (g / (1.0 + np.exp(-g)) * (wu @ x))


def _moe(x, router, wg, wu, wd, scoring, k, renorm):
    T = x.shape[0]
    out = np.zeros_like(x)
    for t in range(T):
        z = router @ x[t]
        if scoring == "sigmoid":
            score = 1.0 / (1.0 + np.exp(-z))
        else:
            e = np.exp(z - z.max())
            score = e / e.sum()
        chosen = np.argsort(-score, kind="stable")[:k]            # equal scores keep the lower index first
        w = score[chosen]
        if renorm:
            w = w / (w.sum() + (1e-20 if scoring == "sigmoid" else 0.0))
        for e_id, weight in zip(chosen, w):                       # in slot order
            out[t] = out[t] + weight * _swiglu(x[t], wg[e_id], wu[e_id], wd[e_id])
    return out


def forward(cfg, weights, tokens):
    """float64 logits [T, V] of one whole sequence."""
    W = {n: _f64(t) for n, t in weights.items()}
    L, Hq, Hkv, hd = cfg["num_hidden_layers"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    qk_eps = cfg.get("qk_norm_eps") or eps
    order = cfg.get("layer_order") or list(range(L))
    borrow = cfg.get("kv_source") or [None] * len(order)
    T = len(tokens)
    h = W["model.embed_tokens.weight"][np.asarray(tokens)]
    caches = {}
    for p, i in enumerate(order):
        pre = f"model.layers.{i}.self_attn."
        x = _rms(h, W[f"model.layers.{i}.input_layernorm.weight"], eps)
        q = (x @ W[pre + "q_proj.weight"].T).reshape(T, Hq, hd)
        rope = (cfg.get("rope_pattern") or [True] * L)[i]
        if cfg.get("qk_norm"):
            q = _rms(q, W[pre + "q_norm.weight"], qk_eps)
        if rope:
            q = _rotate(q, cfg["rope_theta"])
        if borrow[p] is None:
            k = (x @ W[pre + "k_proj.weight"].T).reshape(T, Hkv, hd)
            v = (x @ W[pre + "v_proj.weight"].T).reshape(T, Hkv, hd)
            if cfg.get("qk_norm"):
                k = _rms(k, W[pre + "k_norm.weight"], qk_eps)
            if rope:
                k = _rotate(k, cfg["rope_theta"])
            caches[p] = (k, v)
        else:
            k, v = caches[borrow[p]]
        sliding = (cfg.get("sliding_window_pattern") or [False] * L)[i]
        a = _attend(q, k, v, cfg["sliding_window"] if sliding else None, W[pre + "sinks"] if cfg.get("attn_sinks") else None)
        h = h + a.reshape(T, Hq * hd) @ W[pre + "o_proj.weight"].T
        x = _rms(h, W[f"model.layers.{i}.post_attention_layernorm.weight"], eps)
        mlp = f"model.layers.{i}.mlp."
        if i < cfg.get("first_k_dense_replace", 0):
            f = np.stack([_swiglu(x[t], W[mlp + "gate_proj.weight"], W[mlp + "up_proj.weight"], W[mlp + "down_proj.weight"]) for t in range(T)])
        else:
            f = _moe(x, W[mlp + "gate.weight"], W[mlp + "experts.gate_proj.weight"], W[mlp + "experts.up_proj.weight"],
                     W[mlp + "experts.down_proj.weight"], cfg.get("scoring_func", "softmax"), cfg["num_experts_per_tok"],
                     cfg.get("norm_topk_prob", True))
            if cfg.get("n_shared_experts", 0) > 0:
                sh = mlp + "shared_experts."
                f = f + np.stack([_swiglu(x[t], W[sh + "gate_proj.weight"], W[sh + "up_proj.weight"], W[sh + "down_proj.weight"]) for t in range(T)])
        h = h + f
    x = _rms(h, W["model.norm.weight"], eps)
    head = W["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else W["lm_head.weight"]
    return x @ head.T
