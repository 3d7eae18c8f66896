"""Checks of the plain implementation itself (the yardstick must be right before it measures)."""
import math

import pytest
import torch

import helpers
import plain_flint as P
import tiny_configs


def test_rmsnorm_and_rope_properties():
    x = torch.randn(5, 12, dtype=torch.float64)
    w = torch.rand(12, dtype=torch.float64) + 0.5
    y = P.rmsnorm(x, w, 1e-6)
    assert torch.allclose(y / w, x / x.pow(2).mean(-1, keepdim=True).add(1e-6).sqrt())
    q = torch.randn(6, 2, 8, dtype=torch.float64)
    k = torch.randn(6, 2, 8, dtype=torch.float64)
    pos = torch.arange(6)
    rq, rk = P.rope_neox(q, pos, 100.0), P.rope_neox(k, pos, 100.0)
    assert torch.allclose(rq.norm(dim=-1), q.norm(dim=-1))               # a rotation
    assert torch.allclose(rq[0], q[0])                                   # position 0 is the identity
    # scores depend on the distance only: shift both positions by 3
    rq3, rk3 = P.rope_neox(q, pos + 3, 100.0), P.rope_neox(k, pos + 3, 100.0)
    assert torch.allclose((rq[4] * rk[1]).sum(-1), (rq3[4] * rk3[1]).sum(-1))
    # element pairing: d with d + hd/2
    one = torch.zeros(1, 1, 8, dtype=torch.float64)
    one[0, 0, 1] = 1.0
    r = P.rope_neox(one, torch.tensor([2]), 100.0)
    a = 2 * 100.0 ** (-2 / 8)                                            # the angle itself is a float32 there: to 1e-7
    assert math.isclose(r[0, 0, 1], math.cos(a), abs_tol=2e-7) and math.isclose(r[0, 0, 5], math.sin(a), abs_tol=2e-7)


def test_attention_mask_window_sink_and_groups():
    torch.manual_seed(0)
    T, Hq, Hkv, hd = 9, 4, 2, 8
    q, k, v = (torch.randn(T, h, hd, dtype=torch.float64) for h in (Hq, Hkv, Hkv))
    full = P.attention(q, k, v, None, None, False)
    # causal: row t is a softmax over keys 0..t of head h // 2
    t, h = 5, 3
    s = (k[:t + 1, 1] @ q[t, h]) / math.sqrt(hd)
    want = torch.softmax(s, 0) @ v[:t + 1, 1]
    assert torch.allclose(full[t, h], want)
    # window 3: keys t-2..t
    win = P.attention(q, k, v, 3, None, False)
    want = torch.softmax(s[t - 2:], 0) @ v[t - 2:t + 1, 1]
    assert torch.allclose(win[t, h], want)
    assert torch.allclose(win[1], full[1])                               # nothing cut yet
    # sink: extra denominator term only
    sinks = torch.tensor([0.3, -1.0, 2.0, 0.5], dtype=torch.float64)
    sk = P.attention(q, k, v, None, sinks, False)
    e = torch.exp(s)
    want = (e @ v[:t + 1, 1]) / (e.sum() + math.exp(sinks[h]))
    assert torch.allclose(sk[t, h], want)


def test_route_rules():
    z = torch.tensor([[0.0, 2.0, 2.0, -1.0, 2.0, 1.0]], dtype=torch.float64)
    sel, w = P.route(z, "sigmoid", 3, True)
    assert sel.tolist() == [[1, 2, 4]]                                   # ties go to the lower index
    assert torch.allclose(w.sum(), torch.tensor(1.0, dtype=torch.float64))
    sel, w = P.route(z, "sigmoid", 2, False)
    assert torch.allclose(w, torch.sigmoid(torch.tensor([[2.0, 2.0]], dtype=torch.float64)))
    sel, w = P.route(z, "softmax", 4, False)
    assert sel.tolist() == [[1, 2, 4, 5]]
    assert torch.allclose(w, torch.softmax(z, -1)[0, [1, 2, 4, 5]][None])
    sel, w = P.route(z, "softmax", 4, True)
    assert torch.allclose(w.sum(), torch.tensor(1.0, dtype=torch.float64))


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_model_is_causal_and_precisions_agree(tmp_path, name):
    cfg, weights = helpers.make_model_folder(str(tmp_path), name, seed=1)
    toks = helpers.random_tokens(24, cfg["vocab_size"], 5)
    full = P.forward(cfg, weights, toks)
    assert full.shape == (24, cfg["vocab_size"]) and torch.isfinite(full).all()
    head = P.forward(cfg, weights, toks[:11])
    assert torch.allclose(full[:11], head, atol=1e-12)                   # later tokens do not reach back
    other = list(toks)
    other[20] = (other[20] + 1) % cfg["vocab_size"]
    assert torch.allclose(P.forward(cfg, weights, other)[:20], full[:20], atol=1e-12)
    f32 = P.forward(cfg, weights, toks, dtype=torch.float32)
    assert (f32.double() - full).abs().max() < 1e-4 * full.abs().max()
    em = P.forward(cfg, weights, toks, emulate_bf16=True)
    rel = ((em - full).abs().max() / full.abs().max()).item()
    assert 1e-5 < rel < 5e-2                                             # rounding is visible but small


def test_window_limits_what_a_layer_sees(tmp_path):
    # one sliding layer only: a token further back than the window cannot change the logits
    cfg = tiny_configs.get("B")
    cfg.update(num_hidden_layers=1, sliding_window_pattern=[True], rope_pattern=[True], first_k_dense_replace=0, sliding_window=4)
    from quench6k_b200.config import FlintConfig
    from quench6k_b200.models.decoder import DecoderModel
    from quench6k_b200.models.flint import build_spec
    from quench6k_b200.weights import make_tensor
    spec = build_spec(FlintConfig.from_dict(cfg))
    weights = {t.name: make_tensor(t, 0, 0.02) for t in DecoderModel(spec).tensors()}
    toks = helpers.random_tokens(12, cfg["vocab_size"], 1)
    a = P.forward(cfg, weights, toks)
    other = list(toks)
    other[3] = (other[3] + 7) % cfg["vocab_size"]
    b = P.forward(cfg, weights, other)
    assert torch.allclose(a[7:], b[7:], atol=1e-12)                      # position 7 sees keys 4..7
    assert not torch.allclose(a[6], b[6], atol=1e-9)                     # position 6 sees key 3


def test_splitmix_and_pick():
    # first outputs of splitmix64 seeded with 0 (public test vector of the generator)
    mask = (1 << 64) - 1
    z = (0 + 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z ^= z >> 31
    assert z == 0xE220A8397B1DCDAF
    assert P.splitmix64_uniform(0, 1) == (z >> 11) / float(1 << 53)
    logits = [0.1, 3.0, 3.0, -2.0, 1.0]
    assert P.pick(logits, 0.0, 20, 0.95, 0.0, 0.3) == 1                  # greedy, tie to the lower id
    assert P.pick(logits, 1.0, 1, 0.95, 0.0, 0.9) == 1
    assert P.pick(logits, 1.0, 0, 1.0, 0.0, 0.0) == 1
    assert P.pick(logits, 1.0, 0, 1.0, 0.0, 0.999999) == 3
    assert P.pick(logits, 1.0, 2, 1.0, 0.0, 0.75) == 2
    assert P.pick(logits, 1.0, 0, 0.5, 0.0, 0.999) == 2                  # top-p 0.5 keeps two candidates
    assert P.pick(logits, 1.0, 0, 1.0, 0.2, 0.999) == 2                  # min-p drops exp(-2) = 0.135 and below


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_two_plain_implementations_agree(tmp_path, name):
    """tests/plain_flint.py (tensor operations over whole sequences) and tests/numpy_flint.py
    (loops over tokens and heads), two readings of the reference's formulas that share no code:
    the same logits to 1e-6 of the largest, on the tiny configurations (C: layers named twice and a
    borrowed cache), with matrices wide enough apart for every layer to matter."""
    import helpers
    import numpy_flint
    cfg, weights = helpers.make_model_folder(str(tmp_path), name, seed=13, init_std=0.2)
    toks = helpers.random_tokens(37, cfg["vocab_size"], 5)
    a = P.forward(cfg, weights, toks).numpy()
    b = numpy_flint.forward(cfg, weights, toks)
    assert a.shape == b.shape
    assert abs(a - b).max() <= 1e-6 * abs(a).max()
