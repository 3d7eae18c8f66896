"""Each part of a layer alone, built through its registry with sizes of its own, against the plain
implementation's function for that part; and a toy mixer with state of its own, defined here,
registered, built and stepped without touching the framework's files."""
import math

import pytest
import torch

import helpers
import plain_flint as P

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _bind(part, rt, seed=0, std=0.5):
    from quench6k_b200.weights import make_tensor
    store = {t.name: make_tensor(t, seed, std) for t in part.tensors()}
    part.bind(lambda n: store[n], rt)
    return store


def _rt(dtype):
    from quench6k_b200.parts import Runtime
    return Runtime(torch.device(DEV), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from quench6k_b200.parts import NORMS, make_part
    from quench6k_b200.spec import PartSpec
    n = make_part(NORMS, "norm", PartSpec("rmsnorm", {"eps": 1e-4, "init": "random"}), size=88)
    store = _bind(n, _rt(dtype))
    h = torch.randn(9, 88, device=DEV) * 2
    out = n.forward(h)
    ref = P.rmsnorm(h.double().cpu(), store["weight"].double(), 1e-4)
    assert out.dtype == dtype
    assert (out.double().cpu() - ref).abs().max() <= (1e-5 if dtype == torch.float32 else 1e-2) * ref.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shared", [0, 40])
def test_feed_forward_parts(dtype, shared):
    from quench6k_b200.parts import FEED_FORWARDS, make_part
    from quench6k_b200.spec import PartSpec
    D, T = 56, 23
    em = dtype == torch.bfloat16
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    x = (torch.randn(T, D) * 0.7).to(dtype)
    dense = make_part(FEED_FORWARDS, "feed-forward", PartSpec("dense", {"intermediate_size": 72}), hidden_size=D)
    st = _bind(dense, _rt(dtype), std=0.2)
    out = torch.zeros(T, D, device=DEV)
    dense.forward(x.to(DEV), None, out)
    ref = P.swiglu_mlp(x.double(), st["gate_proj.weight"].double(), st["up_proj.weight"].double(), st["down_proj.weight"].double(), em)
    assert (out.double().cpu() - ref).abs().max() <= tol * ref.abs().max()
    moe = make_part(FEED_FORWARDS, "feed-forward", PartSpec("moe", {"num_experts": 12, "top_k": 5, "intermediate_size": 24,
                    "scoring": "sigmoid", "renormalize": True, "shared_intermediate_size": shared}), hidden_size=D)
    st = _bind(moe, _rt(dtype), seed=2, std=0.2)
    out = torch.full((T, D), 0.25, device=DEV)                      # the part adds into the stream
    moe.forward(x.to(DEV), None, out)
    ref = P.moe(x.double(), st["gate.weight"].double(), st["experts.gate_proj.weight"].double(),
                st["experts.up_proj.weight"].double(), st["experts.down_proj.weight"].double(), "sigmoid", 5, True, em)
    if shared:
        ref = ref + P.swiglu_mlp(x.double(), st["shared_experts.gate_proj.weight"].double(),
                                 st["shared_experts.up_proj.weight"].double(), st["shared_experts.down_proj.weight"].double(), em)
    assert ((out.double().cpu() - 0.25) - ref).abs().max() <= tol * ref.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,sinks,qk_norm,rope", [(None, False, False, True), (7, True, True, True), (None, True, True, False)])
def test_attention_part_over_pages(dtype, window, sinks, qk_norm, rope):
    """Two requests in one step, one of them continuing from a cache an earlier step left."""
    from quench6k_b200.parts import MIXERS, LayerCache, make_part
    from quench6k_b200.spec import PartSpec
    D, Hq, Hkv, hd, ps = 40, 6, 2, 32, 4
    em = dtype == torch.bfloat16
    pos = PartSpec("rope", {"head_dim": hd, "theta": 3000.0}) if rope else PartSpec("none", {"head_dim": hd})
    att = make_part(MIXERS, "mixer", PartSpec("attention", {"num_heads": Hq, "num_kv_heads": Hkv, "head_dim": hd, "eps": 1e-5,
                    "pos": pos, "window": window, "sinks": sinks, "qk_norm": qk_norm, "norm_init": "random"}), hidden_size=D)
    st = _bind(att, _rt(dtype), seed=4, std=0.3)
    req = att.cache_request()
    assert (req.kind, req.window, req.kv_heads, req.head_dim) == ("sliding" if window else "full", window, Hkv, hd)
    lens = [19, 11]
    xs = [(torch.randn(n, D) * 0.8).to(dtype) for n in lens]
    cache = LayerCache(0, torch.zeros(Hkv, 16, ps, hd, dtype=dtype, device=DEV), torch.zeros(Hkv, 16, ps, hd, dtype=dtype, device=DEV), ps)
    tables = [[[9, 2, 14, 5, 0], [7, 3, 11]]]
    # step 1: the first 13 tokens of request 0; step 2: its last 6 beside all of request 1
    def run(x, ctx):
        out = torch.zeros(x.shape[0], D, device=DEV)
        delta = att.forward(x.to(DEV), ctx, cache, None, out)       # a mixer adds into `out` or returns its result
        if delta is None:
            return out
        return delta.sum(0) if delta.dim() == 3 else delta          # split-K partial sums

    out1 = run(xs[0][:13], helpers.make_context([13], [0], [[tables[0][0]]]))
    out2 = run(torch.cat([xs[0][13:], xs[1]]), helpers.make_context([6, 11], [13, 0], tables))
    got = [torch.cat([out1, out2[:6]]).double().cpu(), out2[6:].double().cpu()]
    for r, n in enumerate(lens):
        x = xs[r].double()
        q = (x @ st["q_proj.weight"].double().T).view(n, Hq, hd)
        k = (x @ st["k_proj.weight"].double().T).view(n, Hkv, hd)
        v = (x @ st["v_proj.weight"].double().T).view(n, Hkv, hd)
        if qk_norm:
            q, k = P.rmsnorm(q, st["q_norm.weight"].double(), 1e-5), P.rmsnorm(k, st["k_norm.weight"].double(), 1e-5)
        if rope:
            q, k = P.rope_neox(q, torch.arange(n), 3000.0), P.rope_neox(k, torch.arange(n), 3000.0)
        q, k, v = P._r(q, em), P._r(k, em), P._r(v, em)
        a = P._r(P.attention(q, k, v, window, st["sinks"].double() if sinks else None, em), em).reshape(n, Hq * hd)
        ref = a @ st["o_proj.weight"].double().T
        err = (got[r] - ref).abs().max() / ref.abs().max()
        assert err <= (1e-4 if dtype == torch.float32 else 3e-2), (r, err)


def test_attention_part_mixed_step_at_head_size_128():
    """A prompt portion large enough for the tcgen05 attention kernel beside a decoded token and the
    five-token stub of a prompt that stand deep in their contexts: the short ones go to the kernel
    that splits the keys, the portion to the other, and every row of the step is written once."""
    from quench6k_b200.parts import MIXERS, LayerCache, make_part
    from quench6k_b200.spec import PartSpec
    D, Hq, Hkv, hd, ps = 64, 8, 1, 128, 16
    att = make_part(MIXERS, "mixer", PartSpec("attention", {"num_heads": Hq, "num_kv_heads": Hkv, "head_dim": hd, "eps": 1e-6,
                    "pos": PartSpec("rope", {"head_dim": hd, "theta": 10000.0}), "window": None, "sinks": True, "qk_norm": True,
                    "norm_init": "random"}), hidden_size=D)
    st = _bind(att, _rt(torch.bfloat16), seed=8, std=0.3)
    lens = [2400, 1501, 705]
    xs = [(torch.randn(n, D, generator=torch.Generator().manual_seed(60 + i)) * 0.8).to(torch.bfloat16) for i, n in enumerate(lens)]
    pages = sum(-(-n // ps) for n in lens) + 3
    cache = LayerCache(0, torch.zeros(Hkv, pages, ps, hd, dtype=torch.bfloat16, device=DEV),
                       torch.zeros(Hkv, pages, ps, hd, dtype=torch.bfloat16, device=DEV), ps)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(3)).tolist()
    tables = [[order.pop() for _ in range(-(-n // ps))] for n in lens]

    def run(x, ctx):
        out = torch.zeros(x.shape[0], D, device=DEV)
        delta = att.forward(x.to(DEV), ctx, cache, None, out)
        if delta is None:
            return out
        return delta.sum(0) if delta.dim() == 3 else delta

    calls = []
    from quench6k_b200 import ops
    real_tc, real_mma = ops.attention_tc, ops.attention_mma
    try:
        ops.attention_tc = lambda *a, **k: (calls.append(("tc", a[6].shape[0])), real_tc(*a, **k))[1]
        ops.attention_mma = lambda *a, **k: (calls.append(("mma", a[6].numel())), real_mma(*a, **k))[1]
        got = {}
        got[1] = [run(xs[1][:1500], helpers.make_context([1500], [0], [[tables[1]]]))]
        got[2] = [run(xs[2][:700], helpers.make_context([700], [0], [[tables[2]]]))]
        before = len(calls)
        mixed = run(torch.cat([xs[1][1500:], xs[0], xs[2][700:]]), helpers.make_context([1, 2400, 5], [1500, 0, 700], [[tables[1], tables[0], tables[2]]]))
        assert ops.tc_status() == 0
        # the portion's 150 tiles as 75 pairs on tcgen05; the decoded token and the stub as two tiles of the other kernel
        assert calls[before:] == [("tc", 75), ("mma", 2)], calls[before:]
    finally:
        ops.attention_tc, ops.attention_mma = real_tc, real_mma
    got[1].append(mixed[:1])
    got[0] = [mixed[1:2401]]
    got[2].append(mixed[2401:])
    for r, n in enumerate(lens):
        x = xs[r].double()
        q = (x @ st["q_proj.weight"].double().T).view(n, Hq, hd)
        k = (x @ st["k_proj.weight"].double().T).view(n, Hkv, hd)
        v = (x @ st["v_proj.weight"].double().T).view(n, Hkv, hd)
        q, k = P.rmsnorm(q, st["q_norm.weight"].double(), 1e-6), P.rmsnorm(k, st["k_norm.weight"].double(), 1e-6)
        q, k = P.rope_neox(q, torch.arange(n), 10000.0), P.rope_neox(k, torch.arange(n), 10000.0)
        q, k, v = P._r(q, True), P._r(k, True), P._r(v, True)
        a = P._r(P.attention(q, k, v, None, st["sinks"].double(), True), True).reshape(n, Hq * hd)
        ref = a @ st["o_proj.weight"].double().T
        have = torch.cat(got[r]).double().cpu()
        assert have.shape == ref.shape
        err = (have - ref).abs().max() / ref.abs().max()
        assert err <= 3e-2, (r, err)
        tail = (have[-5:] - ref[-5:]).abs().max() / ref[-5:].abs().max()       # the rows of the mixed step
        assert tail <= 3e-2, (r, tail)


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    """A mixer that keeps a running mean of its inputs per request (fixed-size state, no keys),
    and an architecture that alternates it with attention, are defined here and run through the
    unchanged framework: registry, weights, cache manager (state slots), step function."""
    from dataclasses import dataclass
    from quench6k_b200.config import register_architecture
    from quench6k_b200.engine import ModelRunner, StepEntry
    from quench6k_b200.parts import Mixer, register_mixer
    from quench6k_b200.spec import LayerSpec, ModelSpec, PartSpec, TensorSpec

    @register_mixer("toy_running_mean")
    class RunningMean(Mixer):
        """y_t = w * mean(x_0..x_t); the state is (sum [D], count [1]) per request."""
        def __init__(self, hidden_size):
            self.D = hidden_size

        def tensors(self):
            return [TensorSpec("w", (self.D,), "f32", ("ones_plus", 0.5))]

        def bind(self, get, rt):
            self.rt = rt
            self.w = get("w").to(rt.device, torch.float32)

        def state_shape(self):
            return (self.D + 1,)

        def forward(self, xn, ctx, cache, state, out):
            assert cache is None
            x = xn.float()
            at = 0
            for r, n in enumerate(ctx.q_lens):
                s = state[ctx.slots[r]]
                cs = torch.cumsum(x[at:at + n], 0) + s[:self.D]
                cnt = s[self.D] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                out[at:at + n] += self.w * cs / cnt[:, None]
                s[:self.D] = cs[-1]
                s[self.D] = cnt[-1]
                at += n

    @dataclass
    class ToyConfig:
        hidden_size: int
        vocab_size: int
        architectures: list

        @classmethod
        def from_dict(cls, d):
            return cls(d["hidden_size"], d["vocab_size"], d["architectures"])

        def to_dict(self):
            return dict(self.__dict__)

        def save(self, folder):
            import json, os
            with open(os.path.join(folder, "config.json"), "w") as f:
                json.dump(self.to_dict(), f)

    def build(cfg):
        norm = PartSpec("rmsnorm", {"eps": 1e-5, "init": "random"})
        ffn = PartSpec("dense", {"intermediate_size": 24})
        attn = PartSpec("attention", {"num_heads": 2, "num_kv_heads": 1, "head_dim": 16, "eps": 1e-5,
                                      "pos": PartSpec("rope", {"head_dim": 16, "theta": 1000.0})})
        layers = [LayerSpec("model.layers.0.", PartSpec("toy_running_mean", {}), ffn, norm),
                  LayerSpec("model.layers.1.", attn, ffn, norm)]
        return ModelSpec(cfg.hidden_size, cfg.vocab_size, layers, order=[0, 1, 0], kv_source=[None, None, None], final_norm=norm)

    register_architecture("ToyRunningMeanLM", ToyConfig, build)
    cfg = ToyConfig(32, 50, ["ToyRunningMeanLM"])
    runner = ModelRunner.from_random(cfg, seed=1, dtype="float32", page_size=4, num_pages=12, max_requests=3)
    assert [s is not None for s in runner.states] == [True, False, True]          # layer 0 runs twice: two states
    assert [c is not None for c in runner.caches] == [False, True, False]
    toks = {"a": helpers.random_tokens(21, 50, 1), "b": helpers.random_tokens(17, 50, 2)}
    # whole
    whole = {}
    for rid, t in toks.items():
        runner.add_request(rid)
        whole[rid] = runner.step([StepEntry(rid, t, list(range(len(t))))]).cpu()
        runner.end_request(rid)
    # cut and mixed; slots are reused, so stale state would show
    runner.add_request("a"), runner.add_request("b")
    got = {"a": [], "b": []}
    o = runner.step([StepEntry("a", toks["a"][:9], list(range(9)))])
    got["a"].append(o.cpu())
    o = runner.step([StepEntry("a", toks["a"][9:10], [0]), StepEntry("b", toks["b"][:12], list(range(12)))]).cpu()
    got["a"].append(o[:1]), got["b"].append(o[1:])
    o = runner.step([StepEntry("b", toks["b"][12:], list(range(5))), StepEntry("a", toks["a"][10:], list(range(11)))]).cpu()
    got["b"].append(o[:5]), got["a"].append(o[5:])
    for rid in toks:
        g = torch.cat(got[rid])
        assert (g - whole[rid]).abs().max() <= 1e-5 * whole[rid].abs().max()
    runner.end_request("a"), runner.end_request("b")
    runner.manager.check()


def test_toy_feed_forward_with_routing_and_toy_position_encoding(tmp_path):
    """A feed-forward that routes each token to one of three linear maps, and two position
    encodings (a rotary one that pairs neighbouring dimensions and turns only the first 8 of a
    head's 16, which hands the q/k kernel its table, and one that is no rotation at all and
    implements `apply`), are defined here, registered, chosen by a PartSpec and run through the
    unchanged framework (model folder, loader, step function, cache), in one step and cut into
    portions, against the same model written out in plain tensor code."""
    from dataclasses import dataclass
    from quench6k_b200.config import register_architecture
    from quench6k_b200.engine import ModelRunner, StepEntry
    from quench6k_b200.models.decoder import DecoderModel
    from quench6k_b200.parts import FeedForward, PositionEncoding, register_feed_forward, register_position_encoding
    from quench6k_b200.spec import LayerSpec, ModelSpec, PartSpec, TensorSpec
    from quench6k_b200.weights import index_folder, write_model_folder

    RD = 8

    def rotate_pairs(x, positions, theta):
        """(x[2i], x[2i+1]), i < RD/2, turned by position * theta^(-2i/RD); the other dimensions stay."""
        inv = (theta ** (-torch.arange(0, RD, 2, dtype=torch.float64, device=x.device) / RD)).float()
        ang = (positions.float()[:, None] * inv).double()
        c, s = torch.cos(ang)[:, None, :].to(x.dtype), torch.sin(ang)[:, None, :].to(x.dtype)
        a, b = x[..., 0:RD:2].clone(), x[..., 1:RD:2].clone()
        out = x.clone()
        out[..., 0:RD:2], out[..., 1:RD:2] = a * c - b * s, a * s + b * c
        return out

    def bump(x, positions):
        """x[d] + 0.3 sin(position / (d + 1)): no rotation, so no table for the kernel."""
        d = torch.arange(x.shape[-1], dtype=x.dtype, device=x.device)
        return x + 0.3 * torch.sin(positions.to(x.dtype)[:, None, None] / (d + 1.0))

    @register_position_encoding("toy_pairwise_rotary")
    class PairwiseRotary(PositionEncoding):
        def __init__(self, head_dim, theta):
            self.hd, self.theta = head_dim, theta

        def bind(self, get, rt):
            self.table = (self.theta ** (-torch.arange(0, RD, 2, dtype=torch.float64) / RD)).float().to(rt.device)

        def rotary_table(self):
            return self.table, RD, True       # the q/k kernel turns neighbouring pairs of the first RD dimensions

    @register_position_encoding("toy_bump")
    class Bump(PositionEncoding):
        def __init__(self, head_dim):
            self.hd = head_dim

        def apply(self, x, positions):
            x.copy_(bump(x, positions))

    @register_feed_forward("toy_switch")
    class Switch(FeedForward):
        """y = p_e * (W_e x), e the most likely of `n` maps under softmax(R x)."""
        def __init__(self, hidden_size, n):
            self.D, self.n = hidden_size, n

        def tensors(self):
            return [TensorSpec("router.weight", (self.n, self.D), "f32", ("normal", 0.5)),
                    TensorSpec("maps.weight", (self.n, self.D, self.D), "f32", ("normal", 0.2))]

        def bind(self, get, rt):
            self.rt = rt
            self.r, self.w = get("router.weight").to(rt.device, torch.float32), get("maps.weight").to(rt.device, torch.float32)

        def forward(self, xn, ctx, out):
            x = xn.float()
            p = torch.softmax(x @ self.r.T, -1)
            top, e = p.max(-1)
            out += top[:, None] * torch.einsum("tij,tj->ti", self.w[e], x)

    @dataclass
    class ToyConfig:
        hidden_size: int
        vocab_size: int
        architectures: list

        @classmethod
        def from_dict(cls, d):
            return cls(d["hidden_size"], d["vocab_size"], d["architectures"])

        def to_dict(self):
            return dict(self.__dict__)

        def save(self, folder):
            import json, os
            with open(os.path.join(folder, "config.json"), "w") as f:
                json.dump(self.to_dict(), f)

    D, V, Hq, Hkv, hd, eps, theta = 40, 61, 3, 1, 16, 1e-5, 500.0

    def build(cfg):
        norm = PartSpec("rmsnorm", {"eps": eps, "init": "random"})
        attn = lambda pos: PartSpec("attention", {"num_heads": Hq, "num_kv_heads": Hkv, "head_dim": hd, "eps": eps, "pos": pos, "qk_norm": True,
                                                  "norm_init": "random"})
        layers = [LayerSpec("model.layers.0.", attn(PartSpec("toy_pairwise_rotary", {"head_dim": hd, "theta": theta})),
                            PartSpec("toy_switch", {"n": 3}), norm),
                  LayerSpec("model.layers.1.", attn(PartSpec("toy_bump", {"head_dim": hd})), PartSpec("toy_switch", {"n": 3}), norm)]
        return ModelSpec(cfg.hidden_size, cfg.vocab_size, layers, order=[0, 1], kv_source=[None, None], final_norm=norm, init_std=0.2)

    register_architecture("ToySwitchLM", ToyConfig, build)
    cfg = ToyConfig(D, V, ["ToySwitchLM"])
    spec = build(cfg)
    write_model_folder(str(tmp_path), cfg, DecoderModel(spec).tensors(), 3, spec.init_std)
    w = {n: f.read(n).double() for n, (f, e) in index_folder(str(tmp_path)).items()}
    runner = ModelRunner.from_folder(str(tmp_path), dtype="float32", page_size=4, num_pages=16, max_requests=2)
    toks = helpers.random_tokens(23, V, 5)

    # the same model in plain tensor code
    h = P.embed(torch.tensor(toks), w["model.embed_tokens.weight"])
    n = len(toks)
    for L, place in (("model.layers.0.", lambda x: rotate_pairs(x, torch.arange(n), theta)), ("model.layers.1.", lambda x: bump(x, torch.arange(n)))):
        x = P.rmsnorm(h, w[L + "input_layernorm.weight"], eps)
        q = P.rmsnorm((x @ w[L + "self_attn.q_proj.weight"].T).view(n, Hq, hd), w[L + "self_attn.q_norm.weight"], eps)
        k = P.rmsnorm((x @ w[L + "self_attn.k_proj.weight"].T).view(n, Hkv, hd), w[L + "self_attn.k_norm.weight"], eps)
        v = (x @ w[L + "self_attn.v_proj.weight"].T).view(n, Hkv, hd)
        h = h + P.attention(place(q), place(k), v, None, None, False).reshape(n, Hq * hd) @ w[L + "self_attn.o_proj.weight"].T
        x = P.rmsnorm(h, w[L + "post_attention_layernorm.weight"], eps)
        p = torch.softmax(x @ w[L + "mlp.router.weight"].T, -1)
        top, e = p.max(-1)
        assert len(set(e.tolist())) > 1                        # the routing does choose different maps
        h = h + top[:, None] * torch.einsum("tij,tj->ti", w[L + "mlp.maps.weight"][e], x)
    want = P.rmsnorm(h, w["model.norm.weight"], eps) @ w["lm_head.weight"].T

    runner.add_request("w")
    whole = runner.step([StepEntry("w", toks, list(range(n)))]).double().cpu()
    runner.end_request("w")
    runner.add_request("c")
    parts = []
    for a, b in ((0, 9), (9, 11), (11, 12), (12, 23)):
        parts.append(runner.step([StepEntry("c", toks[a:b], list(range(b - a)))]).double().cpu())
    runner.end_request("c")
    runner.manager.check()
    for got in (whole, torch.cat(parts)):
        assert (got - want).abs().max() <= 1e-4 * want.abs().max()


def test_toy_mixer_with_unequal_key_and_value_widths_and_named_states(tmp_path):
    """A mixer whose keys (12 wide) and values (20 wide) differ in width, whose pages are float32
    whatever the engine's operand dtype, and which keeps two named per-request states of
    different dtypes (how many tokens it has seen, int32; the last input row, float32), is defined
    here and run through the unchanged framework in bfloat16: the runner makes its pages and
    states from what the mixer declares."""
    from dataclasses import dataclass
    from quench6k_b200.config import register_architecture
    from quench6k_b200.engine import ModelRunner, StepEntry
    from quench6k_b200.parts import CacheRequest, Mixer, register_mixer
    from quench6k_b200.spec import LayerSpec, ModelSpec, PartSpec, TensorSpec

    KD, VD, PAGE = 12, 20, 4

    @register_mixer("toy_narrow_keys")
    class NarrowKeys(Mixer):
        """One head; out = softmax(q k^T / sqrt(KD)) v Wo + 0.1 * (the row before this one), causal."""
        def __init__(self, hidden_size):
            self.D = hidden_size

        def tensors(self):
            return [TensorSpec("q.weight", (KD, self.D), "f32", ("normal", 0.3)), TensorSpec("k.weight", (KD, self.D), "f32", ("normal", 0.3)),
                    TensorSpec("v.weight", (VD, self.D), "f32", ("normal", 0.3)), TensorSpec("o.weight", (self.D, VD), "f32", ("normal", 0.3))]

        def bind(self, get, rt):
            self.rt = rt
            self.wq, self.wk, self.wv, self.wo = (get(n + ".weight").to(rt.device, torch.float32) for n in "qkvo")

        def cache_request(self):
            return CacheRequest("full", None, 1, KD, v_dim=VD, dtype=torch.float32)

        def state_shape(self):
            return {"seen": ((1,), torch.int32), "last": ((self.D,), torch.float32)}

        def forward(self, xn, ctx, cache, state, out):
            assert cache.k.shape[-1] == KD and cache.v.shape[-1] == VD and cache.k.dtype == torch.float32
            assert state["seen"].dtype == torch.int32 and state["last"].shape[1:] == (self.D,)
            x = xn.float()
            table = ctx.block_tables[cache.group]
            at = 0
            for r, n in enumerate(ctx.q_lens):
                p0, slot = ctx.pos_starts[r], ctx.slots[r]
                assert int(state["seen"][slot]) == p0            # the state followed the request through its steps
                rows = x[at:at + n]
                pos = torch.arange(p0, p0 + n, device=x.device)
                pages = table[r][(pos // PAGE).long()].long()
                cache.k[0, pages, (pos % PAGE).long()] = rows @ self.wk.T
                cache.v[0, pages, (pos % PAGE).long()] = rows @ self.wv.T
                every = torch.arange(p0 + n, device=x.device)
                k = cache.k[0, table[r][(every // PAGE).long()].long(), (every % PAGE).long()]
                v = cache.v[0, table[r][(every // PAGE).long()].long(), (every % PAGE).long()]
                s = (rows @ self.wq.T) @ k.T / math.sqrt(KD)
                s = s.masked_fill(every[None, :] > pos[:, None], float("-inf"))
                before = torch.cat([state["last"][slot][None], rows[:-1]])
                out[at:at + n] += torch.softmax(s, -1) @ v @ self.wo.T + 0.1 * before
                state["last"][slot] = rows[-1]
                state["seen"][slot] += n
                at += n

    @dataclass
    class ToyConfig:
        hidden_size: int
        vocab_size: int
        architectures: list

        @classmethod
        def from_dict(cls, d):
            return cls(d["hidden_size"], d["vocab_size"], d["architectures"])

    def build(cfg):
        norm = PartSpec("rmsnorm", {"eps": 1e-5, "init": "random"})
        layers = [LayerSpec("model.layers.0.", PartSpec("toy_narrow_keys", {}), PartSpec("dense", {"intermediate_size": 24}), norm)]
        return ModelSpec(cfg.hidden_size, cfg.vocab_size, layers, order=[0, 0], kv_source=[None, None], final_norm=norm, init_std=0.2)

    register_architecture("ToyNarrowKeysLM", ToyConfig, build)
    runner = ModelRunner.from_random(ToyConfig(32, 50, ["ToyNarrowKeysLM"]), seed=2, dtype="bfloat16", page_size=PAGE, num_pages=16, max_requests=2)
    assert not runner.cuda_graphs                               # the toy mixer reads host fields of the step: no graph replay
    for c in runner.caches:
        assert c.k.shape == (1, 17, PAGE, KD) and c.v.shape == (1, 17, PAGE, VD) and c.k.dtype == torch.float32
    toks = {"a": helpers.random_tokens(19, 50, 3), "b": helpers.random_tokens(11, 50, 4)}
    whole = {}
    for rid, t in toks.items():
        runner.add_request(rid)
        whole[rid] = runner.step([StepEntry(rid, t, list(range(len(t))))]).cpu()
        runner.end_request(rid)
    runner.add_request("b"), runner.add_request("a")              # the slots the other way round: stale state would show
    got = {"a": [], "b": []}
    got["b"].append(runner.step([StepEntry("b", toks["b"][:4], list(range(4)))]).cpu())
    o = runner.step([StepEntry("a", toks["a"][:13], list(range(13))), StepEntry("b", toks["b"][4:5], [0])]).cpu()
    got["a"].append(o[:13]), got["b"].append(o[13:])
    o = runner.step([StepEntry("b", toks["b"][5:], list(range(6))), StepEntry("a", toks["a"][13:], list(range(6)))]).cpu()
    got["b"].append(o[:6]), got["a"].append(o[6:])
    for rid in toks:
        g = torch.cat(got[rid])
        assert (g - whole[rid]).abs().max() <= 2e-2 * whole[rid].abs().max()
    runner.end_request("a"), runner.end_request("b")
    runner.manager.check()
