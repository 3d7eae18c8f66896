"""The engine at the layer sizes that bench.py times (hidden 2048, 32 query and 4 KV heads of 128,
256 experts of width 512 with 8 per token, a vocabulary of 151,936, theta 1e6, pages of 16), two
layers deep, against the plain implementation under every cut, in float32 and bfloat16: nothing is
timed at sizes whose logits were never checked (the reference checks before it times,
crates/cli/src/flint.rs:116-131).

The weights are made on the device and handed to the engine and to the plain implementation as
they are (no model folder: 4.5 GB).  The plain implementation runs its float64 arithmetic on the
device here (whole sequences, no cache, as everywhere; on the CPU the vocabulary alone would take
minutes), and scores every position of every request except in the long-prompt test, which scores
the positions listed there."""
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

SHAPE = {
    "architectures": ["FlintForCausalLM"],
    "hidden_size": 2048, "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 4, "head_dim": 128,
    "vocab_size": 151936, "n_routed_experts": 256, "num_experts_per_tok": 8, "moe_intermediate_size": 512,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": False, "scoring_func": "softmax",
    "norm_topk_prob": True, "qk_norm": True, "attn_sinks": True, "kv_page_size": 16,
}


@pytest.fixture(scope="module")
def shape():
    from quench6k_b200.config import FlintConfig
    from quench6k_b200.models.decoder import DecoderModel
    from quench6k_b200.models.flint import build_spec
    from quench6k_b200.weights.random_init import make_tensor
    cfg = FlintConfig.from_dict(SHAPE)
    spec = build_spec(cfg, norm_init="random")
    weights = {t.name: make_tensor(t, 5, spec.init_std, device="cuda") for t in DecoderModel(spec).tensors()}
    yield {"cfg": cfg, "cfg_d": cfg.to_dict(), "weights": weights}
    weights.clear()
    torch.cuda.empty_cache()


def _runner(shape, dtype, max_tokens, max_requests=8):
    from quench6k_b200.engine import ModelRunner
    from quench6k_b200.engine.replay import pool_pages
    from quench6k_b200.engine.runner import parse_dtype
    from quench6k_b200.models.decoder import DecoderModel
    from quench6k_b200.models.flint import build_spec
    from quench6k_b200.parts.base import Runtime
    model = DecoderModel(build_spec(shape["cfg"], norm_init="random"))
    rt = Runtime(torch.device("cuda:0"), parse_dtype(dtype), True)
    model.bind(lambda n: shape["weights"][n], rt)
    return ModelRunner(model, rt, 16, pool_pages(max_tokens, 16), max_requests)


def _replay_and_check(shape, dtype, reqs, steps, max_tokens, what, max_requests=8, positions=None):
    outputs, runner = helpers.run_replay(None, dtype, steps, max_tokens, runner=_runner(shape, dtype, max_tokens, max_requests), tap=True)
    worst, flipped = 0.0, 0
    got = helpers.collect(reqs, steps, outputs) if positions is None else None
    for rid, toks in reqs.items():
        pos = None if positions is None else positions[rid]
        mine = got[rid] if got is not None else helpers.collect_wanted(rid, steps, outputs)
        err, n = helpers.assert_matches_plain(shape["cfg_d"], shape["weights"], toks, mine, dtype, f"bench shape {dtype} {what} {rid}",
                                              routing=runner.routing.get(rid), positions=pos,
                                              device="cuda")
        worst, flipped = max(worst, err), flipped + n
    print(f"bench shape {dtype} {what}: worst error {worst:.3e}, {flipped} positions routed at a near-tie")
    from quench6k_b200 import ops
    assert ops.tc_status() == 0
    return runner


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cut(shape, dtype):
    V = SHAPE["vocab_size"]
    reqs = {f"r{i}": helpers.random_tokens(n, V, 40 + i) for i, n in enumerate([70, 131, 45, 96, 64])}
    for what, (steps, mt) in {"whole": helpers.schedule_whole(reqs), "tail": helpers.schedule_tail(reqs),
                              "portions": helpers.schedule_portions(reqs, seed=4),
                              "mixed": helpers.schedule_mixed(reqs, 16, seed=6)}.items():
        _replay_and_check(shape, dtype, reqs, steps, mt, what)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_in_portions_beside_decoding(shape, dtype, monkeypatch):
    """A prompt of 2,560 tokens in four portions of 640, each deep enough in the cache and wide
    enough to go to the tcgen05 attention kernel in bfloat16 (three of them start past position
    0), beside three requests that decode one token per step.  Scored: the first and last four
    positions of every portion and every 29th between, and every position of the others."""
    from quench6k_b200 import ops
    calls = []
    real = ops.attention_tc
    monkeypatch.setattr(ops, "attention_tc", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    V = SHAPE["vocab_size"]
    reqs = {"long": helpers.random_tokens(2560, V, 60), "d0": helpers.random_tokens(40, V, 61), "d1": helpers.random_tokens(75, V, 62),
            "d2": helpers.random_tokens(23, V, 63)}
    steps = [{"step": 0, "entries": [{"id": r, "tokens": reqs[r][:len(reqs[r]) - 4], "want": list(range(len(reqs[r]) - 4))}
                                     for r in ("d0", "d1", "d2")], "end": []}]
    positions = {r: None for r in ("d0", "d1", "d2")}
    positions["long"] = []
    for i in range(4):
        want = sorted(set(list(range(4)) + list(range(636, 640)) + list(range(4, 636, 29))))
        entries = [{"id": "long", "tokens": reqs["long"][640 * i:640 * (i + 1)], "want": want}]
        positions["long"] += [640 * i + w for w in want]
        for r in ("d0", "d1", "d2"):
            at = len(reqs[r]) - 4 + i
            entries.append({"id": r, "tokens": reqs[r][at:at + 1], "want": [0]})
        steps.append({"step": i + 1, "entries": entries, "end": list(reqs) if i == 3 else []})
    _replay_and_check(shape, dtype, reqs, steps, 2560 + 64 + 128 + 64, "long prompt", positions=positions)
    if dtype == "bfloat16":
        assert len(calls) == 4 * SHAPE["num_hidden_layers"], "the portions did not go to the tcgen05 attention kernel"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_batch_of_37(shape, dtype):
    V = SHAPE["vocab_size"]
    reqs = {f"w{i}": helpers.random_tokens(14 + (i * 7) % 23, V, 900 + i) for i in range(37)}
    steps, mt = helpers.schedule_wide_decode(reqs, 16)
    runner = _replay_and_check(shape, dtype, reqs, steps, mt, "decode batch", max_requests=40)
    assert runner.graph_replays > 0
