"""Generation through the Python entry point and the command line, against the plain implementation."""
import os
import subprocess
import sys

import pytest
import torch

import helpers
import plain_flint as P

pytestmark = pytest.mark.gpu


def plain_greedy(cfg, weights, prompt, n):
    toks = list(prompt)
    margins = []
    for _ in range(n):
        logits = P.forward(cfg, weights, toks, dtype=torch.float64)[-1]
        top = torch.topk(logits, 2).values
        margins.append(float(top[0] - top[1]))
        toks.append(int(torch.argmax(logits)))
    return toks[len(prompt):], margins


# With the default N(0, 0.02) matrices the tiny configurations with tied embeddings or windows repeat one token
# for ever, and a wrong token fed back, a lost placeholder or a stale page would go unseen.  These seeds and standard
# deviations make the plain implementation's greedy continuations vary (asserted where they are used).
VARIED = {"A": dict(seed=21), "B": dict(seed=21, init_std=0.2), "C": dict(seed=41, init_std=0.5), "D": dict(seed=41)}


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("C", "bfloat16"), ("C", "float32")])
def test_greedy_generation_matches_plain(tmp_path, name, dtype):
    from quench6k_b200 import Engine, SamplingParams
    cfg, weights = helpers.make_model_folder(str(tmp_path), name, **VARIED[name])
    prompts = [helpers.random_tokens(n, cfg["vocab_size"], 300 + n) for n in (7, 13, 5)]
    eng = Engine.from_folder(str(tmp_path), dtype=dtype, num_pages=24, max_batch_tokens=6)     # prompts are cut into portions
    outs = eng.generate(prompts, SamplingParams(max_tokens=8, temperature=0.0))
    for p, o in zip(prompts, outs):
        want, margins = plain_greedy(cfg, weights, p, 8)
        assert len(set(want)) >= 4, f"the continuation {want} could not show a wrong token"
        assert o.finish_reason == "length" and len(o.tokens) == 8
        for i, (g, w) in enumerate(zip(o.tokens, want)):
            if g != w:
                # a different token is only acceptable at a near-tie of the reference's two best logits
                assert dtype == "bfloat16" and margins[i] < 2e-3, (i, g, w, margins[i])
                break
    eng.runner.manager.check()
    assert not eng.runner.manager.requests


def test_sampled_generation_is_reproducible_and_batch_independent(tmp_path):
    from quench6k_b200 import Engine, SamplingParams
    cfg, _ = helpers.make_model_folder(str(tmp_path), "B", seed=22)
    prompts = [helpers.random_tokens(n, cfg["vocab_size"], 400 + n) for n in (5, 17, 29)]
    params = [SamplingParams(max_tokens=10, temperature=0.8, top_k=0, top_p=1.0, seed=1000 + i) for i in range(3)]
    eng = Engine.from_folder(str(tmp_path), dtype="float32", num_pages=32, max_batch_tokens=6)
    together = eng.generate(prompts, params)
    alone = [eng.generate([p], [sp])[0] for p, sp in zip(prompts, params)]
    for a, b in zip(together, alone):
        assert a.tokens == b.tokens
    assert len({tuple(o.tokens) for o in together}) == 3
    other = eng.generate(prompts[:1], [SamplingParams(max_tokens=10, temperature=0.8, top_k=0, top_p=1.0, seed=5)])[0]
    assert other.tokens != together[0].tokens


@pytest.mark.parametrize("name,std", [("A", None), ("C", 0.8)])
def test_preemption_gives_the_same_tokens(tmp_path, name, std):
    """C: a window on one of its layers and a position that reads another position's cache, so a
    preempted request gives back pages of two groups and recomputes both."""
    from quench6k_b200 import Engine, SamplingParams
    cfg, _ = helpers.make_model_folder(str(tmp_path), name, seed=23, init_std=std)
    prompts = [helpers.random_tokens(n, cfg["vocab_size"], 500 + n) for n in (9, 11, 6)]
    sp = SamplingParams(max_tokens=14, temperature=0.0)
    roomy = Engine.from_folder(str(tmp_path), dtype="float32", page_size=4, num_pages=64)
    want = [o.tokens for o in roomy.generate(prompts, sp)]
    assert sum(len(set(w)) >= 4 for w in want) >= 2, f"the continuations {want} could not show a wrong token"
    tight = Engine.from_folder(str(tmp_path), dtype="float32", page_size=4, num_pages=12)      # 48 token places for 68 tokens
    outs = tight.generate(prompts, sp)
    assert tight.stats["preemptions"] > 0
    assert [o.tokens for o in outs] == want
    tight.runner.manager.check()


def test_stop_token_ends_generation(tmp_path):
    from quench6k_b200 import Engine, SamplingParams
    cfg, _ = helpers.make_model_folder(str(tmp_path), "A", seed=24)
    eng = Engine.from_folder(str(tmp_path), dtype="float32", num_pages=32)
    prompt = helpers.random_tokens(10, cfg["vocab_size"], 1)
    free = eng.generate([prompt], SamplingParams(max_tokens=12, temperature=0.0))[0].tokens
    stop = free[4]
    out = eng.generate([prompt], SamplingParams(max_tokens=12, temperature=0.0, stop_tokens=[stop]))[0]
    assert out.finish_reason == "stop" and out.tokens == free[:free.index(stop) + 1]


@pytest.mark.parametrize("lookahead", [False, True])
def test_abort_reports_the_cancelled_request_and_what_had_just_ended(tmp_path, lookahead):
    """Aborting the last live request while another has ended but is not yet reported: a caller
    that loops `while has_unfinished(): step()` gets both, the aborted one with reason "cancelled"."""
    from quench6k_b200 import Engine, SamplingParams
    cfg, _ = helpers.make_model_folder(str(tmp_path), "A", seed=27)
    eng = Engine.from_folder(str(tmp_path), dtype="float32", num_pages=32, lookahead=lookahead)
    short = eng.add_request(helpers.random_tokens(5, cfg["vocab_size"], 1), SamplingParams(max_tokens=2, temperature=0.0))
    long = eng.add_request(helpers.random_tokens(6, cfg["vocab_size"], 2), SamplingParams(max_tokens=50, temperature=0.0))
    outs = []
    for _ in range(3):                              # prompts, then decode steps: the short request has produced its two tokens
        outs += eng.step()
    eng.abort(long)
    while eng.has_unfinished():
        outs += eng.step()
    by = {o.rid: o for o in outs}
    assert set(by) == {short, long}
    assert by[short].finish_reason == "length" and len(by[short].tokens) == 2
    assert by[long].finish_reason == "cancelled" and 1 <= len(by[long].tokens) < 50 and -1 not in by[long].tokens
    eng.runner.manager.check()
    assert not eng.runner.manager.requests
    eng.abort(long)                                 # aborting what has ended is a no-op
    assert not eng.has_unfinished()


def test_command_line(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, weights = helpers.make_model_folder(str(tmp_path), "A", seed=25)
    prompt = helpers.random_tokens(7, cfg["vocab_size"], 9)
    r = subprocess.run([sys.executable, "-m", "quench6k_b200", "generate", "--model", str(tmp_path), "--prompt-ids",
                        ",".join(map(str, prompt)), "--n", "8", "--dtype", "float32", "--context", "64"],
                       cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "prompt: 7 tokens" in r.stdout and "first-token top 5:" in r.stdout and "decode 7 tokens" in r.stdout
    want, _ = plain_greedy(cfg, weights, prompt, 8)
    assert f"ids: {want}" in r.stdout


def test_command_line_bench_and_ppl(tmp_path):
    """`bench` (prefill and greedy decode rates per context, graph decoding checked against eager
    decoding, one JSON record per context) and `ppl` (chunks scored on their second half) in the
    reference's manner, on files of token ids."""
    import json
    import math
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, weights = helpers.make_model_folder(str(tmp_path), "A", seed=26)
    ids = helpers.random_tokens(90, cfg["vocab_size"], 12)
    corpus = tmp_path / "ids.txt"
    corpus.write_text(" ".join(map(str, ids[:45])) + "\n" + ",".join(map(str, ids[45:])))
    out = tmp_path / "bench.jsonl"
    run = lambda *args: subprocess.run([sys.executable, "-m", "quench6k_b200", *args], cwd=root, capture_output=True, text=True, timeout=600)
    r = run("bench", "--model", str(tmp_path), "--ids", str(corpus), "--ctx", "16", "40", "--generate", "8", "--json", str(out),
            "--dtype", "float32", "--max-batch-tokens", "12")
    assert r.returncode == 0, r.stderr[-2000:]
    assert "graph decoding matches eager decoding (8 tokens)" in r.stdout
    recs = [json.loads(line) for line in out.read_text().splitlines()]
    assert [x["ctx"] for x in recs] == [16, 40] and all(x["generate"] == 8 and x["kv"] == "fp32" and x["decode_tok_s"] > 0 for x in recs)
    for x in recs:                                  # the tokens it printed are the plain implementation's greedy continuation
        want, _ = plain_greedy(cfg, weights, ids[:x["ctx"]], 8)
        assert f"{want}" in r.stdout
        assert x["copied"] == sum(1 for a, b in zip(want, ids[x["ctx"]:]) if a == b)
    r = run("ppl", "--model", str(tmp_path), "--file", str(corpus), "--ctx", "24", "--chunks", "3", "--dtype", "float32",
            "--max-batch-tokens", "5")
    assert r.returncode == 0, r.stderr[-2000:]
    nll, count = 0.0, 0
    for c in range(3):
        toks = ids[c * 24:(c + 1) * 24]
        logits = helpers.plain_logits(cfg, weights, toks, False)[0]
        for p in range(12, 23):
            nll += float(torch.logsumexp(logits[p], -1) - logits[p][toks[p + 1]])
            count += 1
    got = float(r.stdout.strip().splitlines()[-1].split(":")[1].split("(")[0])
    assert abs(got - math.exp(nll / count)) <= 2e-4 * got, (got, math.exp(nll / count))
    assert r.stdout.count("[") == 3


@pytest.mark.parametrize("name,dtype,lengths", [("B", "float32", (9, 21, 14)), ("B", "bfloat16", (9, 21, 14)),
                                                ("D", "bfloat16", (300, 700, 140)),
                                                ("B", "float32", (9, 21, 14, 5, 8, 11, 6, 17, 10, 12, 7)),
                                                ("D", "bfloat16", (30, 70, 140, 9, 200, 33, 64, 65, 17, 90))])
def test_graph_replay_equals_eager_steps(tmp_path, name, dtype, lengths):
    """Decode-only steps replay a CUDA graph; the logits must equal those of the same steps run
    eagerly (the reference checks graph decoding against eager decoding the same way,
    crates/cli/src/flint.rs:116-131).  D: the head size at which the key splits of decode
    attention are planned on the device; a replay must plan them from its own positions.  Batches
    of 9 to 12 requests share one recording: filler entries bring them to 12 rows, which must not
    change the rows of the real requests (bit for bit in float32)."""
    from quench6k_b200.engine import ModelRunner, StepEntry
    cfg, _ = helpers.make_model_folder(str(tmp_path), name, seed=31)
    prompts = {f"r{i}": helpers.random_tokens(n, cfg["vocab_size"], 600 + n) for i, n in enumerate(lengths)}
    tails = {rid: helpers.random_tokens(12, cfg["vocab_size"], 700 + i) for i, rid in enumerate(prompts)}
    outs = {}
    for graphs in (False, True):
        runner = ModelRunner.from_folder(str(tmp_path), dtype=dtype, num_pages=(32 if name == "B" else 96) * (1 + len(lengths) // 4),
                                         max_requests=len(lengths), cuda_graphs=graphs)
        assert runner.cuda_graphs == graphs
        for rid, p in prompts.items():
            runner.add_request(rid)
        runner.step([StepEntry(rid, p, []) for rid, p in prompts.items()])
        got = []
        for i in range(12):
            live = list(prompts)[: len(prompts) - (0 if i < 4 else 1 if i < 8 else 2)]      # the batch shrinks
            got.append(runner.step([StepEntry(rid, [tails[rid][i]], [0]) for rid in live]).clone().cpu())
        outs[graphs] = got
        assert (runner.graph_replays > 0) == graphs
        if graphs:                # 3, 2, 1 requests: three recordings; 11, 10, 9 requests: one of 12 rows; 10, 9, 8: one of 12 rows and one of 8
            assert runner.graph_captures == {3: 3, 11: 1, 10: 2}[len(lengths)]
    for a, b in zip(outs[False], outs[True]):
        if dtype == "float32":
            assert torch.equal(a, b)
        else:
            assert (a - b).abs().max() <= 1e-2 * a.abs().max()


_LAUNCH_MODE_SCRIPT = r"""
import sys, hashlib, torch
sys.path.insert(0, sys.argv[1])
from quench6k_b200.config import FlintConfig
from quench6k_b200.engine import ModelRunner, StepEntry
# wide enough for the tensor-core products with sliced K and for the decode path of the experts
cfg = FlintConfig.from_dict(dict(architectures=["FlintForCausalLM"], hidden_size=512, num_hidden_layers=3, num_attention_heads=8,
                                 num_key_value_heads=2, head_dim=128, vocab_size=1000, n_routed_experts=16, num_experts_per_tok=4,
                                 moe_intermediate_size=128, rms_norm_eps=1e-6, rope_theta=10000.0, qk_norm=True, kv_page_size=16))
runner = ModelRunner.from_random(cfg, 5, dtype="bfloat16", num_pages=64, max_requests=4)
g = torch.Generator().manual_seed(9)
h = hashlib.sha256()
for rid, n in (("a", 150), ("b", 37)):
    runner.add_request(rid)
    h.update(runner.step([StepEntry(rid, torch.randint(0, 1000, (n,), generator=g).tolist(), [n - 1])]).cpu().numpy().tobytes())
for i in range(20):
    toks = torch.randint(0, 1000, (2,), generator=g).tolist()
    h.update(runner.step([StepEntry("a", [toks[0]], [0]), StepEntry("b", [toks[1]], [0])]).cpu().numpy().tobytes())
torch.cuda.synchronize()
print("digest", h.hexdigest(), runner.graph_replays)
"""


def test_launch_modes_give_the_same_logits(tmp_path):
    """Programmatic dependent launch lets the dense tensor-core product fetch weights while the
    kernel before it still runs.  With it off, on for the marked launches (the default) and on for
    every launch, the same steps (eager prompts, then decode steps replayed from a graph) must give
    the same bits: nothing may be read before it is written."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "launch_modes.py"
    script.write_text(_LAUNCH_MODE_SCRIPT)
    digests = {}
    for mode in ("0", "gemm", "1"):
        env = dict(os.environ, Q6K_PDL=mode)
        proc = subprocess.run([sys.executable, str(script), root], capture_output=True, text=True, timeout=600, env=env)
        assert proc.returncode == 0, proc.stderr[-2000:]
        line = [ln for ln in proc.stdout.splitlines() if ln.startswith("digest")][-1].split()
        digests[mode] = line[1]
        assert int(line[2]) > 0                          # the decode steps did replay a graph
    assert digests["0"] == digests["gemm"] == digests["1"], digests


@pytest.mark.parametrize("name,pages,preempts,dtype", [("A", 64, False, "float32"), ("A", 14, True, "float32"), ("B", 24, False, "float32"),
                                                       ("C", 64, False, "float32"), ("C", 14, True, "float32"), ("D", 64, False, "bfloat16")])
def test_lookahead_gives_the_same_tokens(tmp_path, name, pages, preempts, dtype):
    """Greedy decoding without waiting for each step's tokens (they stay on the device, the host
    reads them one step late) against the engine that waits: the same tokens, finish reasons and
    preemption-safe bookkeeping, with stop tokens that do occur, ends by length, prompts cut into
    portions, and (14 pages) so few pages that requests are preempted."""
    import random
    from quench6k_b200 import Engine, SamplingParams
    cfg, _ = helpers.make_model_folder(str(tmp_path), name, **dict(VARIED[name], seed=41))
    rng = random.Random(7)
    prompts = [helpers.random_tokens(rng.randint(3, 25), cfg["vocab_size"], 900 + i) for i in range(7)]
    page = 4 if preempts else None        # pages of 4 tokens where requests are to be preempted (the configurations' own are 4 to 16)
    plain = Engine.from_folder(str(tmp_path), dtype=dtype, page_size=page, num_pages=pages, max_batch_tokens=9, lookahead=False)
    free = plain.generate(prompts, SamplingParams(max_tokens=18, temperature=0.0))
    if name in ("B", "C"):            # the configurations with windows, sinks, tied embeddings, a borrowed cache
        assert all(len(set(o.tokens)) >= 6 for o in free), [o.tokens for o in free]
    # stop tokens taken from what the requests really produce, at different depths; some never stop
    params = []
    for i, o in enumerate(free):
        stops = [o.tokens[2 + i % 9]] if i % 3 != 2 else []
        params.append(SamplingParams(max_tokens=5 + 3 * i, temperature=0.0, stop_tokens=stops))
    want = plain.generate(prompts, params)
    assert plain.stats["lookahead_steps"] == 0
    ahead = Engine.from_folder(str(tmp_path), dtype=dtype, page_size=page, num_pages=pages, max_batch_tokens=9)
    got = ahead.generate(prompts, params)
    assert ahead.stats["lookahead_steps"] > 0
    for w, g in zip(want, got):
        assert (g.tokens, g.finish_reason) == (w.tokens, w.finish_reason)
    assert {o.finish_reason for o in got} == {"stop", "length"}
    for eng in (plain, ahead):
        eng.runner.manager.check()
        assert not eng.runner.manager.requests and not eng.has_unfinished()
    if preempts:
        assert ahead.stats["preemptions"] > 0 and plain.stats["preemptions"] > 0
    # sampled requests without penalties are chosen on the device and run ahead too: the same tokens as from the host sampler
    trio = [params[0], SamplingParams(max_tokens=9, temperature=0.9, top_k=0, top_p=0.8, min_p=0.02, seed=3), params[2]]
    host_side = plain.generate(prompts[:3], trio)
    mixed = Engine.from_folder(str(tmp_path), dtype=dtype, num_pages=64, max_batch_tokens=9)
    outs = mixed.generate(prompts[:3], trio)
    assert mixed.stats["lookahead_steps"] > 0
    assert [o.tokens for o in outs] == [o.tokens for o in host_side] and len(outs[1].tokens) == 9
    assert (outs[0].tokens, outs[2].tokens) == (want[0].tokens, want[2].tokens)
    # a request with penalties is chosen on the host: while it lives the engine waits for each step
    trio[1] = SamplingParams(max_tokens=6, temperature=0.9, repetition_penalty=1.2, seed=3)
    before = dict(mixed.stats)
    outs = mixed.generate(prompts[:3], trio)
    assert [o.tokens for o in outs] == [o.tokens for o in plain.generate(prompts[:3], trio)]
    assert mixed.stats["lookahead_steps"] - before["lookahead_steps"] <= mixed.stats["steps"] - before["steps"] - 6


@pytest.mark.parametrize("seed", [0, 1])
def test_random_traffic_with_and_without_lookahead(tmp_path, seed):
    """Requests arriving over time (greedy and sampled ones mixed, stop tokens, aborts, so few pages
    that some are preempted) through an engine that waits for each step and one that looks ahead:
    every request that was not aborted ends with the same tokens and reason, the cache manager's
    invariants hold after every step, nothing is left behind."""
    import random
    from quench6k_b200 import Engine, SamplingParams, ops
    helpers.make_model_folder(str(tmp_path), "A", seed=5)

    def run(lookahead):
        rng = random.Random(seed)
        eng = Engine.from_folder(str(tmp_path), dtype="float32", num_pages=30, max_requests=6, max_batch_tokens=rng.choice([7, 16, 40]),
                                 lookahead=lookahead)
        V, n, results, live, aborted = eng.runner.vocab_size, 0, {}, set(), set()
        for step in range(160):
            if n < 28 and rng.random() < 0.3:
                sp = SamplingParams(max_tokens=rng.randint(1, 20), temperature=0.0 if rng.random() < 0.6 else 0.8, seed=rng.randrange(1 << 30),
                                    top_k=rng.choice([20, 0, 5]), top_p=rng.choice([0.95, 1.0, 0.5]), min_p=rng.choice([0.0, 0.05]),
                                    presence_penalty=0.5 if rng.random() < 0.1 else 0.0,
                                    stop_tokens=[rng.randrange(V) for _ in range(rng.choice([0, 0, 3, 40]))])
                eng.add_request([rng.randrange(V) for _ in range(rng.randint(1, 30))], sp, rid=n)
                live.add(n)
                n += 1
            victim = rng.randrange(max(1, n)) if rng.random() < 0.05 else None
            if victim in live and victim not in results:
                eng.abort(victim)
                aborted.add(victim)
                live.discard(victim)
            if eng.has_unfinished():
                for o in eng.step():
                    results[o.rid] = (o.tokens, o.finish_reason)
            eng.runner.manager.check()
        while eng.has_unfinished():
            for o in eng.step():
                results[o.rid] = (o.tokens, o.finish_reason)
        eng.runner.manager.check()
        assert not eng.runner.manager.requests and ops.tc_status() == 0
        return results, aborted, eng.stats

    waits, aborted_w, _ = run(False)
    ahead, aborted_a, stats = run(True)
    assert stats["lookahead_steps"] > 10
    same = [k for k in waits if k not in aborted_w and k not in aborted_a]
    assert len(same) >= 15
    for k in same:
        assert ahead[k] == waits[k], k


def test_graph_cache_is_bounded(tmp_path):
    """Only the most recently replayed step shapes keep their CUDA graph; a shape whose graph was
    dropped is recorded again and gives the same logits as eager steps."""
    from quench6k_b200.engine import ModelRunner, StepEntry
    cfg, _ = helpers.make_model_folder(str(tmp_path), "A", seed=33)
    prompts = {f"r{i}": helpers.random_tokens(5 + i, cfg["vocab_size"], 800 + i) for i in range(3)}
    tails = {rid: helpers.random_tokens(12, cfg["vocab_size"], 900 + i) for i, rid in enumerate(prompts)}
    outs = {}
    for graphs in (False, True):
        runner = ModelRunner.from_folder(str(tmp_path), dtype="float32", num_pages=32, cuda_graphs=graphs)
        runner.max_graphs = 2
        for rid, p in prompts.items():
            runner.add_request(rid)
            runner.step([StepEntry(rid, p, [])])
        got = []
        for i in range(12):
            live = list(prompts)[: 1 + i % 3]                                # three batch sizes in turn: three shapes
            got.append(runner.step([StepEntry(rid, [tails[rid][i]], [0]) for rid in live]).clone().cpu())
            assert len(runner._graphs) <= 2
        outs[graphs] = got
    for a, b in zip(outs[False], outs[True]):
        assert torch.equal(a, b)
