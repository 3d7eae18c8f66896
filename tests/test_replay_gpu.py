"""Replay of the same requests under every way of cutting the work, in float32 and bfloat16,
against the plain implementation: whole; most in one step and the last 32 tokens one by one;
portions of changing size down to two tokens; mixed batches with so few pages that they are reused.

A, B, C are the tiny configurations; D and E have head size 128 and widths at which the bfloat16
path runs its tensor-core kernels (tests/tiny_configs.py).  In bfloat16 the engine's choice of
router logits and experts are recorded, checked, and the experts forced on the plain implementation
(tests/helpers.py says why), so every position is held to the tolerance."""
import json
import os
import subprocess
import sys

import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [71, 130, 45, 96, 64, 33, 120, 58, 77], "B": [85, 140, 37, 101, 66, 50, 90, 125, 44],
           "C": [90, 57, 129, 48, 75, 40, 110, 66, 83], "D": [71, 130, 45, 200, 64, 33, 160, 58, 77],
           "E": [85, 140, 37, 101, 66, 210, 90, 125, 44]}


@pytest.fixture(scope="module", params=["A", "B", "C", "D", "E"])
def model(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp(f"tiny_{name}"))
    cfg, weights = helpers.make_model_folder(folder, name, seed=11)
    reqs = {f"r{i}": helpers.random_tokens(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(LENGTHS[name])}
    return {"name": name, "folder": folder, "cfg": cfg, "weights": weights, "requests": reqs}


def _check(model, dtype, steps, max_tokens, what):
    """Replay the steps, compare every request's logits with the plain implementation."""
    outputs, runner = helpers.run_replay(model["folder"], dtype, steps, max_tokens, tap=True)
    got = helpers.collect(model["requests"], steps, outputs)
    worst, flipped = 0.0, 0
    for rid, toks in model["requests"].items():
        err, n = helpers.assert_matches_plain(model["cfg"], model["weights"], toks, got[rid], dtype, f"{model['name']} {dtype} {what} {rid}",
                                              routing=runner.routing[rid])
        worst, flipped = max(worst, err), flipped + n
    print(f"{model['name']} {dtype} {what}: worst error {worst:.3e}, {flipped} positions routed at a near-tie")
    from quench6k_b200 import ops
    assert ops.tc_status() == 0
    return got, worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole(model, dtype):
    steps, mt = helpers.schedule_whole(model["requests"])
    _check(model, dtype, steps, mt, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_32_one_by_one(model, dtype):
    steps, mt = helpers.schedule_tail(model["requests"])
    _check(model, dtype, steps, mt, "tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_changing_size(model, dtype):
    steps, mt = helpers.schedule_portions(model["requests"], seed=3)
    assert any(len(s["entries"][0]["tokens"]) == 2 for s in steps)
    _check(model, dtype, steps, mt, "portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_with_reused_pages(model, dtype):
    page = model["cfg"]["kv_page_size"]
    steps, mt = helpers.schedule_mixed(model["requests"], page, seed=5)
    assert max(len(s["entries"]) for s in steps) == 4
    assert any(len(e["tokens"]) > 1 for s in steps for e in s["entries"][1:]) and any(
        len(e["tokens"]) == 1 for s in steps for e in s["entries"])
    total = sum(-(-len(t) // page) for t in model["requests"].values())
    from quench6k_b200.engine.replay import pool_pages
    assert pool_pages(mt, page) < total                     # fewer pages than the requests need together: reuse
    _check(model, dtype, steps, mt, "mixed")


def test_cuts_agree_with_each_other_in_float32(model):
    """Beyond the comparison with the plain implementation: in the 32-bit path the same position
    gives the same logits, bit for bit, however the work was cut."""
    whole, _ = _check(model, "float32", *helpers.schedule_whole(model["requests"]), "whole")
    page = model["cfg"]["kv_page_size"]
    for what, (steps, mt) in {"tail": helpers.schedule_tail(model["requests"]),
                              "portions": helpers.schedule_portions(model["requests"], seed=9),
                              "mixed": helpers.schedule_mixed(model["requests"], page, seed=2)}.items():
        got, _ = _check(model, "float32", steps, mt, what)
        for rid in model["requests"]:
            same = torch.equal(got[rid], whole[rid])
            err = (got[rid] - whole[rid]).abs().max().item() / whole[rid].abs().max().item()
            assert same, f"{what} {rid}: differs from the whole run (by {err:.2e} of the largest logit)"


def test_decode_batches_of_17_to_64(model):
    """Decoding in batches of up to 37 requests (recorded at the next bucket of the runner's
    list, with filler rows), which shrink as requests end: the grouped expert path above 16 rows."""
    if model["name"] not in ("B", "D", "E"):
        pytest.skip("one tiny and the two tensor-core configurations")
    cfg = model["cfg"]
    reqs = {f"w{i}": helpers.random_tokens(14 + (i * 7) % 23, cfg["vocab_size"], 900 + i) for i in range(37)}
    steps, mt = helpers.schedule_wide_decode(reqs, cfg["kv_page_size"])
    assert max(len(s["entries"]) for s in steps) == 37 and any(17 <= len(s["entries"]) < 37 for s in steps)
    for dtype in ("float32", "bfloat16"):
        outputs, runner = helpers.run_replay(model["folder"], dtype, steps, mt, max_requests=40, tap=True)
        got = helpers.collect(reqs, steps, outputs)
        for rid, toks in reqs.items():
            helpers.assert_matches_plain(cfg, model["weights"], toks, got[rid], dtype, f"{model['name']} {dtype} wide decode {rid}",
                                         routing=runner.routing[rid])
        assert runner.graph_replays > 0


def test_first_tokens_and_long_decoding(model):
    """The first tokens of a sequence (one token, two tokens) and decoding far past the prompt."""
    if model["name"] == "E":
        pytest.skip("D covers the head size; E's window is longer than the sequence")
    cfg, folder = model["cfg"], model["folder"]
    toks = helpers.random_tokens(230, cfg["vocab_size"], 77)
    for dtype in ("float32", "bfloat16"):
        steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:1], "want": [0]}], "end": []},
                 {"step": 1, "entries": [{"id": "x", "tokens": toks[1:3], "want": [0, 1]}], "end": []}]
        for i in range(3, len(toks)):
            steps.append({"step": i - 1, "entries": [{"id": "x", "tokens": toks[i:i + 1], "want": [0]}],
                          "end": ["x"] if i == len(toks) - 1 else []})
        outputs, runner = helpers.run_replay(folder, dtype, steps, len(toks), tap=True)
        got = helpers.collect({"x": toks}, steps, outputs)["x"]
        helpers.assert_matches_plain(cfg, model["weights"], toks, got, dtype, f"{model['name']} {dtype} long decoding",
                                     routing=runner.routing.get("x"))


@pytest.mark.parametrize("name", ["D", "E"])
def test_tensor_core_kernels_inside_the_model(tmp_path, name):
    """Configurations with head size 128 and widths the tcgen05 products take (D; E has every option
    the other way: windows, groups of 8, sigmoid scores, a shared expert, a dense layer, tied
    embeddings, pages of 32), in bfloat16: a 2,400-token prompt in one step (prompt-portion
    attention on tensor cores) beside a decoded token and the stub of another prompt (the
    key-splitting kernel writes their rows), prompts alone (wide tiles), decoding in a changing
    batch (narrow tiles, the decode router and the per-pair expert products), against the plain
    implementation on the experts the engine chose; then the same steps in true 32-bit arithmetic."""
    cfg, weights = helpers.make_model_folder(str(tmp_path), name, seed=23)
    V = cfg["vocab_size"]
    reqs = {"long": helpers.random_tokens(2400, V, 1), "r1": helpers.random_tokens(300, V, 2), "r2": helpers.random_tokens(150, V, 3),
            "r3": helpers.random_tokens(90, V, 4)}
    every = lambda n: list(range(n))
    steps = [{"step": 0, "entries": [{"id": "r1", "tokens": reqs["r1"][:280], "want": every(280)}], "end": []},
             {"step": 1, "entries": [{"id": "r2", "tokens": reqs["r2"][:140], "want": every(140)}], "end": []},
             {"step": 2, "entries": [{"id": "r1", "tokens": reqs["r1"][280:281], "want": [0]},
                                     {"id": "long", "tokens": reqs["long"], "want": every(2400)},
                                     {"id": "r2", "tokens": reqs["r2"][140:145], "want": every(5)}], "end": ["long"]},
             {"step": 3, "entries": [{"id": "r3", "tokens": reqs["r3"][:80], "want": every(80)},
                                     {"id": "r1", "tokens": reqs["r1"][281:282], "want": [0]}], "end": []}]
    at = {"r1": 282, "r2": 145, "r3": 80}
    n = 4
    while at:
        entries, end = [], []
        for rid in list(at):
            entries.append({"id": rid, "tokens": reqs[rid][at[rid]:at[rid] + 1], "want": [0]})
            at[rid] += 1
            if at[rid] == len(reqs[rid]):
                end.append(rid)
                del at[rid]
        steps.append({"step": n, "entries": entries, "end": end})
        n += 1
    for dtype in ("bfloat16", "float32"):
        outputs, runner = helpers.run_replay(str(tmp_path), dtype, steps, 2432 + 320 + 192 + 128, tap=True)
        got = helpers.collect(reqs, steps, outputs)
        for rid, toks in reqs.items():
            worst, flipped = helpers.assert_matches_plain(cfg, weights, toks, got[rid], dtype, f"{name} {dtype} {rid}",
                                                          routing=runner.routing.get(rid))
            print(f"{name} {dtype} {rid}: worst error {worst:.3e}, {flipped} positions routed at a near-tie")
            assert flipped <= 0.03 * len(toks) + 1, f"{rid}: too many positions routed differently to be rounding"
    from quench6k_b200 import ops
    assert ops.tc_status() == 0


def test_trace_run_program(model, tmp_path):
    """The program itself, as a user runs it: JSON lines in, `done` lines and .f32 files out."""
    if model["name"] != "B":
        pytest.skip("one configuration is enough for the subprocess")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    page = model["cfg"]["kv_page_size"]
    steps, mt = helpers.schedule_mixed(model["requests"], page, seed=8)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model["folder"], "--dtype", "float32",
                           "--out", str(out), "--max-tokens", str(mt)],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:len(steps)] == [f"done {s['step']}" for s in steps]
    import numpy as np
    V = model["cfg"]["vocab_size"]
    outputs = {}
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        data = np.fromfile(out / f"{s['step']}.f32", dtype="<f4")
        assert data.size == n * V
        outputs[s["step"]] = torch.from_numpy(data.reshape(n, V))
    got = helpers.collect(model["requests"], steps, outputs)
    for rid, toks in model["requests"].items():
        helpers.assert_matches_plain(model["cfg"], model["weights"], toks, got[rid], "float32", f"trace_run {rid}")
