"""Replay of the same requests under every way of cutting the work, in float32 and bfloat16,
against the plain implementation: whole; most in one step and the last 32 tokens one by one;
portions of changing size down to two tokens; mixed batches with so few pages that they are reused."""
import json
import os
import subprocess
import sys

import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [71, 130, 45, 96, 64, 33, 120, 58, 77], "B": [85, 140, 37, 101, 66, 50, 90, 125, 44],
           "C": [90, 57, 129, 48, 75, 40, 110, 66, 83]}


@pytest.fixture(scope="module", params=["A", "B", "C"])
def model(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp(f"tiny_{name}"))
    cfg, weights = helpers.make_model_folder(folder, name, seed=11)
    reqs = {f"r{i}": helpers.random_tokens(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(LENGTHS[name])}
    ref = {}
    for emulate in (False, True):
        ref[emulate] = {rid: helpers.plain_logits(cfg, weights, t, emulate) for rid, t in reqs.items()}
    return {"name": name, "folder": folder, "cfg": cfg, "requests": reqs, "ref": ref}


def _check(model, dtype, steps, max_tokens, what):
    outputs, runner = helpers.run_replay(model["folder"], dtype, steps, max_tokens)
    got = helpers.collect(model["requests"], steps, outputs)
    ref = model["ref"][dtype == "bfloat16"]
    worst = 0.0
    reach = max(8, model["cfg"].get("sliding_window") or 0)
    for rid in model["requests"]:
        worst = max(worst, helpers.assert_close(got[rid], ref[rid], dtype, f"{model['name']} {dtype} {what} {rid}", reach))
    print(f"{model['name']} {dtype} {what}: worst error {worst:.3e}")
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
    """Beyond the comparison with the plain implementation: the same position gives the same
    logits however the work was cut (to rounding far below the tolerance)."""
    whole, _ = _check(model, "float32", *helpers.schedule_whole(model["requests"]), "whole")
    page = model["cfg"]["kv_page_size"]
    for what, (steps, mt) in {"tail": helpers.schedule_tail(model["requests"]),
                              "portions": helpers.schedule_portions(model["requests"], seed=9),
                              "mixed": helpers.schedule_mixed(model["requests"], page, seed=2)}.items():
        got, _ = _check(model, "float32", steps, mt, what)
        for rid in model["requests"]:
            scale = whole[rid].abs().max().item()
            err = (got[rid] - whole[rid]).abs().max().item() / scale
            assert err < 2e-6, f"{what} {rid}: differs from the whole run by {err:.2e}"


def test_first_tokens_and_long_decoding(model):
    """The first tokens of a sequence (one token, two tokens) and decoding far past the prompt."""
    cfg, folder = model["cfg"], model["folder"]
    toks = helpers.random_tokens(230, cfg["vocab_size"], 77)
    import plain_flint
    from quench6k_b200.weights import index_folder
    weights = {n: f.read(n) for n, (f, e) in index_folder(folder).items()}
    for dtype in ("float32", "bfloat16"):
        ref = helpers.plain_logits(cfg, weights, toks, dtype == "bfloat16")
        steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:1], "want": [0]}], "end": []},
                 {"step": 1, "entries": [{"id": "x", "tokens": toks[1:3], "want": [0, 1]}], "end": []}]
        for i in range(3, len(toks)):
            steps.append({"step": i - 1, "entries": [{"id": "x", "tokens": toks[i:i + 1], "want": [0]}],
                          "end": ["x"] if i == len(toks) - 1 else []})
        outputs, _ = helpers.run_replay(folder, dtype, steps, len(toks))
        got = helpers.collect({"x": toks}, steps, outputs)["x"]
        helpers.assert_close(got, ref, dtype, f"{model['name']} {dtype} long decoding", max(8, cfg.get("sliding_window") or 0))


@pytest.mark.parametrize("name", ["D", "E"])
def test_tensor_core_kernels_inside_the_model(tmp_path, name):
    """Configurations with head size 128 and widths the tcgen05 products take (D; E has every option
    the other way: windows, groups of 8, sigmoid scores, a shared expert, a dense layer, tied
    embeddings, pages of 32), in bfloat16: a
    2,400-token prompt in one step (prompt-portion attention on tensor cores) beside a decoded
    token and the stub of another prompt (the key-splitting kernel writes their rows), prompts
    alone (wide tiles), decoding in a changing batch (narrow tiles, the decode router and the
    per-pair expert products), against the plain implementation.

    Measured on this model: positions whose routing agrees differ from the plain implementation by
    2.5e-3 of the scale in the median and 6.8e-3 at most (TOL is 1e-2, as everywhere); positions
    where a near-tie of two router logits went the other way differ by 1e-2 to 6e-2, and their
    margins reach 0.0100 of the rms of the token's router logits (sums over four times the width of
    the tiny configurations carry more rounding), so a margin below 1.5e-2 counts as a possible
    flip here; no more than 3 % of the positions may need that explanation."""
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
    outputs, runner = helpers.run_replay(str(tmp_path), "bfloat16", steps, 2432 + 320 + 192 + 128)
    got = helpers.collect(reqs, steps, outputs)
    for rid, toks in reqs.items():
        ref = helpers.plain_logits(cfg, weights, toks, True)
        worst = helpers.assert_close(got[rid], ref, "bfloat16", f"{name} bfloat16 {rid}", 16, fragile=1.5e-2)
        print(f"{name} bfloat16 {rid}: worst error {worst:.3e}")
        err = (got[rid].double() - ref[0].double()).abs().reshape(len(toks), -1).max(-1).values / float(ref[0].abs().max())
        assert int((err > helpers.TOL["bfloat16"]).sum()) <= 0.03 * len(toks) + 1, f"{rid}: too many positions beyond the tolerance"
    from quench6k_b200 import ops
    assert ops.tc_status() == 0
    # the same steps in true 32-bit arithmetic: no flips to explain, every position within 5e-6
    outputs, _ = helpers.run_replay(str(tmp_path), "float32", steps, 2432 + 320 + 192 + 128)
    got = helpers.collect(reqs, steps, outputs)
    for rid, toks in reqs.items():
        helpers.assert_close(got[rid], helpers.plain_logits(cfg, weights, toks, False), "float32", f"{name} float32 {rid}")


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
    for rid in model["requests"]:
        helpers.assert_close(got[rid], model["ref"][False][rid], "float32", f"trace_run {rid}")
