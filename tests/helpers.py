"""Shared helpers of the tests: model folders with random weights, replay schedules, comparisons."""
import json
import os
import random

import torch

import plain_flint
import tiny_configs


def make_model_folder(folder, name, seed=0, init_std=None):
    """Write config.json + model.safetensors for tiny config `name`; returns (config dict, weights dict).
    The weights handed back are the generated tensors themselves, not what a reader makes of the
    file, so that the plain implementation does not depend on the product's reader agreeing with
    its writer.  init_std: standard deviation of the matrices instead of the default 0.02 (larger
    values make the layers outweigh the embedding, so that greedy continuations vary)."""
    from quench6k_b200.config import FlintConfig
    from quench6k_b200.models.decoder import DecoderModel
    from quench6k_b200.models.flint import build_spec
    from quench6k_b200.weights.random_init import make_tensor
    from quench6k_b200.weights.safetensors_io import write_safetensors

    cfg_d = tiny_configs.get(name) if isinstance(name, str) else name
    cfg = FlintConfig.from_dict(cfg_d)
    norm_init = tiny_configs.NORM_INIT[name] if isinstance(name, str) else "random"
    spec = build_spec(cfg, norm_init=norm_init)
    model = DecoderModel(spec)
    weights = {t.name: make_tensor(t, seed, init_std or spec.init_std) for t in model.tensors()}
    os.makedirs(folder, exist_ok=True)
    cfg.save(folder)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights.items())
    with open(os.path.join(folder, "config.json")) as f:
        cfg_d = json.load(f)
    return cfg_d, weights


def random_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def plain_logits(cfg_d, weights, tokens, emulate_bf16):
    """(logits [T, V], routing margins [T]) of the plain implementation."""
    return plain_flint.forward(cfg_d, weights, tokens, dtype=torch.float64, emulate_bf16=emulate_bf16, return_margins=True)


# --------------------------------------------------------------------------- schedules
def _ceil64(n, page):
    unit = max(64, page)
    return (n + unit - 1) // unit * unit


def schedule_whole(requests):
    """Each request alone and whole, one after the other."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
    return steps, max(len(t) for t in requests.values())


def schedule_tail(requests, tail=32):
    """Most of each request in one step, the last `tail` tokens one by one."""
    steps = []
    n = 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        n += 1
        for i in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[i:i + 1], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
            n += 1
    return steps, max(len(t) for t in requests.values())


def schedule_portions(requests, seed=0):
    """Each request alone, in portions of changing size down to two tokens (and single tokens)."""
    rng = random.Random(seed)
    steps = []
    n = 0
    for rid, toks in requests.items():
        at = 0
        while at < len(toks):
            size = rng.choice([2, 2, 3, 5, 7, 1, 11, 16, 17, 4])
            size = min(size, len(toks) - at)
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[at:at + size], "want": list(range(size))}],
                          "end": [rid] if at + size == len(toks) else []})
            at += size
            n += 1
    return steps, max(len(t) for t in requests.values())


def schedule_mixed(requests, page, seed=0, max_live=4):
    """Up to max_live live requests; portions of some beside single tokens of others; requests
    skip steps at random; finished requests give way to new ones, whose pages are reused.
    Returns (steps, max_tokens) with max_tokens the peak of the live requests' rounded-up sizes."""
    rng = random.Random(seed)
    pending = list(requests.items())
    live = {}                         # rid -> [tokens, at, prefill_end]
    steps = []
    n = 0
    peak = 0
    while pending or live:
        while pending and len(live) < max_live:
            rid, toks = pending.pop(0)
            live[rid] = [toks, 0, rng.randint(len(toks) // 3, max(len(toks) // 3, len(toks) - 8))]
        peak = max(peak, sum(_ceil64(len(v[0]), page) for v in live.values()))
        entries, end = [], []
        for rid, st in list(live.items()):
            toks, at, pre = st
            if len(live) > 1 and rng.random() < 0.25:
                continue                # this request sits the step out
            if at < pre:
                size = min(rng.choice([2, 3, 6, 9, 13, 24]), pre - at)
            else:
                size = 1
            entries.append({"id": rid, "tokens": toks[at:at + size], "want": list(range(size))})
            st[1] = at + size
            if st[1] == len(toks):
                end.append(rid)
                del live[rid]
        if not entries:
            continue
        steps.append({"step": n, "entries": entries, "end": end})
        n += 1
    return steps, peak


def schedule_wide_decode(requests, page, per_step=6):
    """Many requests live at once: the prompts (all but each request's last 6 to 10 tokens) come in
    steps of `per_step` whole portions, then every live request decodes one token per step until
    its tokens end, so the batch shrinks."""
    steps, n = [], 0
    items = list(requests.items())
    head = {rid: len(t) - (6 + i % 5) for i, (rid, t) in enumerate(items)}
    for i in range(0, len(items), per_step):
        entries = [{"id": rid, "tokens": t[:head[rid]], "want": list(range(head[rid]))} for rid, t in items[i:i + per_step]]
        steps.append({"step": n, "entries": entries, "end": []})
        n += 1
    at = dict(head)
    while at:
        entries, end = [], []
        for rid, t in items:
            if rid not in at:
                continue
            entries.append({"id": rid, "tokens": t[at[rid]:at[rid] + 1], "want": [0]})
            at[rid] += 1
            if at[rid] == len(t):
                end.append(rid)
                del at[rid]
        steps.append({"step": n, "entries": entries, "end": end})
        n += 1
    return steps, sum(_ceil64(len(t), page) for t in requests.values())


def collect(requests, steps, outputs):
    """Per-request logits [len, V] assembled from the per-step outputs (dict step -> tensor [wanted, V])."""
    got = {rid: [None] * len(t) for rid, t in requests.items()}
    at = {rid: 0 for rid in requests}
    for msg in steps:
        out = outputs.get(msg["step"])
        row = 0
        for e in msg["entries"]:
            for w in e["want"]:
                got[e["id"]][at[e["id"]] + w] = out[row]
                row += 1
            at[e["id"]] += len(e["tokens"])
    return {rid: torch.stack(rows) for rid, rows in got.items()}


def collect_wanted(rid, steps, outputs):
    """The logits of one request at the places the steps asked for, in the steps' order: [wanted, V]."""
    rows = []
    for msg in steps:
        out = outputs.get(msg["step"])
        row = 0
        for e in msg["entries"]:
            n = len(e["want"])
            if e["id"] == rid and n:
                rows.append(out[row:row + n])
            row += n
    return torch.cat(rows)


def run_replay(folder, dtype, steps, max_tokens, page_size=None, max_requests=8, runner=None, tap=False):
    """Replay `steps` through the engine's ModelRunner in this process; returns (step -> logits on
    the CPU, runner).  tap: also record which experts every routed layer chose for every row; the
    runner then carries `routing`: request -> {"experts": {executed position: int64 [tokens, k]},
    "router_logits": {executed position: float32 [tokens, E]}}."""
    from quench6k_b200.config.registry import load_config
    from quench6k_b200.engine import ModelRunner
    from quench6k_b200.engine.replay import pool_pages, replay

    if runner is None:
        _, cfg = load_config(folder)
        page = page_size or cfg.kv_page_size or 16
        runner = ModelRunner.from_folder(folder, dtype=dtype, page_size=page, num_pages=pool_pages(max_tokens, page),
                                         max_requests=max_requests)
    outputs = {}
    by_step = {s["step"]: s for s in steps}
    routing = {}
    the_tap = attach_routing_tap(runner, max(sum(len(e["tokens"]) for e in s["entries"]) for s in steps)) if tap else None

    def emit(step, logits):
        if logits is not None:
            outputs[step] = logits.detach().cpu()
        if the_tap is not None:
            row = 0
            for e in by_step[step]["entries"]:
                n = len(e["tokens"])
                for (name, p), buf in the_tap.buffers.items():
                    part = buf[row:row + n].cpu()
                    routing.setdefault(e["id"], {}).setdefault(name, {}).setdefault(p, []).append(part.long() if name == "experts" else part)
                row += n

    replay(runner, steps, emit)
    runner.manager.check()
    assert not runner.manager.requests, "requests left alive after the trace"
    runner.routing = {rid: {name: {p: torch.cat(parts) for p, parts in per.items()} for name, per in names.items()}
                      for rid, names in routing.items()}
    return outputs, runner


def attach_routing_tap(runner, capacity_rows):
    """Give every routed feed-forward of the runner's model one Tap (the debugging hook of
    parts.base) and return it."""
    from quench6k_b200.parts.base import Tap
    tap = Tap(capacity_rows)
    for b in runner.model.blocks:
        if hasattr(b.ffn, "routing_tap"):
            b.ffn.routing_tap = tap
    return tap


# Tolerances, relative to the largest reference logit of the sequence.  float32: the engine against
# float64 arithmetic (measured at the first pass: 7e-7).  bfloat16: the engine against the plain
# implementation rounding to bfloat16 at the same places (measured at the first pass: at most 0.6
# percent).  They were set when the first kernels passed and are not to be widened.
#
# A mixture of experts is discontinuous: where the router's last chosen and first rejected logits
# nearly tie, bfloat16 rounding may choose the other expert, and the logits of that position (and
# of those that attend to it) move by far more than rounding.  So in bfloat16 the engine reports
# its router logits and the experts it chose (parts.base.Tap), and the plain implementation is run
# on those experts (forced_routing).  Then every position must meet TOL, with no exception, and
# the routing itself is checked in two parts: the engine's router logits are held to the same TOL
# against the plain implementation's (relative to the layer's largest router logit), and the
# engine's experts must be the k best of its own router logits.  The float32 runs are compared the
# same way with their own TOL: among thousands of tokens and hundreds of experts even float32
# rounding meets a tie now and then.
TOL = {"float32": 5e-6, "bfloat16": 1e-2}


def assert_close(got, want, dtype, what):
    """Every position of `got` within TOL[dtype] of `want`, relative to the largest logit of `want`."""
    if isinstance(want, tuple):
        want = want[0]
    want = want.to(torch.float64)
    got = got.to(device=want.device, dtype=torch.float64)
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} against {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: the engine produced non-finite logits"
    scale = float(want.abs().max())
    per_pos = (got - want).abs().reshape(want.shape[0], -1).max(dim=-1).values / scale
    worst = int(per_pos.argmax())
    assert float(per_pos[worst]) <= TOL[dtype], (f"{what}: error {float(per_pos[worst]):.3e} of scale {scale:.3f} at position {worst} "
                                                 f"exceeds {TOL[dtype]:.1e} ({int((per_pos > TOL[dtype]).sum())} of {len(per_pos)} positions do)")
    return float(per_pos[worst])


def assert_matches_plain(cfg_d, weights, tokens, got, dtype, what, routing=None, positions=None, device=None):
    """The engine's logits of one request against the plain implementation.  `routing`
    ({"experts" | "router_logits": {executed position: [tokens, ...]}}, from run_replay(tap=True);
    bfloat16 needs it, float32 may do without) is checked and forced on the plain implementation.  positions: the positions `got` holds
    (default: all).  Returns (worst error, number of positions at which the plain implementation's
    own router would have chosen another set of experts)."""
    flipped = 0
    if dtype == "bfloat16" or routing is not None:
        assert routing is not None or not any_routed(cfg_d), f"{what}: a bfloat16 comparison needs the engine's routing"
        experts = routing["experts"] if routing else {}
        want, routers = plain_flint.forward(cfg_d, weights, tokens, emulate_bf16=dtype == "bfloat16", forced_routing=experts,
                                            logit_positions=positions, device=device)
        differs = torch.zeros(len(tokens), dtype=torch.bool)
        for p, (z_plain, own) in routers.items():
            z = routing["router_logits"][p].to(device=z_plain.device, dtype=torch.float64)
            chosen = experts[p].to(z_plain.device)
            scale = float(z_plain.abs().max())
            err = (z - z_plain).abs().max(dim=-1).values / scale
            over = err > TOL[dtype]
            assert not bool(over.any()), (f"{what}: router logits of executed layer {p} differ by {float(err[over].max()):.3e} of their "
                                          f"scale {scale:.3f} at position {int(over.nonzero()[0])} ({int(over.sum())} positions beyond the tolerance)")
            # the k best of the engine's own logits: no chosen logit below an unchosen one (beyond FP32 rounding)
            picked = torch.zeros_like(z, dtype=torch.bool).scatter_(1, chosen, True)
            assert int(picked.sum(-1).min()) == chosen.shape[1], f"{what}: layer {p} chose an expert twice"
            lowest_in = z.masked_fill(~picked, float("inf")).min(-1).values
            highest_out = z.masked_fill(picked, float("-inf")).max(-1).values
            bad = lowest_in < highest_out - 1e-6 * scale
            assert not bool(bad.any()), f"{what}: layer {p}, position {int(bad.nonzero()[0])}: the chosen experts are not the best of the engine's own router logits"
            differs |= (chosen.sort(-1).values != own.sort(-1).values).any(-1).cpu()
        flipped = int(differs.sum())
        if dtype == "float32":
            assert flipped <= 1 + len(tokens) // 500, f"{what}: {flipped} positions routed differently: more than float32 rounding meets ties"
    else:
        want = plain_flint.forward(cfg_d, weights, tokens, logit_positions=positions, device=device)
    return assert_close(got, want, dtype, what), flipped


def any_routed(cfg_d):
    return cfg_d.get("first_k_dense_replace", 0) < cfg_d["num_hidden_layers"]


def make_context(q_lens, pos_starts, tables, n_groups=1, device="cuda"):
    """A StepContext for tests of single parts: tables[g][r] is request r's page list in group g."""
    from quench6k_b200.engine.batch import StepContext
    i32 = dict(dtype=torch.int32, device=device)
    pos, rot = [], []
    for r, (n, p0) in enumerate(zip(q_lens, pos_starts)):
        pos += list(range(p0, p0 + n))
        rot += [r] * n
    T, R = len(pos), len(q_lens)
    qs = [0]
    for n in q_lens:
        qs.append(qs[-1] + n)
    bts = []
    for g in range(n_groups):
        width = max(len(t) for t in tables[g])
        bts.append(torch.tensor([list(t) + [-1] * (width - len(t)) for t in tables[g]], **i32))
    return StepContext(T=T, R=R, token_ids=torch.zeros(T, **i32), positions=torch.tensor(pos, **i32),
                       req_of_token=torch.tensor(rot, **i32), q_start=torch.tensor(qs, **i32),
                       pos_start=torch.tensor(pos_starts, **i32), slot_ids=torch.arange(R, **i32), block_tables=bts,
                       logit_rows=torch.arange(T, **i32), n_logit_rows=T, q_lens=list(q_lens), pos_starts=list(pos_starts),
                       slots=list(range(R)), max_context=max(p + n for p, n in zip(pos_starts, q_lens)), max_q_len=max(q_lens))
