"""Shared helpers of the tests: model folders with random weights, replay schedules, comparisons."""
import json
import os
import random

import torch

import plain_flint
import tiny_configs


def make_model_folder(folder, name, seed=0):
    """Write config.json + model.safetensors for tiny config `name`; returns (config dict, weights dict)."""
    from quench6k_b200.config import FlintConfig
    from quench6k_b200.models.decoder import DecoderModel
    from quench6k_b200.models.flint import build_spec
    from quench6k_b200.weights import index_folder, write_model_folder

    cfg_d = tiny_configs.get(name)
    cfg = FlintConfig.from_dict(cfg_d)
    spec = build_spec(cfg, norm_init=tiny_configs.NORM_INIT[name])
    model = DecoderModel(spec)
    write_model_folder(folder, cfg, model.tensors(), seed, spec.init_std)
    idx = index_folder(folder)
    weights = {n: f.read(n) for n, (f, e) in idx.items()}
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


def run_replay(folder, dtype, steps, max_tokens, page_size=None):
    """Replay `steps` through the engine's ModelRunner in this process; returns step -> logits (CPU)."""
    from quench6k_b200.config.registry import load_config
    from quench6k_b200.engine import ModelRunner
    from quench6k_b200.engine.replay import pool_pages, replay

    _, cfg = load_config(folder)
    page = page_size or cfg.kv_page_size or 16
    runner = ModelRunner.from_folder(folder, dtype=dtype, page_size=page, num_pages=pool_pages(max_tokens, page), max_requests=8)
    outputs = {}

    def emit(step, logits):
        if logits is not None:
            outputs[step] = logits.detach().cpu()

    replay(runner, steps, emit)
    runner.manager.check()
    assert not runner.manager.requests, "requests left alive after the trace"
    return outputs, runner


# Tolerances, relative to the largest reference logit of the sequence.  float32: the engine against
# float64 arithmetic (measured at the first pass: 7e-7).  bfloat16: the engine against the plain implementation rounding to bfloat16
# at the same places (measured at the first pass: at most 0.6 percent at positions with decisive
# routing).  They were set when the first kernels passed and are not to be widened.
#
# A mixture of experts is discontinuous: where the router's last chosen and first rejected logits
# nearly tie, rounding may choose the other expert, and the logits of that position move by far
# more than rounding; its changed keys and values then disturb the positions that attend to it
# (measured: for a sliding window's length), where a second near-tie may flip in turn.  In bfloat16
# a position may therefore exceed the tolerance only if a routing flip explains it: its own routing
# margin in the plain implementation (gap of the two router logits over the rms of the token's
# router logits, smallest over the layers) is below FRAGILE, or a position that exceeded the
# tolerance lies within `reach` positions before it.  Such positions must still stay within
# BF16_FLIPPED_TOL.  Every other position, and every position in float32, must meet TOL.
TOL = {"float32": 5e-6, "bfloat16": 1e-2}
FRAGILE = 1e-2
BF16_FLIPPED_TOL = 0.5


def assert_close(got, ref, dtype, what, reach=16, fragile=FRAGILE):
    """ref: (logits, margins) from plain_logits, or a plain tensor.  reach: how far a flipped
    position's keys are seen (the configuration's sliding window, at least 8).  fragile: the
    routing margin below which a flip may explain a bfloat16 difference (a caller with a wider
    model states its own and why; TOL and BF16_FLIPPED_TOL are the same for everyone)."""
    want, margins = ref if isinstance(ref, tuple) else (ref, None)
    want = want.to(torch.float64)
    got = got.to(torch.float64)
    assert torch.isfinite(got).all(), f"{what}: the engine produced non-finite logits"
    scale = float(want.abs().max())
    per_pos = ((got - want).abs().reshape(want.shape[0], -1).max(dim=-1).values / scale).tolist()
    tol = TOL[dtype]
    explained = 0
    over = [False] * len(per_pos)
    for p, err in enumerate(per_pos):
        if err <= tol:
            continue
        over[p] = True
        ok = False
        if dtype == "bfloat16" and margins is not None and err <= BF16_FLIPPED_TOL:
            ok = float(margins[p]) < fragile or any(over[max(0, p - reach):p])
        if not ok:
            raise AssertionError(f"{what}: error {err:.3e} of scale {scale:.3f} at position {p} exceeds {tol:.1e} "
                                 f"(routing margin {float(margins[p]) if margins is not None else float('nan'):.4f}; "
                                 f"{explained} earlier positions were explained by routing flips)")
        explained += 1
    if explained > 0.2 * len(per_pos):
        raise AssertionError(f"{what}: {explained} of {len(per_pos)} positions differ by routing flips: too many to be rounding")
    return max(per_pos)


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
