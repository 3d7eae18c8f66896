"""Command line in the manner of the reference's `quench6k flint generate`
(crates/cli/src/flint.rs:13-27, :217-288): `--model DIR --n 64 --context 32768`, greedy by
default, printing the prompt's token count, the first token's top 5, the generated ids and the
prefill and decode rates in the reference's wording.  The reference tokenizes `--prompt` text;
this engine takes token ids (`--prompt-ids 1,2,3`, or `--prompt-len N` seeded random ids).

`bench` and `ppl` follow `flint bench` and `flint ppl` (:28-55) with files of token ids in place of
text files.

    python -m quench6k_b200.cli generate --model DIR --prompt-ids 1,2,3 --n 16
    python -m quench6k_b200.cli bench --model DIR --ctx 512 8192 --generate 128 --json bench.jsonl
    python -m quench6k_b200.cli ppl --model DIR --file ids.txt --ctx 2048 --chunks 8
    python -m quench6k_b200.cli random-weights --config config.json --seed 0 --out DIR
"""
from __future__ import annotations

import argparse
import sys
import time


def _generate(a) -> int:
    import torch
    from . import ops
    from .engine import Engine
    from .sampling import SamplingParams

    page = a.page_size
    if a.model:
        from .config.registry import load_config
        _, cfg = load_config(a.model)
        page = page or getattr(cfg, "kv_page_size", None) or 16
        num_pages = a.num_pages or (a.context + page - 1) // page
        eng = Engine.from_folder(a.model, dtype=a.dtype, page_size=page, num_pages=num_pages,
                                 max_batch_tokens=a.max_batch_tokens)
    else:
        from .config.registry import load_config
        _, cfg = load_config(a.random)
        page = page or getattr(cfg, "kv_page_size", None) or 16
        num_pages = a.num_pages or (a.context + page - 1) // page
        eng = Engine.from_random(cfg, seed=a.seed, dtype=a.dtype, page_size=page, num_pages=num_pages,
                                 max_batch_tokens=a.max_batch_tokens)
    vocab = eng.runner.vocab_size
    if a.prompt_ids:
        ids = [int(x) for x in a.prompt_ids.split(",") if x.strip()]
    else:
        g = torch.Generator().manual_seed(a.seed)
        ids = torch.randint(0, vocab, (a.prompt_len,), generator=g).tolist()
    print(f"prompt: {len(ids)} tokens")
    params = SamplingParams(max_tokens=a.n, temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, min_p=a.min_p,
                            seed=a.sample_seed)
    rid = eng.add_request(ids, params)
    req = eng.scheduler.by_id[rid]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    first_top = None
    while not req.output and not req.finished:
        plan = eng.scheduler.schedule()
        logits = eng.runner.step(plan.step_entries())
        sampled = []
        if logits is not None:
            tid, tval = ops.topk_pool(logits, min(5, vocab))
            first_top = list(zip(tid[0].tolist(), tval[0].tolist()))
            sampled = eng.sampler.sample(logits, [req.params], [req.output], [req.rng])
        eng.scheduler.update(plan, sampled)
    torch.cuda.synchronize()
    prefill = time.perf_counter() - t0
    if first_top:
        print("first-token top 5: " + ", ".join(f"{t} {v:.3f}" for t, v in first_top))
    t1 = time.perf_counter()
    while eng.has_unfinished():
        eng.step()
    torch.cuda.synchronize()
    decode = time.perf_counter() - t1
    out = req.output
    print(f"ids: {out}")
    print(f"prefill {len(ids)} tokens in {prefill:.3f}s ({len(ids) / prefill:.0f} tok/s); "
          f"decode {len(out) - 1} tokens in {decode:.3f}s ({(len(out) - 1) / max(decode, 1e-9):.1f} tok/s)")
    return 0


def _runner(a, tokens: int):
    """A model runner with room for `tokens` cached tokens of one request."""
    from .config.registry import load_config
    from .engine import ModelRunner
    _, cfg = load_config(a.model or a.random)
    page = a.page_size or getattr(cfg, "kv_page_size", None) or 16
    num_pages = (tokens + page - 1) // page + 1
    if a.model:
        return ModelRunner.from_folder(a.model, dtype=a.dtype, page_size=page, num_pages=num_pages, max_requests=2)
    return ModelRunner.from_random(cfg, a.seed, dtype=a.dtype, page_size=page, num_pages=num_pages, max_requests=2)


def _corpus(path, need: int, vocab: int, seed: int):
    """Token ids from a file of integers (any of space, comma, newline between them), or seeded
    uniform-random ids where the reference would tokenize a text file."""
    import torch
    if path:
        with open(path) as f:
            ids = [int(x) for x in f.read().replace(",", " ").split()]
        if len(ids) < need:
            raise SystemExit(f"corpus has {len(ids)} tokens, {need} needed")
        bad = [t for t in ids[:need] if not 0 <= t < vocab]
        if bad:
            raise SystemExit(f"corpus holds token id {bad[0]} outside 0..{vocab - 1}")
        return ids
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (need,), generator=g).tolist()


def _prefill(runner, rid, ids, portion: int):
    """The prompt in portions of at most `portion` tokens; logits of its last token."""
    from .engine import StepEntry
    logits = None
    for at in range(0, len(ids), portion):
        part = ids[at:at + portion]
        logits = runner.step([StepEntry(rid, part, [len(part) - 1] if at + len(part) == len(ids) else [])])
    return logits


def _bench(a) -> int:
    """Prefill and greedy decode throughput at each context length, as the reference's
    `flint bench` measures them (crates/cli/src/flint.rs:83-152): prefill from the first upload to
    the first argmax; decode = generate - 1 steps, each followed by the 4-byte download of its
    argmax; at the first context, decoding that replays CUDA graphs must give the same tokens as
    eager decoding; one JSON record per context is appended to --json."""
    import json
    import torch
    from . import ops
    from .engine import StepEntry
    gen = a.generate
    runner = _runner(a, max(a.ctx) + gen + 8)
    ids = _corpus(a.ids, max(a.ctx) + gen, runner.vocab_size, a.seed)

    def decode_run(ctx, n):
        runner.add_request("b")
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        nxt = int(ops.argmax(_prefill(runner, "b", ids[:ctx], a.max_batch_tokens))[0])
        prefill = time.perf_counter() - t0
        out = [nxt]
        t1 = time.perf_counter()
        while len(out) < n:
            nxt = int(ops.argmax(runner.step([StepEntry("b", [nxt], [0])]))[0])
            out.append(nxt)
        decode = time.perf_counter() - t1
        runner.end_request("b")
        return out, prefill, decode

    for i, ctx in enumerate(a.ctx):
        out, prefill, decode = decode_run(ctx, gen)
        copied = sum(1 for x, y in zip(out, ids[ctx:]) if x == y)
        if i == 0 and runner.cuda_graphs:
            runner.cuda_graphs = False
            eager, _, _ = decode_run(ctx, min(gen, 64))
            runner.cuda_graphs = True
            if eager != out[:len(eager)]:
                raise SystemExit(f"graph decoding differs from eager decoding: {eager} vs {out[:len(eager)]}")
            print(f"graph decoding matches eager decoding ({len(eager)} tokens)")
        pf, tg = ctx / prefill, (gen - 1) / max(decode, 1e-9)
        print(f"ctx {ctx:>6}: prefill {pf:>7.0f} tok/s ({prefill:.2f}s), decode {tg:>6.1f} tok/s; corpus continuation {copied}/{gen}; {out[:24]}")
        if a.json:
            rec = {"engine": "quench6k_b200", "model": a.model or a.random, "mode": "plain", "kv": "bf16" if a.dtype in ("bfloat16", "bf16") else "fp32",
                   "ctx": ctx, "generate": gen, "prefill_tok_s": round(pf, 1), "decode_tok_s": round(tg, 1), "copied": copied}
            with open(a.json, "a") as f:
                f.write(json.dumps(rec) + "\n")
    return 0


def _ppl(a) -> int:
    """Perplexity of a file of token ids as the reference's `flint ppl` computes it
    (crates/cli/src/flint.rs:154-203, after llama-perplexity): chunks of `ctx` tokens, each scored on
    its second half (the logits of positions ctx/2 .. ctx-2 predict the next token)."""
    import math
    import torch
    from . import ops
    from .engine import StepEntry
    ctx = a.ctx
    half = ctx // 2
    if half < 1 or ctx - 1 <= half:
        raise SystemExit("--ctx must be at least 4")
    with open(a.file) as f:
        ids = [int(x) for x in f.read().replace(",", " ").split()]
    n_chunks = min(len(ids) // ctx, a.chunks)
    if n_chunks < 1:
        raise SystemExit(f"{len(ids)} tokens: fewer than one chunk of {ctx}")
    runner = _runner(a, ctx + 8)
    piece = min(a.max_batch_tokens, half)
    nll, count = 0.0, 0
    t0 = time.perf_counter()
    for c in range(n_chunks):
        toks = ids[c * ctx:(c + 1) * ctx]
        runner.add_request("p")
        _prefill(runner, "p", toks[:half], a.max_batch_tokens)
        at = half
        while at < ctx - 1:
            rows = min(piece, ctx - 1 - at)
            logits = runner.step([StepEntry("p", toks[at:at + rows], list(range(rows)))])
            target = torch.tensor(toks[at + 1:at + 1 + rows], dtype=torch.int32, device=logits.device)
            lse, tl = ops.row_logsumexp(logits, target)
            nll += float((lse - tl).double().sum())
            count += rows
            at += rows
        runner.end_request("p")
        print(f"[{c + 1}] {math.exp(nll / count):.4f}")
    print(f"PPL over {n_chunks} chunks of {ctx}: {math.exp(nll / count):.4f} ({time.perf_counter() - t0:.1f}s)")
    return 0


def _random_weights(a) -> int:
    from .config.registry import load_config
    from .models.decoder import DecoderModel
    from .weights import write_model_folder

    arch, cfg = load_config(a.config)
    spec = arch.build_spec(cfg)
    model = DecoderModel(spec)
    write_model_folder(a.out, cfg, model.tensors(), a.seed, spec.init_std)
    print(f"wrote {a.out}/config.json and {a.out}/model.safetensors ({len(model.tensors())} tensors, seed {a.seed})")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="quench6k_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="generate from token ids, printing ids and timings")
    src = g.add_mutually_exclusive_group(required=True)
    src.add_argument("--model", help="folder with config.json and model.safetensors")
    src.add_argument("--random", metavar="CONFIG.json", help="random weights from this configuration")
    g.add_argument("--seed", type=int, default=0, help="seed of the random weights and of --prompt-len ids")
    p = g.add_mutually_exclusive_group(required=True)
    p.add_argument("--prompt-ids", help="comma-separated token ids")
    p.add_argument("--prompt-len", type=int, help="this many seeded uniform-random token ids")
    g.add_argument("--n", type=int, default=64, help="tokens to generate")
    g.add_argument("--context", type=int, default=32768, help="token places in the cache")
    g.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    g.add_argument("--top-k", type=int, default=20)
    g.add_argument("--top-p", type=float, default=0.95)
    g.add_argument("--min-p", type=float, default=0.0)
    g.add_argument("--sample-seed", type=int, default=0)
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    g.add_argument("--page-size", type=int, default=None)
    g.add_argument("--num-pages", type=int, default=None)
    g.add_argument("--max-batch-tokens", type=int, default=2048)
    g.set_defaults(fn=_generate)
    def source(q):
        src = q.add_mutually_exclusive_group(required=True)
        src.add_argument("--model", help="folder with config.json and model.safetensors")
        src.add_argument("--random", metavar="CONFIG.json", help="random weights from this configuration")
        q.add_argument("--seed", type=int, default=0, help="seed of the random weights (and of random token ids)")
        q.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
        q.add_argument("--page-size", type=int, default=None)
        q.add_argument("--max-batch-tokens", type=int, default=2048, help="tokens of a prompt portion")

    b = sub.add_parser("bench", help="prefill and greedy decode throughput at each context length")
    source(b)
    b.add_argument("--ids", help="file of token ids (the reference's --text, tokenized); default: seeded random ids")
    b.add_argument("--ctx", type=int, nargs="+", default=[512, 8192, 65536, 131072, 260000])
    b.add_argument("--generate", type=int, default=128)
    b.add_argument("--json", help="append one JSON record per context to this file")
    b.set_defaults(fn=_bench)
    q = sub.add_parser("ppl", help="perplexity of a file of token ids, chunks of --ctx tokens scored on their second half")
    source(q)
    q.add_argument("--file", required=True, help="file of token ids (the reference tokenizes a text file)")
    q.add_argument("--ctx", type=int, default=2048)
    q.add_argument("--chunks", type=int, default=8)
    q.set_defaults(fn=_ppl)
    r = sub.add_parser("random-weights", help="write a model folder from a configuration and a seed")
    r.add_argument("--config", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.set_defaults(fn=_random_weights)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
