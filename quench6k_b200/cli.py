"""Command line in the manner of the reference's `quench6k flint generate`
(crates/cli/src/flint.rs:13-27, :217-288): `--model DIR --n 64 --context 32768`, greedy by
default, printing the prompt's token count, the first token's top 5, the generated ids and the
prefill and decode rates in the reference's wording.  The reference tokenizes `--prompt` text;
this engine takes token ids (`--prompt-ids 1,2,3`, or `--prompt-len N` seeded random ids).

    python -m quench6k_b200.cli generate --model DIR --prompt-ids 1,2,3 --n 16
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
    r = sub.add_parser("random-weights", help="write a model folder from a configuration and a seed")
    r.add_argument("--config", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.set_defaults(fn=_random_weights)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
