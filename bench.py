#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of the half-depth Flint configuration (24 layers, hidden 2048,
32 query / 4 KV heads of 128, 256 experts of width 512, top-8, vocabulary 151,936) with random
weights, a batch of 8 requests that each hold 32,768 cached tokens, bfloat16.  One JSON line:
`value` is decoded tokens a second timed on the device (CUDA events around K decode steps of
ModelRunner.step plus the device argmax); `e2e` is the same through Engine.step() with host token
ids in (pinned host memory -> device) and sampled ids out (device -> host) every step; `prefill`
is one 2,048-token prompt in one step; `points` are decode at batch 1 and 64; `roofline` is the
decode step's bytes (every weight it uses once, and the cache of the live requests) over its time
over the peak copy bandwidth.  Peaks come from MEASURED_PEAKS.json beside this file when the
measuring harness wrote it, else from the fallback figures below.

The caches are filled with random values instead of by a prefill (the weights are random too), so
every request stands at the context length at once; what the decode step reads and computes is the
same.  Inputs are larger than L2: one decode step streams gigabytes of weights and cache.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

CONFIG2 = {
    "architectures": ["FlintForCausalLM"], "hidden_size": 2048, "num_hidden_layers": 24, "num_attention_heads": 32,
    "num_key_value_heads": 4, "head_dim": 128, "vocab_size": 151936, "n_routed_experts": 256, "num_experts_per_tok": 8,
    "moe_intermediate_size": 512, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "kv_page_size": 16,
}


# the further shapes this file can run: the full-depth model (about 80 GB of weights) at 8,192 cached tokens
SHAPES = {2: {"layers": 24, "context": 32768, "label": "Recursive Flint MoE, half-depth shape"},
          3: {"layers": 48, "context": 8192, "label": "Recursive Flint MoE, 40B-A2.5B shape"}}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in d.items() if k in out and isinstance(v, (int, float))})
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """SM clock and throttle reasons of GPU 0 while a timed region runs: read through NVML every
    5 ms when its Python binding is there (a timed region of a few dozen milliseconds still gets
    several samples), else from `nvidia-smi -lms 200`.  Reading only; nothing is set."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.lines, self.proc, self.nvml, self.samples, self.stop_flag = [], None, None, [], False

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(int(os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0] or 0)
                                                            if os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0].isdigit() else 0)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll(self):
        nv = self.nvml
        bits = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self.stop_flag:
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = int(reasons_fn(self.handle))
                self.samples.append((mhz, {n for n, b in bits.items() if mask & b}))
            except Exception:
                pass
            time.sleep(0.005)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self.stop_flag = True
            self.thread.join(timeout=1)
            sm = sorted(m for m, _ in self.samples)
            reasons = set().union(*[r for _, r in self.samples]) if self.samples else set()
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(reasons),
                    "samples": len(sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])), mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(self.NAMES, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi"}


def expected_experts(E, k, B):
    return E * (1.0 - (1.0 - k / E) ** B)


def decode_bytes(cfg, layers, B, ctx, experts_read=None):
    """Bytes one decode step has to read: every weight it uses once, and the cache of the live requests.
    experts_read: distinct experts per layer that the router really chose (measured); else the expectation."""
    D, Hq, Hkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    E, k, I, V = cfg["n_routed_experts"], cfg["num_experts_per_tok"], cfg["moe_intermediate_size"], cfg["vocab_size"]
    attn = ((Hq + 2 * Hkv) * hd * D + D * Hq * hd) * 2
    router = E * D * 2
    experts = (experts_read if experts_read is not None else expected_experts(E, k, B)) * 3 * I * D * 2
    weights = layers * (attn + router + experts) + V * D * 2
    kv = B * ctx * layers * 2 * Hkv * hd * 2
    return weights + kv, weights, kv


def prefill_bytes(cfg, layers, T):
    """Bytes a prefill step of T tokens has to read at least: every weight once (with T * k pairs far above the number of
    experts, all of them), the logits' row of the head aside."""
    D, Hq, Hkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    E, k, I, V = cfg["n_routed_experts"], cfg["num_experts_per_tok"], cfg["moe_intermediate_size"], cfg["vocab_size"]
    per_layer = ((Hq + 2 * Hkv) * hd * D + D * Hq * hd + E * D + expected_experts(E, k, T) * 3 * I * D) * 2
    return layers * per_layer + V * D * 2


def prefill_flops(cfg, layers, T):
    D, Hq, Hkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    E, k, I, V = cfg["n_routed_experts"], cfg["num_experts_per_tok"], cfg["moe_intermediate_size"], cfg["vocab_size"]
    per_token = (Hq + 2 * Hkv) * hd * D + D * Hq * hd + E * D + k * 3 * I * D
    matmul = 2.0 * T * layers * per_token + 2.0 * V * D
    attention = layers * 4.0 * Hq * hd * T * (T / 2.0)
    return matmul + attention


def kernel_attention_prefill(args):
    """The prompt-portion attention kernel alone: T query tokens of one request whose last token stands
    at position `context - 1`, over a cache of `context` keys (so T = context is a whole prompt from
    position 0); FLOPs counted under the causal mask; CUDA events, warm-up, cache larger than L2 from
    32,768 keys on."""
    import torch
    from quench6k_b200 import ops
    from quench6k_b200.engine.batch import StepContext
    c = CONFIG2
    Hq, Hkv, hd, ps = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"], args.page_size or c["kv_page_size"]
    n, T, dev = args.context, min(args.prefill_tokens, args.context), "cuda:0"
    pages = (n + ps - 1) // ps
    kp = torch.randn(Hkv, pages, ps, hd, device=dev).to(torch.bfloat16)
    vp = torch.randn(Hkv, pages, ps, hd, device=dev).to(torch.bfloat16)
    q = torch.randn(T, Hq, hd, device=dev).to(torch.bfloat16)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    ctx = StepContext(T=T, R=1, token_ids=i32([0] * T), positions=i32(list(range(n - T, n))), req_of_token=i32([0] * T), q_start=i32([0, T]),
                      pos_start=i32([n - T]), slot_ids=i32([0]), block_tables=[i32([list(range(pages))])], logit_rows=i32([]), n_logit_rows=0,
                      q_lens=[T], pos_starts=[n - T], slots=[0], max_context=n, max_q_len=T)
    tok0, ntok, n_tiles = ctx.query_tile_pairs(ops.attention_tc_tile_tokens(Hq // Hkv), False)
    run = lambda: ops.attention_tc(q, kp, vp, ctx.block_tables[0], ctx.req_of_token, ctx.positions, tok0, ntok, None, None)
    for _ in range(max(3, args.warmup)):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    assert ops.tc_status() == 0
    ms = e0.elapsed_time(e1) / args.steps
    flops = 4.0 * Hq * hd * T * (n - T + (T + 1) / 2.0)
    pk = peaks()
    print(json.dumps({"kernel": "attention_tc (prompt portions)", "tokens": T, "context": n, "us": round(ms * 1e3, 1),
                      "tflops": round(flops / ms / 1e9, 1), "frac_of_bf16_peak": round(flops / ms / 1e9 / pk["bf16_tflops"], 3),
                      "peaks": pk["source"], "ctas": n_tiles * Hkv, "steps": args.steps}))
    return 0


def profile_ops(args, runner, cfg_d, layers, ctx, stand_at_context, rand_ids):
    """Where the time of an eager decode step (batch --batch at the context) and of a prefill step goes, launcher by
    launcher: CUDA events around every launch (quench6k_b200.ops.profile_begin/profile_end), no profiler involved.  Eager
    launches leave gaps that a replayed graph does not have, so the sum is the step's kernel time, not its duration."""
    import torch
    from quench6k_b200 import ops
    from quench6k_b200.engine import StepEntry
    runner.cuda_graphs = False
    B, T = args.batch, args.prefill_tokens
    rids = [f"q{i}" for i in range(B)]
    stand_at_context(rids)
    toks = [rand_ids(args.steps + args.warmup) for _ in rids]
    step = lambda i: runner.step([StepEntry(r, [toks[j][i]], [0]) for j, r in enumerate(rids)])
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    ops.profile_begin()
    for i in range(args.warmup, args.warmup + args.steps):
        step(i)
    decode = ops.profile_end()
    for r in rids:
        runner.end_request(r)
    prefill = {}
    for it in range(2):
        runner.add_request("p")
        ids = rand_ids(T)
        if it:
            ops.profile_begin()
        runner.step([StepEntry("p", ids, [T - 1])])
        if it:
            prefill = ops.profile_end()
        runner.end_request("p")
    table = lambda rec, n: [{"op": tag, "launcher": fn, "calls_per_step": calls / n, "us_per_step": round(ms * 1e3 / n, 1)}
                            for (tag, fn), (calls, ms) in rec.items()]
    print(json.dumps({"profile": "CUDA events around every launch of eager steps", "layers": layers, "batch": B, "context": ctx,
                      "decode_step": table(decode, args.steps), "decode_us": round(sum(ms for _, ms in decode.values()) * 1e3 / args.steps, 1),
                      "prefill_tokens": T, "prefill_step": table(prefill, 1), "prefill_us": round(sum(ms for _, ms in prefill.values()) * 1e3, 1)}))
    return 0


def workload_stress(args, shape):
    """A long prompt beside many short sampled requests, through the engine's own scheduler and
    paged cache: one request of `--context` (131,072) uniform-random tokens, greedy, 128 new tokens;
    `--batch - 1` (63) requests of 256 to 16,384 tokens at temperature 1.0, 128 new tokens each.
    Host wall clock around Engine.step() until everything has finished; one JSON line."""
    import torch
    from quench6k_b200 import Engine, SamplingParams, ops
    from quench6k_b200.config import FlintConfig
    torch.cuda.set_device(0)
    long_len, n_req, new = args.context or 131072, args.batch or 64, 128
    cfg_d = dict(CONFIG2)
    layers = args.layers or shape["layers"]
    cfg_d["num_hidden_layers"] = layers
    if args.page_size:
        cfg_d["kv_page_size"] = args.page_size
    cfg = FlintConfig.from_dict(cfg_d)
    page, budget = cfg.kv_page_size, args.prefill_tokens
    gen = torch.Generator().manual_seed(4)
    lens = [long_len] + [int(x) for x in torch.randint(256, min(16384, long_len) + 1, (n_req - 1,), generator=gen)]
    num_pages = sum((n + new + page - 1) // page + 1 for n in lens)      # every request fits at once: no preemption is forced
    t0 = time.time()
    eng = Engine.from_random(cfg, seed=0, dtype=args.dtype, page_size=page, num_pages=num_pages, max_requests=n_req,
                             max_batch_tokens=budget)
    torch.cuda.synchronize()
    print(f"[bench] model and cache ready in {time.time() - t0:.1f}s ({torch.cuda.memory_allocated() / 2**30:.1f} GiB on the device)",
          file=sys.stderr, flush=True)
    V = cfg.vocab_size
    ids = lambda n: torch.randint(0, V, (n,), generator=gen).tolist()
    warm = eng.generate([ids(budget), ids(300)], SamplingParams(max_tokens=4, temperature=0.0))      # first-call costs stay outside
    assert all(len(o.tokens) == 4 for o in warm)
    torch.cuda.synchronize()
    base = dict(eng.stats)
    clocks = ClockSampler()
    clocks.start()
    t1 = time.perf_counter()
    rids = [eng.add_request(ids(n), SamplingParams(max_tokens=new, temperature=0.0 if i == 0 else 1.0, seed=100 + i), rid=f"s{i}")
            for i, n in enumerate(lens)]
    done, first_long, decode_only_s, decode_only_tokens, last = {}, None, 0.0, 0, t1
    while len(done) < len(rids):
        prompts_left = any(not r.output for r in list(eng.scheduler.running) + list(eng.scheduler.waiting))
        tokens_before = eng.stats["tokens"]
        for out in eng.step():
            done[out.rid] = out
        now = time.perf_counter()
        if not prompts_left:                      # a step of decode tokens only
            decode_only_s += now - last
            decode_only_tokens += eng.stats["tokens"] - tokens_before
        if first_long is None and any(r.rid == "s0" and r.output for r in eng.scheduler.running):
            first_long = now - t1
        last = now
    torch.cuda.synchronize()
    total_s = time.perf_counter() - t1
    clock_info = clocks.stop()
    assert ops.tc_status() == 0
    generated = sum(len(o.tokens) for o in done.values())
    print(json.dumps({
        "workload": "stress: a long greedy prompt in portions beside sampled requests, continuous batching", "impl": "ours",
        "config": {"model": shape["label"], "layers": layers, "layers_full": shape["layers"], "requests": n_req, "long_prompt": long_len,
                   "other_prompts": "uniform 256..16384", "new_tokens": new, "token_budget": budget, "page_size": page,
                   "pages": num_pages, "dtype": args.dtype},
        "prompt_tokens": sum(lens), "generated_tokens": generated, "seconds": round(total_s, 3),
        "tokens_per_s": round((sum(lens) + generated) / total_s, 1),
        "long_prompt_first_token_s": None if first_long is None else round(first_long, 3),
        "decode_only": {"tokens": decode_only_tokens, "tok_per_s": round(decode_only_tokens / decode_only_s, 1) if decode_only_s else None},
        "steps": eng.stats["steps"] - base["steps"], "preemptions": eng.stats["preemptions"] - base["preemptions"],
        "gib_on_device": round(torch.cuda.max_memory_allocated() / 2**30, 1), "clocks": clock_info}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--config", type=int, default=2, choices=sorted(SHAPES),
                    help="2: 24 layers at 32,768 cached tokens (the default run); 3: the full 48 layers at 8,192 cached tokens")
    ap.add_argument("--workload", default="decode", choices=["decode", "stress"],
                    help="stress: one 131,072-token prompt in 2,048-token portions and 128 decoded tokens beside 63 sampled requests "
                         "of 256 to 16,384 tokens, all through Engine.step() (its own JSON line; --context and --batch scale it down)")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--context", type=int, default=None)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--points", default="1,64", help="further decode batch sizes, comma separated ('' for none)")
    ap.add_argument("--temperature", type=float, default=0.0, help="sampling temperature of the end-to-end part (0: greedy, the headline)")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--page-size", type=int, default=None, help="KV page size (default: the configuration's 16)")
    ap.add_argument("--profile-ops", action="store_true",
                    help="instead of the benchmark line: where an eager decode step and a prefill step spend their time, launcher by "
                         "launcher (CUDA events around every launch; its own JSON line)")
    ap.add_argument("--kernel", default=None, choices=["attention_prefill"],
                    help="time one kernel alone at the configuration's head sizes instead of the model: attention_prefill runs "
                         "--prefill-tokens query tokens that end at position --context (one request, contiguous pages)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "lkarlslund/quench6k is a Rust workspace (Cargo.toml, no setup.py or "
                          "pyproject.toml): pip cannot install it offline, cargo/rustc are absent, and its kernels are sm_120a-only"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from quench6k_b200 import Engine, SamplingParams, ops
    from quench6k_b200.config import FlintConfig
    from quench6k_b200.engine import StepEntry

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    if args.kernel == "attention_prefill":
        return kernel_attention_prefill(args)
    torch.cuda.set_device(0)
    pk = peaks()
    shape = SHAPES[args.config]
    if args.workload == "stress":
        return workload_stress(args, shape)
    args.batch = args.batch or 8
    args.context = args.context or shape["context"]
    cfg_d = dict(CONFIG2)
    full_layers = shape["layers"]
    layers = args.layers or full_layers
    cfg_d["num_hidden_layers"] = layers
    if args.page_size:
        cfg_d["kv_page_size"] = args.page_size
    cfg = FlintConfig.from_dict(cfg_d)
    page = cfg.kv_page_size
    point_batches = [int(x) for x in args.points.split(",") if x.strip()]
    max_b = max([args.batch] + point_batches)
    ctx = args.context
    headroom = max(96, args.steps + args.warmup + 16)            # every timed request decodes that many tokens past its context
    pages_per_req = (ctx + headroom + page - 1) // page + 1
    num_pages = max(max_b * pages_per_req, (args.prefill_tokens + page - 1) // page + 1)
    t0 = time.time()
    eng = Engine.from_random(cfg, seed=0, dtype=args.dtype, page_size=page, num_pages=num_pages, max_requests=max_b,
                             max_batch_tokens=max(args.prefill_tokens, max_b))
    runner = eng.runner
    for c in runner.caches:                      # stand-in for the keys and values a prefill would have left
        c.k.normal_(0.0, 0.5)
        c.v.normal_(0.0, 0.5)
    torch.cuda.synchronize()
    print(f"[bench] model and cache ready in {time.time() - t0:.1f}s ({torch.cuda.memory_allocated() / 2**30:.1f} GiB on the device)",
          file=sys.stderr, flush=True)
    gen = torch.Generator().manual_seed(1)
    V = cfg.vocab_size

    def rand_ids(n):
        return torch.randint(0, V, (n,), generator=gen).tolist()

    def stand_at_context(rids):
        for r in rids:
            runner.add_request(r)
        chunk = args.prefill_tokens              # pages are taken as a chunked prefill would take them:
        for at in range(0, ctx, chunk):          # one portion of each request in turn
            for r in rids:
                runner.assume_cached(r, min(chunk, ctx - at))

    def graphs_equal_eager(B, n=64, prompt=4096):
        """The reference times nothing before it has checked it (crates/cli/src/flint.rs:116-131: 64 graph-decoded
        tokens must equal eager decoding): B prompts are prefilled in portions, then n greedy tokens are decoded by
        replaying CUDA graphs; the same again with eager launches; the ids must be equal.  (Real prompts, not the
        random cache contents of the timed part: those differ from page to page, and the two passes get other pages.)"""
        prompt = min(prompt, ctx)
        prompts = [rand_ids(prompt) for _ in range(B)]
        seqs = []
        for graphs in (True, False):
            rids = [f"g{B}_{i}" for i in range(B)]
            keep, runner.cuda_graphs = runner.cuda_graphs, runner.cuda_graphs and graphs
            cur = []
            for r, toks in zip(rids, prompts):
                runner.add_request(r)
                for at in range(0, prompt, args.prefill_tokens):
                    part = toks[at:at + args.prefill_tokens]
                    logits = runner.step([StepEntry(r, part, [len(part) - 1])])
                cur.append(int(ops.argmax(logits)[0]))
            ids = [cur]
            for _ in range(n):
                cur = ops.argmax(runner.step([StepEntry(r, [cur[j]], [0]) for j, r in enumerate(rids)])).tolist()
                ids.append(cur)
            runner.cuda_graphs = keep
            for r in rids:
                runner.end_request(r)
            seqs.append(ids)
        return seqs[0] == seqs[1], len({t for step in seqs[0] for t in step})

    def experts_read(one, first, B, n=2):
        """Distinct experts per routed layer that n further (eager) decode steps really chose, on average."""
        from quench6k_b200.parts.base import Tap
        tap = Tap(max(64, B))
        routed = [b.ffn for b in runner.model.blocks if hasattr(b.ffn, "routing_tap")]
        for f in routed:
            f.routing_tap = tap
        keep, runner.cuda_graphs = runner.cuda_graphs, False
        total, count = 0, 0
        for i in range(first, first + n):
            one(i)
            for (what, _), buf in tap.buffers.items():
                if what == "experts":
                    total += int(torch.unique(buf[:B]).numel())
                    count += 1
        runner.cuda_graphs = keep
        for f in routed:
            f.routing_tap = None
        return total / count if count else None

    def timed_decode(B, steps, warmup, sampler=None):
        """Device-timed decode steps of B requests standing at `ctx` cached tokens: (ms per step, launches, distinct
        experts per layer the router chose in two further steps)."""
        rids = [f"d{B}_{i}" for i in range(B)]
        stand_at_context(rids)
        toks = [rand_ids(steps + warmup + 2) for _ in rids]

        def one(i):
            logits = runner.step([StepEntry(r, [toks[j][i]], [0]) for j, r in enumerate(rids)])
            return ops.argmax(logits)

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        l0 = ops.launch_count
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler is not None:
            sampler.start()                      # the clocks are read while the timed steps run, and only then
        a.record()
        for i in range(warmup, warmup + steps):
            one(i)
        b.record()
        torch.cuda.synchronize()
        if sampler is not None:
            sampler.result = sampler.stop()
        ms = a.elapsed_time(b) / steps
        launches = ops.launch_count - l0
        chosen = experts_read(one, warmup + steps, B)
        for r in rids:
            runner.end_request(r)
        return ms, launches, chosen

    if args.profile_ops:
        return profile_ops(args, runner, cfg_d, layers, ctx, stand_at_context, rand_ids)
    checked, distinct = graphs_equal_eager(args.batch)
    if not checked:
        print("bench.py: decoding by CUDA-graph replay and by eager launches gave different tokens; nothing is timed", file=sys.stderr)
        return 1
    clocks = ClockSampler()
    ms, launches, chosen = timed_decode(args.batch, args.steps, args.warmup, clocks)
    clock_info = clocks.result
    value = args.batch * 1000.0 / ms
    total_b, w_b, kv_b = decode_bytes(cfg_d, layers, args.batch, ctx, chosen)
    achieved = total_b / (ms * 1e-3) / 1e9

    # prefill: one prompt of T tokens in one step, the logits of its last token wanted
    T = args.prefill_tokens
    pre_ms = []
    for it in range(3):
        runner.add_request("p")
        ids = rand_ids(T)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        runner.step([StepEntry("p", ids, [T - 1])])
        b.record()
        torch.cuda.synchronize()
        pre_ms.append(a.elapsed_time(b))
        runner.end_request("p")
    pms = min(pre_ms[1:])
    pf = prefill_flops(cfg_d, layers, T)
    pb = prefill_bytes(cfg_d, layers, T)
    prefill = {"value": round(T * 1000.0 / pms, 1), "tokens": T, "ms": round(pms, 3),
               "frac": round(pf / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               # a step of milliseconds runs under the power cap: the sustained product rate is its yardstick; and the step
               # cannot be shorter than its weights take to stream, nor than that plus its products one after the other
               "frac_sustained": round(pf / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
               "bytes_floor_ms": round(pb / pk["hbm_gbs"] / 1e6, 3),
               "flops_floor_ms": round(pf / pk["bf16_tflops_sustained"] / 1e9, 3)}

    # end to end: Engine.step() with host ids in and sampled ids out each step
    for i in range(args.batch):
        sp = SamplingParams(max_tokens=args.steps + args.warmup + 8, temperature=args.temperature, seed=1000 + i)
        eng.adopt_request(rand_ids(ctx), rand_ids(1)[0], sp)
    for _ in range(args.warmup):
        eng.step()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    for _ in range(args.steps):
        eng.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t1
    for r in list(eng.scheduler.running):
        eng.abort(r.rid)
    R = args.batch
    h2d = 4 * (3 * R + (R + 1) + 2 * R + R + R * ((ctx + 64 + page - 1) // page))       # the step's int32 block, tables included
    e2e = {"value": round(args.batch * args.steps / e2e_s, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": 4 * R}
    if args.temperature > 0:
        e2e["temperature"] = args.temperature
        e2e["h2d_bytes_per_step"] += 32 * R               # the rows' sampling records

    # further batch sizes last: their long steps at batch 64 warm the GPU up, which the headline numbers should not feel
    points, points_roofline, points_ms = {}, {}, {}
    for B in point_batches:
        bms, _, bchosen = timed_decode(B, args.steps, 3)
        points[f"decode_b{B}"] = round(B * 1000.0 / bms, 1)
        points_ms[f"decode_b{B}"] = round(bms, 3)
        points_roofline[f"decode_b{B}"] = round(decode_bytes(cfg_d, layers, B, ctx, bchosen)[0] / (bms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)

    out = {
        "metric": f"decode tok/s at batch {args.batch} (context {ctx}); prefill tok/s at {T} tokens; % of roofline",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype in ("bfloat16", "bf16") else "fp32",
        "data": "synthetic: seeded random weights N(0,0.02), uniform-random token ids, caches filled with random values",
        "config": {"model": shape["label"], "layers": layers, "layers_full": full_layers,
                   "hidden": cfg.hidden_size, "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "experts": cfg.n_routed_experts, "top_k": cfg.num_experts_per_tok,
                   "expert_width": cfg.moe_intermediate_size, "vocab": cfg.vocab_size, "rope_theta": cfg.rope_theta,
                   "page_size": page, "global_batch": args.batch, "seq_len": ctx, "prefill_tokens": T,
                   "parallelism": "single-gpu", "l2": "inputs larger than L2 (weights and cache stream from HBM every step)",
                   "kv_fill": "random values; pages taken in portions of prefill_tokens per request in turn", "peaks": pk["source"]},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes": int(total_b), "weight_bytes": int(w_b), "kv_bytes": int(kv_b),
                     "experts_read_per_layer": None if chosen is None else round(chosen, 1)},
        "points": points, "points_roofline": points_roofline, "points_ms": points_ms,
        "checked": {"graph_replay_equals_eager": True, "tokens": 64, "distinct_ids": distinct},
        "e2e": e2e, "gpu_launches": launches, "clocks": clock_info, "impl": "ours",
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
