"""Configurations drawn at random over everything config.json allows (head sizes in steps of 16 up
to 256, any number of heads and groups, widths and vocabularies that are no power of two or
multiple of 8, expert counts down to the top-k itself, pages of odd sizes, windows shorter than a
page), each replayed in mixed batches in float32 and bfloat16 against the plain implementation:
a size the kernels do not take must be refused or handed to a kernel that does, never computed wrongly."""
import random

import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def draw(seed, head_dim=None):
    rng = random.Random(seed)
    kv = rng.choice([1, 2, 3, 5])
    group = rng.choice([1, 2, 3, 4, 7, 8, 16])
    layers = rng.choice([1, 2, 3])
    experts = rng.choice([2, 3, 5, 9, 33, 70])
    hd = head_dim or rng.choice([16, 32, 48, 64, 80, 112, 128, 144, 256])
    while kv * group * hd > 4096 and group > 1:      # no output projection over more than 4,096 inputs: float32 sums that long leave
        group = max(1, group // 2)                   # the tolerance through their length alone, which is not what this test is after
    cfg = {
        "architectures": ["FlintForCausalLM"],
        "hidden_size": rng.choice([24, 40, 72, 100, 136, 264, 520]), "num_hidden_layers": layers,
        "num_attention_heads": kv * group, "num_key_value_heads": kv, "head_dim": hd,
        "vocab_size": rng.choice([17, 100, 257, 1001]), "n_routed_experts": experts,
        "num_experts_per_tok": rng.randint(1, min(experts, 9)), "moe_intermediate_size": rng.choice([8, 24, 40, 100, 136]),
        "rms_norm_eps": rng.choice([1e-6, 1e-5, 3e-4]), "rope_theta": rng.choice([100.0, 10000.0, 1e6]),
        "tie_word_embeddings": rng.random() < 0.5, "scoring_func": rng.choice(["softmax", "sigmoid"]),
        "norm_topk_prob": rng.random() < 0.5, "qk_norm": rng.random() < 0.5, "attn_sinks": rng.random() < 0.5,
        "kv_page_size": rng.choice([1, 3, 4, 5, 8, 16, 24, 32, 64]),
    }
    if rng.random() < 0.6:
        cfg["sliding_window"] = rng.choice([1, 2, 7, 30, 64])
        cfg["sliding_window_pattern"] = [rng.random() < 0.6 for _ in range(layers)]
        cfg["rope_pattern"] = [rng.random() < 0.7 for _ in range(layers)]
    if rng.random() < 0.4:
        cfg["n_shared_experts"] = 1
        cfg["shared_expert_intermediate_size"] = rng.choice([8, 56, 120])
    if rng.random() < 0.3 and layers > 1:
        cfg["first_k_dense_replace"] = 1
        cfg["intermediate_size"] = rng.choice([16, 72])
    if rng.random() < 0.3:
        cfg["qk_norm_eps"] = 1e-4
    return cfg


# the last six with the head sizes the mma.sync attention kernel takes, whatever group size and page size come with them
@pytest.mark.parametrize("seed,head_dim", [(s, None) for s in range(10)] + [(10, 64), (11, 128), (12, 64), (13, 128), (14, 128), (15, 64)])
def test_random_configuration(tmp_path, seed, head_dim):
    cfg = draw(seed, head_dim)
    cfg_d, weights = helpers.make_model_folder(str(tmp_path), cfg, seed=seed)      # N(0, 0.02) matrices, as where the tolerances were set
    V, page = cfg["vocab_size"], cfg["kv_page_size"]
    rng = random.Random(100 + seed)
    reqs = {f"r{i}": helpers.random_tokens(rng.randint(3, 90), V, 7 * seed + i) for i in range(5)}
    steps, mt = helpers.schedule_mixed(reqs, page, seed=seed, max_live=3)
    for dtype in ("float32", "bfloat16"):
        outputs, runner = helpers.run_replay(str(tmp_path), dtype, steps, mt, tap=True)
        got = helpers.collect(reqs, steps, outputs)
        for rid, toks in reqs.items():
            helpers.assert_matches_plain(cfg_d, weights, toks, got[rid], dtype, f"configuration {seed} {dtype} {rid}: {cfg}",
                                         routing=runner.routing.get(rid))
    from quench6k_b200 import ops
    assert ops.tc_status() == 0
