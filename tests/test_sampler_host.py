"""The host half of the sampler against the plain implementation's reading of the reference."""
import random

import plain_flint as P
from quench6k_b200.sampling import SamplingParams, SplitMix64, pick_from_pool, pool_size


def test_rng_matches_plain():
    r = SplitMix64(12345)
    for n in range(1, 6):
        assert r.uniform() == P.splitmix64_uniform(12345, n)


def test_pool_sizes_follow_the_reference():
    assert pool_size(SamplingParams(temperature=0.0), 1000) == 1
    assert pool_size(SamplingParams(temperature=1.0, top_k=1), 1000) == 1
    assert pool_size(SamplingParams(temperature=1.0, top_k=20), 1000) == 20
    assert pool_size(SamplingParams(temperature=1.0, top_k=0), 1000) == 256
    assert pool_size(SamplingParams(temperature=1.0, top_k=0), 100) == 100
    assert pool_size(SamplingParams(temperature=0.0, presence_penalty=0.5), 1000) == 64
    assert pool_size(SamplingParams(temperature=1.0, top_k=500), 1000) == 256


def test_pick_matches_plain_on_random_rows():
    rng = random.Random(0)
    for case in range(200):
        n = rng.choice([5, 40, 300])
        logits = [round(rng.gauss(0, 2), rng.choice([1, 4])) for _ in range(n)]     # coarse values make ties
        p = SamplingParams(temperature=rng.choice([0.0, 0.5, 1.0, 1.7]), top_k=rng.choice([0, 1, 3, 20]),
                           top_p=rng.choice([1.0, 0.95, 0.5]), min_p=rng.choice([0.0, 0.1]))
        seed = rng.getrandbits(64)
        k = min(pool_size(p, n), n)
        order = sorted(range(n), key=lambda i: (-logits[i], i))[:k]
        ids = list(order)
        rng.shuffle(ids)                                                            # the pool may come in any order
        got = pick_from_pool(ids, [logits[i] for i in ids], p, [], SplitMix64(seed))
        want = P.pick(logits, p.temperature, p.top_k, p.top_p, p.min_p, P.splitmix64_uniform(seed, 1))
        assert got == want, (case, p)


def test_penalties():
    ids, vals = [0, 1, 2], [2.0, 1.9, -1.0]
    p = SamplingParams(temperature=0.0, presence_penalty=0.5)
    assert pick_from_pool(ids, vals, p, [0], SplitMix64(0)) == 1          # 2.0 - 0.5 < 1.9
    p = SamplingParams(temperature=0.0, repetition_penalty=2.0)
    assert pick_from_pool(ids, vals, p, [0, 1], SplitMix64(0)) == 0       # 1.0 vs 0.95
    assert pick_from_pool([0, 2], [-0.4, -1.0], p, [0], SplitMix64(0)) == 0   # -0.8 still above -1.0
    assert pick_from_pool([0, 2], [-0.6, -1.0], p, [0], SplitMix64(0)) == 2   # -1.2 below -1.0
