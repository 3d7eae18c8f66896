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


def test_native_rows_match_the_python_twin():
    """The C++ choice over a block of rows against pick_from_pool row by row: greedy and sampled
    rows, penalties, rows that are skipped, ties, and the same advance of each row's random stream."""
    import numpy as np
    from quench6k_b200.sampling.sampler import pick_rows_native
    rng = random.Random(5)
    for case in range(60):
        rows, pool = rng.randint(1, 9), rng.choice([4, 64, 256])
        ids = np.zeros((rows, pool), dtype=np.int32)
        vals = np.zeros((rows, pool), dtype=np.float32)
        params, sizes, generated, seeds = [], [], [], []
        for r in range(rows):
            n = rng.randint(1, pool)
            cand = rng.sample(range(5000), n)
            ids[r, :n] = cand
            vals[r, :n] = [round(rng.gauss(0, 2), rng.choice([1, 5])) for _ in range(n)]
            params.append(SamplingParams(temperature=rng.choice([0.0, 0.3, 1.0, 2.5]), top_k=rng.choice([0, 1, 5, 40]),
                                         top_p=rng.choice([1.0, 0.9, 0.3]), min_p=rng.choice([0.0, 0.05, 0.1]),
                                         presence_penalty=rng.choice([0.0, 0.7]), repetition_penalty=rng.choice([1.0, 1.3])))
            sizes.append(0 if rng.random() < 0.15 else n)
            generated.append(rng.sample(cand, min(n, 3)) + [7777])
            seeds.append(rng.getrandbits(64))
        a, b = [SplitMix64(s) for s in seeds], [SplitMix64(s) for s in seeds]
        got = pick_rows_native(ids, vals, sizes, params, generated, a)
        for r in range(rows):
            if sizes[r] == 0:
                assert a[r].state == seeds[r]                     # a skipped row draws nothing
                continue
            want = pick_from_pool(ids[r, :sizes[r]], vals[r, :sizes[r]], params[r], generated[r], b[r])
            assert got[r] == want, (case, r, params[r])
            assert a[r].state == b[r].state


def test_device_rows_records():
    """The per-row records of the device sampler: pool sizes, options as 32-bit values, a uniform
    drawn exactly for the rows that sample, and no penalties."""
    import numpy as np
    import pytest
    from quench6k_b200.sampling.sampler import ROW_RECORD, device_rows
    assert ROW_RECORD.itemsize == 32
    params = [SamplingParams(temperature=0.0), SamplingParams(temperature=0.7, top_k=0, top_p=0.9, min_p=0.05),
              SamplingParams(temperature=1.0, top_k=1), SamplingParams(temperature=1.3, top_k=40)]
    rngs = [SplitMix64(s) for s in (1, 2, 3, 4)]
    rec = np.zeros(6, dtype=ROW_RECORD)
    k = device_rows(params, rngs, 1000, rec)
    assert k == 256 and rec["size"][:4].tolist() == [1, 256, 1, 40] and rec["top_k"][:4].tolist() == [20, 0, 1, 40]
    assert rec["u"][0] == 0.0 and rec["u"][2] == 0.0
    assert rec["u"][1] == P.splitmix64_uniform(2, 1) and rec["u"][3] == P.splitmix64_uniform(4, 1)
    assert [r.state for r in rngs[::2]] == [1, 3]                     # greedy rows draw nothing
    assert rec["temperature"][1] == np.float32(0.7) and rec["min_p"][1] == np.float32(0.05)
    assert device_rows(params[:1], rngs[:1], 100, rec) == 1
    with pytest.raises(ValueError):
        device_rows([SamplingParams(temperature=0.5, presence_penalty=0.1)], rngs[:1], 1000, rec)


def test_sampled_frequencies_follow_the_distribution():
    """1,500 draws from one request's stream at min_p 0.2 (the reference's own check of its sampler):
    candidates below a fifth of the best one's probability never come, the others as often as their
    renormalised probabilities say (each within four standard deviations)."""
    import math
    import numpy as np
    from quench6k_b200.sampling.sampler import pick_rows_native
    ids = list(range(100, 112))
    vals = [2.0, 1.7, 1.5, 1.1, 0.9, 0.4, 0.1, -0.5, -1.0, -2.0, -3.0, -6.0]
    p = SamplingParams(temperature=0.8, top_k=0, top_p=1.0, min_p=0.2)
    probs = [math.exp((v - vals[0]) / 0.8) for v in vals]
    probs = [q if q >= 0.2 else 0.0 for q in probs]
    total = sum(probs)
    n = 1500
    for native in (False, True):
        rng, counts = SplitMix64(2024), {i: 0 for i in ids}
        for _ in range(n):
            if native:
                tok = pick_rows_native(np.asarray([ids], dtype=np.int32), np.asarray([vals], dtype=np.float32), [len(ids)], [p], [[]], [rng])[0]
            else:
                tok = pick_from_pool(ids, vals, p, [], rng)
            counts[tok] += 1
        for i, q in zip(ids, probs):
            expect = n * q / total
            if q == 0.0:
                assert counts[i] == 0
            else:
                assert abs(counts[i] - expect) <= 4.0 * math.sqrt(expect * (1 - q / total)), (native, i, counts[i], expect)
