"""The step's launch plans that are made on the host: query tiles and their pairs."""
import random

import pytest
import torch

from quench6k_b200.engine.batch import StepContext


def make_ctx(q_lens, pos_starts=None):
    T, R = sum(q_lens), len(q_lens)
    z = torch.zeros(0, dtype=torch.int32)
    return StepContext(T=T, R=R, token_ids=torch.zeros(T, dtype=torch.int32), positions=z, req_of_token=z, q_start=z, pos_start=z,
                       slot_ids=z, block_tables=[], logit_rows=z, n_logit_rows=0, q_lens=list(q_lens), pos_starts=list(pos_starts or [0] * R),
                       slots=list(range(R)), max_context=max(q_lens), max_q_len=max(q_lens))


def request_of(row, q_lens):
    at = 0
    for r, n in enumerate(q_lens):
        if row < at + n:
            return r
        at += n
    raise AssertionError(row)


@pytest.mark.parametrize("seed", range(5))
@pytest.mark.parametrize("zigzag", [False, True])
def test_tile_pairs_cover_every_token_once(seed, zigzag):
    rng = random.Random(seed)
    q_lens = [rng.choice([1, 2, 15, 16, 17, 100, 333]) for _ in range(rng.randint(1, 6))]
    per = rng.choice([1, 5, 16, 128])
    ctx = make_ctx(q_lens)
    tok0, ntok, n = ctx.query_tile_pairs(per, zigzag)
    assert tuple(tok0.shape) == (n, 2) and tuple(ntok.shape) == (n, 2)
    seen = [0] * sum(q_lens)
    for (a0, b0), (an, bn) in zip(tok0.tolist(), ntok.tolist()):
        assert 1 <= an <= per and 0 <= bn <= per           # the first tile of a pair is never empty
        for t0, tn in ((a0, an), (b0, bn)):
            for row in range(t0, t0 + tn):
                seen[row] += 1
            if tn:                                          # a tile stays inside one request
                assert request_of(t0, q_lens) == request_of(t0 + tn - 1, q_lens)
        if bn:
            assert request_of(a0, q_lens) == request_of(b0, q_lens) and a0 > b0      # one request; the later tile first
            if not zigzag:
                assert b0 + bn == a0                        # neighbours
    assert seen == [1] * sum(q_lens)
    # the same tiles as the single-tile plan
    s0, sn, m = ctx.query_tiles(per)
    singles = sorted(zip(s0.tolist(), sn.tolist()))
    paired = sorted((t0, tn) for (a0, b0), (an, bn) in zip(tok0.tolist(), ntok.tolist()) for t0, tn in ((a0, an), (b0, bn)) if tn)
    assert singles == paired and m == len(singles)


def test_zigzag_pairs_the_last_tile_with_the_first():
    ctx = make_ctx([70])
    tok0, ntok, n = ctx.query_tile_pairs(16, True)          # tiles at 0, 16, 32, 48, 64 (6 tokens)
    assert tok0.tolist() == [[64, 0], [48, 16], [32, 32]] and ntok.tolist() == [[6, 16], [16, 16], [16, 0]] and n == 3


def test_short_requests_go_one_way_and_the_others_another():
    ctx = make_ctx([1, 40, 5, 1, 33], [100, 0, 7, 9, 64])
    assert ctx.short_requests(8) == (3, 0, 47, 5, 101)            # rows 0..46 span them; deepest position 100
    tok0, ntok, n = ctx.query_tiles(2, at_most=8)
    assert n == 5 and tok0.tolist() == [0, 41, 43, 45, 46] and ntok.tolist() == [1, 2, 2, 1, 1]
    p0, pn, pairs = ctx.query_tile_pairs(16, False, more_than=8)
    # request 4 (positions 64..96) sees the most keys: its pairs come first
    assert pairs == 4 and p0.tolist() == [[79, 79], [63, 47], [33, 33], [17, 1]] and pn.tolist() == [[1, 0], [16, 16], [8, 0], [16, 16]]
    covered = sorted(r for a, c in zip(tok0.tolist(), ntok.tolist()) for r in range(a, a + c)) + sorted(
        r for a2, c2 in zip(p0.tolist(), pn.tolist()) for a, c in zip(a2, c2) for r in range(a, a + c))
    assert sorted(covered) == list(range(80))                      # every row of the step exactly once
    none0, nonen, zero = ctx.query_tile_pairs(16, False, more_than=64)
    assert zero == 0 and tuple(none0.shape) == (0, 2)


def test_decode_batches_are_recorded_at_a_few_sizes():
    from quench6k_b200.engine.runner import ModelRunner
    b = ModelRunner.decode_bucket
    assert [b(n) for n in range(1, 10)] == [1, 2, 3, 4, 5, 6, 7, 8, 12]
    assert [b(n) for n in (12, 13, 31, 32, 33, 40, 64, 65, 80, 81, 200)] == [12, 16, 32, 32, 40, 40, 64, 80, 80, 96, 208]
    assert all(n <= b(n) < n + (1 if n <= 8 else 4 if n <= 32 else 8 if n <= 64 else 16) for n in range(1, 600))
