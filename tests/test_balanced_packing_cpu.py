"""Solver-packed, attention-balanced microbatches of a data-parallel step (CPU)."""

import numpy as np
import pytest

from lorafusion_b200.train.data import LengthDistribution, pack_balanced_dp_step

DISTS = [LengthDistribution(256, 0.5, 32, 8192), LengthDistribution(512, 0.6, 32, 8192),
         LengthDistribution(1024, 0.7, 32, 8192), LengthDistribution(2048, 0.8, 32, 8192)]


def _pool(rng, tokens, start=()):
    pool, a = list(start), 0
    while sum(n for _, n in pool) < tokens:
        pool.append((a, int(DISTS[a].sample(1, int(rng.integers(1 << 31)))[0])))
        a = (a + 1) % 4
    return pool


@pytest.mark.parametrize("world", [1, 2, 8])
def test_every_rank_gets_full_microbatches_and_equal_attention_work(world):
    rng = np.random.default_rng(world)
    cap, per_rank, left = 16384, 2, []
    for _ in range(3):
        pool = _pool(rng, world * per_rank * cap * 1.08, left)
        dealt, left = pack_balanced_dp_step(pool, world, per_rank, cap)
        assert len(dealt) == world and all(len(d) == per_rank for d in dealt)
        used = [(a, n) for d in dealt for s in d for a, lens in s.segments for n in lens]
        assert sorted(used + left) == sorted(pool)                       # exact cover, nothing invented
        assert all(s.padded_total_tokens <= cap for d in dealt for s in d)
        toks = [sum(s.total_tokens for s in d) for d in dealt]
        assert min(toks) > 0.97 * per_rank * cap                        # nearly full
        sq = [sum(n * n for s in d for _, lens in s.segments for n in lens) for d in dealt]
        assert max(sq) <= 1.12 * (sum(sq) / world)                      # attention cost within 12 % of the mean


def test_too_small_a_pool_is_refused():
    with pytest.raises(ValueError):
        pack_balanced_dp_step([(0, 512)] * 8, 2, 2, 16384)
