"""The buckets of captured decode steps: what is captured ahead of the first
request covers every bucket that a step can ask for later."""
from velox_b200.engine.graphs import SPLIT_KEYS, all_buckets, batch_bucket, keys_bucket


def test_batch_buckets_pad_little_and_never_beyond_the_slots():
    for cap in (1, 4, 7, 8, 20, 64):
        for n in range(1, cap + 1):
            b = batch_bucket(n, False, cap)
            assert n <= b <= cap and b - n < 8
            assert b == n or b % 8 == 0 or b == cap
            assert batch_bucket(n, True, cap) == n      # a model with per-request state is never padded


def test_key_buckets_are_powers_of_two_of_the_piece():
    for kv in (1, 255, 256, 257, 1000, 4096, 4097):
        b = keys_bucket(kv)
        assert b >= kv and b % SPLIT_KEYS == 0 and (b // SPLIT_KEYS) & (b // SPLIT_KEYS - 1) == 0
        assert b == SPLIT_KEYS or b // 2 < kv


def test_the_buckets_captured_ahead_cover_every_step():
    for cap, max_batch, max_kv in ((64, 64, 4368), (4, 4, 256), (7, 100, 1000), (20, 13, 5000)):
        ahead = set(all_buckets(max_batch, cap, max_kv))
        for n in range(1, min(max_batch, cap) + 1):
            for kv in list(range(1, max_kv + 1, 37)) + [max_kv]:
                assert (batch_bucket(n, False, cap), keys_bucket(kv)) in ahead, (cap, max_batch, max_kv, n, kv)
        assert len(ahead) == len(all_buckets(max_batch, cap, max_kv))  # none twice
