"""Arithmetic of the random fills (csrc/pxe_backward.cu), restated in integers: the folding reduction modulo 2^31-1
and the jump from one of a thread's elements to the next reproduce thrust::default_random_engine (the minimal-standard
generator x <- 48271 x mod 2^31-1 from seed 1) advanced i + 1 steps for element i, as src/CudaUtils.cu:53-60 draws it."""
import random

M = 2147483647


def minstd_mul(a, b):
    p = a * b
    r = (p & M) + (p >> 31)
    r = (r & M) + (r >> 31)
    return r - M if r >= M else r


def minstd_after(steps):
    result, base = 1, 48271
    while steps:
        if steps & 1:
            result = minstd_mul(result, base)
        base = minstd_mul(base, base)
        steps >>= 1
    return result


def test_folding_is_the_remainder():
    rng = random.Random(5)
    for _ in range(200_000):
        a, b = rng.randrange(1, M), rng.randrange(1, M)
        assert minstd_mul(a, b) == a * b % M
    for a, b in ((M - 1, M - 1), (1, 1), (M - 1, 1), (48271, M - 1), (1 << 30, 1 << 30)):
        assert minstd_mul(a, b) == a * b % M


def test_jump_ahead_walks_the_engine_sequence():
    engine, seq = 1, []
    for _ in range(5000):
        engine = engine * 48271 % M
        seq.append(engine)                              # seq[i] = state after i + 1 steps = element i
    for stride, first in ((256, 0), (256, 255), (606208, 3), (7, 6), (1, 0)):
        state, jump = minstd_after(first + 1), minstd_after(stride)
        i = first
        while i < len(seq):
            assert state == seq[i]
            state = minstd_mul(state, jump)
            i += stride
    assert all(1 <= v <= M - 1 for v in seq)            # never 0: (x - 1) / 2^31 stays in [0, 1)
