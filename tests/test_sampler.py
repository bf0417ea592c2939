"""The host sampler: the reference's options, order and arithmetic (no GPU).
Modelled on mischief/lgml's test/test_sample.lua: greedy, determinism under a seed,
penalties, logit_bias, logprobs, the sets top-k / top-p / min-p keep, and a frequency fit."""
import math

import numpy as np
import pytest

from lgml_b200.sampling import DEFAULTS, Sampler, SamplingParams, Xoshiro256


def test_defaults_are_the_reference_defaults():
    p = SamplingParams()
    assert (p.temperature, p.top_k, p.top_p, p.min_p, p.repeat_penalty, p.repeat_last_n) == (0.8, 40, 0.95, 0.05, 1.0, 64)
    assert DEFAULTS["frequency_penalty"] == 0.0 and DEFAULTS["presence_penalty"] == 0.0
    assert not p.is_neutral and SamplingParams.neutral(0.8).is_neutral
    assert SamplingParams.preset("greedy").greedy
    with pytest.raises(ValueError):
        SamplingParams.preset("nope")
    with pytest.raises(ValueError):
        SamplingParams(repeat_penalty=0.0)


def _plain_xoshiro(seed, n):
    """xoshiro256** seeded by four splitmix64 outputs, restated from the published algorithms
    (``src/sample.c:93-139``): the first n outputs."""
    M = (1 << 64) - 1
    rotl = lambda x, k: ((x << k) | (x >> (64 - k))) & M
    s, z = [], seed & M
    for _ in range(4):
        z = (z + 0x9E3779B97F4A7C15) & M
        x = z
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & M
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & M
        s.append(x ^ (x >> 31))
    out = []
    for _ in range(n):
        out.append((rotl((s[1] * 5) & M, 7) * 9) & M)
        t = (s[1] << 17) & M
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = rotl(s[3], 45)
    return out


def test_generator_is_xoshiro256_starstar_seeded_by_splitmix64():
    # splitmix64(0) gives the well-known first outputs; xoshiro256** then runs on that state
    g = Xoshiro256(0)
    assert g.s == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F, 0xF88BB8A8724C81EC]
    # the first output for that state, worked by hand from the definition: rotl(s1 * 5, 7) * 9
    s1 = 0x6E789E6AA1B965F4
    x = (s1 * 5) & ((1 << 64) - 1)
    assert g.next() == ((((x << 7) | (x >> 57)) & ((1 << 64) - 1)) * 9) & ((1 << 64) - 1)
    for seed in (0, 42, 7, (1 << 64) - 1, 0x5EED):
        g = Xoshiro256(seed)
        want = _plain_xoshiro(seed, 20)
        assert [g.next() for _ in range(20)] == want, seed
    # a uniform double is the top 53 bits of the next output (src/sample.c:126-130)
    g, want = Xoshiro256(7), _plain_xoshiro(7, 3)
    assert [g.double() for _ in range(3)] == [(w >> 11) * 2.0 ** -53 for w in want]
    s = Sampler(SamplingParams(seed=7))
    assert s.uniform() == (want[0] >> 11) * 2.0 ** -53


def test_min_p_keeps_a_candidate_exactly_on_its_bound():
    """The bound is max + logf(p) in float32 (``src/sample.c:841``, ``:847``); a logit equal to
    it stays, the next float32 below it goes."""
    from lgml_b200.sampling import log_min_p

    for p in (0.05, 0.3, 0.123456, 1e-3):
        ln = np.float32(log_min_p(p))
        assert abs(float(ln) - math.log(np.float32(p))) <= 2e-7 * abs(math.log(p)) + 1e-7
        for top in (np.float32(0.0), np.float32(3.25), np.float32(-7.5)):
            on = np.float32(top + ln)
            below = np.nextafter(on, np.float32(-np.inf), dtype=np.float32)
            row = np.array([below, top, on, below], dtype=np.float32)
            s = Sampler(SamplingParams(temperature=1.0, seed=3, top_k=0, top_p=1.0, min_p=p))
            seen = {s.sample(row) for _ in range(300)}
            assert seen <= {1, 2} and 1 in seen, (p, top, seen)
            # on the bound means kept: with the top logit lowered out of the way of chance, index 2 shows
            flat = np.array([below, on - ln, on, below], dtype=np.float32)      # the two kept ones p apart
            s = Sampler(SamplingParams(temperature=100.0, seed=4, top_k=0, top_p=1.0, min_p=p))
            assert {s.sample(flat) for _ in range(300)} == {1, 2}, (p, top)


def test_greedy_and_ties():
    s = Sampler(SamplingParams(temperature=0.0))
    l = np.array([0.1, 3.0, -1.0, 3.0], dtype=np.float32)
    assert s.sample(l) == 1                              # lowest index wins a tie


def test_same_seed_same_draws():
    l = np.random.default_rng(0).normal(size=500).astype(np.float32)
    a = Sampler(SamplingParams(seed=5))
    b = Sampler(SamplingParams(seed=5))
    c = Sampler(SamplingParams(seed=6))
    da, db, dc = [a.sample(l) for _ in range(50)], [b.sample(l) for _ in range(50)], [c.sample(l) for _ in range(50)]
    assert da == db and da != dc


def test_top_k_top_p_min_p_keep_the_right_sets():
    l = np.log(np.array([0.5, 0.25, 0.125, 0.0625, 0.0625], dtype=np.float64)).astype(np.float32)
    def support(**kw):
        s = Sampler(SamplingParams(temperature=1.0, seed=1, **{**dict(top_k=0, top_p=1.0, min_p=0.0), **kw}))
        return {s.sample(l) for _ in range(400)}
    assert support(top_k=2) == {0, 1}
    assert support(top_p=0.7) == {0, 1}                   # 0.5 < 0.7 <= 0.75
    assert support(top_p=0.5) == {0}
    assert support(min_p=0.3) == {0, 1}                   # p >= 0.3 * 0.5
    assert support() == {0, 1, 2, 3, 4}


def test_penalties_and_bias():
    l = np.array([2.0, 1.9, -1.0, 0.0], dtype=np.float32)
    s = Sampler(SamplingParams(temperature=0.0, repeat_penalty=2.0))
    assert s.sample(l) == 0
    s.accept(0)
    assert s.sample(l) == 1                               # 2.0 / 2 < 1.9
    s = Sampler(SamplingParams(temperature=0.0, frequency_penalty=0.2, presence_penalty=0.0))
    s.accept(0); s.accept(0)
    assert s.sample(l) == 1                               # 2.0 - 2 * 0.2 < 1.9
    s = Sampler(SamplingParams(temperature=0.0, repeat_penalty=2.0))
    s.accept(2)
    s.sample(l)
    assert s.last_logits[2] == -2.0                       # a negative logit is multiplied
    s = Sampler(SamplingParams(temperature=0.0, logit_bias={3: 5.0}))
    assert s.sample(l) == 3
    s = Sampler(SamplingParams(temperature=0.0, repeat_penalty=2.0, repeat_last_n=1))
    s.accept(0); s.accept(1)                              # only the last id is remembered
    assert s.sample(l) == 0
    s.reset()
    assert s.hist == []


def test_logprobs():
    l = np.array([1.0, 2.0, 3.0], dtype=np.float32)
    s = Sampler(SamplingParams(temperature=0.0))
    with pytest.raises(RuntimeError):
        s.logprobs(0)
    s.sample(l)
    lp, top = s.logprobs(2, 2)
    lse = math.log(sum(math.exp(x) for x in (1.0, 2.0, 3.0)))
    assert abs(lp - (3.0 - lse)) < 1e-6 and [t[0] for t in top] == [2, 1]


def test_draw_frequencies_fit_the_softmax():
    """20 000 draws at temperature 0.8 stay within 4 sigma of softmax(l / 0.8) (test/test_sample.lua:182-185)."""
    l = np.array([0.0, 1.0, 2.0, 0.5, -1.0], dtype=np.float32)
    p = np.exp(l.astype(np.float64) / 0.8)
    p /= p.sum()
    s = Sampler(SamplingParams.neutral(0.8, seed=123))
    n = 20000
    counts = np.bincount([s.sample(l) for _ in range(n)], minlength=5)
    for i in range(5):
        sigma = math.sqrt(n * p[i] * (1 - p[i]))
        assert abs(counts[i] - n * p[i]) < 4 * sigma


def test_candidates_from_top_k_give_the_same_draws_as_the_whole_row():
    """The chain run on the top_k candidates (as the device hands them over: logit descending,
    id ascending) picks what the chain on the whole row picks, draw after draw."""
    import numpy as np
    from lgml_b200.sampling import Sampler, SamplingParams

    rng = np.random.default_rng(4)
    for kw in (dict(), dict(top_k=7, top_p=0.8, min_p=0.1, temperature=1.3), dict(top_k=50, top_p=1.0, min_p=0.0, temperature=0.5)):
        a, b = Sampler(SamplingParams(seed=9, **kw)), Sampler(SamplingParams(seed=9, **kw))
        assert a.p.top_k_on_device
        for _ in range(40):
            row = (rng.standard_normal(500) * 2).astype(np.float32)
            row[rng.integers(0, 500, 30)] = row[3]                       # ties
            k = a.p.top_k
            order = np.lexsort((np.arange(500), -row.astype(np.float64)))[:k]
            got = b.sample_candidates(order, row[order])
            want = a.sample(row)
            assert got == want
            a.accept(want), b.accept(got)
    assert not SamplingParams(temperature=0.0).top_k_on_device and not SamplingParams(top_k=0).top_k_on_device
    assert SamplingParams(repeat_penalty=1.1).top_k_on_device and SamplingParams(repeat_penalty=1.1).edits_logits
    assert SamplingParams(logit_bias={3: 1.0}).edits_logits and not SamplingParams().edits_logits
    s = Sampler(SamplingParams(seed=1, repeat_penalty=1.2, repeat_last_n=4, logit_bias={5: 0.5}))
    for t in (9, 3, 9, 9, 2):
        s.accept(t)
    bias, hist, pen = s.device_edits()
    assert bias == [(5, 0.5)] and sorted(hist) == [(2, 1), (3, 1), (9, 2)] and pen == (1.2, 0.0, 0.0)


def test_history_is_a_ring_of_the_last_ids():
    s = Sampler(SamplingParams(temperature=0.0, repeat_last_n=3))
    for t in (5, 6, 7, 8, 9):
        s.accept(t)
    assert s.hist == [7, 8, 9]
    s.reset()
    s.accept(1)
    assert s.hist == [1]
    with pytest.raises(ValueError):
        s.accept(-1)
    none = Sampler(SamplingParams(temperature=0.0, repeat_last_n=0))
    none.accept(3)
    assert none.hist == []


def test_top_k_of_a_large_row_is_in_the_sampler_order():
    """The k best, logit descending and id ascending among equals, whatever k and the row's size."""
    rng = np.random.default_rng(3)
    l = rng.integers(-5, 5, size=5000).astype(np.float32)          # many ties
    s = Sampler(SamplingParams(temperature=0.0))
    s.sample(l)
    for k in (1, 7, 40, 5000):
        _, top = s.logprobs(0, k)
        want = np.lexsort((np.arange(l.size), -l.astype(np.float64)))[:k]
        assert [t[0] for t in top] == want.tolist()
