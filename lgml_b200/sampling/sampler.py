"""The sampler: one per request, with mischief/lgml's options, order and arithmetic.

Options and defaults are those of ``lgml.sampler`` (``src/sample.c:493-559``,
``lua/lgml/sampler.lua:14-28``): temperature 0.8, top_k 40, top_p 0.95, min_p 0.05,
repeat_penalty 1, frequency_penalty 0, presence_penalty 0, repeat_last_n 64,
logit_bias, seed.  The chain's order is bias -> penalties -> top_k -> top_p -> min_p
-> temperature -> draw (``src/sample.c:1050-1055``, ``chain`` ``:929-962``);
temperature <= 0 is the argmax with ties to the lowest index (``:937-940``,
``:913-926``).  The generator is xoshiro256** seeded by splitmix64 (``:93-139``) and a
draw uses one double ``(next() >> 11) * 2^-53`` (``:126-130``).

When the chain is *neutral* (no bias, no penalties, top_k 0, top_p 1, min_p 0) a draw
is exactly "softmax(logits / T), inverse CDF in id order"; the engine then samples on
the device with the uniform number this sampler supplies, and the host chain below is
its plain twin.  With top_k set (the default chain) the device applies bias and penalties to
the rows, picks the k best in this chain's order, and ``sample_candidates`` finishes the chain
on those k pairs; a chain without top_k that sorts the whole row stays on the host.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np

MASK64 = (1 << 64) - 1

DEFAULTS = dict(temperature=0.8, top_k=40, top_p=0.95, min_p=0.05, repeat_penalty=1.0,
                frequency_penalty=0.0, presence_penalty=0.0, repeat_last_n=64)

# lua/lgml/sampler.lua:14-20 (the qwen3 presets belong to other model families)
PRESETS = {"default": {}, "greedy": {"temperature": 0.0}}

#: the chain with every filter off: what tests and the device path use
NEUTRAL = dict(top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0, frequency_penalty=0.0, presence_penalty=0.0)


class Xoshiro256:
    """xoshiro256** seeded with splitmix64 (``src/sample.c:93-139``)."""

    def __init__(self, seed: int):
        x = seed & MASK64
        self.s = []
        for _ in range(4):
            x = (x + 0x9E3779B97F4A7C15) & MASK64
            z = x
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
            self.s.append(z ^ (z >> 31))

    @staticmethod
    def _rotl(x: int, k: int) -> int:
        return ((x << k) | (x >> (64 - k))) & MASK64

    def next(self) -> int:
        s = self.s
        r = (self._rotl((s[1] * 5) & MASK64, 7) * 9) & MASK64
        t = (s[1] << 17) & MASK64
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = self._rotl(s[3], 45)
        return r

    def double(self) -> float:
        return (self.next() >> 11) * 2.0 ** -53


@dataclass
class SamplingParams:
    temperature: float = DEFAULTS["temperature"]
    top_k: int = DEFAULTS["top_k"]
    top_p: float = DEFAULTS["top_p"]
    min_p: float = DEFAULTS["min_p"]
    repeat_penalty: float = DEFAULTS["repeat_penalty"]
    frequency_penalty: float = DEFAULTS["frequency_penalty"]
    presence_penalty: float = DEFAULTS["presence_penalty"]
    repeat_last_n: int = DEFAULTS["repeat_last_n"]
    logit_bias: Optional[Dict[int, float]] = None
    seed: Optional[int] = None

    def __post_init__(self):
        if self.repeat_last_n < 0:
            raise ValueError("repeat_last_n must be >= 0")
        if not self.repeat_penalty > 0:
            raise ValueError("repeat_penalty must be > 0")

    @classmethod
    def preset(cls, name: str = "default", **over) -> "SamplingParams":
        if name not in PRESETS:
            raise ValueError(f"unknown sampler preset '{name}'")
        return cls(**{**PRESETS[name], **over})

    @classmethod
    def neutral(cls, temperature: float = 0.8, seed: Optional[int] = None) -> "SamplingParams":
        return cls(temperature=temperature, seed=seed, **NEUTRAL)

    @property
    def greedy(self) -> bool:
        return not self.temperature > 0.0

    @property
    def on_device(self) -> bool:
        """The device kernels give this chain's result: nothing alters the logits before the
        draw, and either the draw is the argmax (temperature <= 0: the filters always keep the
        maximum, ``src/sample.c:937-940``) or every filter is off."""
        plain = (not self.logit_bias and self.repeat_penalty == 1.0 and self.frequency_penalty == 0.0
                 and self.presence_penalty == 0.0)
        return plain and (self.greedy or self.is_neutral)

    @property
    def top_k_on_device(self) -> bool:
        """Bias, penalties and top_k can run on the device and the rest of the chain on the k
        candidates: a draw follows, and k is within the kernel's reach."""
        return self.temperature > 0.0 and 0 < self.top_k <= 128

    @property
    def edits_logits(self) -> bool:
        """A bias or a penalty alters logits before top_k."""
        return bool(self.logit_bias) or self.repeat_penalty != 1.0 or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0

    @property
    def is_neutral(self) -> bool:
        """No step of the chain but temperature and the draw changes the logits."""
        return (not self.logit_bias and self.repeat_penalty == 1.0 and self.frequency_penalty == 0.0
                and self.presence_penalty == 0.0 and (self.top_k <= 0) and self.top_p >= 1.0 and self.min_p <= 0.0)


class Sampler:
    def __init__(self, params: Optional[SamplingParams] = None, **over):
        p = params or SamplingParams(**over)
        self.p = p
        seed = p.seed if p.seed is not None else (time.time_ns() ^ id(self))
        self.rng = Xoshiro256(seed)
        self.hist: List[int] = []          # ring of the last repeat_last_n ids, oldest first
        self.last_logits: Optional[np.ndarray] = None

    # ---- history (src/sample.c:603-650) -------------------------------------------------
    def accept(self, token: int) -> None:
        if token < 0:
            raise ValueError("bad token id")
        if self.p.repeat_last_n == 0:
            return
        self.hist.append(int(token))
        if len(self.hist) > self.p.repeat_last_n:
            self.hist.pop(0)

    def reset(self) -> None:
        self.hist.clear()

    def device_edits(self):
        """What the device needs to apply this sampler's bias and penalties to a row of logits:
        ([(id, bias)], [(id, count)] over the distinct ids of the history, (repeat, frequency,
        presence))."""
        p = self.p
        bias = [(int(t), float(b)) for t, b in (p.logit_bias or {}).items()]
        counts: Dict[int, int] = {}
        if p.repeat_penalty != 1.0 or p.frequency_penalty != 0.0 or p.presence_penalty != 0.0:
            for t in self.hist:
                counts[t] = counts.get(t, 0) + 1
        return bias, list(counts.items()), (float(p.repeat_penalty), float(p.frequency_penalty), float(p.presence_penalty))

    def uniform(self) -> float:
        """The next uniform double of this request's stream (for the device draw)."""
        return self.rng.double()

    # ---- the chain -----------------------------------------------------------------------
    def _penalties(self, l: np.ndarray) -> None:
        """Each distinct id of the history once (``apply_penalties``, ``src/sample.c:652-677``)."""
        p = self.p
        if not self.hist or (p.repeat_penalty == 1.0 and p.frequency_penalty == 0.0 and p.presence_penalty == 0.0):
            return
        counts: Dict[int, int] = {}
        for t in self.hist:
            if t < l.shape[0]:
                counts[t] = counts.get(t, 0) + 1
        rep = np.float32(p.repeat_penalty)
        for t, c in counts.items():
            v = l[t]
            v = v * rep if v <= 0 else v / rep
            l[t] = np.float32(v - np.float32(np.float32(c) * np.float32(p.frequency_penalty) + np.float32(p.presence_penalty)))

    def sample(self, logits: Sequence[float]) -> int:
        """One id from a row of float32 logits (``sampler_sample``, ``src/sample.c:1045-1060``)."""
        l = np.array(logits, dtype=np.float32, copy=True)
        p = self.p
        if p.logit_bias:
            for t, b in p.logit_bias.items():
                if 0 <= t < l.shape[0]:
                    l[t] += np.float32(b)
        self._penalties(l)
        self.last_logits = l
        n = l.shape[0]
        if not p.temperature > 0.0:
            return int(np.argmax(l))                      # first maximum: the lowest index wins a tie
        ids = np.arange(n, dtype=np.int64)
        vals = l
        is_sorted = False
        if 0 < p.top_k < n:
            order = np.lexsort((ids, -vals.astype(np.float64)))[: p.top_k]   # logit descending, then id ascending
            ids, vals, is_sorted = ids[order], vals[order], True
        return self._after_top_k(ids, vals, is_sorted)

    def sample_candidates(self, ids: Sequence[int], vals: Sequence[float]) -> int:
        """The chain from top_p on, for candidates that top_k has already chosen on the device
        (``ops.topk_rows``: the top_k best, logit descending, id ascending).  The same id as
        ``sample`` on the whole row when no bias and no penalty is set and temperature > 0."""
        if not self.p.temperature > 0.0:
            raise ValueError("sample_candidates is for temperature > 0 (the argmax needs no candidates)")
        self.last_logits = None
        return self._after_top_k(np.asarray(ids, dtype=np.int64), np.asarray(vals, dtype=np.float32), True)

    def _after_top_k(self, ids: np.ndarray, vals: np.ndarray, is_sorted: bool) -> int:
        p = self.p
        if p.top_p < 1.0:
            if not is_sorted:
                order = np.lexsort((ids, -vals.astype(np.float64)))
                ids, vals, is_sorted = ids[order], vals[order], True
            w = np.exp((vals - vals[0]).astype(np.float32)).astype(np.float32)
            # float32 running sums, as apply_top_p (:808-831); cumsum adds in order in the array's type
            total = np.cumsum(w, dtype=np.float32)[-1]
            cum = np.cumsum((w / total).astype(np.float32), dtype=np.float32)
            reached = np.flatnonzero(cum >= np.float32(p.top_p))
            keep = int(reached[0]) + 1 if reached.size else len(w)
            ids, vals = ids[:keep], vals[:keep]
        if p.min_p > 0.0:
            thr = np.float32(vals.max() + np.float32(math.log(p.min_p)))   # apply_min_p (:834-852)
            mask = vals >= thr
            ids, vals = ids[mask], vals[mask]
        if p.temperature != 1.0:
            vals = (vals / np.float32(p.temperature)).astype(np.float32)
        return self._draw(ids, vals)

    def _draw(self, ids: np.ndarray, vals: np.ndarray) -> int:
        """``draw`` (``src/sample.c:855-877``): float32 weights, float64 sums, first
        candidate whose running sum reaches sum * u; a zero weight never wins."""
        m = vals.max()
        w = np.exp((vals - m).astype(np.float32)).astype(np.float32).astype(np.float64)
        run = np.cumsum(w)                                  # sequential float64 sums
        tgt = run[-1] * self.rng.double()
        ok = (w > 0) & (run >= tgt)
        hit = np.flatnonzero(ok)
        if hit.size:
            return int(ids[hit[0]])
        nz = np.flatnonzero(w > 0)
        return int(ids[nz[-1]] if nz.size else ids[0])

    def logprobs(self, token: int, k: int = 0):
        """Log-softmax of the last sampled row after bias and penalties, before temperature
        and truncation (``sampler_logprobs``, ``src/sample.c:1075-1110``)."""
        l = self.last_logits
        if l is None:
            raise RuntimeError("no logits: sample first")
        if not 0 <= token < l.shape[0] or not 0 <= k <= l.shape[0]:
            raise ValueError("bad token id or count")
        m = float(l.max())
        lse = m + math.log(float(np.exp(l.astype(np.float64) - m).sum()))
        top = []
        if k > 0:
            order = np.lexsort((np.arange(l.shape[0]), -l.astype(np.float64)))[:k]
            top = [(int(i), float(l[i]) - lse) for i in order]
        return float(l[token]) - lse, top
