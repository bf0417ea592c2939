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
the device with the uniform number this sampler supplies, and the host chain is its plain
twin.  The chain, the history and the generator are the host library's (C, as in mischief/lgml:
``csrc/host/lgml_host.c``); this module holds the options and the bindings.  With top_k set (the default chain) the device applies bias and penalties to
the rows, picks the k best in this chain's order, and ``sample_candidates`` finishes the chain
on those k pairs; a chain without top_k that sorts the whole row stays on the host.
"""
from __future__ import annotations

import ctypes
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

from .. import host

MASK64 = (1 << 64) - 1

DEFAULTS = dict(temperature=0.8, top_k=40, top_p=0.95, min_p=0.05, repeat_penalty=1.0,
                frequency_penalty=0.0, presence_penalty=0.0, repeat_last_n=64)

# lua/lgml/sampler.lua:14-20 (the qwen3 presets belong to other model families)
PRESETS = {"default": {}, "greedy": {"temperature": 0.0}}

#: the chain with every filter off: what tests and the device path use
NEUTRAL = dict(top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0, frequency_penalty=0.0, presence_penalty=0.0)


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


class Xoshiro256:
    """xoshiro256** seeded with splitmix64 (``src/sample.c:93-139``): the generator of the host
    library's sampler, on its own."""

    def __init__(self, seed: int):
        self._lib = host.lib()
        self._h = self._lib.lgml_sampler_new(ctypes.byref(_c_params(SamplingParams())), seed & MASK64)
        if not self._h:
            raise RuntimeError(host.last_error())

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.lgml_sampler_free(self._h)
            self._h = None

    def __reduce__(self):
        raise TypeError(f"a {type(self).__name__} holds state of the host library and cannot be copied or pickled")

    @property
    def s(self) -> List[int]:
        out = (ctypes.c_uint64 * 4)()
        self._lib.lgml_sampler_state(self._h, out)
        return list(out)

    def next(self) -> int:
        return int(self._lib.lgml_sampler_next_u64(self._h))

    def double(self) -> float:
        return float(self._lib.lgml_sampler_uniform(self._h))


def log_min_p(min_p: float) -> float:
    """ln(min_p) as the host chain computes it (float32 ``logf``, ``src/sample.c:841``): the
    device's copy of the chain gets its bound from here."""
    return float(host.lib().lgml_log_min_p(float(min_p)))


def _c_params(p: "SamplingParams") -> host.SamplerParams:
    return host.SamplerParams(p.temperature, p.top_k, p.top_p, p.min_p, p.repeat_penalty, p.frequency_penalty, p.presence_penalty,
                              p.repeat_last_n)


class Sampler:
    """One request's sampler: the host library's, with its history and generator."""

    def __init__(self, params: Optional[SamplingParams] = None, **over):
        p = params or SamplingParams(**over)
        self.p = p
        seed = p.seed if p.seed is not None else (time.time_ns() ^ id(self))
        self._lib = host.lib()
        self._h = self._lib.lgml_sampler_new(ctypes.byref(_c_params(p)), seed & MASK64)
        if not self._h:
            raise ValueError(host.last_error())
        if p.logit_bias:
            ids = np.asarray([int(t) for t in p.logit_bias], dtype=np.int32)
            bias = np.asarray([float(b) for b in p.logit_bias.values()], dtype=np.float32)
            if self._lib.lgml_sampler_set_bias(self._h, ids.ctypes.data, bias.ctypes.data, len(ids)):
                raise RuntimeError(host.last_error())
        self.last_logits: Optional[np.ndarray] = None

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.lgml_sampler_free(self._h)
            self._h = None

    def __reduce__(self):
        raise TypeError(f"a {type(self).__name__} holds state of the host library and cannot be copied or pickled")

    # ---- history (src/sample.c:603-650) -------------------------------------------------
    @property
    def hist(self) -> List[int]:
        """The last repeat_last_n accepted ids, oldest first."""
        n = self.p.repeat_last_n
        if n == 0:
            return []
        out = np.empty(n, dtype=np.int32)
        k = self._lib.lgml_sampler_history(self._h, out.ctypes.data, n)
        return out[:k].tolist()

    def accept(self, token: int) -> None:
        if token < 0 or self._lib.lgml_sampler_accept(self._h, int(token)):
            raise ValueError("bad token id")

    def reset(self) -> None:
        self._lib.lgml_sampler_reset(self._h)

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
        return float(self._lib.lgml_sampler_uniform(self._h))

    # ---- the chain -----------------------------------------------------------------------
    def sample(self, logits: Sequence[float]) -> int:
        """One id from a row of float32 logits (``sampler_sample``, ``src/sample.c:1045-1060``)."""
        l = np.ascontiguousarray(logits, dtype=np.float32)
        edited = np.empty_like(l)
        tok = self._lib.lgml_sampler_sample(self._h, l.ctypes.data, l.shape[0], edited.ctypes.data)
        if tok < 0:
            raise RuntimeError(host.last_error())
        self.last_logits = edited
        return int(tok)

    def sample_candidates(self, ids: Sequence[int], vals: Sequence[float]) -> int:
        """The chain from top_p on, for candidates that top_k has already chosen on the device
        (``ops.topk_rows``: the top_k best, logit descending, id ascending).  The same id as
        ``sample`` on the whole row when no bias and no penalty is set and temperature > 0."""
        if not self.p.temperature > 0.0:
            raise ValueError("sample_candidates is for temperature > 0 (the argmax needs no candidates)")
        i = np.ascontiguousarray(ids, dtype=np.int64)
        v = np.ascontiguousarray(vals, dtype=np.float32)
        self.last_logits = None
        tok = self._lib.lgml_sampler_sample_candidates(self._h, i.ctypes.data, v.ctypes.data, i.shape[0])
        if tok < 0:
            raise RuntimeError(host.last_error())
        return int(tok)

    def logprobs(self, token: int, k: int = 0):
        """Log-softmax of the last sampled row after bias and penalties, before temperature
        and truncation (``sampler_logprobs``, ``src/sample.c:1075-1110``)."""
        if self.last_logits is None:
            raise RuntimeError("no logits: sample first")
        n = self.last_logits.shape[0]
        if not 0 <= token < n or not 0 <= k <= n:
            raise ValueError("bad token id or count")
        lp = ctypes.c_double()
        ids = np.empty(max(k, 1), dtype=np.int32)
        lps = np.empty(max(k, 1), dtype=np.float64)
        if self._lib.lgml_sampler_logprobs(self._h, int(token), int(k), ctypes.byref(lp), ids.ctypes.data, lps.ctypes.data):
            raise RuntimeError(host.last_error())
        return float(lp.value), [(int(ids[i]), float(lps[i])) for i in range(k)]
