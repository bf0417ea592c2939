"""Shared test material: the tiny configurations, model folders, traces and the oracle."""
from __future__ import annotations

import json
import random
from pathlib import Path
from typing import Dict, List, Tuple

import torch

from tests.plain import llama_plain as P

# Two tiny Llama configurations that differ in every size and option.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 4, "head_dim": 16,
    "intermediate_size": 176, "vocab_size": 256, "rope_theta": 10000.0, "rope_scaling": None, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "attention_bias": False, "mlp_bias": False, "max_position_embeddings": 128,
    "hidden_act": "silu",
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32,
    "intermediate_size": 256, "vocab_size": 320, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "attention_bias": True, "mlp_bias": False,
    "max_position_embeddings": 256, "hidden_act": "silu",
}
# A third one with sizes that are no power of two: odd head count, head_dim 48, mlp bias.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 120, "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48,
    "intermediate_size": 200, "vocab_size": 331, "rope_theta": 25000.0,
    "rope_scaling": {"rope_type": "linear", "factor": 2.0},
    "rms_norm_eps": 3e-6, "tie_word_embeddings": False, "attention_bias": False, "mlp_bias": True,
    "max_position_embeddings": 320, "hidden_act": "silu",
}
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2)}


def make_folder(tmp: Path, cfg: dict, seed: int, dtype: str = "float32", sharpen: float = 1.0) -> Path:
    """A model folder with random weights.  ``sharpen`` scales the q and k projections so
    that attention is far from uniform and a wrong key or a stale page shows in the logits."""
    from lgml_b200.config import config_from_dict
    from lgml_b200.weights import index_folder, read_tensor, write_random_model, write_safetensors

    folder = write_random_model(tmp, config_from_dict(cfg), seed, dtype=dtype)
    if sharpen != 1.0:
        idx = index_folder(folder)
        tensors = {}
        for name, ent in idx.items():
            t = read_tensor(ent)
            if ".q_proj.weight" in name or ".k_proj.weight" in name:
                t = (t.float() * sharpen).to(t.dtype)
            tensors[name] = t
        write_safetensors(folder / "model.safetensors", tensors)
    return folder


_oracle_cache: Dict[Tuple[str, Tuple[int, ...]], torch.Tensor] = {}


def oracle_logits(folder: Path, ids: List[int]) -> torch.Tensor:
    """float64 logits [n, V] of the whole sequence from the plain implementation."""
    key = (str(folder), tuple(ids))
    if key not in _oracle_cache:
        cfg, w = P.load_folder(folder)
        _oracle_cache[key] = P.forward(cfg, w, ids)
    return _oracle_cache[key]


def random_ids(n: int, vocab: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


# ----------------------------------------------------------------------------------------
# traces: lists of steps in trace_run's input format
# ----------------------------------------------------------------------------------------

def trace_whole(seqs: Dict[str, List[int]]) -> List[dict]:
    return [{"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]}
            for i, (rid, ids) in enumerate(seqs.items())]


def trace_tail(seqs: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of each request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, ids in seqs.items():
        head = max(len(ids) - tail, 1)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[:head], "want": list(range(head))}], "end": []})
        for p in range(head, len(ids)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [ids[p]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    return steps


def trace_portions(seqs: Dict[str, List[int]], sizes=(7, 2, 19, 3, 64, 2, 33, 5, 2, 70)) -> List[dict]:
    """Each request alone, in portions of changing size, down to two tokens."""
    steps = []
    k = 0
    for rid, ids in seqs.items():
        p = 0
        while p < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - p)
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[p:p + n], "want": list(range(n))}], "end": []})
            p += n
        steps[-1]["end"] = [rid]
    return steps


def trace_mixed(seqs: Dict[str, List[int]], max_tokens: int, seed: int = 0, max_live: int = 4, page: int = 64,
                choices=(1, 1, 1, 2, 2, 5, 17, 40, 64, 90), tail: int = 0, skip: float = 0.2, first: int = 0) -> List[dict]:
    """Up to ``max_live`` requests at once: portions of some beside single tokens of others,
    a request sometimes left out of a step, and a pool of ``max_tokens`` so small that the
    pages of finished requests are used again by later ones.  ``choices``: the portion sizes
    drawn from; the last ``tail`` tokens of a request come one by one; a request that has more
    than ``first`` tokens before its tail starts with a portion of ``first``."""
    rng = random.Random(seed)
    waiting = list(seqs.items())
    live: Dict[str, int] = {}      # id -> tokens fed
    steps = []

    def held(extra=None):
        n = sum(-(-len(seqs[r]) // page) * page for r in live)
        if extra is not None:
            n += -(-len(seqs[extra]) // page) * page
        return n

    while waiting or live:
        while waiting and len(live) < max_live and held(waiting[0][0]) <= max_tokens:
            live[waiting.pop(0)[0]] = 0
        assert live, "the pool cannot hold the next request at all"
        entries, end = [], []
        for rid in list(live):
            fed, ids = live[rid], seqs[rid]
            if len(live) > 1 and rng.random() < skip:
                continue                                            # left out of this step
            left = len(ids) - fed
            n = 1 if left <= tail else min(rng.choice(choices), left - tail)
            if first and fed == 0 and left - tail > first:
                n = first
            entries.append({"id": rid, "tokens": ids[fed:fed + n], "want": list(range(n))})
            live[rid] = fed + n
            if live[rid] == len(ids):
                end.append(rid)
        if not entries:
            continue
        steps.append({"step": len(steps), "entries": entries, "end": end})
        for rid in end:
            del live[rid]
    return steps


def run_trace(runner, steps: List[dict]) -> Dict[Tuple[str, int], torch.Tensor]:
    """Drive ``runner.step`` with a trace; (request, position) -> float32 logits row on the host."""
    live, fed = {}, {}
    out = {}
    for st in steps:
        entries = []
        for e in st["entries"]:
            if e["id"] not in live:
                live[e["id"]] = runner.open(e["id"])
                fed[e["id"]] = 0
            entries.append((live[e["id"]], e["tokens"], e["want"]))
        logits = runner.step(entries).float().cpu()
        runner.rt.check_status()
        r = 0
        for e in st["entries"]:
            for i in e["want"]:
                out[(e["id"], fed[e["id"]] + i)] = logits[r]
                r += 1
            fed[e["id"]] += len(e["tokens"])
        assert r == logits.shape[0]
        for rid in st["end"]:
            runner.close(live.pop(rid))
        runner.cache.check()
    return out


def compare_with_oracle(got: Dict[Tuple[str, int], torch.Tensor], folder: Path, seqs: Dict[str, List[int]], atol: float, rtol: float):
    """Largest error over all rows; raises naming the first wrong (request, position)."""
    worst = 0.0
    for rid, ids in seqs.items():
        ref = oracle_logits(folder, ids)
        for p in range(len(ids)):
            row = got[(rid, p)].double()
            err = (row - ref[p]).abs()
            bound = atol + rtol * ref[p].abs()
            if bool((err > bound).any()):
                j = int((err - bound).argmax())
                raise AssertionError(f"request {rid} position {p} (page {p // 64}, cell {p % 64}): logit {j} is {row[j]:.6g}, "
                                     f"oracle {ref[p, j]:.6g}, |diff| {err[j]:.3g} > {bound[j]:.3g}")
            worst = max(worst, float(err.max()))
    return worst
