"""Generation through the entry points: greedy and seeded temperature sampling equal the
plain implementation's; a pool too small for all requests (preemption) changes no reply;
bin/trace_run as a separate process; the command line."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests.plain import llama_plain as P

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {
        ("A", "float32"): H.make_folder(tmp_path_factory.mktemp("engA"), H.TINY_A, 0, dtype="float32", sharpen=12.0),
        ("B", "float32"): H.make_folder(tmp_path_factory.mktemp("engB"), H.TINY_B, 1, dtype="float32", sharpen=12.0),
        ("B", "bfloat16"): H.make_folder(tmp_path_factory.mktemp("engBh"), H.TINY_B, 1, dtype="bfloat16", sharpen=6.0),
    }


def test_greedy_generation_equals_the_plain_implementation(folders):
    """tiny-A: prompts of 5 / 17 / 31 tokens, 16 greedy tokens each, in one call."""
    import lgml_b200

    folder = folders[("A", "float32")]
    cfg, w = P.load_folder(folder)
    prompts = [H.random_ids(n, 256, 40 + n) for n in (5, 17, 31)]
    eng = lgml_b200.Engine(str(folder), dtype="float32", slots=4)
    got = eng.generate(prompts, max_tokens=16, temperature=0.0)
    for p, g in zip(prompts, got):
        assert g == P.greedy(cfg, w, p, 16)
    # Engine.greedy, the counterpart of generate.greedy, with a stop id
    ids, t = eng.greedy(prompts[1], 16)
    assert ids == got[1] and t["n_decode"] == 15 and t["prefill"] > 0
    stop_at = got[1][4]
    ids, _ = eng.greedy(prompts[1], 16, stop=[stop_at])
    assert ids == got[1][: got[1].index(stop_at) + 1]
    assert not eng.runner.cache.live and eng.runner.cache.n_free_pages == eng.runner.cache.n_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_weights_by_seed_are_the_written_folder(dtype, tmp_path):
    """``Engine(config=C, random_weights=s)`` fills its weights on the device; ``write_random_model(dir, C, s)``
    draws them on the host.  One generator: the same tensors bit for bit, so the same replies."""
    import lgml_b200
    from lgml_b200.config import config_from_dict
    from lgml_b200.weights import write_random_model

    cfg = config_from_dict(H.TINY_B)
    folder = write_random_model(tmp_path / "m", cfg, 5, dtype=dtype)
    by_seed = lgml_b200.Engine(config=cfg, random_weights=5, dtype=dtype, n_ctx=256)
    by_folder = lgml_b200.Engine(str(folder), dtype=dtype, n_ctx=256)
    a, b = by_seed.runner.model, by_folder.runner.model
    for x, y in ((a.embedding.table, b.embedding.table), (a.blocks[2].mixer.wqkv, b.blocks[2].mixer.wqkv), (a.blocks[0].mixer.bqkv, b.blocks[0].mixer.bqkv),
                 (a.blocks[1].ffn.wgu, b.blocks[1].ffn.wgu), (a.final_norm.weight, b.final_norm.weight), (a.head.weight, b.head.weight)):
        assert x.dtype == y.dtype and torch.equal(x, y)
    prompts = [H.random_ids(n, 320, 700 + n) for n in (3, 50)]
    assert by_seed.generate(prompts, max_tokens=12, temperature=0.0) == by_folder.generate(prompts, max_tokens=12, temperature=0.0)


def plain_sampled(cfg, w, prompt, n_new, temperature, seed):
    """Seeded sampling replayed on the plain implementation's logits with the host sampler."""
    from lgml_b200.sampling import Sampler, SamplingParams

    s = Sampler(SamplingParams.neutral(temperature, seed=seed))
    ids, out = list(prompt), []
    for _ in range(n_new):
        logits = P.forward(cfg, w, ids)[-1].float().numpy()
        t = s.sample(logits)
        s.accept(t)
        out.append(t)
        ids.append(t)
    return out


def test_seeded_sampling_with_chunked_prefill_mixed_with_decodes(folders):
    """tiny-B: prompts of 1 / 40 / 77 / 130 tokens, portions of 32 beside decoded tokens,
    24 samples each at temperature 0.8 from per-request seeded streams."""
    import lgml_b200
    from lgml_b200.sampling import NEUTRAL

    folder = folders[("B", "float32")]
    cfg, w = P.load_folder(folder)
    prompts = [H.random_ids(n, 320, 60 + n) for n in (1, 40, 77, 130)]
    eng = lgml_b200.Engine(str(folder), dtype="float32", slots=4, ubatch=32, max_batch_tokens=64, kv_tokens=64 * 12)
    got = eng.generate(prompts, max_tokens=24, temperature=0.8, seed=11, **NEUTRAL)
    assert any(t["decode"] > 0 and not t["pure_decode"] for t in eng.turn_log)       # a decoded token beside a prompt portion
    for i, (p, g) in enumerate(zip(prompts, got)):
        assert g == plain_sampled(cfg, w, p, 24, 0.8, 11 + i), i


def test_preemption_keeps_every_reply_whole(folders):
    """A pool that cannot hold all requests as they grow: requests are preempted and
    prefilled again, and every reply equals the reply with room to spare."""
    import lgml_b200

    folder = folders[("B", "float32")]
    prompts = [H.random_ids(n, 320, 80 + n) for n in (60, 50, 40, 30)]
    roomy = lgml_b200.Engine(str(folder), dtype="float32", slots=4, kv_tokens=64 * 16)
    want = roomy.generate(prompts, max_tokens=90, temperature=0.0)
    tight = lgml_b200.Engine(str(folder), dtype="float32", slots=4, kv_tokens=64 * 5)
    reqs = tight.generate(prompts, max_tokens=90, temperature=0.0, return_details=True)
    assert tight.scheduler.stats["preemptions"] >= 1
    assert [r.generated for r in reqs] == want
    assert all(r.finish_reason == "length" for r in reqs)
    tight.runner.cache.check()
    assert tight.runner.cache.n_free_pages == 5


def test_preemption_keeps_seeded_draws_whole(folders):
    """The same with temperature sampling: a preempted request keeps its sampler (history and
    generator), so the reply it goes on with is the one it would have drawn with room to spare; and
    against the plain implementation's logits through the host sampler."""
    import lgml_b200
    from lgml_b200.sampling import NEUTRAL

    folder = folders[("B", "float32")]
    cfg, w = P.load_folder(folder)
    prompts = [H.random_ids(n, 320, 180 + n) for n in (60, 50, 40)]
    roomy = lgml_b200.Engine(str(folder), dtype="float32", slots=3, kv_tokens=64 * 12)
    want = roomy.generate(prompts, max_tokens=80, temperature=0.9, seed=31, **NEUTRAL)
    tight = lgml_b200.Engine(str(folder), dtype="float32", slots=3, kv_tokens=64 * 4)
    reqs = tight.generate(prompts, max_tokens=80, temperature=0.9, seed=31, return_details=True, **NEUTRAL)
    assert tight.scheduler.stats["preemptions"] >= 1
    assert [r.generated for r in reqs] == want
    assert want[2][:20] == plain_sampled(cfg, w, prompts[2], 20, 0.9, 33)
    tight.runner.cache.check()
    assert tight.runner.cache.n_free_pages == 4


def test_prefix_cache_changes_no_reply(folders):
    """With the prefix cache on, prompts that begin like earlier ones take up the pages that hold
    those tokens and compute only the rest: the replies equal those of an engine without it, in
    32-bit token for token; a pool too small for everything (preemption, cached pages taken
    away again) included."""
    import lgml_b200

    folder = folders[("B", "float32")]
    common = H.random_ids(150, 320, 901)
    prompts = [common + H.random_ids(n, 320, 910 + n) for n in (1, 20, 70)] + [common[:130], H.random_ids(90, 320, 950)]
    plain = lgml_b200.Engine(str(folder), dtype="float32", slots=2, kv_tokens=64 * 16)
    want = plain.generate(prompts, max_tokens=40, temperature=0.0)
    for kv_pages in (16, 7):
        eng = lgml_b200.Engine(str(folder), dtype="float32", slots=2, kv_tokens=64 * kv_pages, prefix_cache=True)
        got = eng.generate(prompts, max_tokens=40, temperature=0.0)
        assert got == want, kv_pages
        again = eng.generate(prompts[:2], max_tokens=40, temperature=0.0)      # everything of these is cached by now
        assert again == want[:2]
        assert eng.scheduler.stats["prefix_tokens"] >= 128 * 3
        eng.runner.cache.check()
        assert not eng.runner.cache.live and eng.runner.cache.n_free_pages == kv_pages
    # bfloat16: the same replies as the same engine without the cache computes for each prompt alone
    folder = folders[("B", "bfloat16")]
    eng = lgml_b200.Engine(str(folder), dtype="bfloat16", slots=1, kv_tokens=64 * 16, prefix_cache=True)
    base = lgml_b200.Engine(str(folder), dtype="bfloat16", slots=1, kv_tokens=64 * 16)
    for p in prompts[:3]:
        assert eng.generate([p], max_tokens=8, temperature=0.0) == base.generate([p], max_tokens=8, temperature=0.0)
    assert eng.scheduler.stats["prefix_tokens"] >= 128 * 2


def test_replies_do_not_depend_on_the_schedule(folders):
    """Seeded random workloads (prompts that share beginnings, a sampler of its own per prompt,
    end tokens, reply limits) through engines that differ in slots, pool size, portion size, token
    budget, prefix cache and launching ahead: in 32-bit every reply and every reason equals
    those of one roomy engine that takes the prompts one at a time and waits for every step."""
    import random

    import lgml_b200

    folder = folders[("B", "float32")]
    V, maxpos = 320, 256
    roomy = lgml_b200.Engine(str(folder), dtype="float32", slots=1, kv_tokens=64 * 8, run_ahead=False)
    preemptions = from_cache = 0
    for trial in range(8):
        rng = random.Random(trial)
        common = H.random_ids(rng.choice([64, 70, 128]), V, 5 + trial)
        prompts = []
        for i in range(rng.randint(3, 7)):
            own = H.random_ids(rng.choice([1, 2, 30, 63, 64, 65, rng.randint(1, 120)]), V, 1000 * trial + i)
            prompts.append((common[:rng.choice([len(common), 64, 10])] + own) if rng.random() < 0.6 else own)
        per = []
        for _ in prompts:
            o = {"temperature": 0.0}
            if rng.random() < 0.7:
                o = {"temperature": rng.choice([0.5, 0.9, 1.3])}
                if rng.random() < 0.5:
                    o["top_k"] = rng.choice([1, 5, 40])
                if rng.random() < 0.5:
                    o["top_p"] = rng.choice([0.5, 0.9])
                if rng.random() < 0.3:
                    o["repeat_penalty"] = 1.2
            per.append(o)
        stop = [rng.randrange(V) for _ in range(rng.choice([0, 3, 20]))]
        limit = rng.choice([5, 40, 60])
        common_kw = dict(max_tokens=limit, stop=stop, seed=trial, per_prompt=per, return_details=True)
        want = [(r.generated, r.finish_reason) for r in roomy.generate(prompts, **common_kw)]
        for _ in range(2):
            pages = -(-(max(len(p) for p in prompts) + limit) // 64) + rng.choice([0, 0, 1, 4])
            ubatch = rng.choice([2, 7, 64, 512])
            eng = lgml_b200.Engine(str(folder), dtype="float32", slots=rng.randint(1, 6), kv_tokens=64 * pages, ubatch=ubatch,
                                   max_batch_tokens=max(ubatch, rng.choice([8, 64, 2048])), prefix_cache=rng.random() < 0.5,
                                   run_ahead=rng.random() < 0.7)
            got = [(r.generated, r.finish_reason) for r in eng.generate(prompts, **common_kw)]
            assert got == want, (trial, pages, ubatch)
            eng.runner.cache.check()
            assert not eng.runner.cache.live and eng.runner.cache.n_free_pages == pages
            preemptions += eng.scheduler.stats["preemptions"]
            from_cache += eng.scheduler.stats.get("prefix_tokens", 0)
    assert preemptions > 0 and from_cache > 0          # the hard paths were on the way


@pytest.mark.parametrize("n_requests", [100, 150])
def test_a_hundred_requests_at_once(folders, n_requests):
    """Decode steps of 100 and 150 tokens (the products on pairs of CTAs: the y^T tile up to 128
    tokens, tokens as rows beyond; captured steps of the next larger size on the ladder with their
    spare rows): in 32-bit every reply equals the reply of the same prompt alone."""
    import lgml_b200

    folder = folders[("B", "float32")]
    prompts = [H.random_ids(5 + (i * 7) % 40, 320, 100 + i) for i in range(n_requests)]
    alone = lgml_b200.Engine(str(folder), dtype="float32", slots=1, kv_tokens=64 * 4, run_ahead=False)
    want = alone.generate(prompts, max_tokens=10, temperature=0.0, stop=[])
    many = lgml_b200.Engine(str(folder), dtype="float32", slots=n_requests, kv_tokens=64 * (n_requests + 8), max_batch_tokens=4096)
    got = many.generate(prompts, max_tokens=10, temperature=0.0, stop=[])
    assert got == want
    assert max(t["decode"] for t in many.turn_log) == n_requests and many.runner.graph_replays > 0
    many.runner.cache.check()
    assert not many.runner.cache.live


@pytest.mark.parametrize("key", [("B", "float32"), ("B", "bfloat16")])
def test_launching_ahead_of_the_host_changes_no_reply(folders, key):
    """Decode steps launched before the host has seen the ids of the step before: replies,
    end tokens and reasons equal those of an engine that waits for every step; six requests
    on three slots, end tokens that strike in mid-flight, greedy and seeded draws."""
    import lgml_b200

    folder = folders[key]
    prompts = [H.random_ids(n, 320, 300 + n) for n in (9, 33, 70, 21, 64, 5)]
    for opts in (dict(temperature=0.0), dict(temperature=0.9, seed=5)):
        waits = lgml_b200.Engine(str(folder), dtype=key[1], slots=3, kv_tokens=64 * 9, run_ahead=False)
        base = waits.generate(prompts, max_tokens=48, **opts)
        # end tokens: ids that some replies produce part-way
        stop = [base[0][10], base[2][30], base[4][3]]
        want = waits.generate(prompts, max_tokens=48, stop=stop, return_details=True, **opts)
        ahead = lgml_b200.Engine(str(folder), dtype=key[1], slots=3, kv_tokens=64 * 9)
        got = ahead.generate(prompts, max_tokens=48, stop=stop, return_details=True, **opts)
        if key[1] == "float32":
            # 32-bit results do not depend on what else is in the batch: the replies are equal
            assert [r.generated for r in got] == [r.generated for r in want]
            assert [r.finish_reason for r in got] == [r.finish_reason for r in want]
            assert any(r.finish_reason == "stop" for r in got)
        for r in got:
            # in bfloat16 a batch of another size may round a near tie the other way, so
            # only what must hold of any reply: it ends at its first end token, or at the limit
            hits = [i for i, t in enumerate(r.generated) if t in stop]
            if hits:
                assert r.finish_reason == "stop" and hits[0] == len(r.generated) - 1
            else:
                assert r.finish_reason == "length" and len(r.generated) == 48
        ahead.runner.cache.check()
        assert not ahead.runner.cache.live and ahead.runner.cache.n_free_pages == 9
        assert sum(t["decode"] for t in ahead.turn_log) == sum(len(r.generated) - 1 for r in got)


def test_full_sampler_chain_is_reproducible_and_stops(folders):
    import lgml_b200

    folder = folders[("B", "bfloat16")]
    eng = lgml_b200.Engine(str(folder), dtype="bfloat16", slots=2)
    prompts = [H.random_ids(20, 320, 1), H.random_ids(9, 320, 2)]
    a = eng.generate(prompts, max_tokens=12, seed=3, temperature=0.9, top_k=20, top_p=0.9, min_p=0.02, repeat_penalty=1.1)
    b = eng.generate(prompts, max_tokens=12, seed=3, temperature=0.9, top_k=20, top_p=0.9, min_p=0.02, repeat_penalty=1.1)
    assert a == b and all(len(x) == 12 and all(0 <= t < 320 for t in x) for x in a)
    stop = a[0][3]
    c = eng.generate(prompts[:1], max_tokens=12, seed=3, stop=[stop], temperature=0.9, top_k=20, top_p=0.9, min_p=0.02, repeat_penalty=1.1)
    assert c[0] == a[0][: a[0].index(stop) + 1]


def test_chains_with_top_k_run_on_the_device(folders, monkeypatch):
    """The reference's default chain (top_k 40, top_p 0.95, min_p 0.05, temperature 0.8), and a
    chain with a logit bias and all three history penalties.  The first runs on the device to
    the chosen id (top_k, then the rest on its candidates), also beside a greedy request; for the
    second, bias, penalties and top_k run on the device and the host finishes on k candidates
    per row.  The replies equal those of the chain run on whole rows of logits on the host."""
    import lgml_b200
    from lgml_b200 import ops
    from lgml_b200.sampling import SamplingParams

    folder = folders[("B", "float32")]
    prompts = [H.random_ids(n, 320, 500 + n) for n in (12, 31, 70)]
    eng = lgml_b200.Engine(str(folder), dtype="float32", slots=3)
    chains = [dict(), dict(top_k=25, temperature=1.1, repeat_penalty=1.3, frequency_penalty=0.2, presence_penalty=0.1, repeat_last_n=16,
                           logit_bias={7: 2.5, 300: -4.0, 11: 0.75})]
    for opts in chains:
        calls = []
        real_topk, real_edits, real_rest = ops.topk_rows, ops.sampler_edits, ops.sample_candidates
        monkeypatch.setattr(ops, "topk_rows", lambda *a, **k: (calls.append("topk"), real_topk(*a, **k))[1])
        monkeypatch.setattr(ops, "sampler_edits", lambda *a, **k: (calls.append("edits"), real_edits(*a, **k))[1])
        monkeypatch.setattr(ops, "sample_candidates", lambda *a, **k: (calls.append("rest"), real_rest(*a, **k))[1])
        got = eng.generate(prompts, max_tokens=24, seed=21, **opts)
        assert "topk" in calls and (("edits" in calls) == bool(opts)) and (("rest" in calls) == (not opts)), calls
        # the same chain on whole rows on the host
        with monkeypatch.context() as m:
            m.setattr(SamplingParams, "top_k_on_device", property(lambda self: False))
            want = eng.generate(prompts, max_tokens=24, seed=21, **opts)
        assert got == want and all(len(x) == 24 for x in got)
        monkeypatch.undo()
    # a greedy request beside two with the default chain: one batch, all chosen on the device
    own = [{}, dict(temperature=0.0), {}]
    calls = []
    real_rest = ops.sample_candidates
    monkeypatch.setattr(ops, "sample_candidates", lambda *a, **k: (calls.append("rest"), real_rest(*a, **k))[1])
    got = eng.generate(prompts, max_tokens=12, seed=5, per_prompt=own)
    assert calls
    monkeypatch.undo()
    alone = [eng.generate([p], max_tokens=12, seed=5 + i, **own[i])[0] for i, p in enumerate(prompts)]
    assert got == alone


def replay_in_a_process(folder, dtype, seqs, vocab, tmp_path, extra_env=None, pool_pages=7):
    """bin/trace_run in a separate process on a mixed trace with page reuse: (request, position) -> logits row."""
    steps = H.trace_mixed(seqs, max_tokens=64 * pool_pages, seed=5)
    out = tmp_path / "out"
    env = dict(os.environ, PYTHONPATH=str(ROOT), **(extra_env or {}))
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
                           "--max-tokens", str(64 * pool_pages)], input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                          capture_output=True, env=env, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    fed = {k: 0 for k in seqs}
    got = {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        rows = np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(n_want, vocab)
        r = 0
        for e in st["entries"]:
            for i in e["want"]:
                got[(e["id"], fed[e["id"]] + i)] = torch.from_numpy(rows[r].copy())
                r += 1
            fed[e["id"]] += len(e["tokens"])
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_as_a_process(folders, dtype, tmp_path):
    """bin/trace_run in a separate process: a mixed trace with page reuse, logits files and
    'done' lines, compared with the plain implementation."""
    folder = folders[("B", dtype)]
    seqs = {f"r{i}": H.random_ids(n, 320, 300 + i) for i, n in enumerate([25, 101, 154, 64, 130])}
    got = replay_in_a_process(folder, dtype, seqs, 320, tmp_path)
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == "float32" else dict(atol=1.5e-2, rtol=1.5e-2)
    H.compare_with_oracle(got, folder, seqs, **tol)


@pytest.mark.parametrize("switch", ["LGML_PDL=0", "LGML_ATTN_EARLY=0", "LGML_PREFILL_ATTENTION=single", "LGML_PREFILL_ATTENTION=mma",
                                    "LGML_ATTN_TMA=0", "LGML_GEMM_PAIR=0", "LGML_NORM_GROUPED=0", "LGML_L2_AHEAD=0"])
def test_every_switch_still_gives_the_plain_implementations_logits(switch, tmp_path):
    """Each environment switch selects the older of two implementations of one thing (read once
    per process, so a process each): the same mixed trace in bfloat16 on a tiny model with head
    size 64 (the two-tile prompt attention's size), against the plain implementation."""
    cfg = dict(H.TINY_B, head_dim=64, num_attention_heads=4, num_key_value_heads=2, hidden_size=128, intermediate_size=320,
               max_position_embeddings=256)
    folder = H.make_folder(tmp_path / "model", cfg, 3, dtype="bfloat16", sharpen=4.0)
    seqs = {f"r{i}": H.random_ids(n, 320, 700 + i) for i, n in enumerate([25, 101, 200, 64, 130])}
    name, value = switch.split("=")
    got = replay_in_a_process(folder, "bfloat16", seqs, 320, tmp_path, {name: value})
    H.compare_with_oracle(got, folder, seqs, atol=1.5e-2, rtol=1.5e-2)


def test_command_line(folders):
    folder = folders[("A", "float32")]
    cfg, w = P.load_folder(folder)
    prompt = H.random_ids(9, 256, 5)
    proc = subprocess.run([sys.executable, "-m", "lgml_b200", "-m", str(folder), "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
                           "-n", "6", "--temperature", "0", "-c", "128", "-np", "2", "-ub", "4"], cwd=ROOT, text=True, capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [int(t) for t in proc.stdout.strip().splitlines()[-1].split(",")] == P.greedy(cfg, w, prompt, 6)


def test_kernel_times_and_turn_csv(folders, tmp_path):
    """Events around every launcher give device time by kernel class (steps then run eagerly, a replayed
    graph would hide its kernels); the command line writes them and one line per turn."""
    import lgml_b200
    from lgml_b200 import ops

    folder = folders[("B", "bfloat16")]
    eng = lgml_b200.Engine(str(folder), dtype="bfloat16", slots=2)
    prompts = [H.random_ids(20, 320, 1), H.random_ids(9, 320, 2)]
    want = eng.generate(prompts, max_tokens=6, temperature=0.0)
    replays = eng.runner.graph_replays
    with ops.KernelTimes() as kt:
        got = eng.generate(prompts, max_tokens=6, temperature=0.0)
    assert got == want and eng.runner.graph_replays == replays          # the same replies, no replay meanwhile
    tot = kt.totals()
    for name in ("gemm_tcgen05", "rmsnorm", "rope_kv_write", "decode_attention", "embed_rows", "argmax_rows"):
        assert tot[name] > 0.0 and tot[name + " calls"] >= 1, name
    assert tot["rmsnorm calls"] == (2 * 3 + 1) * len(eng.turn_log)      # two a layer and the final one, every turn
    assert ops.KernelTimes.active is None
    # every new token is told once, in order, as it becomes known (with steps launched ahead of the host too)
    told = {0: [], 1: []}
    end = want[0][3]
    again = eng.generate(prompts, max_tokens=6, temperature=0.0, stop=[end], on_token=lambda i, t: told[i].append(t))
    assert [told[0], told[1]] == again
    for w, a in zip(want, again):
        assert a == (w[: w.index(end) + 1] if end in w else w)
    eng.write_turn_csv(tmp_path / "turns.csv")
    lines = (tmp_path / "turns.csv").read_text().splitlines()
    assert lines[0].startswith("turn,seconds,tokens") and len(lines) == 1 + len(eng.turn_log)
    proc = subprocess.run([sys.executable, "-m", "lgml_b200", "-m", str(folder), "--prompt-ids", "1,2,3", "-n", "4", "--temperature", "0",
                           "--kernel-times", "--turn-csv", str(tmp_path / "cli.csv")], cwd=ROOT, text=True, capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "gemm_tcgen05" in proc.stderr and (tmp_path / "cli.csv").read_text().count("\n") >= 2


def test_errors_are_loud(folders, tmp_path):
    import lgml_b200
    from lgml_b200.engine.runner import ModelRunner, StepError
    from lgml_b200.cache import PoolFull

    folder = folders[("A", "float32")]
    runner = ModelRunner.from_folder(folder, torch.float32, "cuda:0", n_pages=1, max_slots=2)
    r = runner.open("r")
    with pytest.raises(StepError, match="vocabulary"):
        runner.step([(r, [256], [0])])
    with pytest.raises(StepError, match="twice"):
        runner.step([(r, [1], [0]), (r, [2], [0])])
    with pytest.raises(StepError, match="wanted place"):
        runner.step([(r, [1, 2], [2])])
    with pytest.raises(PoolFull, match="kv pool full"):
        runner.step([(r, [1] * 65, [])])
    big = ModelRunner.from_folder(folder, torch.float32, "cuda:0", n_pages=4, max_slots=1)
    with pytest.raises(StepError, match="context full"):
        big.step([(big.open("s"), [1] * 129, [])])
    with pytest.raises(RuntimeError, match="CUDA"):
        lgml_b200.Engine(str(folder), device="cpu")
