"""The engine against the plain implementation, under every way of cutting the work.

Each request alone and whole; most of it in one step and the last 32 tokens one by
one; in portions of changing size down to two tokens; and mixed, up to four live
requests, portions of some beside decoded tokens of others, with so few pages that
they are used again.  In float32 and in bfloat16, on tiny configurations that differ
in every size and option, with attention sharpened so that a wrong key shows.  In
float32 the four ways must agree bit for bit (the kernels sum in an order that does
not depend on the batch), as mischief/lgml demands of its own passes
(``test/replay_check.lua:63-76``, ``test/test_qwen_moe.lua:466-509``).
"""
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu

# Tolerances.  float32 kernels against a float64 oracle: a few units of float32 rounding on
# logits of size ~1, amplified by the sharpened attention.  bfloat16 has a unit roundoff of
# 2^-9 ~ 0.002 and a handful of roundings per layer: ~8 x 0.002 of the logits' size.
TOL = {"float32": dict(atol=2e-5, rtol=1e-4), "bfloat16": dict(atol=1.5e-2, rtol=1.5e-2)}
# The q and k projections are scaled so that attention is far from uniform and a wrong key,
# a stale page or a wrong position moves the logits by much more than the tolerance.  The
# scores' spread is ~4 in float32 and ~1 in bfloat16, where a larger spread would amplify
# bfloat16's own rounding of q and k past any useful bound.
SHARPEN = {"float32": 12.0, "bfloat16": 6.0}


def sequences(cfg, which):
    V = cfg["vocab_size"]
    lens = {"A": [21, 33, 47, 70, 100, 128], "B": [25, 64, 101, 154, 200, 65, 130], "C": [40, 129, 257, 64, 310]}[which]
    return {f"r{i}": H.random_ids(n, V, 100 + i) for i, n in enumerate(lens)}


@pytest.fixture(scope="module", params=["A", "B", "C"])
def tiny(request, tmp_path_factory):
    cfg, seed = H.TINY[request.param]
    out = {}
    for dtype in ("float32", "bfloat16"):
        out[dtype] = H.make_folder(tmp_path_factory.mktemp(f"tiny{request.param}_{dtype}"), cfg, seed, dtype=dtype, sharpen=SHARPEN[dtype])
    return request.param, cfg, out


def make_runner(folder, dtype, n_pages, slots=4):
    from lgml_b200.engine.engine import parse_dtype
    from lgml_b200.engine.runner import ModelRunner

    return ModelRunner.from_folder(folder, parse_dtype(dtype), "cuda:0", n_pages=n_pages, max_slots=slots)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_cuttings_match_oracle(tiny, dtype):
    which, cfg, folders = tiny
    folder = folders[dtype]
    seqs = sequences(cfg, which)
    longest = max(len(s) for s in seqs.values())
    pages_one = -(-longest // 64)
    results = {}
    # alone and whole; tail one by one; portions
    for name, trace in (("whole", H.trace_whole(seqs)), ("tail", H.trace_tail(seqs)), ("portions", H.trace_portions(seqs))):
        runner = make_runner(folder, dtype, n_pages=pages_one)
        results[name] = H.run_trace(runner, trace)
        assert runner.cache.groups[0].pool.n_held == 0
    # mixed, with a pool that cannot hold all requests at once: pages are used again
    total_pages = sum(-(-len(s) // 64) for s in seqs.values())
    max_tokens = 64 * min(2 * pages_one + 2, total_pages - 2)
    trace = H.trace_mixed(seqs, max_tokens=max_tokens, seed=7)
    assert max(len(st["entries"]) for st in trace) >= 3
    runner = make_runner(folder, dtype, n_pages=max_tokens // 64)
    results["mixed"] = H.run_trace(runner, trace)
    pool = runner.cache.groups[0].pool
    assert pool.taken_total > pool.n_pages, "the trace never used a page twice"
    for name, got in results.items():
        worst = H.compare_with_oracle(got, folder, seqs, **TOL[dtype])
        print(f"tiny-{which} {dtype} {name}: max |diff| {worst:.3g}")
    if dtype == "float32":
        for name in ("tail", "portions", "mixed"):
            for key, row in results["whole"].items():
                assert torch.equal(row, results[name][key]), f"float32 {name} differs from whole at {key}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_single_token_prompt(tiny, dtype):
    """The first tokens of a sequence, a one-token prompt, and a two-token portion at a page's edge."""
    which, cfg, folders = tiny
    folder = folders[dtype]
    V = cfg["vocab_size"]
    seqs = {"one": H.random_ids(1, V, 5), "two": H.random_ids(2, V, 6), "edge": H.random_ids(66, V, 8)}
    steps = [
        {"step": 0, "entries": [{"id": "one", "tokens": seqs["one"], "want": [0]}, {"id": "two", "tokens": seqs["two"], "want": [0, 1]}], "end": ["one", "two"]},
        {"step": 1, "entries": [{"id": "edge", "tokens": seqs["edge"][:63], "want": list(range(63))}], "end": []},
        {"step": 2, "entries": [{"id": "edge", "tokens": seqs["edge"][63:65], "want": [0, 1]}], "end": []},
        {"step": 3, "entries": [{"id": "edge", "tokens": seqs["edge"][65:], "want": [0]}], "end": ["edge"]},
    ]
    runner = make_runner(folder, dtype, n_pages=4)
    got = H.run_trace(runner, steps)
    H.compare_with_oracle(got, folder, seqs, **TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(tiny, dtype):
    """A short prompt, then token by token to the end of the context, on pages another request used."""
    which, cfg, folders = tiny
    folder = folders[dtype]
    n = cfg["max_position_embeddings"]
    ids = H.random_ids(n, cfg["vocab_size"], 77)
    junk = H.random_ids(n, cfg["vocab_size"], 78)
    runner = make_runner(folder, dtype, n_pages=-(-n // 64))
    # dirty every page first
    H.run_trace(runner, [{"step": 0, "entries": [{"id": "junk", "tokens": junk, "want": []}], "end": ["junk"]}])
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": ids[:3], "want": [0, 1, 2]}], "end": []}]
    for p in range(3, n):
        steps.append({"step": p, "entries": [{"id": "x", "tokens": [ids[p]], "want": [0]}], "end": ["x"] if p == n - 1 else []})
    got = H.run_trace(runner, steps)
    H.compare_with_oracle(got, folder, {"x": ids}, **TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_five_thousand_tokens_of_context(dtype, tmp_path):
    """Positions in the thousands (rotation angles of thousands of radians in 32-bit, block
    tables of 80 pages, key ranges cut for a long context): tiny-B with room for 16k positions,
    one request of 5,000 tokens read in portions of up to 2,048 on pages another request
    dirtied, its last 40 tokens one by one beside a second request's portions."""
    cfg = dict(H.TINY_B, max_position_embeddings=16384)
    folder = H.make_folder(tmp_path, cfg, 1, dtype=dtype, sharpen=SHARPEN[dtype])
    n, V = 5000, cfg["vocab_size"]
    ids, other, junk = H.random_ids(n, V, 42), H.random_ids(300, V, 43), H.random_ids(4000, V, 44)
    from lgml_b200.engine.engine import parse_dtype
    from lgml_b200.engine.runner import ModelRunner

    runner = ModelRunner.from_folder(folder, parse_dtype(dtype), "cuda:0", n_pages=-(-n // 64) + 5, max_slots=2, max_step_tokens=2048)
    steps = [{"step": 0, "entries": [{"id": "junk", "tokens": junk[:2048], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "junk", "tokens": junk[2048:], "want": []}], "end": ["junk"]}]
    p = 0
    for m in (2048, 1, 2047, 864):
        steps.append({"step": len(steps), "entries": [{"id": "long", "tokens": ids[p:p + m], "want": sorted({0, m // 2, m - 1})}], "end": []})
        p += m
    q = 0
    while p < n:
        entries = [{"id": "long", "tokens": [ids[p]], "want": [0]}]
        if q < len(other):
            m = min(9, len(other) - q)
            entries.append({"id": "other", "tokens": other[q:q + m], "want": [m - 1]})
            q += m
        p += 1
        steps.append({"step": len(steps), "entries": entries, "end": ["long", "other"] if p == n else []})
    assert q == len(other)
    got = H.run_trace(runner, steps)
    # only the rows that were asked for
    for rid, seq in (("long", ids), ("other", other)):
        ref = H.oracle_logits(folder, seq)
        rows = [pos for (r, pos) in got if r == rid]
        assert len(rows) >= 34
        for pos in rows:
            err = (got[(rid, pos)].double() - ref[pos]).abs()
            bound = TOL[dtype]["atol"] + TOL[dtype]["rtol"] * ref[pos].abs()
            assert bool((err <= bound).all()), (rid, pos, float(err.max()))
    runner.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_short_portions_replayed_from_captured_steps(tiny, dtype):
    """A short portion of one request that starts on a page's edge is padded to the next edge and
    replayed from a captured graph: prompts of 70, 3 and 64 tokens, each decoded on through the
    cells that the padding wrote, a second portion of 130 tokens behind a first of 64, and the same
    shapes again on pages that were used before (replays, not captures).  Against the plain
    implementation, and in 32-bit bit for bit against a runner without graphs."""
    which, cfg, folders = tiny
    folder, V = folders[dtype], cfg["vocab_size"]
    n_max = min(cfg["max_position_embeddings"], 250)
    seqs = {"a": H.random_ids(min(70 + 50, n_max), V, 11), "b": H.random_ids(3 + 40, V, 12), "c": H.random_ids(min(64 + 130 + 6, n_max), V, 13),
            "d": H.random_ids(min(70 + 50, n_max), V, 14), "e": H.random_ids(64 + 20, V, 15)}
    first = {"a": 70, "b": 3, "c": 64, "d": 70, "e": 64}
    steps = []
    for rid, ids in seqs.items():
        p = first[rid]
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[:p], "want": [p - 1]}], "end": []})
        if rid == "c":
            q = min(130, len(ids) - p - 2)
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[p:p + q], "want": []}], "end": []})
            p += q
        while p < len(ids):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [ids[p]], "want": [0]}], "end": [rid] if p == len(ids) - 1 else []})
            p += 1
    runner = make_runner(folder, dtype, n_pages=5)
    got = H.run_trace(runner, steps)
    assert runner._prompt_graphs and runner.graph_replays > 0
    from lgml_b200.engine.runner import prompt_graph_length as padded

    assert sorted(runner._prompt_graphs) == sorted({(padded(n, 64), 1) for n in (70, 3, 64)} | {(padded(min(130, len(seqs["c"]) - 66), 64), 0)})
    assert [padded(n, 64) for n in (2, 16, 17, 32, 33, 64, 65, 128, 129)] == [16, 16, 32, 32, 64, 64, 128, 128, 192]
    for rid, ids in seqs.items():
        ref = H.oracle_logits(folder, ids)
        for (r, pos), row in got.items():
            if r == rid:
                err = (row.double() - ref[pos]).abs()
                assert bool((err <= TOL[dtype]["atol"] + TOL[dtype]["rtol"] * ref[pos].abs()).all()), (rid, pos, float(err.max()))
    if dtype == "float32":
        from lgml_b200.engine.engine import parse_dtype
        from lgml_b200.engine.runner import ModelRunner

        plain = ModelRunner.from_folder(folder, parse_dtype(dtype), "cuda:0", n_pages=5, max_slots=4, use_graphs=False)
        want = H.run_trace(plain, steps)
        assert not plain._prompt_graphs
        assert all(torch.equal(got[k], want[k]) for k in want)
