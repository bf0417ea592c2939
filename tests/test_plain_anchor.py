"""The plain implementation against the one independent anchor the reference carries:
llama.cpp's logits for its tiny llama (``test/test_qwen_moe.lua:208-225``), kept as
data in ``tests/golden/ref_llama.json``.  Also the plain implementation's own
consistency (no GPU)."""
import json
from pathlib import Path

import torch

from tests import helpers as H
from tests.golden import make_ref_llama as G
from tests.plain import llama_plain as P

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_plain_matches_recorded_llama_cpp_rows():
    ref = json.loads((GOLDEN / "ref_llama.json").read_text())
    ids = [r["id"] for r in ref["rows"]]
    logits = P.forward(G.CONFIG, G.build(), ids, pairing="adjacent")
    idx = [i - 1 for i in ref["idx"]]
    for t, row in enumerate(ref["rows"]):
        assert int(torch.argmax(logits[t])) == row["best"], f"row {t}: argmax differs"
        got = logits[t, idx]
        err = (got - torch.tensor(row["v"], dtype=torch.float64)).abs().max()
        assert float(err) <= ref["tol"], f"row {t}: {float(err)} over the reference's own tolerance"


def test_half_pairing_on_permuted_rows_is_the_same_model():
    """safetensors rows with half pairing == gguf rows with adjacent pairing."""
    w = G.build()
    ids = [104, 101, 108, 108, 111, 256, 32, 119]
    a = P.forward(G.CONFIG, w, ids, pairing="adjacent")
    b = P.forward(G.CONFIG, G.to_half_pairing(w), ids, pairing="half")
    assert float((a - b).abs().max()) < 1e-12


def test_committed_plain_rows_are_current():
    stored = json.loads((GOLDEN / "ref_llama_plain.json").read_text())
    ref = json.loads((GOLDEN / "ref_llama.json").read_text())
    ids = [r["id"] for r in ref["rows"]]
    logits = P.forward(G.CONFIG, G.build(), ids, pairing="adjacent")
    idx = [i - 1 for i in ref["idx"]]
    for t, row in enumerate(stored["rows"]):
        assert torch.allclose(logits[t, idx], torch.tensor(row["v"], dtype=torch.float64), atol=1e-9)


def test_causality_and_greedy(tmp_path):
    folder = H.make_folder(tmp_path, H.TINY_B, seed=1, sharpen=40.0)
    cfg, w = P.load_folder(folder)
    ids = H.random_ids(70, cfg["vocab_size"], 1)
    full = P.forward(cfg, w, ids)
    part = P.forward(cfg, w, ids[:33])
    assert float((full[:33] - part).abs().max()) < 1e-10      # a position does not see later tokens
    out = P.greedy(cfg, w, ids[:5], 3)
    assert out[0] == int(torch.argmax(P.forward(cfg, w, ids[:5])[-1]))


def test_llama3_factors():
    s = H.TINY_B["rope_scaling"]
    f = P.rope_inv_freq(32, 500000.0, s)
    base = P.rope_inv_freq(32, 500000.0, None)
    ratio = base / f
    assert float(ratio[0]) == 1.0 and abs(float(ratio[-1]) - 8.0) < 1e-12
    assert all(1.0 <= float(r) <= 8.0 + 1e-9 for r in ratio)
    assert any(1.0 < float(r) < 8.0 for r in ratio)           # the blended band is hit


def test_window_limits_the_keys():
    torch.manual_seed(0)
    q, k, v = torch.randn(10, 2, 8, dtype=torch.float64), torch.randn(10, 1, 8, dtype=torch.float64), torch.randn(10, 1, 8, dtype=torch.float64)
    pos = list(range(10))
    full = P.attention(q, k, v, pos)
    win = P.attention(q, k, v, pos, window=4)
    assert torch.allclose(full[:4], win[:4]) and not torch.allclose(full[9], win[9])
    tail = P.attention(q[6:], k[6:], v[6:], pos[6:])
    assert torch.allclose(win[9], tail[3])
