"""The engine itself on the one model the reference records output for.

mischief/lgml's ``test/test_qwen_moe.lua`` feeds its tiny llama the batches
``{104,101,108,108,111}`` and ``{256,32,119}`` (``:203-204``), then six recorded ids one
by one (``:359-376``), and compares 8 logits of each of the 14 rows with llama.cpp's
(``REF.llama`` ``:210-225``, tolerance 2e-3 ``:378``).  Here ``bin/trace_run`` gets the
same model as a safetensors folder (rows in safetensors order, the frequency factors
as ``rope_freqs.weight``, the reference's only way to scale the rotation,
``lua/lgml/transformer.lua:410``) and the same steps, in float32 and in bfloat16.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.golden import make_ref_llama as G
from tests.plain import llama_plain as P

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"


def replay(folder, dtype, steps, out):
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
                           "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", text=True, capture_output=True,
                          env=dict(os.environ, PYTHONPATH=str(ROOT)), timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    rows = []
    for st in steps:
        n = sum(len(e["want"]) for e in st["entries"])
        rows.append(np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(n, G.V))
    return torch.from_numpy(np.concatenate(rows))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_reproduces_the_recorded_rows(dtype, tmp_path):
    ref = json.loads((GOLDEN / "ref_llama.json").read_text())
    ids = [r["id"] for r in ref["rows"]]
    assert ids[:8] == [104, 101, 108, 108, 111, 256, 32, 119]
    folder = G.write_folder(tmp_path / "model", dtype)
    cuts = [ids[:5], ids[5:8]] + [[t] for t in ids[8:]]
    steps = [{"step": i, "entries": [{"id": "llama", "tokens": c, "want": list(range(len(c)))}], "end": []} for i, c in enumerate(cuts)]
    steps[-1]["end"] = ["llama"]
    got = replay(folder, dtype, steps, tmp_path / "out")
    assert got.shape == (14, G.V)
    idx = [i - 1 for i in ref["idx"]]
    want = torch.tensor([r["v"] for r in ref["rows"]], dtype=torch.float64)
    err = (got[:, idx].double() - want).abs()
    if dtype == "float32":
        # the reference's own bound for another engine on this model
        assert float(err.max()) <= ref["tol"], f"row {int(err.max(dim=1).values.argmax())}: {float(err.max())}"
        assert got.argmax(dim=1).tolist() == [r["best"] for r in ref["rows"]]
    else:
        # bfloat16 weights, activations and cache: a unit roundoff of 2^-9 on a dozen stages,
        # relative to the logits' size; the best token wherever it leads by more than that
        full = P.forward(G.CONFIG, G.build(), ids, pairing="adjacent")
        bound = 1.5e-2 * float(full.abs().max())
        assert float(err.max()) <= bound, (float(err.max()), bound)
        for t, r in enumerate(ref["rows"]):
            top2 = full[t].topk(2).values
            if float(top2[0] - top2[1]) > 2 * bound:
                assert int(got[t].argmax()) == r["best"], t
