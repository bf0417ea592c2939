"""Rebuild the reference's tiny llama and store the plain implementation's logits for it.

mischief/lgml's ``test/test_qwen_moe.lua`` makes a tiny llama from a fixed linear
congruential generator (``:32-38``, ``build`` ``:70-198``), feeds it two prompt
batches and six recorded ids (``:203-204``, ``:359-376``) and compares 8 logits per
row with numbers recorded from llama.cpp on the CPU with an f16 KV cache
(``REF.llama`` ``:210-225``, indices ``IDX`` ``:208``, tolerance 2e-3 ``:378``).
The reference's own model code (Lua on ggml) cannot run here, so those recorded
rows are the one independent anchor there is.  They are kept in
``ref_llama.json`` beside this script as data; this script regenerates the
weights, runs ``tests/plain/llama_plain.py`` on them and writes
``ref_llama_plain.json`` with the plain implementation's values at the same
places, for the record of how close the two are.

Run from the repository root:  python tests/golden/make_ref_llama.py
"""
import json
import math
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from tests.plain import llama_plain as P  # noqa: E402

HERE = Path(__file__).resolve().parent
E, H, HKV, D, NL, V = 64, 4, 2, 16, 2, 259
MASK = (1 << 64) - 1


def lcg(seed):
    x = seed

    def r():
        nonlocal x
        x = (x * 6364136223846793005 + 1442695040888963407) & MASK
        return (x >> 11) / 2.0**53

    return r


def build():
    """Weights in the reference's draw order, under safetensors names, rows in the
    gguf order (adjacent rotation pairs)."""
    r = lcg(len("llama") * 7919)
    w = {}

    def rand(shape, lo, hi):
        n = math.prod(shape)
        vals = [lo + (hi - lo) * r() for _ in range(n)]
        return torch.tensor(vals, dtype=torch.float64).to(torch.float32).reshape(shape)

    def mat(name, shape, gain=1.0):
        s = gain * math.sqrt(3.0 / shape[-1])
        w[name] = rand(shape, -s, s)

    def norm(name, d):
        w[name] = rand((d,), 0.9, 1.1)

    mat("model.embed_tokens.weight", (V, E), 3.0)
    norm("model.norm.weight", E)
    mat("lm_head.weight", (V, E))
    w["rope_freqs.weight"] = rand((D // 2,), 1.0, 8.0)
    for i in range(NL):
        p = f"model.layers.{i}."
        norm(p + "input_layernorm.weight", E)
        mat(p + "self_attn.q_proj.weight", (H * D, E))
        mat(p + "self_attn.k_proj.weight", (HKV * D, E))
        mat(p + "self_attn.v_proj.weight", (HKV * D, E))
        mat(p + "self_attn.o_proj.weight", (E, H * D))
        norm(p + "post_attention_layernorm.weight", E)
        mat(p + "mlp.gate_proj.weight", (2 * E, E))
        mat(p + "mlp.up_proj.weight", (2 * E, E))
        mat(p + "mlp.down_proj.weight", (E, 2 * E))
    return w


CONFIG = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": NL, "hidden_size": E, "num_attention_heads": H,
    "num_key_value_heads": HKV, "head_dim": D, "intermediate_size": 2 * E,
    "vocab_size": V, "rms_norm_eps": 1e-6, "rope_theta": 1e6,
    "max_position_embeddings": 4096, "tie_word_embeddings": False, "hidden_act": "silu",
}


def to_half_pairing(w):
    """Undo the gguf row order of q and k: gguf row h*D + 2j + x holds the
    safetensors row h*D + x*D/2 + j (``lua/lgml/lora.lua:164-184``)."""
    out = dict(w)
    for name, heads in (("q_proj", H), ("k_proj", HKV)):
        for i in range(NL):
            key = f"model.layers.{i}.self_attn.{name}.weight"
            g = w[key].reshape(heads, D // 2, 2, E)
            out[key] = g.permute(0, 2, 1, 3).reshape(heads * D, E).contiguous()
    return out


def write_folder(folder, dtype="float32"):
    """The same model as a safetensors folder: rows in safetensors order (half pairing), the
    frequency factors under ``rope_freqs.weight`` as the reference's loader takes them
    (``lua/lgml/transformer.lua:410``).  ``dtype`` is the stored type of the matrices."""
    from lgml_b200.weights import write_safetensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    w = to_half_pairing(build())
    if dtype == "bfloat16":
        w = {k: (v.to(torch.bfloat16) if v.dim() == 2 else v) for k, v in w.items()}
    (folder / "config.json").write_text(json.dumps({**CONFIG, "model_type": "llama", "torch_dtype": dtype}, indent=1))
    write_safetensors(folder / "model.safetensors", w, metadata={"format": "pt"})
    return folder


def main():
    ref = json.loads((HERE / "ref_llama.json").read_text())
    ids = [row["id"] for row in ref["rows"]]
    w = build()
    logits = P.forward(CONFIG, w, ids, pairing="adjacent")
    idx = [i - 1 for i in ref["idx"]]
    rows, err = [], 0.0
    for t, row in enumerate(ref["rows"]):
        got = [float(logits[t, j]) for j in idx]
        err = max(err, max(abs(a - b) for a, b in zip(got, row["v"])))
        rows.append({"id": row["id"], "best": int(torch.argmax(logits[t])), "v": got})
    (HERE / "ref_llama_plain.json").write_text(json.dumps({"idx": ref["idx"], "max_abs_diff_to_ref": err, "rows": rows}, indent=1))
    print("max |plain - llama.cpp| =", err)


if __name__ == "__main__":
    main()
