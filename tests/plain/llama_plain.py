"""Plain, slow Llama decoder: the oracle of the test-suite.

Whole sequences, no cache, one function per part, float64 on the CPU. It shares
no code with ``lgml_b200``: it has its own safetensors reader, its own config
reading and its own formulas, each written from mischief/lgml's graph builder
(``lua/lgml/transformer.lua``) and C binding (``src/lgml.c``); the citation
beside each function is a path inside that project.

mischief/lgml's own model code is Lua on ggml and can be neither imported nor
compiled here (no Lua, no ggml), so this file rests on the formulas.  It is
anchored once on numbers the reference records from another engine: the
llama.cpp logits of its tiny llama (``test/test_qwen_moe.lua:210-225``), see
``tests/golden/`` and ``tests/test_plain_anchor.py``.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64

_ST_DTYPES = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "I64": np.int64, "I32": np.int32}


def read_safetensors(path):
    """name -> float64/int64 torch tensor.  Format as ``src/safetensors.c:278-332``:
    8-byte little-endian header length, JSON header, raw data."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + hlen].decode("utf-8"))
    data = raw[8 + hlen :]
    out = {}
    for name, ent in header.items():
        if name == "__metadata__":
            continue
        b, e = ent["data_offsets"]
        buf = data[b:e]
        shape = tuple(ent["shape"])
        if ent["dtype"] == "BF16":
            u16 = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            arr = u16.view(np.float32).astype(np.float64)
        else:
            arr = np.frombuffer(buf, dtype=np.dtype(_ST_DTYPES[ent["dtype"]]).newbyteorder("<"))
            arr = arr.astype(np.int64 if ent["dtype"].startswith("I") else np.float64)
        out[name] = torch.from_numpy(arr.reshape(shape).copy())
    return out


def load_folder(folder):
    """(config dict, weights dict) of a model folder."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = {}
    for f in sorted(folder.glob("*.safetensors")):
        weights.update(read_safetensors(f))
    return cfg, weights


# ----------------------------------------------------------------------------
# configuration
# ----------------------------------------------------------------------------

def sizes(cfg):
    """The sizes the formulas need, with the defaults of ``M.config``
    (``lua/lgml/transformer.lua:135-150``): KV heads default to the heads, the
    head size to hidden // heads, the rope base to 10000."""
    H = cfg["num_attention_heads"]
    rp = cfg.get("rope_parameters") or {}
    scaling = cfg.get("rope_scaling")
    if scaling is None and rp.get("rope_type", "default") != "default":
        scaling = rp
    return dict(
        L=cfg["num_hidden_layers"],
        E=cfg["hidden_size"],
        H=H,
        Hkv=cfg.get("num_key_value_heads") or H,
        D=cfg.get("head_dim") or cfg["hidden_size"] // H,
        F=cfg["intermediate_size"],
        V=cfg["vocab_size"],
        eps=cfg["rms_norm_eps"],
        theta=float(rp.get("rope_theta", cfg.get("rope_theta", 10000.0))),
        scaling=scaling,
        tied=bool(cfg.get("tie_word_embeddings", False)),
        window=cfg.get("sliding_window"),
    )


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------

def embed(table, ids):
    """``x = get_rows(tok_embd, ids)``, no scale for llama
    (``lua/lgml/transformer.lua:2303-2306``)."""
    return table[torch.as_tensor(ids, dtype=torch.long)].to(F64)


def rms_norm(x, weight, eps):
    """``rms_norm(x, eps) * w``: x / sqrt(mean(x^2) + eps), eps inside the root,
    the weight a separate multiply (``src/lgml.c:1626-1633``,
    ``lua/lgml/transformer.lua:1760``)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * weight


def linear(x, w, b=None):
    """``mul_mat(W (M,K), x (N,K)) -> (N,M)``: y = x W^T (``src/lgml.c:1811-1839``).
    The bias (``attention_bias``/``mlp_bias``) is added after the product; the
    reference loads none (``lua/lgml/transformer.lua:304-319``)."""
    y = x @ w.T
    return y if b is None else y + b


def rope_inv_freq(D, theta, scaling=None, n_rot=None):
    """Per-pair angular frequency ``theta^(-2i/n_rot) / ff_i``
    (``lua/lgml/transformer.lua:1756`` with ``src/lgml.c:2067-2078``).  The
    reference takes the factors ``ff`` ready-made from ``rope_freqs.weight``
    (``lua/lgml/transformer.lua:410``); for ``rope_type: llama3`` they follow
    from the wavelength of each pair: short waves are kept, long ones slowed by
    ``factor``, and a smooth blend lies between."""
    n_rot = n_rot or D
    i = torch.arange(0, n_rot // 2, dtype=F64)
    f = theta ** (-2.0 * i / n_rot)
    if not scaling:
        return f
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    if kind == "default":
        return f
    if kind == "linear":
        return f / float(scaling["factor"])
    assert kind == "llama3", kind
    factor = float(scaling["factor"])
    low = float(scaling.get("low_freq_factor", 1.0))
    high = float(scaling.get("high_freq_factor", 4.0))
    orig = float(scaling["original_max_position_embeddings"])
    wavelen = 2.0 * math.pi / f
    out = f.clone()
    for j in range(f.numel()):
        if wavelen[j] < orig / high:
            continue
        if wavelen[j] > orig / low:
            out[j] = f[j] / factor
        else:
            s = (orig / wavelen[j] - low) / (high - low)
            out[j] = (1.0 - s) * f[j] / factor + s * f[j]
    return out


def rope(x, pos, inv_freq, pairing="half"):
    """Rotate pairs of x (n, heads, D) by ``pos * inv_freq``.  ``adjacent`` pairs
    (2i, 2i+1) is the reference's "normal" mode on gguf-ordered rows;
    ``half`` pairs (i, i + n_rot/2), which is what safetensors checkpoints
    hold (the reference permutes rows between the two:
    ``lua/lgml/lora.lua:164-184``).  Dimensions past n_rot pass through."""
    n_rot = 2 * inv_freq.numel()
    ang = torch.as_tensor(pos, dtype=F64)[:, None] * inv_freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if pairing == "adjacent":
        a, b = x[..., 0:n_rot:2], x[..., 1:n_rot:2]
        out[..., 0:n_rot:2] = a * c - b * s
        out[..., 1:n_rot:2] = a * s + b * c
    else:
        h = n_rot // 2
        a, b = x[..., :h], x[..., h:n_rot]
        out[..., :h] = a * c - b * s
        out[..., h:n_rot] = a * s + b * c
    return out


def attention(q, k, v, pos, scale=None, window=None):
    """softmax over keys of ``(q.k) * scale + mask`` then the weighted sum of v
    (``lua/lgml/transformer.lua:1805-1816``); scale 1/sqrt(D) (``:1845``); row i
    sees keys at positions <= its own (``src/lgml.c:2863-2865``), and with a
    window only the last ``window`` of them; q head h reads KV head
    h // (H / Hkv).  q (n,H,D), k, v (n,Hkv,D) -> (n, H*D)."""
    n, H, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    p = torch.as_tensor(pos, dtype=torch.long)
    ok = p[None, :] <= p[:, None]
    if window:
        ok &= p[None, :] > p[:, None] - window
    out = torch.empty(n, H, D, dtype=F64)
    for h in range(H):
        g = h // (H // Hkv)
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(~ok, float("-inf"))
        out[:, h, :] = torch.softmax(s, dim=-1) @ v[:, g, :]
    return out.reshape(n, H * D)


def swiglu(h, wg, wu, wd, bg=None, bu=None, bd=None):
    """``Wd . (silu(Wg.h) * (Wu.h))``, silu(a) = a * sigmoid(a)
    (``lua/lgml/transformer.lua:2047-2049``, ``src/lgml.c:1476-1482``)."""
    g = linear(h, wg, bg)
    u = linear(h, wu, bu)
    return linear(g * torch.sigmoid(g) * u, wd, bd)


# ----------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------

def forward(cfg, w, ids, pairing="half", inv_freq=None, names="hf"):
    """Logits (n, V) of one whole sequence.  Layer loop as
    ``lua/lgml/transformer.lua:2312-2345``: norm, q/k/v, rope, attention,
    out-projection + residual, norm, feed-forward + residual; then the final
    norm and the head (``:2095-2096``), which falls back to the embedding when
    the file has no head (``:408``)."""
    z = sizes(cfg)
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in w.items()}
    if inv_freq is None:
        inv_freq = rope_inv_freq(z["D"], z["theta"], z["scaling"])
        if "rope_freqs.weight" in w:
            inv_freq = rope_inv_freq(z["D"], z["theta"], None) / w["rope_freqs.weight"]
    n = len(ids)
    pos = list(range(n))
    x = embed(w["model.embed_tokens.weight"], ids)
    for il in range(z["L"]):
        p = f"model.layers.{il}."
        a = p + "self_attn."
        h = rms_norm(x, w[p + "input_layernorm.weight"], z["eps"])
        q = linear(h, w[a + "q_proj.weight"], w.get(a + "q_proj.bias")).reshape(n, z["H"], z["D"])
        k = linear(h, w[a + "k_proj.weight"], w.get(a + "k_proj.bias")).reshape(n, z["Hkv"], z["D"])
        v = linear(h, w[a + "v_proj.weight"], w.get(a + "v_proj.bias")).reshape(n, z["Hkv"], z["D"])
        q = rope(q, pos, inv_freq, pairing)
        k = rope(k, pos, inv_freq, pairing)
        o = attention(q, k, v, pos, window=z["window"])
        x = x + linear(o, w[a + "o_proj.weight"], w.get(a + "o_proj.bias"))
        m = p + "mlp."
        h = rms_norm(x, w[p + "post_attention_layernorm.weight"], z["eps"])
        x = x + swiglu(
            h, w[m + "gate_proj.weight"], w[m + "up_proj.weight"], w[m + "down_proj.weight"],
            w.get(m + "gate_proj.bias"), w.get(m + "up_proj.bias"), w.get(m + "down_proj.bias"),
        )
    x = rms_norm(x, w["model.norm.weight"], z["eps"])
    head = w.get("lm_head.weight")
    if head is None:
        head = w["model.embed_tokens.weight"]
    return linear(x, head)


def greedy(cfg, w, prompt, n_new, **kw):
    """Greedy continuation by whole-sequence passes: the lowest index wins a tie
    (``src/sample.c:913-926``)."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(cfg, w, ids, **kw)[-1]
        t = int(torch.argmax(logits))
        out.append(t)
        ids.append(t)
    return out
