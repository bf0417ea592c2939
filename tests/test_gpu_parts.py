"""Each part of a layer alone, built by name from the registry with sizes unlike the tiny
models', against the plain functions of tests/plain/llama_plain.py, in float32 and bfloat16."""
import pytest
import torch

from tests.plain import llama_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=3e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=4e-2, rtol=3e-2)


def runtime(dtype):
    from lgml_b200.engine.runtime import Runtime

    return Runtime(DEV, dtype)


def bind(part, prefix, rt, seed, scale=0.1):
    """Random tensors for a part's specs; returns them as float64 on the host too."""
    from lgml_b200.weights.loader import target_dtype

    g = torch.Generator().manual_seed(seed)
    host, dev = {}, {}
    for s in part.tensor_specs(prefix):
        if s.optional:
            continue
        t = torch.randn(s.shape, generator=g) * scale + s.init[0]
        t = t.to(target_dtype(s.kind, rt.dtype))
        host[s.name], dev[s.name] = t.double(), t.to(DEV)
    part.bind(prefix, dev, rt)
    return host


def one_batch(cm, lens, pos0s):
    """A StepBatch of requests that already hold pos0 tokens and bring lens new ones."""
    from lgml_b200.engine.batch import StepBatch

    reqs = []
    for i, (n, p0) in enumerate(zip(lens, pos0s)):
        r = cm.open(i)
        assert cm.reserve(r, p0 + n)
        r.n_tokens = p0
        reqs.append(r)
    return StepBatch(cm, reqs, [[0] * n for n in lens], [[] for _ in lens], DEV), reqs


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    from lgml_b200.parts import make_part

    rt = runtime(dtype)
    norm = make_part("norm", "rmsnorm", width=200, eps=2e-5)
    w = bind(norm, "n", rt, 1)
    x = torch.randn(6, 200, generator=torch.Generator().manual_seed(2))
    delta = torch.randn(6, 200, generator=torch.Generator().manual_seed(3)).to(dtype)
    xd = x.to(DEV)
    h = norm.forward(rt, xd, dtype, delta=delta.to(DEV))
    want = P.rms_norm(x.double() + delta.double(), w["n.weight"], 2e-5)
    assert torch.allclose(h.double().cpu(), want, **tol(dtype))
    assert torch.allclose(xd.double().cpu(), x.double() + delta.double(), atol=1e-6, rtol=1e-6)   # the sum stays in x, float32


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    from lgml_b200.parts import make_part

    rt = runtime(dtype)
    ffn = make_part("feed_forward", "gated_mlp", width=120, inner=200, activation="silu", bias=True)
    w = bind(ffn, "m", rt, 4)
    h = (torch.randn(9, 120, generator=torch.Generator().manual_seed(5))).to(dtype)
    y = ffn.forward(rt, h.to(DEV))
    if not torch.is_tensor(y):
        y = y.sum()
    want = P.swiglu(h.double(), w["m.gate_proj.weight"], w["m.up_proj.weight"], w["m.down_proj.weight"],
                    w["m.gate_proj.bias"], w["m.up_proj.bias"], w["m.down_proj.bias"])
    assert torch.allclose(y.double().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pairing,n_rot,window", [("half", 48, None), ("adjacent", 32, None), ("half", 48, 50)])
def test_attention_part_with_cache(dtype, pairing, n_rot, window):
    """Attention alone over a real cache: a request is fed in two portions (the second reads
    the first from its pages), beside a second request, and compared with whole-sequence
    plain attention."""
    from lgml_b200.cache import CacheManager
    from lgml_b200.config.llama import RopeScaling
    from lgml_b200.engine.batch import StepBatch
    from lgml_b200.parts import make_part

    rt = runtime(dtype)
    E, H, G, D = 120, 6, 2, 48
    scaling = RopeScaling("llama3", 4.0, 1.0, 4.0, 32)
    pos = make_part("position", "rope", head_dim=D, theta=7000.0, scaling=scaling, n_rot=n_rot, pairing=pairing)
    att = make_part("mixer", "attention", width=E, n_heads=H, n_kv_heads=G, head_dim=D, position=pos, bias=True, window=window)
    # float32: weights large enough for peaked attention; bfloat16: a spread of scores of ~1, since
    # a larger one amplifies bfloat16's own rounding of q and k past any useful bound
    w = bind(att, "a", rt, 6, scale=0.15 if dtype == torch.float32 else 0.08)
    cm = CacheManager({0: att.cache_spec()}, n_pages=8, max_slots=2, dtype=dtype, device=DEV)
    g = torch.Generator().manual_seed(7)
    lens = {"x": 100, "y": 70}
    hs = {k: torch.randn(n, E, generator=g).to(dtype) for k, n in lens.items()}
    reqs = {k: cm.open(k) for k in lens}
    outs = {k: [] for k in lens}
    for step in ([("x", 0, 61)], [("x", 61, 100), ("y", 0, 70)]):
        rs = [reqs[k] for k, _, _ in step]
        for (k, a, b), r in zip(step, rs):
            assert cm.reserve(r, b - a)
        batch = StepBatch(cm, rs, [[0] * (b - a) for _, a, b in step], [[] for _ in step], DEV)
        h = torch.cat([hs[k][a:b] for k, a, b in step]).to(DEV)
        y = att.forward(rt, h, batch, batch.cache_view(0))
        y = y if torch.is_tensor(y) else y.sum()
        o = 0
        for (k, a, b), r in zip(step, rs):
            outs[k].append(y[o:o + b - a].double().cpu())
            o += b - a
            cm.commit(r, b - a)
    rt.check_status()
    inv = P.rope_inv_freq(D, 7000.0, {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                      "original_max_position_embeddings": 32}, n_rot=n_rot)
    for k, n in lens.items():
        h = hs[k].double()
        q = P.linear(h, w["a.q_proj.weight"], w["a.q_proj.bias"]).reshape(n, H, D)
        kk = P.linear(h, w["a.k_proj.weight"], w["a.k_proj.bias"]).reshape(n, G, D)
        v = P.linear(h, w["a.v_proj.weight"], w["a.v_proj.bias"]).reshape(n, G, D)
        p = list(range(n))
        o = P.attention(P.rope(q, p, inv, pairing), P.rope(kk, p, inv, pairing), v, p, window=window)
        want = P.linear(o, w["a.o_proj.weight"], w["a.o_proj.bias"])
        assert torch.allclose(torch.cat(outs[k]), want, **tol(dtype)), k


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_embedding_and_head(dtype):
    from lgml_b200.cache import CacheManager
    from lgml_b200.engine.batch import StepBatch
    from lgml_b200.parts import LMHead, TokenEmbedding, make_part

    rt = runtime(dtype)
    E, H, G, D, F, V = 96, 3, 3, 32, 130, 211
    pos = make_part("position", "none")
    block = make_part("block", "pre_norm",
                      mixer_norm=make_part("norm", "rmsnorm", width=E, eps=1e-5),
                      mixer=make_part("mixer", "attention", width=E, n_heads=H, n_kv_heads=G, head_dim=D, position=pos),
                      ffn_norm=make_part("norm", "rmsnorm", width=E, eps=1e-5),
                      ffn=make_part("feed_forward", "gated_mlp", width=E, inner=F))
    w = bind(block, "b", rt, 8, scale=0.1)
    emb = TokenEmbedding(V, E, name="emb")
    head = LMHead(V, E, tied_to=emb)
    wt = bind(emb, "", rt, 9, scale=0.5)
    head.bind("", {}, rt)
    assert [s.optional for s in head.tensor_specs("")] == [True] and head.weight is emb.table    # tied: one tensor, unless the folder has a head
    cm = CacheManager({0: block.cache_spec()}, n_pages=2, max_slots=1, dtype=dtype, device=DEV)
    r = cm.open("r")
    ids = [5, 210, 0, 77, 5, 9, 100]
    n = len(ids)
    assert cm.reserve(r, n)
    batch = StepBatch(cm, [r], [ids], [[n - 1]], DEV)
    x = emb.forward(rt, batch.token_ids)
    assert torch.equal(x.double().cpu(), wt["emb"][ids])
    x, pending = block.forward(rt, x, None, batch, batch.cache_view(0))
    xs = x.double().cpu() + (pending if torch.is_tensor(pending) else pending.sum()).double().cpu()
    # plain: no position encoding, full attention
    x0 = wt["emb"][ids]
    h = P.rms_norm(x0, w["b.input_layernorm.weight"], 1e-5)
    a = "b.self_attn."
    q = P.linear(h, w[a + "q_proj.weight"]).reshape(n, H, D)
    k = P.linear(h, w[a + "k_proj.weight"]).reshape(n, G, D)
    v = P.linear(h, w[a + "v_proj.weight"]).reshape(n, G, D)
    x1 = x0 + P.linear(P.attention(q, k, v, list(range(n))), w[a + "o_proj.weight"])
    h = P.rms_norm(x1, w["b.post_attention_layernorm.weight"], 1e-5)
    x2 = x1 + P.swiglu(h, w["b.mlp.gate_proj.weight"], w["b.mlp.up_proj.weight"], w["b.mlp.down_proj.weight"])
    assert torch.allclose(xs, x2, **tol(dtype))
    # the head on normed rows gives float32 logits whatever the mode
    hrow = torch.randn(2, E, generator=torch.Generator().manual_seed(10)).to(dtype)
    logits = head.forward(rt, hrow.to(DEV))
    assert logits.dtype == torch.float32
    assert torch.allclose(logits.double().cpu(), hrow.double() @ wt["emb"].t(), **tol(dtype))
