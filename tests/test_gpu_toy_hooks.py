"""A position part that is no rotation, and the attention mixer's optional extras, in a toy
architecture defined here and registered without a change to the framework's files.

Layer 0: a position encoding that adds a learnt vector per position to every head of q and k
(nothing is rotated), attention with a norm of q and of k per head and a cap on the scores.
Layer 1: the framework's rotary encoding and plain attention.  The model scales its embedding
rows and scales and caps its logits.  The toy position part is written with torch operations
and hands the cache write back to the framework (``store_kv``): only the interfaces are under
test.  Everything is compared with a plain float64 restatement over whole sequences."""
import math
from dataclasses import dataclass

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
E, H, G, D, INNER, V, MAXPOS = 40, 4, 2, 16, 56, 91, 256
SCORE_CAP, LOGIT_CAP, LOGIT_SCALE, QK_EPS = 4.0, 3.0, 0.5, 1e-4


def define_toy():
    from lgml_b200 import ops
    from lgml_b200.config import ModelConfig, register_architecture
    from lgml_b200.models import DecoderModel
    from lgml_b200.parts import LMHead, Part, TokenEmbedding, make_part, register_part, store_kv
    from lgml_b200.weights import MATRIX, TensorSpec

    class AddedPositions(Part):
        """q and k of every head get ``table[position]`` added; v is left alone."""

        def __init__(self, head_dim, max_positions):
            self.head_dim, self.max_positions = head_dim, max_positions
            self.table = None

        def tensor_specs(self, prefix):
            return [TensorSpec(prefix + ".position_table", (self.max_positions, self.head_dim), MATRIX)]

        def bind(self, prefix, tensors, rt):
            self.table = tensors[prefix + ".position_table"]

        def apply(self, rt, qkv, batch, cache, n_heads, n_kv_heads, head_dim):
            full = (qkv.sum() if isinstance(qkv, ops.Partials) else qkv).float()
            n, qk = full.shape[0], (n_heads + n_kv_heads) * head_dim
            add = self.table.float()[batch.positions.long()]
            moved = full[:, :qk].reshape(n, n_heads + n_kv_heads, head_dim) + add[:, None, :]
            out = torch.cat([moved.reshape(n, qk), full[:, qk:]], dim=1).to(rt.dtype)
            return store_kv(rt, out, batch, cache, n_heads, n_kv_heads, head_dim)

    @dataclass
    class ToyConfig(ModelConfig):
        architecture: str = "ToyHooksForCausalLM"
        vocab_size: int = V
        hidden_size: int = E
        max_position_embeddings: int = MAXPOS

        @classmethod
        def from_dict(cls, d):
            return cls(vocab_size=d["vocab_size"], hidden_size=d["hidden_size"], max_position_embeddings=d["max_position_embeddings"])

        def validate(self):
            pass

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                    "max_position_embeddings": self.max_position_embeddings}

    def build(cfg):
        norm = lambda w=E, eps=1e-5: make_part("norm", "rmsnorm", width=w, eps=eps)
        ffn = lambda: make_part("feed_forward", "gated_mlp", width=E, inner=INNER)
        first = make_part("mixer", "attention", width=E, n_heads=H, n_kv_heads=G, head_dim=D,
                          position=make_part("position", "toy_added", head_dim=D, max_positions=MAXPOS),
                          q_norm=norm(D, QK_EPS), k_norm=norm(D, QK_EPS), softcap=SCORE_CAP)
        second = make_part("mixer", "attention", width=E, n_heads=H, n_kv_heads=G, head_dim=D,
                           position=make_part("position", "rope", head_dim=D, theta=10000.0))
        blocks = [make_part("block", "pre_norm", mixer_norm=norm(), mixer=m, ffn_norm=norm(), ffn=ffn()) for m in (first, second)]
        emb = TokenEmbedding(cfg.vocab_size, E)
        return DecoderModel(cfg, emb, blocks, norm(), LMHead(cfg.vocab_size, E), embed_scale=math.sqrt(E), logit_scale=LOGIT_SCALE,
                            logit_softcap=LOGIT_CAP)

    register_part("position", "toy_added", AddedPositions)
    register_architecture("ToyHooksForCausalLM", ToyConfig, build)
    return ToyConfig


def plain_forward(w, ids):
    """The same toy model, whole sequence, no cache, float64."""
    from tests.plain import llama_plain as P

    n = len(ids)
    pos = list(range(n))
    x = w["model.embed_tokens.weight"][ids] * math.sqrt(E)

    def capped_attention(q, k, v):
        out = torch.empty(n, H, D, dtype=torch.float64)
        causal = torch.tril(torch.ones(n, n, dtype=torch.bool))
        for h in range(H):
            g = h // (H // G)
            s = (q[:, h] @ k[:, g].T) / math.sqrt(D)
            s = SCORE_CAP * torch.tanh(s / SCORE_CAP)
            out[:, h] = torch.softmax(s.masked_fill(~causal, float("-inf")), dim=-1) @ v[:, g]
        return out.reshape(n, H * D)

    for i in range(2):
        p = f"model.layers.{i}.self_attn."
        h = P.rms_norm(x, w[f"model.layers.{i}.input_layernorm.weight"], 1e-5)
        q = P.linear(h, w[p + "q_proj.weight"]).reshape(n, H, D)
        k = P.linear(h, w[p + "k_proj.weight"]).reshape(n, G, D)
        v = P.linear(h, w[p + "v_proj.weight"]).reshape(n, G, D)
        if i == 0:
            add = w[p + "position_table"][pos]
            q = P.rms_norm(q, w[p + "q_norm.weight"], QK_EPS) + add[:, None, :]
            k = P.rms_norm(k, w[p + "k_norm.weight"], QK_EPS) + add[:, None, :]
            o = capped_attention(q, k, v)
        else:
            inv = P.rope_inv_freq(D, 10000.0)
            o = P.attention(P.rope(q, pos, inv, "half"), P.rope(k, pos, inv, "half"), v, pos)
        x = x + P.linear(o, w[p + "o_proj.weight"])
        m = f"model.layers.{i}.mlp."
        h = P.rms_norm(x, w[f"model.layers.{i}.post_attention_layernorm.weight"], 1e-5)
        x = x + P.swiglu(h, w[m + "gate_proj.weight"], w[m + "up_proj.weight"], w[m + "down_proj.weight"])
    logits = P.linear(P.rms_norm(x, w["model.norm.weight"], 1e-5), w["lm_head.weight"]) * LOGIT_SCALE
    return LOGIT_CAP * torch.tanh(logits / LOGIT_CAP)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_position_part_that_is_no_rotation_and_the_optional_extras(dtype, tmp_path):
    ToyConfig = define_toy()
    from lgml_b200.engine.engine import parse_dtype
    from lgml_b200.engine.runner import ModelRunner
    from lgml_b200.weights import write_random_model
    from tests import helpers as Hp
    from tests.plain import llama_plain as P

    cfg = ToyConfig()
    folder = write_random_model(tmp_path, cfg, seed=9, std=0.15, dtype=dtype)
    runner = ModelRunner.from_folder(folder, parse_dtype(dtype), DEV, n_pages=6, max_slots=3)
    assert not runner.use_graphs                       # the toy part is not declared safe to capture: every step runs eagerly
    _, w = P.load_folder(folder)
    seqs = {"a": Hp.random_ids(150, V, 1), "b": Hp.random_ids(33, V, 2), "c": Hp.random_ids(70, V, 3)}
    want = {k: plain_forward(w, ids) for k, ids in seqs.items()}
    # the extras do something: without the caps and the added positions the logits are other logits
    assert float(want["a"].abs().max()) > 0.5
    tol = dict(atol=5e-5, rtol=1e-4) if dtype == "float32" else dict(atol=4e-2, rtol=2e-2)
    results = []
    for trace in (Hp.trace_whole(seqs), Hp.trace_tail(seqs, tail=20), Hp.trace_mixed(seqs, max_tokens=64 * 5, seed=4, max_live=2)):
        got = Hp.run_trace(runner, trace)
        results.append(got)
        for k, ids in seqs.items():
            rows = torch.stack([got[(k, p)] for p in range(len(ids))]).double()
            assert torch.allclose(rows, want[k], **tol), (k, float((rows - want[k]).abs().max()))
    if dtype == "float32":
        for got in results[1:]:
            assert all(torch.equal(results[0][key], got[key]) for key in results[0])
    assert not runner.cache.live
