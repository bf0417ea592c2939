"""Two more toy parts, defined here and registered without a change to the framework's files:
a feed-forward with routing (every token goes to the one of three small experts that a router
scores highest) and another position encoding (frequencies that fall off linearly, on the first
12 of 16 dimensions, adjacent pairs).  A toy architecture puts them in its first layer and the
framework's own rotary encoding and gated feed-forward in its second, so one model holds
different feed-forwards and position encodings in different layers.  The toy parts are written
with torch operations: only the framework's interfaces are under test."""
from dataclasses import dataclass

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
E, INNER, EXPERTS = 48, 40, 3


def define_toy():
    from lgml_b200.config import ModelConfig, register_architecture
    from lgml_b200.models import DecoderModel
    from lgml_b200.parts import LMHead, Part, TokenEmbedding, make_part, register_part
    from lgml_b200.weights import MATRIX, TensorSpec

    class RoutedFeedForward(Part):
        """y = down_e(relu(up_e(h))) for the expert e = argmax(router(h)) of each token; the router's
        scores in float32."""

        def __init__(self, width, inner, experts):
            self.width, self.inner, self.experts = width, inner, experts

        def tensor_specs(self, prefix):
            specs = [TensorSpec(prefix + ".router.weight", (self.experts, self.width), MATRIX)]
            for e in range(self.experts):
                specs += [TensorSpec(f"{prefix}.experts.{e}.up.weight", (self.inner, self.width), MATRIX),
                          TensorSpec(f"{prefix}.experts.{e}.down.weight", (self.width, self.inner), MATRIX)]
            return specs

        def bind(self, prefix, tensors, rt):
            self.router = tensors[prefix + ".router.weight"]
            self.up = [tensors[f"{prefix}.experts.{e}.up.weight"] for e in range(self.experts)]
            self.down = [tensors[f"{prefix}.experts.{e}.down.weight"] for e in range(self.experts)]

        def forward(self, rt, h):
            choice = (h.float() @ self.router.float().t()).argmax(dim=1)
            out = torch.zeros_like(h)
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    x = h[rows].float()
                    out[rows] = (torch.relu(x @ self.up[e].float().t()).to(h.dtype).float() @ self.down[e].float().t()).to(h.dtype)
            return out

    class LinearFrequencies(Part):
        """What the attention mixer asks of a position encoding: `inv_freq` (float32, one angular
        frequency per rotated pair, on the device), `n_rot` and `pairing`."""
        graph_safe = True
        pairing = "adjacent"

        def __init__(self, head_dim, n_rot):
            self.n_rot = n_rot
            self.inv_freq = None

        def tensor_specs(self, prefix):
            return []

        def bind(self, prefix, tensors, rt):
            half = self.n_rot // 2
            self.inv_freq = torch.tensor([0.5 * (1.0 - i / half) for i in range(half)], dtype=torch.float32, device=rt.device)

    @dataclass
    class ToyConfig(ModelConfig):
        architecture: str = "ToyPartsForCausalLM"
        vocab_size: int = 83
        hidden_size: int = E
        max_position_embeddings: int = 256

        @classmethod
        def from_dict(cls, d):
            return cls(vocab_size=d["vocab_size"], hidden_size=d["hidden_size"], max_position_embeddings=d["max_position_embeddings"])

        def validate(self):
            pass

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                    "max_position_embeddings": self.max_position_embeddings}

    def build(cfg):
        norm = lambda: make_part("norm", "rmsnorm", width=E, eps=1e-5)
        attn = lambda pos: make_part("mixer", "attention", width=E, n_heads=3, n_kv_heads=1, head_dim=16, position=pos)
        blocks = [
            make_part("block", "pre_norm", mixer_norm=norm(), mixer=attn(make_part("position", "toy_linear", head_dim=16, n_rot=12)),
                      ffn_norm=norm(), ffn=make_part("feed_forward", "toy_routed", width=E, inner=INNER, experts=EXPERTS)),
            make_part("block", "pre_norm", mixer_norm=norm(), mixer=attn(make_part("position", "rope", head_dim=16, theta=10000.0)),
                      ffn_norm=norm(), ffn=make_part("feed_forward", "gated_mlp", width=E, inner=64)),
        ]
        emb = TokenEmbedding(cfg.vocab_size, E)
        return DecoderModel(cfg, emb, blocks, norm(), LMHead(cfg.vocab_size, E, tied_to=emb))

    register_part("feed_forward", "toy_routed", RoutedFeedForward)
    register_part("position", "toy_linear", LinearFrequencies)
    register_architecture("ToyPartsForCausalLM", ToyConfig, build)
    return ToyConfig


def plain_forward(w, ids):
    """The same toy model, whole sequence, no cache, float64."""
    from tests.plain import llama_plain as P

    n = len(ids)
    pos = list(range(n))
    x = w["model.embed_tokens.weight"][ids]

    def attn(x, i, inv, pairing):
        p = f"model.layers.{i}.self_attn."
        h = P.rms_norm(x, w[f"model.layers.{i}.input_layernorm.weight"], 1e-5)
        q = P.rope(P.linear(h, w[p + "q_proj.weight"]).reshape(n, 3, 16), pos, inv, pairing)
        k = P.rope(P.linear(h, w[p + "k_proj.weight"]).reshape(n, 1, 16), pos, inv, pairing)
        v = P.linear(h, w[p + "v_proj.weight"]).reshape(n, 1, 16)
        return x + P.linear(P.attention(q, k, v, pos), w[p + "o_proj.weight"])

    lin = torch.tensor([0.5 * (1.0 - i / 6) for i in range(6)], dtype=torch.float32).double()
    x = attn(x, 0, lin, "adjacent")
    h = P.rms_norm(x, w["model.layers.0.post_attention_layernorm.weight"], 1e-5)
    choice = (h @ w["model.layers.0.mlp.router.weight"].t()).argmax(dim=1)
    y = torch.zeros_like(h)
    for t in range(n):
        e = int(choice[t])
        mid = torch.relu(h[t] @ w[f"model.layers.0.mlp.experts.{e}.up.weight"].t())
        y[t] = mid @ w[f"model.layers.0.mlp.experts.{e}.down.weight"].t()
    x = x + y
    x = attn(x, 1, P.rope_inv_freq(16, 10000.0), "half")
    m = "model.layers.1.mlp."
    h = P.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], 1e-5)
    x = x + P.swiglu(h, w[m + "gate_proj.weight"], w[m + "up_proj.weight"], w[m + "down_proj.weight"])
    return P.linear(P.rms_norm(x, w["model.norm.weight"], 1e-5), w["model.embed_tokens.weight"]), choice


def test_toy_routed_feed_forward_and_toy_position_encoding(tmp_path):
    ToyConfig = define_toy()
    from lgml_b200.engine.runner import ModelRunner
    from lgml_b200.weights import write_random_model
    from tests import helpers as H
    from tests.plain import llama_plain as P

    cfg = ToyConfig()
    folder = write_random_model(tmp_path, cfg, seed=5, std=0.1, dtype="float32")
    runner = ModelRunner.from_folder(folder, torch.float32, DEV, n_pages=6, max_slots=3)
    _, w = P.load_folder(folder)
    seqs = {"a": H.random_ids(140, 83, 1), "b": H.random_ids(30, 83, 2), "c": H.random_ids(66, 83, 3)}
    want = {}
    for k, ids in seqs.items():
        want[k], choice = plain_forward(w, ids)
        if k == "a":
            assert len(set(choice.tolist())) == EXPERTS          # the router really spreads the tokens over the experts
    for trace in (H.trace_whole(seqs), H.trace_mixed(seqs, max_tokens=64 * 5, seed=4, max_live=2)):
        got = H.run_trace(runner, trace)
        for k, ids in seqs.items():
            rows = torch.stack([got[(k, p)] for p in range(len(ids))]).double()
            assert torch.allclose(rows, want[k], atol=5e-5, rtol=1e-4), (k, float((rows - want[k]).abs().max()))
    assert not runner.cache.live
