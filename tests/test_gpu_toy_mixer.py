"""A toy mixer with state of its own, defined here, is registered, built into a model and
stepped without a change to the framework's files.

The mixer keeps, per request, the running sum of its inputs and a token count in a slot of
fixed size; its output for a token is W . (mean of the inputs up to and including it).  It
is written with torch operations: only the framework's interfaces are under test.  A toy
architecture puts it beside real attention layers (different mixers in different layers),
runs one block twice, and lets a late layer read an early layer's cache."""
from dataclasses import dataclass

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def define_toy():
    from lgml_b200.cache import FixedState
    from lgml_b200.config import ModelConfig, register_architecture
    from lgml_b200.models import DecoderModel, LayerCall
    from lgml_b200.parts import LMHead, Part, TokenEmbedding, make_part, register_part
    from lgml_b200.weights import MATRIX, TensorSpec

    class RunningMean(Part):
        def __init__(self, width):
            self.width = width
            self.w = None

        def cache_spec(self):
            return FixedState((self.width + 1,), torch.float32)       # the sum, and the count

        def tensor_specs(self, prefix):
            return [TensorSpec(prefix + ".mix.weight", (self.width, self.width), MATRIX)]

        def bind(self, prefix, tensors, rt):
            self.w = tensors[prefix + ".mix.weight"]

        def forward(self, rt, h, batch, cache):
            out = torch.empty_like(h)
            start = 0
            for s, n in enumerate(batch.seq_lens):                   # tokens of a request in order
                slot = batch.requests[s].slot
                st = cache.state[slot]
                x = h[start:start + n].float()
                sums = st[: self.width] + torch.cumsum(x, 0)
                counts = st[self.width] + torch.arange(1, n + 1, device=h.device, dtype=torch.float32)
                mean = sums / counts[:, None]
                out[start:start + n] = (mean @ self.w.float().t()).to(h.dtype)
                if cache.writable:
                    st[: self.width] = sums[-1]
                    st[self.width] = counts[-1]
                start += n
            return out

    @dataclass
    class ToyConfig(ModelConfig):
        architecture: str = "ToyStateForCausalLM"
        vocab_size: int = 97
        hidden_size: int = 64
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
        E = cfg.hidden_size
        norm = lambda: make_part("norm", "rmsnorm", width=E, eps=1e-5)
        ffn = lambda: make_part("feed_forward", "gated_mlp", width=E, inner=96)
        rope = make_part("position", "rope", head_dim=16, theta=10000.0)
        blocks = [
            make_part("block", "pre_norm", mixer_norm=norm(), mixer=make_part("mixer", "attention", width=E, n_heads=4, n_kv_heads=2, head_dim=16, position=rope), ffn_norm=norm(), ffn=ffn()),
            make_part("block", "pre_norm", mixer_norm=norm(), mixer=make_part("mixer", "running_mean", width=E), ffn_norm=norm(), ffn=ffn()),
            make_part("block", "pre_norm", mixer_norm=norm(), mixer=make_part("mixer", "attention", width=E, n_heads=4, n_kv_heads=2, head_dim=16, position=rope), ffn_norm=None, ffn=None),
        ]
        emb = TokenEmbedding(cfg.vocab_size, E)
        # block 1 (the stateful one) runs twice, each call with state of its own; the last call
        # runs attention block 2 on the cache that call 0 wrote
        schedule = [LayerCall(0), LayerCall(1), LayerCall(1), LayerCall(2, cache=0)]
        return DecoderModel(cfg, emb, blocks, norm(), LMHead(cfg.vocab_size, E, tied_to=emb), schedule=schedule)

    register_part("mixer", "running_mean", RunningMean)
    register_architecture("ToyStateForCausalLM", ToyConfig, build)
    return ToyConfig


def plain_forward(w, ids, E=64):
    """The same toy model, whole sequence, no cache, float64."""
    from tests.plain import llama_plain as P

    n = len(ids)
    pos = list(range(n))
    inv = P.rope_inv_freq(16, 10000.0)
    x = w["model.embed_tokens.weight"][ids]

    def attn(x, i, kv=None):
        p = f"model.layers.{i}.self_attn."
        h = P.rms_norm(x, w[f"model.layers.{i}.input_layernorm.weight"], 1e-5)
        q = P.rope(P.linear(h, w[p + "q_proj.weight"]).reshape(n, 4, 16), pos, inv)
        if kv is None:
            k = P.rope(P.linear(h, w[p + "k_proj.weight"]).reshape(n, 2, 16), pos, inv)
            v = P.linear(h, w[p + "v_proj.weight"]).reshape(n, 2, 16)
            kv = (k, v)
        return x + P.linear(P.attention(q, kv[0], kv[1], pos), w[p + "o_proj.weight"]), kv

    def mean_mix(x, i):
        h = P.rms_norm(x, w[f"model.layers.{i}.input_layernorm.weight"], 1e-5)
        mean = torch.cumsum(h, 0) / torch.arange(1, n + 1, dtype=torch.float64)[:, None]
        return x + mean @ w[f"model.layers.{i}.self_attn.mix.weight"].t()

    def ffn(x, i):
        m = f"model.layers.{i}.mlp."
        h = P.rms_norm(x, w[f"model.layers.{i}.post_attention_layernorm.weight"], 1e-5)
        return x + P.swiglu(h, w[m + "gate_proj.weight"], w[m + "up_proj.weight"], w[m + "down_proj.weight"])

    x, kv0 = attn(x, 0)
    x = ffn(x, 0)
    x = ffn(mean_mix(x, 1), 1)
    x = ffn(mean_mix(x, 1), 1)
    x, _ = attn(x, 2, kv=kv0)
    return P.linear(P.rms_norm(x, w["model.norm.weight"], 1e-5), w["model.embed_tokens.weight"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype, tmp_path):
    ToyConfig = define_toy()
    from lgml_b200.config import load_config
    from lgml_b200.engine.runner import ModelRunner
    from lgml_b200.models import build_model
    from lgml_b200.weights import write_random_model
    from tests import helpers as H
    from tests.plain import llama_plain as P

    cfg = ToyConfig()
    folder = write_random_model(tmp_path, cfg, seed=3, std=0.08, dtype="float32" if dtype == torch.float32 else "bfloat16")
    assert load_config(folder) == cfg
    model = build_model(cfg)
    layout = model.cache_layout()
    assert sorted(layout) == [0, 1, 2]                      # call 3 owns no cache
    runner = ModelRunner.from_folder(folder, dtype, DEV, n_pages=6, max_slots=3)
    assert len(runner.cache.state_groups) == 1 and sorted(runner.cache.state_groups[0].layers) == [1, 2]
    _, w = P.load_folder(folder)
    seqs = {"a": H.random_ids(150, 97, 1), "b": H.random_ids(33, 97, 2), "c": H.random_ids(70, 97, 3)}
    want = {k: plain_forward(w, ids) for k, ids in seqs.items()}
    # whole, then a mixed trace with portions, single tokens and a slot used again
    for trace in (H.trace_whole(seqs), H.trace_mixed(seqs, max_tokens=64 * 5, seed=3, max_live=2)):
        got = H.run_trace(runner, trace)
        for k, ids in seqs.items():
            rows = torch.stack([got[(k, p)] for p in range(len(ids))]).double()
            tol = dict(atol=5e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=6e-2, rtol=5e-2)
            assert torch.allclose(rows, want[k], **tol), (k, float((rows - want[k]).abs().max()))
    assert not runner.cache.live
