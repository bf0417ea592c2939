"""The Llama dense decoder: which parts a ``LlamaConfig`` asks for.

Per layer (``lua/lgml/transformer.lua:2312-2345``): RMSNorm, attention with
grouped KV heads and rotary positions, residual; RMSNorm, SiLU-gated
feed-forward, residual; then a final RMSNorm and the head, tied to the embedding
when ``tie_word_embeddings`` (``:408``).  The family flags of the reference for
llama are "normal" rope over the whole head and nothing else
(``family.llama``, ``:62``).  Tensor names are the safetensors names of
``lua/lgml/convert.lua:52-75``.
"""
from __future__ import annotations

from ..config import LlamaConfig, register_architecture
from ..parts import LMHead, TokenEmbedding, make_part
from .decoder import DecoderModel


def layer_descriptors(cfg: LlamaConfig):
    """One descriptor per layer: the names and arguments of its parts.  Every Llama layer
    is alike; the list form is what lets another architecture differ layer by layer
    (the reference keeps ``hp.layers[i]``, ``lua/lgml/transformer.lua:222-245``)."""
    rope = dict(head_dim=cfg.head_dim, theta=cfg.rope_theta, scaling=cfg.rope_scaling, pairing="half",
                factors_tensor="rope_freqs.weight")
    return [
        dict(
            block="pre_norm",
            norm=("rmsnorm", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps)),
            position=("rope", rope),
            mixer=("attention", dict(width=cfg.hidden_size, n_heads=cfg.num_attention_heads,
                                     n_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, bias=cfg.attention_bias)),
            feed_forward=("gated_mlp", dict(width=cfg.hidden_size, inner=cfg.intermediate_size,
                                            activation=cfg.hidden_act, bias=cfg.mlp_bias)),
        )
        for _ in range(cfg.num_hidden_layers)
    ]


def build_block(desc):
    norm_name, norm_args = desc["norm"]
    pos_name, pos_args = desc["position"]
    mixer_name, mixer_args = desc["mixer"]
    ffn_name, ffn_args = desc["feed_forward"]
    position = make_part("position", pos_name, **pos_args)
    return make_part(
        "block", desc["block"],
        mixer_norm=make_part("norm", norm_name, **norm_args),
        mixer=make_part("mixer", mixer_name, position=position, **mixer_args),
        ffn_norm=make_part("norm", norm_name, **norm_args),
        ffn=make_part("feed_forward", ffn_name, **ffn_args),
    )


def build_llama(cfg: LlamaConfig) -> DecoderModel:
    embedding = TokenEmbedding(cfg.vocab_size, cfg.hidden_size)
    head = LMHead(cfg.vocab_size, cfg.hidden_size, tied_to=embedding if cfg.tie_word_embeddings else None)
    blocks = [build_block(d) for d in layer_descriptors(cfg)]
    final_norm = make_part("norm", "rmsnorm", width=cfg.hidden_size, eps=cfg.rms_norm_eps)
    # older exports of this architecture still carry each layer's rotary frequencies as a buffer
    return DecoderModel(cfg, embedding, blocks, final_norm, head, ignored_tensors=("model.layers.*.self_attn.rotary_emb.inv_freq",))


register_architecture("LlamaForCausalLM", LlamaConfig, build_llama)
