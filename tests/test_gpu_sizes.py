"""Every size that config.json allows goes through the engine and comes out right.

The tiny configurations of the replay tests have head sizes 16, 32 and 48.  Here the
whole engine (mixed steps, decoded tokens beside portions, pages used again) runs on
configurations whose sizes the kernels may not like: head sizes that are no multiple
of 16 (2, 6, 20, 40, 72), every multiple of 16 up to 256, groups of 3, 5, 7, 9 and 12
query heads per key head, H * D far from the width, widths, inner sizes and
vocabularies that are no multiple of anything (34, 35, 33, 1001), with and without
biases, tied head, and the three kinds of rotary scaling.  A kernel that cannot take
a size has to refuse it with an error; none of these is refused today, so a refusal
fails the test like a wrong logit does.
"""
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu

LLAMA3 = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
LINEAR = {"rope_type": "linear", "factor": 3.5}

#         D   heads kv  width inner vocab layers  scaling  attention_bias mlp_bias tied
SIZES = [(2, 4, 1, 66, 176, 64, 1, LLAMA3, False, False, False),
         (6, 15, 5, 50, 96, 100, 2, None, True, False, False),
         (20, 6, 3, 64, 200, 100, 1, None, False, False, True),
         (40, 60, 5, 256, 96, 1001, 1, LINEAR, False, True, True),
         (72, 14, 2, 34, 96, 64, 1, LINEAR, True, False, True),
         (80, 24, 3, 120, 512, 64, 3, None, True, False, False),
         (96, 4, 1, 34, 130, 331, 1, LINEAR, False, False, False),
         (112, 21, 3, 34, 333, 256, 1, None, False, False, True),
         (128, 35, 5, 50, 200, 1001, 3, LINEAR, False, False, False),
         (144, 9, 1, 120, 64, 1001, 2, None, False, True, False),
         (160, 10, 5, 66, 35, 33, 2, None, True, False, False),
         (192, 25, 5, 96, 512, 331, 2, None, False, True, False),
         (256, 24, 2, 130, 333, 33, 2, LLAMA3, True, True, False),
         (8, 7, 1, 1000, 200, 256, 2, None, False, True, False)]


def config_of(row):
    D, heads, kv, width, inner, vocab, layers, scaling, abias, mbias, tied = row
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": layers, "hidden_size": width,
            "num_attention_heads": heads, "num_key_value_heads": kv, "head_dim": D, "intermediate_size": inner, "vocab_size": vocab,
            "rope_theta": 10000.0 if D < 100 else 777.0, "rope_scaling": scaling, "rms_norm_eps": 1e-5 if layers > 1 else 3e-4,
            "tie_word_embeddings": tied, "attention_bias": abias, "mlp_bias": mbias, "max_position_embeddings": 200, "hidden_act": "silu"}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("row", SIZES, ids=lambda r: f"D{r[0]}-H{r[1]}-kv{r[2]}-E{r[3]}-F{r[4]}-V{r[5]}")
def test_sizes_under_the_mixed_schedule(row, dtype, tmp_path):
    from lgml_b200.engine.engine import parse_dtype
    from lgml_b200.engine.runner import ModelRunner

    cfg = config_of(row)
    width = cfg["hidden_size"]
    # attention sharpened as in the replay tests, less for a wide model (its q and k are longer sums)
    sharpen = max(1.0, {"float32": 8.0, "bfloat16": 4.0}[dtype] * (64.0 / width) ** 0.5)
    folder = H.make_folder(tmp_path, cfg, seed=row[0] + row[1], dtype=dtype, sharpen=sharpen)
    lens = [65, 2, 129, 64, 200, 1, 63]
    seqs = {f"r{i}": H.random_ids(n, cfg["vocab_size"], 300 + 7 * i + row[0]) for i, n in enumerate(lens)}
    max_tokens = 64 * 6                                    # the longest request needs 4 pages; all of them would need 13
    trace = H.trace_mixed(seqs, max_tokens=max_tokens, seed=row[0], max_live=4, choices=(1, 1, 2, 2, 5, 17, 40, 64, 90), tail=12, skip=0.2)
    runner = ModelRunner.from_folder(folder, parse_dtype(dtype), "cuda:0", n_pages=max_tokens // 64, max_slots=4)
    got = H.run_trace(runner, trace)
    assert runner.cache.groups[0].pool.taken_total > runner.cache.groups[0].pool.n_pages      # pages were used again
    if dtype == "float32":
        tol = dict(atol=3e-5, rtol=1e-4)
    else:
        # bfloat16 rounds to 2^-9 of a value's size: the bound of the replay tests, for logits of
        # size ~1, grows with the logits of a wide model (width 1000: about three times as large)
        span = max(float(H.oracle_logits(folder, ids).abs().max()) for ids in seqs.values())
        tol = dict(atol=1.5e-2 * max(1.0, span / 2.0), rtol=1.5e-2)
    H.compare_with_oracle(got, folder, seqs, **tol)
