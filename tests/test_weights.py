"""safetensors reader and writer, loader errors, random-weights mode (no GPU)."""
import json
import struct

import pytest
import torch

from lgml_b200.config import config_from_dict
from lgml_b200.models import tensor_specs_for
from lgml_b200.weights import (SafetensorsError, TensorSpec, WeightError, check_index, index_folder, load_tensors, read_index,
                               read_tensor, write_random_model, write_safetensors)
from tests import helpers as H
from tests.plain import llama_plain as P


def raw_file(path, header: dict, data: bytes = b"", hlen=None):
    h = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(h) if hlen is None else hlen) + h + data)
    return path


def test_write_then_read_every_type(tmp_path):
    tensors = {
        "a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
        "d": torch.randn(2, 2, 2).double(), "e": torch.randn(4).half(), "f": torch.arange(3, dtype=torch.int64),
    }
    write_safetensors(tmp_path / "model.safetensors", tensors)
    idx = read_index(tmp_path / "model.safetensors")
    assert list(idx) == list(tensors)
    for name, t in tensors.items():
        got = read_tensor(idx[name])
        assert got.dtype == t.dtype and torch.equal(got, t)
    # the independent reader of the plain implementation sees the same values
    plain = P.read_safetensors(tmp_path / "model.safetensors")
    assert torch.equal(plain["b"], tensors["b"].double())


@pytest.mark.parametrize("header,data,hlen,match", [
    ({"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4, None, "do not fit"),      # data too short
    ({"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 8, None, "do not fit"),      # size mismatch
    ({"x": {"dtype": "F32", "shape": [2], "data_offsets": [4, 0]}}, b"\0" * 8, None, "do not fit"),      # begin > end
    ({"x": {"dtype": "Q8", "shape": [2], "data_offsets": [0, 2]}}, b"\0" * 2, None, "unsupported dtype"),
    ({"x": {"dtype": "F32", "shape": [1, 1, 1, 1, 1], "data_offsets": [0, 4]}}, b"\0" * 4, None, "bad shape"),
    ({"x": {"dtype": "F32", "shape": [0], "data_offsets": [0, 0]}}, b"", None, "bad shape"),
    ({"y" * 64: {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4, None, "bad tensor name"),
    ({"x": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4, 1 << 40, "bad header length"),
    ({"x": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4, 1, "bad header length"),
])
def test_malformed_files_are_refused(tmp_path, header, data, hlen, match):
    f = raw_file(tmp_path / "model.safetensors", header, data, hlen)
    with pytest.raises(SafetensorsError, match=match):
        read_index(f)


def test_header_reader_is_strict_json(tmp_path):
    """The host library's own JSON reader: escapes in names, metadata of any shape skipped,
    and the faults a lenient reader would let through."""
    def raw(text: bytes, data: bytes = b"\0" * 4):
        f = tmp_path / "h.safetensors"
        f.write_bytes(struct.pack("<Q", len(text)) + text + data)
        return f

    ok = b'{"__metadata__": {"a": [1, 2.5e3, {"b": null}], "c": true}, "w\\u00e9\\n": {"dtype":"F32","shape":[1],"data_offsets":[0,4], "extra": -0.5}}   '
    idx = read_index(raw(ok))
    assert list(idx) == ["w\u00e9\n"] and idx["w\u00e9\n"].shape == (1,)
    entry = b'{"dtype":"F32","shape":[1],"data_offsets":[0,4]}'
    for text, match in [
        (b'{"x": ' + entry + b', "x": ' + entry + b'}', "twice"),
        (b'{"x": ' + entry + b'} trailing', "not JSON"),
        (b'{"x": ' + entry + b',}', "not JSON"),
        (b"{'x': " + entry + b'}', "not JSON"),
        (b'{"x": {"dtype":"F32","shape":[1.0],"data_offsets":[0,4]}}', "bad shape"),
        (b'{"x": {"dtype":"F32","shape":[1],"data_offsets":[0,"4"]}}', "bad data_offsets"),
        (b'{"x": {"dtype":"F32","shape":[1],"data_offsets":[0,4,8]}}', "bad data_offsets"),
        (b'{"x": {"dtype":"F32","shape":[4611686018427387904, 4],"data_offsets":[0,4]}}', "do not fit"),
        (b'{"x": [1, 2]}', "must be an object"),
        (b'[1]', "not JSON"),
        (b'{"x\xff": ' + entry + b'}', "not JSON"),                                  # not UTF-8
        (b'{"x": ' + b'[' * 64 + b']' * 64 + b'}', "not JSON"),
    ]:
        with pytest.raises(SafetensorsError, match=match):
            read_index(raw(text))


def test_truncated_and_not_json(tmp_path):
    (tmp_path / "a.safetensors").write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="shorter"):
        read_index(tmp_path / "a.safetensors")
    (tmp_path / "b.safetensors").write_bytes(struct.pack("<Q", 5) + b"nope!")
    with pytest.raises(SafetensorsError, match="not JSON"):
        read_index(tmp_path / "b.safetensors")


def test_folder_rules(tmp_path):
    with pytest.raises(SafetensorsError, match="no safetensors"):
        index_folder(tmp_path)
    write_safetensors(tmp_path / "one.safetensors", {"w": torch.ones(2)})
    write_safetensors(tmp_path / "two.safetensors", {"w": torch.ones(2)})
    with pytest.raises(SafetensorsError, match="both"):
        index_folder(tmp_path)
    (tmp_path / "two.safetensors").unlink()
    write_safetensors(tmp_path / "two.safetensors", {"v": torch.ones(3)})
    assert set(index_folder(tmp_path)) == {"w", "v"}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"w": "one.safetensors"}}))
    assert set(index_folder(tmp_path)) == {"w"}


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(H.TINY_A)
    folder = write_random_model(tmp_path, cfg, seed=0, dtype="float32")
    idx = index_folder(folder)
    tensors = {n: read_tensor(e) for n, e in idx.items()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    tensors["model.layers.0.self_attn.extra.weight"] = torch.ones(3)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.ones(64, 32)
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(WeightError) as ei:
        load_tensors(folder, tensor_specs_for(cfg), torch.float32, "cpu")
    e = ei.value
    assert set(e.missing) == {"model.layers.1.mlp.up_proj.weight", "model.norm.weight"}
    assert e.unexpected == ["model.layers.0.self_attn.extra.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]
    # the architecture's builder names what a folder may carry unread (old exports keep each layer's
    # rotary frequencies as a buffer): that one is no fault, the other still is
    from lgml_b200.models import build_model
    with pytest.raises(WeightError) as ei2:
        load_tensors(folder, tensor_specs_for(cfg), torch.float32, "cpu", ignore=build_model(cfg).ignored_tensors)
    assert ei2.value.unexpected == ["model.layers.0.self_attn.extra.weight"]
    assert [w[0] for w in e.wrong_shape] == ["model.layers.0.self_attn.q_proj.weight"]
    msg = str(e)
    for name in e.missing + e.unexpected:
        assert name in msg
    assert "(64, 32)" in msg and "(64, 64)" in msg


def test_tied_head_and_optional_tensors(tmp_path):
    cfg = config_from_dict(H.TINY_A)                       # tied: no lm_head in the folder
    folder = write_random_model(tmp_path / "a", cfg, seed=0, dtype="float32")
    names = set(index_folder(folder))
    assert "lm_head.weight" not in names and "rope_freqs.weight" not in names
    load_tensors(folder, tensor_specs_for(cfg), torch.float32, "cpu")          # optional factors may be absent
    # a tied folder that still carries a head of its own is taken, and that head is the one used
    # (the reference takes ``output.weight`` whenever the file has it, ``lua/lgml/transformer.lua:408``)
    tensors = {n: read_tensor(e) for n, e in index_folder(folder).items()}
    tensors["lm_head.weight"] = torch.full((256, 64), 0.5)
    write_safetensors(folder / "model.safetensors", tensors)
    got = load_tensors(folder, tensor_specs_for(cfg), torch.float32, "cpu")
    assert torch.equal(got["lm_head.weight"], tensors["lm_head.weight"])
    from lgml_b200.models import build_model
    model = build_model(cfg)

    class Rt:
        device, dtype = torch.device("cpu"), torch.float32
    model.head.bind("", got, Rt)
    assert model.head.weight is got["lm_head.weight"]
    del got["lm_head.weight"]
    model.embedding.bind("", got, Rt)
    model.head.bind("", got, Rt)
    assert model.head.weight is model.embedding.table
    cfg_b = config_from_dict(H.TINY_B)
    names_b = set(index_folder(write_random_model(tmp_path / "b", cfg_b, seed=1, dtype="float32")))
    assert "lm_head.weight" in names_b and "model.layers.2.self_attn.k_proj.bias" in names_b


def test_types_kept(tmp_path):
    cfg = config_from_dict(H.TINY_B)
    folder = write_random_model(tmp_path, cfg, seed=1, dtype="bfloat16")
    idx = index_folder(folder)
    assert idx["model.layers.0.mlp.up_proj.weight"].dtype == "BF16"
    assert idx["model.norm.weight"].dtype == "F32"
    t = load_tensors(folder, tensor_specs_for(cfg), torch.bfloat16, "cpu")
    assert t["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16      # a matrix stays bfloat16
    assert t["model.norm.weight"].dtype == torch.float32                       # stored in 32-bit, stays so
    assert t["model.layers.0.self_attn.q_proj.bias"].dtype == torch.float32
    t32 = load_tensors(folder, tensor_specs_for(cfg), torch.float32, "cpu")
    assert all(v.dtype == torch.float32 for v in t32.values())
    # an integer table becomes int32
    write_safetensors(tmp_path / "x.safetensors", {"table": torch.arange(4, dtype=torch.int64)})
    (tmp_path / "model.safetensors").unlink()
    got = load_tensors(tmp_path, [TensorSpec("table", (4,), "int")], torch.bfloat16, "cpu")
    assert got["table"].dtype == torch.int32


def test_random_weights_are_seeded_and_shaped(tmp_path):
    cfg = config_from_dict(H.TINY_B)
    a = write_random_model(tmp_path / "a", cfg, seed=1, dtype="float32")
    b = write_random_model(tmp_path / "b", cfg, seed=1, dtype="float32")
    c = write_random_model(tmp_path / "c", cfg, seed=2, dtype="float32")
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    _, w = P.load_folder(a)
    big = w["model.layers.0.mlp.gate_proj.weight"]
    assert abs(float(big.mean())) < 2e-3 and abs(float(big.std()) - 0.02) < 2e-3
    norm = w["model.layers.1.input_layernorm.weight"]
    assert abs(float(norm.mean()) - 1.0) < 0.02
    assert json.loads((a / "config.json").read_text())["num_key_value_heads"] == 2
    check_index(index_folder(a), tensor_specs_for(cfg))


def test_header_reader_agrees_with_a_json_library_and_survives_damage(tmp_path):
    """Random well-formed headers (names with escapes and other alphabets, metadata of any shape)
    give the index a JSON library gives; the same headers with bytes damaged either still parse
    or are refused with SafetensorsError, never anything else."""
    from hypothesis import given, settings, strategies as st

    names = st.text(alphabet=st.characters(blacklist_categories=("Cs",), blacklist_characters="\0"), min_size=1, max_size=12).filter(
        lambda n: len(n.encode()) <= 63 and n != "__metadata__")
    meta = st.recursive(st.none() | st.booleans() | st.integers(-10**6, 10**6) | st.floats(allow_nan=False, allow_infinity=False) | st.text(max_size=5),
                        lambda c: st.lists(c, max_size=3) | st.dictionaries(st.text(max_size=4), c, max_size=3), max_leaves=8)
    f = tmp_path / "fuzz.safetensors"

    @settings(max_examples=60, deadline=None)
    @given(st.dictionaries(names, st.lists(st.integers(1, 5), max_size=4), max_size=6), meta, st.booleans(), st.data())
    def run(shapes, metadata, ascii_only, data):
        header, off = {"__metadata__": {"m": metadata}}, 0
        for name, shape in shapes.items():
            n = 1
            for d in shape:
                n *= d
            header[name] = {"dtype": "I16", "shape": shape, "data_offsets": [off, off + 2 * n]}
            off += 2 * n
        text = json.dumps(header, ensure_ascii=ascii_only).encode()
        f.write_bytes(struct.pack("<Q", len(text)) + text + b"\0" * off)
        idx = read_index(f)
        assert {k: v.shape for k, v in idx.items()} == {k: tuple(v) for k, v in shapes.items()}
        # damage: a few bytes of the header replaced
        raw = bytearray(text)
        for _ in range(data.draw(st.integers(1, 3))):
            raw[data.draw(st.integers(0, len(raw) - 1))] = data.draw(st.integers(0, 255))
        f.write_bytes(struct.pack("<Q", len(raw)) + bytes(raw) + b"\0" * off)
        try:
            read_index(f)
        except SafetensorsError:
            pass

    run()
