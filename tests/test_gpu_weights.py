"""The upload of weights: file -> pinned chunks -> device gives the bytes a plain read gives."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_staged_upload_equals_a_plain_read(tmp_path):
    from lgml_b200.weights import index_folder, read_tensor, write_safetensors
    from lgml_b200.weights.loader import StagedUpload

    g = torch.Generator().manual_seed(0)
    tensors = {"big": torch.randn(301, 77, generator=g).to(torch.bfloat16), "odd": torch.randn(1001, generator=g),
               "one": torch.randn(1, generator=g), "ids": torch.arange(5000, dtype=torch.int64),
               "exact": torch.randn(250, generator=g)}                    # 1000 bytes: exactly one chunk
    write_safetensors(tmp_path / "model.safetensors", tensors)
    idx = index_folder(tmp_path)
    up = StagedUpload("cuda:0", stage_bytes=1000)                         # many chunks, the last one short
    for name, want in tensors.items():
        got = up.upload(idx[name])
        assert got.dtype == want.dtype and got.shape == want.shape
        assert torch.equal(got.cpu(), read_tensor(idx[name])) and torch.equal(got.cpu(), want), name
    up.finish()
    assert up.bytes == sum(t.numel() * t.element_size() for t in tensors.values())


def test_loader_converts_on_the_device(tmp_path):
    from lgml_b200.config import config_from_dict
    from lgml_b200.models import tensor_specs_for
    from lgml_b200.weights import load_tensors, write_random_model
    from tests import helpers as H

    cfg = config_from_dict(H.TINY_B)
    folder = write_random_model(tmp_path, cfg, seed=1, dtype="float32")
    on_dev = load_tensors(folder, tensor_specs_for(cfg), torch.bfloat16, "cuda:0")
    on_host = load_tensors(folder, tensor_specs_for(cfg), torch.bfloat16, "cpu")
    assert set(on_dev) == set(on_host)
    for name, t in on_host.items():
        assert on_dev[name].dtype == t.dtype and torch.equal(on_dev[name].cpu(), t), name
