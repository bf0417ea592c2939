"""Model builders.  Importing this package registers the architectures it holds."""
from ..config import lookup_architecture
from .decoder import DecoderModel, LayerCall
from . import llama  # noqa: F401  (registers LlamaForCausalLM)


def build_model(config):
    """The assembled (unbound) model of a configuration."""
    _, builder = lookup_architecture(config.architecture)
    return builder(config)


def tensor_specs_for(config):
    return build_model(config).tensor_specs()


__all__ = ["DecoderModel", "LayerCall", "build_model", "tensor_specs_for"]
