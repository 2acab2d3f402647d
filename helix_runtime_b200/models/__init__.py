from . import llama  # noqa: F401  (registers the architecture)
from .decoder import Block, DecoderModel, register_arrangement
from .llama import build_llama_spec

__all__ = ["Block", "DecoderModel", "build_llama_spec", "register_arrangement"]
