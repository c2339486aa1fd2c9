"""GenerationConfig, streamers and the ModelForCausalLM entry point."""
from .config import GenerationConfig
from .streamer import AsyncTextStreamer, ListStreamer, TextStreamer, TokenStreamer

__all__ = ["GenerationConfig", "TokenStreamer", "ListStreamer", "TextStreamer", "AsyncTextStreamer",
           "ModelForCausalLM"]


def __getattr__(name):
    if name == "ModelForCausalLM":
        from .model import ModelForCausalLM
        return ModelForCausalLM
    raise AttributeError(name)
