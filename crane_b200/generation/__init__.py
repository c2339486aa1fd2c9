"""GenerationConfig, streamers and the ModelForCausalLM entry point."""
from .chat import apply_chat_template, format_chat
from .config import GenerationConfig
from .streamer import AsyncTextStreamer, ListStreamer, TextStreamer, TokenStreamer

__all__ = ["GenerationConfig", "TokenStreamer", "ListStreamer", "TextStreamer", "AsyncTextStreamer",
           "ModelForCausalLM", "apply_chat_template", "format_chat"]


def __getattr__(name):
    if name == "ModelForCausalLM":
        from .model import ModelForCausalLM
        return ModelForCausalLM
    raise AttributeError(name)
