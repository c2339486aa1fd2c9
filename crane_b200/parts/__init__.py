"""Parts of a decoder and their registries."""
from .base import (CacheNeed, LayerCache, Part, Workspace, block_class, build_part, part_class,
                   register_block, register_part)
from .runtime import DeviceFault, Runtime
from . import attention, block, embedding, feed_forward, norm, position   # register the parts
from .model import DecoderModel, model_manifest

__all__ = ["CacheNeed", "LayerCache", "Part", "Workspace", "block_class", "build_part",
           "part_class", "register_block", "register_part", "Runtime", "DeviceFault",
           "DecoderModel", "model_manifest"]
