"""Weights: safetensors by tensor name, manifest check, random weights."""
from .loader import TensorSpec, WeightsError, load_weights, open_folder
from .safetensors_io import (DictSource, SafetensorsError, SafetensorsFile, TensorSource,
                             model_files, save_file)

__all__ = ["TensorSpec", "WeightsError", "load_weights", "open_folder", "DictSource",
           "SafetensorsError", "SafetensorsFile", "TensorSource", "model_files", "save_file"]
