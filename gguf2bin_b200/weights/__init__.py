"""Weights: safetensors reading/writing, by-name binding with one clear error, and the
random-weights model writer."""
from .safetensors_io import SafetensorsFile, WeightsError, open_model_files, write_safetensors
from .loader import Expected, check_names_and_shapes, load_weights, runtime_dtype
from .random_init import (fill_random_on_device, normal_values, random_tensor,
                          random_tensors_on_device, write_random_model)

__all__ = ["SafetensorsFile", "WeightsError", "open_model_files", "write_safetensors", "Expected",
           "check_names_and_shapes", "load_weights", "runtime_dtype", "random_tensor", "normal_values",
           "fill_random_on_device", "random_tensors_on_device",
           "write_random_model"]
