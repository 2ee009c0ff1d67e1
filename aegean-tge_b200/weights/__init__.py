"""Checkpoint reading, binding by name, and the random-weights mode."""
from .loader import WeightError, check_against_manifest, load_checkpoint, load_tensors, write_model_folder
from .draws import Draw, normal, tensor_key, uniform
from .random_init import fill_random, parse_dtype, random_tensor, random_tensors, write_random_model
from .safetensors_io import ModelFiles, SafetensorsFile, WeightFileError, write_safetensors

__all__ = ["WeightError", "check_against_manifest", "load_checkpoint", "load_tensors", "write_model_folder",
           "fill_random", "parse_dtype", "write_random_model", "random_tensor", "random_tensors", "Draw", "normal",
           "uniform", "tensor_key", "ModelFiles", "SafetensorsFile", "WeightFileError",
           "write_safetensors"]
