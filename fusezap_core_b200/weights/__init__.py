from .params import ParamSpec
from .safetensors_io import read_file, read_model_dir, write_file, read_header, SafetensorsError
from .loader import load_weights, check_tensors, WeightsError
from .random_weights import write_random_model, random_tensors

__all__ = ["ParamSpec", "read_file", "read_model_dir", "write_file", "read_header", "SafetensorsError", "load_weights",
           "check_tensors", "WeightsError", "write_random_model", "random_tensors"]
