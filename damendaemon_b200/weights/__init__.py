from .loader import DictSource, WeightError, check_and_place, load_weights
from .random_init import write_random_model
from .safetensors_io import CheckpointFormatError, SafetensorsFile, read_header, write_safetensors

__all__ = ["DictSource", "WeightError", "check_and_place", "load_weights", "write_random_model",
           "CheckpointFormatError", "SafetensorsFile", "read_header", "write_safetensors"]
