from .loader import (FolderSource, RandomSource, WeightSource, WeightsMismatch, check_tensors,
                     draw_tensor, load_tensors, write_model_folder)
from .safetensors_io import SafetensorsFile, WeightsError, find_weight_files, write_safetensors

__all__ = ["FolderSource", "RandomSource", "WeightSource", "WeightsMismatch", "check_tensors",
           "draw_tensor", "load_tensors", "write_model_folder", "SafetensorsFile", "WeightsError",
           "find_weight_files", "write_safetensors"]
