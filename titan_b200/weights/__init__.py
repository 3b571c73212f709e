from .loader import DictWeights, FolderWeights, WeightError, WeightSource, WeightSpec, check_names, held_dtype
from .random_init import RandomWeights, make_tensor, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, write_safetensors

__all__ = ["DictWeights", "FolderWeights", "WeightError", "WeightSource", "WeightSpec", "check_names",
           "held_dtype", "RandomWeights", "make_tensor", "write_model_folder", "SafetensorsError",
           "SafetensorsFile", "open_model_files", "write_safetensors"]
