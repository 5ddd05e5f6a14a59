from .loader import Fetcher, ParamSpec, WeightError, check_names
from .safetensors_file import SafetensorsError, SafetensorsFile, write_safetensors
from .sources import FolderSource, RandomSource

__all__ = ["Fetcher", "ParamSpec", "WeightError", "check_names", "SafetensorsError",
           "SafetensorsFile", "write_safetensors", "FolderSource", "RandomSource"]
