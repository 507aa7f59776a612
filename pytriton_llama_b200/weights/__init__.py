from .loader import WeightError, check_tensors  # noqa: F401
from .random_init import random_tensors, write_random_model  # noqa: F401
from .safetensors_io import SafetensorsError, read_file, read_folder, write_file  # noqa: F401
