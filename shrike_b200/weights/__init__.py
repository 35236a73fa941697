from .expected import expected_tensors, tensor_names  # noqa: F401
from .loader import WeightError, load_weights  # noqa: F401
from .random_init import random_tensors, write_model_folder  # noqa: F401
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors  # noqa: F401
