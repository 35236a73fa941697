from .expected import expected_tensors, tensor_names  # noqa: F401
from .loader import WeightError, load_weights  # noqa: F401
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors  # noqa: F401


def __getattr__(name):
    # random_init is also a program (python -m shrike_b200.weights.random_init): import it on demand
    if name in ("random_tensors", "random_tensor", "write_model_folder"):
        from . import random_init

        return getattr(random_init, name)
    raise AttributeError(name)
