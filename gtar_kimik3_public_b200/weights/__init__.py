"""Model folders: safetensors by tensor name, the loader's checks, the random-weights mode."""

from .loader import WeightsError, load_weights  # noqa: F401
from .random_init import load_random_weights, write_random_model  # noqa: F401
from .safetensors_io import ModelFolderTensors, SafetensorsError, SafetensorsFile, write_safetensors  # noqa: F401
