"""Checkpoint reading by tensor name, and the random-weights mode."""
from .loader import check_against, load_folder, load_tensors  # noqa: F401
from .random_init import random_tensors, write_model_folder  # noqa: F401
from .safetensors_io import Checkpoint, SafetensorsFile, write_safetensors  # noqa: F401
