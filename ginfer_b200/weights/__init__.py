from .loader import WeightError, load_weights
from .random_init import load_random_weights, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
