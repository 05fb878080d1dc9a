from .loader import WeightError, check_names, init_random, load_weights, write_random_model
from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, write_safetensors
