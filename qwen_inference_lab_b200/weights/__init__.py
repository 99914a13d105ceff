from .loader import WeightError, load_weights
from .random_init import init_random, random_state, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
