from .loader import WeightError, load_model, load_weights_into
from .random_init import init_random, write_random_model
from .safetensors_io import SafetensorsFile, write_safetensors
