from .safetensors_io import SafetensorsFolder, SafetensorsFile, SafetensorsError, write_safetensors
from .loader import WeightError, load_weights, load_model, check_folder
from .random_init import write_random_model, random_weights
