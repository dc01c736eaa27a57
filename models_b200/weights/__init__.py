from .loader import ParamRequest, WeightsError, check_names_and_shapes, load_tensors
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
