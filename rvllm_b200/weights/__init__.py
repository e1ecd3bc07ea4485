from .safetensors_io import SafetensorsFile, write_safetensors, open_model_files
from .loader import WeightSource, engine_dtype_of
from .random_init import write_random_model, random_tensors
