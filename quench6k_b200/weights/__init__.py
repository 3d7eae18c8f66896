from .loader import WeightError, check_against, load_folder
from .random_init import make_tensor, random_getter, write_model_folder, standard_normal
from .safetensors_io import SafetensorsError, SafetensorsFile, index_folder, write_safetensors
