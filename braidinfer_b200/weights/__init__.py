"""Weights: the safetensors container, loading by tensor name, random model folders."""
from .loader import RoundedWeightsWarning, UnexpectedTensorsWarning, WeightsError, load_tensors
from .random_init import draw_tensors, tensor_specs_of, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_folder, save_file
