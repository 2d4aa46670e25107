from .loader import WeightsError, check_checkpoint, load_weights, read_header
from .random_init import random_tensors, random_tensors_on_device, write_random_model
