from .loader import WeightError, check_rules, load_weights, storage_dtype
from .plan import Source, TensorRule, single
from .random_init import random_device_weights, random_file_tensors, write_model_folder
