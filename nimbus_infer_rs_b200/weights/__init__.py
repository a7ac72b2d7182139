from .loader import (Recipe, Source, TensorDict, WeightError, WeightPlan, find_weight_file,
                     load_params, target_dtype)
from .safetensors_io import SafeTensorsError, SafeTensorsFile, write_safetensors
from .random_init import write_random_model
