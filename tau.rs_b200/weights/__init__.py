from .loader import check_contract, device_dtype, load_weights
from .random_init import random_tensor, random_tensors, write_random_model
from .safetensors_io import SafetensorsFolder, TensorInfo, write_safetensors
from .tensor_spec import TensorSpec
