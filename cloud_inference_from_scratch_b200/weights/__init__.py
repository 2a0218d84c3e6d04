from .loader import check_tensors, device_tensors
from .random_init import write_random_model
from .source import RandomSource, SafetensorsSource, WeightsError

__all__ = [
    "RandomSource", "SafetensorsSource", "WeightsError", "check_tensors", "device_tensors",
    "write_random_model",
]
