"""Weight sources: safetensors by tensor name, seeded random weights, model folders."""
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from .store import (RandomWeightStore, WeightError, WeightStore, random_store, random_tensors,
                    write_model_folder)

__all__ = ["SafetensorsError", "SafetensorsFile", "write_safetensors", "WeightError",
           "WeightStore", "RandomWeightStore", "random_store", "random_tensors", "write_model_folder"]
