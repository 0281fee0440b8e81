from .spec import MATRIX, NORM, TensorSource, WeightError, WeightSpec
from .loader import SafetensorsSource, check_against_manifest
from .random_weights import RandomSource, write_model_folder

__all__ = ["MATRIX", "NORM", "TensorSource", "WeightError", "WeightSpec", "SafetensorsSource",
           "check_against_manifest", "RandomSource", "write_model_folder"]
