from .loader import (CheckpointSource, RandomSource, TensorDecl, WeightError,  # noqa: F401
                     WeightSource, check, materialize)
from .safetensors_io import Checkpoint, SafetensorsError, write_safetensors  # noqa: F401
