from .executor import Executor, StepEntry, StepError  # noqa: F401
from .runtime import Runtime, load_model, parse_dtype  # noqa: F401
