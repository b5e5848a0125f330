"""B200-native framework for pretraining and serving depth-recurrent language models."""
__version__ = "0.1.0"

from .config import Config, ModelConfig  # noqa: F401
from .registry import name_to_config  # noqa: F401
