from .config import ModelConfig, get_config  # noqa: F401
from .registry import build_model, get_model_class, register_model  # noqa: F401
