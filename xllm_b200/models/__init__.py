from .config import ModelArgs, load_model_args, model_args_from_dict, preset  # noqa: F401
from .registry import create_model, register_model, supported_models  # noqa: F401
