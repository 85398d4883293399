from .config import ModelArgs, update_model_cfg, LLAMA_PRESETS  # noqa
from .llama import LlamaModelPipe, StageIO, build_model, get_layer_info, llama_custom  # noqa
from . import losses  # noqa
