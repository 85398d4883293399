from .yaml_loader import load_yaml, apply_overwrites, clear_include_cache  # noqa
from .cfg_helper import merge_opts_into_cfg, try_decode  # noqa
from .parser import parse_args, build_parser  # noqa
from .registry import *  # noqa
