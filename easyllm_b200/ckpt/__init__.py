from .layer_files import save_engine_checkpoint, load_engine_checkpoint, layer_file, read_latest  # noqa
from .helper import load_checkpoint, save_checkpoint  # noqa
