from .grid import *  # noqa
from .grid import get_grid, set_grid, grid_layout, ParallelGrid, initialize_distributed, initialize_model_parallel  # noqa
from .mappings import *  # noqa
from .data import broadcast_data  # noqa
from .buffers import get_global_memory_buffer, GlobalMemoryBuffer  # noqa
from .rng import set_random_seed, get_rng_tracker, get_cuda_rng_tracker, model_parallel_manual_seed  # noqa
