from .tokenizer import build_tokenizer, SimpleTokenizer  # noqa
from .parsers import *  # noqa
from .parsers import build_parser, build_transformer, build_augmentation, NLPCompose  # noqa
from .datasets import build_dataset, build_location_idx_py  # noqa
from .samplers import build_batch_sampler, InfiniteBatchSampler  # noqa
from .collators import BatchCollector, BatchAlignCollector, RewardBatchCollector, MiniRLHFBatchCollector  # noqa
from .loader import (build_data_loader, build_batch_collator, build_batch_pipe_fn, build_data_iterator,  # noqa
                     get_ltor_masks_and_position_ids)
from .synthetic import synthetic_batches, SyntheticTokenDataset  # noqa
from . import tokenizers_hf  # noqa
