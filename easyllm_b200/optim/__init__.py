from .zero import ZeroOptimizer, DynamicLossScaler  # noqa
from .builder import build_optimizer  # noqa
from .lr import build_learning_rate_scheduler, IterBaseAnnealingLR, SampleBaseAnnealingLR, HFCosineLR  # noqa
from .microbatches import build_num_microbatches_calculator, get_train_iters  # noqa
from .sophia import SophiaG  # noqa
from .novograd import NovoGrad  # noqa
from .adam8bit import Adam8bit  # noqa
