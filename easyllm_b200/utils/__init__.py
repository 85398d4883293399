from .log import default_logger, init_log, is_master  # noqa
from .timers import Timers, DeviceTimer, report_memory  # noqa
