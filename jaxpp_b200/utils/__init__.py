from .config import (BoolEnvVar, EnvVar, IntEnvVar, OverwriteableVar, StrEnvVar, parse_bool)
from .misc import (format_bytes, groupby, hbytes, log_elapsed_time, logger, partition,
                   unique_in_order, unzip_multi)
