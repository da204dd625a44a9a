"""Process-wide singleton: config, loggers, timer, tokenizer (reference: ironcore/global_vars.py:21-128)."""

from ironcore_b200.global_vars import (GlobalStates, get_config, get_logger, get_timer, get_tokenizer,  # noqa: F401
                                       log_histogram, log_metric, log_metrics, set_global_states)
from ironcore_b200.tokenizer import build_tokenizer  # noqa: F401
