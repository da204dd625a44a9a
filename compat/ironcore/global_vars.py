"""Process-wide singleton: config, loggers, timer, tokenizer (reference: ironcore/global_vars.py:21-128)."""

from ironcore_b200.global_vars import (GlobalStates, get_config, get_global_states, get_logger,  # noqa: F401
                                       get_timer, get_tokenizer, global_states_cleanup, log_histogram, log_metric,
                                       log_metrics, set_global_states)
from ironcore_b200.tokenizer import build_tokenizer  # noqa: F401
