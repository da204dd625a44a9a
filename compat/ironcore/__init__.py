"""``ironcore``: the public names of haanjack/ironcore served by :mod:`ironcore_b200`.

A user of the reference can keep ``import ironcore`` / ``from ironcore.trainer import Trainer`` /
``from ironcore.parallel.parallel_states import get_tensor_model_parallel_rank`` and the ``ironcore``
console script; every module here is a thin re-export (no logic of its own). Where the reference's name
differs from the native one, the docstring of the re-export says which native object it is.
(Reference: ironcore/__init__.py:11-20.)"""

from ironcore_b200.global_vars import (get_config, get_logger, get_timer, get_tokenizer,  # noqa: F401
                                       set_global_states)

__all__ = ["get_config", "get_tokenizer", "set_global_states", "get_logger", "get_timer"]
